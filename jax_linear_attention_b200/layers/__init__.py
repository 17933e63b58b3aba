"""Callers of the hot path that the reference keeps in ``jla.layers``: the Mamba-2 SSD mapping, the gate
activations of the Gated DeltaNet / KDA mixers and their gated output norm."""
from .gates import gate_prologue  # noqa: F401
from .norm import gated_rms_norm  # noqa: F401
from .ssm import mamba2_ssd  # noqa: F401
