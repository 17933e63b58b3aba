"""Callers of the hot path that the reference keeps in ``jla.layers``: the Mamba-2 SSD mapping, the q / k prologue
(short convolution + SiLU + L2 norm), the gate activations of the Gated DeltaNet / KDA mixers and their gated output
norm."""
from .conv import short_conv  # noqa: F401
from .gates import gate_prologue  # noqa: F401
from .norm import gated_rms_norm  # noqa: F401
from .ssm import mamba2_ssd  # noqa: F401
