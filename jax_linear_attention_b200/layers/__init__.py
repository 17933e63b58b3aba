"""Callers of the hot path that the reference keeps in ``jla.layers``: the Mamba-2 SSD mapping."""
from .ssm import mamba2_ssd  # noqa: F401
