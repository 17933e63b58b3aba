"""Gated RMS norm after the linear-attention kernels (mirror of ``GatedRMSNorm`` in the reference's
``src/jla/layers/norm.py:60-112``), one fused CUDA pass forward and one backward (``jla_gated_rmsnorm_fwd/bwd``).

``norm_before_gate=True``: ``rms_norm(x) * weight * act(z)`` (Gated DeltaNet with ``activation="silu"``, KDA with
``"sigmoid"``); ``False``: ``rms_norm(x * act(z)) * weight`` (Mamba-2). ``group_size`` normalises each group of that
many consecutive channels of the last axis on its own (``None``: the whole axis). Computed in float32, returned in
``x``'s dtype.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _call(name, x, *args):
    lib = _lib.load()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        _lib.check(getattr(lib, name)(*args, C.c_void_p(stream)), name)


def _ptr(t):
    return C.c_void_p(t.data_ptr())


class _GatedRMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, z, weight, eps, sigmoid_gate, norm_before_gate, group):
        dim = x.shape[-1]
        rows = x.numel() // dim
        y = torch.empty_like(x)
        _call("jla_gated_rmsnorm_fwd", x, _DTYPES[x.dtype], C.c_int64(rows), dim, group, _ptr(x), _ptr(z), _ptr(weight),
              C.c_float(eps), int(sigmoid_gate), int(norm_before_gate), _ptr(y))
        ctx.save_for_backward(x, z, weight)
        ctx.cfg = (eps, sigmoid_gate, norm_before_gate, group)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        x, z, weight = ctx.saved_tensors
        eps, sigmoid_gate, norm_before_gate, group = ctx.cfg
        dim = x.shape[-1]
        rows = x.numel() // dim
        dy = dy.contiguous()
        dx, dz, dw = torch.empty_like(x), torch.empty_like(z), torch.empty_like(weight)
        _call("jla_gated_rmsnorm_bwd", x, _DTYPES[x.dtype], C.c_int64(rows), dim, group, _ptr(x), _ptr(z), _ptr(weight),
              C.c_float(eps), int(sigmoid_gate), int(norm_before_gate), _ptr(dy), _ptr(dx), _ptr(dz), _ptr(dw))
        return dx, dz, dw, None, None, None, None


def gated_rms_norm(x, z, weight, *, eps: float = 1e-6, activation: str = "silu", norm_before_gate: bool = True,
                   group_size: int | None = None):
    """``GatedRMSNorm(dim, eps=..., activation=..., norm_before_gate=..., group_size=...)(x, z)`` with ``weight [dim]``."""
    if activation not in ("silu", "sigmoid"):
        raise ValueError(f"unsupported gate activation {activation!r}")
    if z.shape != x.shape:
        raise ValueError(f"gate shape {tuple(z.shape)} must match input shape {tuple(x.shape)}")
    dim = x.shape[-1]
    group = group_size or dim
    if group < 1 or dim % group:
        raise ValueError(f"group_size {group_size} must divide dim {dim}")
    if weight.shape != (dim,):
        raise ValueError(f"weight must be [{dim}]; got {tuple(weight.shape)}")
    if not x.is_cuda:
        raise ValueError("gated_rms_norm runs on CUDA tensors only: the 'cuda' implementation has no CPU fallback")
    if x.dtype not in _DTYPES or z.dtype != x.dtype:
        raise ValueError(f"x and z must share one of {sorted(str(d) for d in _DTYPES)}; got {x.dtype}, {z.dtype}")
    return _GatedRMSNorm.apply(x.contiguous(), z.contiguous(), weight.float().contiguous(), float(eps),
                               activation == "sigmoid", bool(norm_before_gate), int(group))
