"""Gate activations of the Gated DeltaNet and KDA mixers (mirror of ``_mamba_gate`` and ``_write_strength`` in the
reference's ``src/jla/layers/linear_attention.py:84-86, 159-162``), fused into one CUDA pass forward and one
backward (``jla_gate_prologue_fwd/bwd``):

``g = -exp(A_log) * softplus(a + dt_bias)`` in float32 with ``a [B, T, H]`` (one decay per head, ``dt_bias [H]``)
or ``a [B, T, H, K]`` (KDA: ``dt_bias [H, K]``), ``A_log [H]``; ``beta = sigmoid(b)``, doubled when
``allow_neg_eigval``. The results feed ``ops.linear_attention`` as ``g`` and ``beta``.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _call(name: str, a: torch.Tensor, *args):
    lib = _lib.load()
    stream = torch.cuda.current_stream(a.device).cuda_stream
    with torch.cuda.device(a.device):
        _lib.check(getattr(lib, name)(*args, C.c_void_p(stream)), name)


def _ptr(t):
    return C.c_void_p(None if t is None else t.data_ptr())


class _GatePrologue(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, a_log, dt_bias, b, allow_neg: bool):
        heads = a.shape[2]
        width = a.shape[3] if a.ndim == 4 else 1
        tokens = a.shape[0] * a.shape[1]
        g = torch.empty(a.shape, dtype=torch.float32, device=a.device)
        beta = None if b is None else torch.empty(b.shape, dtype=torch.float32, device=a.device)
        _call("jla_gate_prologue_fwd", a, _DTYPES[a.dtype], C.c_int64(tokens), heads, width, _ptr(a), _ptr(a_log),
              _ptr(dt_bias), _ptr(b), int(allow_neg), _ptr(g), _ptr(beta))
        ctx.save_for_backward(a, a_log, dt_bias, b)
        ctx.allow_neg = allow_neg
        return g, beta

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dg, dbeta):
        a, a_log, dt_bias, b = ctx.saved_tensors
        heads = a.shape[2]
        width = a.shape[3] if a.ndim == 4 else 1
        tokens = a.shape[0] * a.shape[1]
        dg = torch.zeros(a.shape, dtype=torch.float32, device=a.device) if dg is None else dg.float().contiguous()
        if b is not None:
            dbeta = torch.zeros(b.shape, dtype=torch.float32, device=a.device) if dbeta is None else dbeta.float().contiguous()
        da = torch.empty_like(a)
        db = None if b is None else torch.empty_like(b)
        da_log = torch.empty_like(a_log)
        ddt_bias = torch.empty_like(dt_bias)
        _call("jla_gate_prologue_bwd", a, _DTYPES[a.dtype], C.c_int64(tokens), heads, width, _ptr(a), _ptr(a_log),
              _ptr(dt_bias), _ptr(b), int(ctx.allow_neg), _ptr(dg), _ptr(None if b is None else dbeta), _ptr(da),
              _ptr(db), _ptr(da_log), _ptr(ddt_bias))
        return da, da_log, ddt_bias, db, None


def gate_prologue(a, a_log, dt_bias, b=None, *, allow_neg_eigval: bool = False):
    """``(g, beta)`` for the mixers' gate projections ``a`` (``[B, T, H]`` or ``[B, T, H, K]``) and ``b``
    (``[B, T, H]``, optional: ``beta`` is ``None`` without it)."""
    if not a.is_cuda:
        raise ValueError("gate_prologue runs on CUDA tensors only: the 'cuda' implementation has no CPU fallback")
    if a.ndim not in (3, 4) or a_log.shape != (a.shape[2],):
        raise ValueError(f"expected a [B, T, H] or [B, T, H, K] and A_log [H]; got {tuple(a.shape)}, {tuple(a_log.shape)}")
    if dt_bias.numel() != a.shape[2] * (a.shape[3] if a.ndim == 4 else 1):
        raise ValueError(f"dt_bias must have one entry per gate column; got {tuple(dt_bias.shape)} for a {tuple(a.shape)}")
    if b is not None and (b.shape != a.shape[:3] or b.dtype != a.dtype):
        raise ValueError(f"b must be [B, T, H] in a's dtype; got {tuple(b.shape)} {b.dtype}")
    if a.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {a.dtype}")
    g, beta = _GatePrologue.apply(a.contiguous(), a_log.float().contiguous(), dt_bias.float().contiguous(),
                                  None if b is None else b.contiguous(), bool(allow_neg_eigval))
    return g, beta
