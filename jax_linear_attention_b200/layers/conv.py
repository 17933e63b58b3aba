"""Short causal convolution + SiLU + per-head L2 norm in front of the delta-rule kernels (mirror of ``ShortConv``
in the reference's ``src/jla/layers/conv.py:97-142`` and of ``conv_l2norm`` in ``src/jla/layers/conv_l2norm.py``),
one fused CUDA pass forward and one backward (``jla_short_conv_fwd/bwd``).

``y_t = act(bias + sum_i weight[:, i] * x_ext[t + i])`` with ``x_ext = [state; x]``; taps that reach into an earlier
document (``segment_ids``) contribute zero; with ``head_dim`` every head's channels are scaled to unit L2 norm
(eps 1e-6) before the single rounding to ``x``'s dtype, so the kernels downstream run with ``use_qk_l2norm=False``.
Returns ``(y, new_state)`` like the reference; ``new_state`` is the last ``K - 1`` inputs, zeroed where they belong
to an earlier document than the last token.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib

_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _ptr(t):
    return C.c_void_p(None if t is None else t.data_ptr())


def _call(name, x, *args):
    lib = _lib.load()
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        _lib.check(getattr(lib, name)(*args, C.c_void_p(stream)), name)


class _ShortConv(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, state, seg, head_dim, activation):
        B, T, Cn = x.shape
        K = weight.shape[1]
        y = torch.empty_like(x)
        _call("jla_short_conv_fwd", x, _DTYPES[x.dtype], B, T, Cn, K, head_dim, int(activation), _ptr(x), _ptr(weight),
              _ptr(bias), _ptr(seg), _ptr(state), _ptr(y))
        ctx.save_for_backward(x, weight, bias, state, seg)
        ctx.cfg = (head_dim, activation)
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        x, weight, bias, state, seg = ctx.saved_tensors
        head_dim, activation = ctx.cfg
        B, T, Cn = x.shape
        K = weight.shape[1]
        dy = dy.contiguous()
        dx = torch.empty_like(x)
        dw = torch.empty_like(weight)
        db = None if bias is None else torch.empty_like(bias)
        dstate = None if state is None else torch.empty_like(state)
        _call("jla_short_conv_bwd", x, _DTYPES[x.dtype], B, T, Cn, K, head_dim, int(activation), _ptr(x), _ptr(weight),
              _ptr(bias), _ptr(seg), _ptr(state), _ptr(dy), _ptr(dx), _ptr(dw), _ptr(db), _ptr(dstate))
        return dx, dw, db, dstate, None, None, None


def _final_state(x, state, segment_ids, width: int):
    """The last ``width - 1`` inputs, zeroed where they precede the last token's document (conv.py:190-210)."""
    B, T, Cn = x.shape
    if state is None:
        state = x.new_zeros(B, width - 1, Cn)
    if T >= width - 1:
        tail = x[:, T - (width - 1):]
    else:
        tail = torch.cat([state[:, T:], x], dim=1)
    if segment_ids is not None and width > 1:
        seg = segment_ids
        if T >= width - 1:
            seg_tail = seg[:, T - (width - 1):]
        else:
            seg_tail = torch.cat([seg[:, :1].expand(B, width - 1 - T), seg], dim=1)
        tail = torch.where((seg_tail == seg[:, -1:])[..., None], tail, torch.zeros((), dtype=x.dtype, device=x.device))
    return tail


def short_conv(x, weight, bias=None, *, activation: bool = True, head_dim: int | None = None, segment_ids=None,
               state=None):
    """``(y [B, T, C], new_state [B, K - 1, C])``; ``head_dim`` adds the per-head L2 norm of ``conv_l2norm``."""
    if x.ndim != 3 or weight.ndim != 2 or x.shape[-1] != weight.shape[0]:
        raise ValueError(f"expected x [B, T, C] and weight [C, K]; got {tuple(x.shape)}, {tuple(weight.shape)}")
    if not x.is_cuda:
        raise ValueError("short_conv runs on CUDA tensors only: the 'cuda' implementation has no CPU fallback")
    B, T, Cn = x.shape
    K = weight.shape[1]
    if state is not None and state.shape != (B, K - 1, Cn):
        raise ValueError(f"conv state must be {(B, K - 1, Cn)}; got {tuple(state.shape)}")
    if segment_ids is not None and segment_ids.shape != (B, T):
        raise ValueError(f"segment_ids must be {(B, T)}; got {tuple(segment_ids.shape)}")
    if x.dtype not in _DTYPES:
        raise ValueError(f"unsupported dtype {x.dtype}")
    seg = None if segment_ids is None else segment_ids.to(torch.int32).contiguous()
    st = None if state is None or K == 1 else state.to(x.dtype).contiguous()
    y = _ShortConv.apply(x.contiguous(), weight.float().contiguous(), None if bias is None else bias.float().contiguous(),
                         st, seg, int(head_dim or 0), bool(activation))
    with torch.no_grad():
        new_state = _final_state(x, state, segment_ids, K)
    return y, new_state
