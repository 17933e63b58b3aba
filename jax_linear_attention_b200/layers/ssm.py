"""Mamba-2 SSD scan on top of ``simple_gla`` (mirror of ``mamba2_ssd`` in the reference's
``src/jla/layers/ssm.py:183-230``): ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t^T x_t``, ``y_t = C_t h_t + D x_t``.

``x [B, T, H, P]``, ``dt [B, T, H]`` (positive, after softplus), ``a [H]`` (negative), ``b, c [B, T, G, N]`` with
``H % G == 0``, ``d [H]``; the state is ``[B, H, N, P]`` float32. Runs
``ops.linear_attention("simple_gla", q=C, k=B, v=dt*x, g=dt*A, scale=1.0)``: the grouped ``B, C`` go to the kernels
un-repeated (value head ``h`` reads group ``h // (H / G)``; the kernels sum ``dB, dC`` over a group's heads in
float32, as the reference does in ``scalar_gate_grouped.py``). The elementwise glue (``dt*x`` rounded to the
activation dtype, ``dt*A`` in float32, ``+ D*x`` in float32) and its transpose ``dx = dv*dt + D*dy``,
``ddt = sum_p dv*x + dg*A``, ``dA = sum dg*dt``, ``dD = sum dy*x`` (``ssm.py:76-84``) run as the fused
``jla_ssd_*`` kernels for 16-bit activations (one pass over each ``[B, T, H, P]`` tensor); float32 activations, which
take the token-scan kernels anyway, keep plain torch glue. With a ``D`` term the two halves of ``dx`` are formed in one
kernel (``jla_ssd_layer_bwd``): the output side hands ``dy`` to the input side instead of writing ``D*dy`` for autograd
to add to ``dv*dt``.
"""

from __future__ import annotations

import ctypes as C

import torch

from .. import _lib, ops

_DTYPES = {torch.bfloat16: 0, torch.float16: 1}


def mamba2_ssd(x, dt, a, b, c, *, d=None, segment_ids=None, initial_state=None, output_final_state=False,
               impl: str = "auto", chunk_size: int = 64, grouped_key_grads: bool = False, precision=None):
    """Returns ``(y [B, T, H, P], final_state [B, H, N, P] | None)``."""
    del grouped_key_grads  # the CUDA kernels always sum grouped key gradients in float32
    if x.ndim != 4 or dt.shape != x.shape[:3]:
        raise ValueError(f"expected x [B, T, H, P] and dt [B, T, H]; got {tuple(x.shape)}, {tuple(dt.shape)}")
    heads = x.shape[2]
    if b.shape != c.shape or b.ndim != 4 or b.shape[:2] != x.shape[:2] or heads % b.shape[2]:
        raise ValueError(f"b, c must be [B, T, G, N] with H % G == 0; got {tuple(b.shape)}, {tuple(c.shape)}")
    if a.shape != (heads,):
        raise ValueError(f"a must be [H] = {(heads,)}; got {tuple(a.shape)}")
    fused = x.is_cuda and x.dtype in (torch.bfloat16, torch.float16) and x.shape[3] % 8 == 0
    # the output side's backward leaves dy here for the input side's backward (which runs after it: v and g lie
    # between them), so that dx = dv * dt + D * dy, ddt, dA and dD come from one pass over x, dv and dy
    link = {} if fused and d is not None and c.dtype == x.dtype else None
    if fused:
        x = x.contiguous()
        skip = d.float().contiguous() if link is not None else None
        v, g = _SsdInputs.apply(x, dt.float().contiguous(), a.float().contiguous(), skip, link)
        v = v.to(c.dtype)
    else:
        dt32 = dt.float()
        v = (x.float() * dt32[..., None]).to(x.dtype).to(c.dtype)
        g = dt32 * a.float()
    y, state = ops.linear_attention("simple_gla", c, b.to(c.dtype), v, g=g, impl=impl, scale=1.0,
                                    chunk_size=chunk_size, segment_ids=segment_ids, initial_state=initial_state,
                                    output_final_state=output_final_state, precision=precision)
    if d is not None:
        if link is not None:
            y = _SsdOutput.apply(y, x, skip, link)
        elif fused and y.dtype == x.dtype:
            y = _SsdOutput.apply(y, x, d.float().contiguous(), None)
        else:
            y = (y.float() + d.float()[:, None] * x.float()).to(y.dtype)
    return y, state


def _glue_call(name: str, x: torch.Tensor, *args):
    lib = _lib.load()
    tokens, heads, p = x.shape[0] * x.shape[1], x.shape[2], x.shape[3]
    stream = torch.cuda.current_stream(x.device).cuda_stream
    ptrs = [C.c_void_p(t.data_ptr()) for t in args]
    with torch.cuda.device(x.device):
        _lib.check(getattr(lib, name)(_DTYPES[x.dtype], C.c_int64(tokens), heads, p, *ptrs, C.c_void_p(stream)), name)


class _SsdInputs(torch.autograd.Function):
    """``(v, g) = (round(x * dt), dt * A)``. ``d`` and ``link`` (both None for a layer without a skip term) only
    matter backward: when the output side left ``dy`` in ``link``, this node returns the whole ``dx`` and ``dD``."""

    @staticmethod
    def forward(ctx, x, dt, a, d, link):
        v = torch.empty_like(x)
        g = torch.empty_like(dt)
        _glue_call("jla_ssd_inputs_fwd", x, x, dt, a, v, g)
        ctx.save_for_backward(x, dt, a, d)
        ctx.link = link
        return v, g

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dv, dg):
        x, dt, a, d = ctx.saved_tensors
        dv = torch.zeros_like(x) if dv is None else dv.contiguous()
        dg = torch.zeros_like(dt) if dg is None else dg.float().contiguous()
        dx, ddt, da = torch.empty_like(x), torch.empty_like(dt), torch.empty_like(a)
        dy = ctx.link.pop("dy", None) if ctx.link is not None else None
        if dy is None:  # no skip term, or no gradient reached y
            _glue_call("jla_ssd_inputs_bwd", x, x, dt, a, dv, dg, dx, ddt, da)
            return dx, ddt, da, None, None
        dd = torch.empty_like(d)
        _glue_call("jla_ssd_layer_bwd", x, x, dt, a, d, dv, dg, dy, dx, ddt, da, dd)
        return dx, ddt, da, dd, None


class _SsdOutput(torch.autograd.Function):
    """``y = round(o + D * x)``. With ``link`` the gradients of ``x`` and ``D`` are left to ``_SsdInputs.backward``."""

    @staticmethod
    def forward(ctx, o, x, d, link):
        y = torch.empty_like(o)
        _glue_call("jla_ssd_output_fwd", x, o, x, d, y)
        ctx.save_for_backward(x, d)
        ctx.link = link
        return y

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dy):
        x, d = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.link is not None:
            ctx.link["dy"] = dy
            return dy, None, None, None
        dx, dd = torch.empty_like(x), torch.empty_like(d)
        _glue_call("jla_ssd_output_bwd", x, dy, x, d, dx, dd)
        return dy, dx, dd, None
