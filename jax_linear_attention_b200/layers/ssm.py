"""Mamba-2 SSD scan on top of ``simple_gla`` (mirror of ``mamba2_ssd`` in the reference's
``src/jla/layers/ssm.py:183-230``): ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t^T x_t``, ``y_t = C_t h_t + D x_t``.

``x [B, T, H, P]``, ``dt [B, T, H]`` (positive, after softplus), ``a [H]`` (negative), ``b, c [B, T, G, N]`` with
``H % G == 0``, ``d [H]``; the state is ``[B, H, N, P]`` float32. Runs
``ops.linear_attention("simple_gla", q=C, k=B, v=dt*x, g=dt*A, scale=1.0)``: the grouped ``B, C`` go to the kernels
un-repeated (value head ``h`` reads group ``h // (H / G)``; the kernels sum ``dB, dC`` over a group's heads in
float32, as the reference does in ``scalar_gate_grouped.py``). The elementwise glue (``dt*x`` rounded to the
activation dtype, ``dt*A`` in float32, ``+ D*x`` in float32) is plain torch, so autograd supplies the chain rule
``dx = dv*dt + D*dy``, ``ddt = sum_p dv*x + dg*A``, ``dA = sum dg*dt``, ``dD = sum dy*x`` (``ssm.py:76-84``).
"""

from __future__ import annotations

import torch

from .. import ops


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
    dt32 = dt.float()
    v = (x.float() * dt32[..., None]).to(x.dtype).to(c.dtype)
    g = dt32 * a.float()
    y, state = ops.linear_attention("simple_gla", c, b.to(c.dtype), v, g=g, impl=impl, scale=1.0,
                                    chunk_size=chunk_size, segment_ids=segment_ids, initial_state=initial_state,
                                    output_final_state=output_final_state, precision=precision)
    if d is not None:
        y = (y.float() + d.float()[:, None] * x.float()).to(y.dtype)
    return y, state
