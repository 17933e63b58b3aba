"""CPU restatement of the mixers' gate activations (test infrastructure only; nothing under the package imports it).

Follows ``src/jla/layers/linear_attention.py:84-86`` (``_mamba_gate``: ``-exp(A_log) * softplus(a + dt_bias)`` in
float32, ``A_log`` broadcast per head) and ``:159-162`` (``_write_strength``: ``sigmoid``, doubled with
``allow_neg_eigval``), in torch float64 so that autograd supplies the gradients. Parity of these two: pinned to the
reference's float64 oracle, whose ``gate="softplus"`` branch applies the same activations in front of the KDA
recurrence (``benchmarks/diff_vector_gate.py:215-225``; fixture ``tests/golden/kda_softplus.npz``, checked by
``tests/test_oracle_golden.py``), and by closed-form values (``tests/test_oracle.py``). The norm and the short
convolution below are restated from the layers' source and checked by closed forms only (parity unpinned: the
reference's layers need JAX to run).
"""

from __future__ import annotations

import torch


def mamba_gate(a, a_log, dt_bias):
    a = a.double()
    a_log = a_log.double()
    dt_bias = dt_bias.double().reshape(a.shape[2:])
    neg = -torch.exp(a_log)
    if a.ndim == 4:
        neg = neg[:, None]
    return neg * torch.nn.functional.softplus(a + dt_bias)


def write_strength(b, allow_neg_eigval: bool = False):
    s = torch.sigmoid(b.double())
    return 2.0 * s if allow_neg_eigval else s


def gated_rms_norm(x, z, weight, *, eps=1e-6, activation="silu", norm_before_gate=True, group_size=None):
    """``GatedRMSNorm.__call__`` (``src/jla/layers/norm.py:96-109``) in float64."""
    x64, z64 = x.double(), z.double()
    gate = torch.nn.functional.silu(z64) if activation == "silu" else torch.sigmoid(z64)
    if not norm_before_gate:
        x64 = x64 * gate
    dim = x.shape[-1]
    group = group_size or dim
    grouped = x64.reshape(*x.shape[:-1], dim // group, group)
    y = grouped * torch.rsqrt((grouped * grouped).mean(-1, keepdim=True) + eps)
    y = y.reshape(x.shape) * weight.double()
    if norm_before_gate:
        y = y * gate
    return y


def short_conv(x, weight, bias=None, *, activation=True, head_dim=None, segment_ids=None, state=None):
    """``ShortConv.__call__`` (``src/jla/layers/conv.py:97-142``) followed by the per-head ``l2norm`` of
    ``src/jla/ops/reference.py:65-69`` (as the fused ``short_conv_l2norm`` does, without rounding in between), in
    float64. Returns ``(y, new_state)``."""
    B, T, Cn = x.shape
    K = weight.shape[1]
    x64 = x.double()
    st = x64.new_zeros(B, K - 1, Cn) if state is None else state.double()
    x_ext = torch.cat([st, x64], dim=1)
    seg_ext = None
    if segment_ids is not None:
        seg_ext = torch.cat([segment_ids[:, :1].expand(B, K - 1), segment_ids], dim=1)
    y = x64.new_zeros(B, T, Cn)
    if bias is not None:
        y = y + bias.double()
    w = weight.double()
    for i in range(K):
        tap = x_ext[:, i:i + T] * w[:, i]
        if seg_ext is not None and i < K - 1:
            same = seg_ext[:, i:i + T] == segment_ids
            tap = torch.where(same[..., None], tap, torch.zeros((), dtype=tap.dtype))
        y = y + tap
    if activation:
        y = torch.nn.functional.silu(y)
    if head_dim:
        yh = y.reshape(B, T, Cn // head_dim, head_dim)
        y = (yh * torch.rsqrt((yh * yh).sum(-1, keepdim=True) + 1e-6)).reshape(B, T, Cn)
    new_state = x_ext[:, T:]
    if seg_ext is not None and K > 1:
        keep = seg_ext[:, T:] == segment_ids[:, -1:]
        new_state = torch.where(keep[..., None], new_state, torch.zeros((), dtype=new_state.dtype))
    return y, new_state
