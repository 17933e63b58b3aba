"""CPU oracle: chunk-parallel form of the linear-attention family (torch, CPU).

TEST INFRASTRUCTURE ONLY (see ``oracle/recurrence.py``); also the timed CPU baseline of
``bench.py``. It restates the six-stage chunk algorithm of the reference's
``src/jla/ops/chunked.py``:

* ``segment_masks``        follows ``chunked.py:108-121`` (same run / carry_in / tail);
* ``decayed_scores``       follows ``chunked.py:133-182`` (scalar gates: masked exponent of
  ``G_i - G_j``; vector gates: ``sub_chunk`` blocks, off-diagonal blocks referenced to the first
  decay of the row block so both factors are at most one, diagonal blocks from exact per-channel
  differences);
* ``solve_unit_lower``     follows ``chunked.py:213-217``;
* ``wy_factors``           follows ``chunked.py:226-252`` (``recompute_w_u``);
* ``state_pass``           follows ``chunked.py:255-307`` (``chunk_state_pass``);
* ``chunk_output``         follows ``chunked.py:310-331``;
* ``chunked``              follows ``chunked.py:334-402`` (``_chunked``: zero padding is inert).

Gradients come from torch autograd. Validated against ``oracle/recurrence.py`` (itself pinned to
the reference's float64 oracles) in ``tests/test_oracle.py``.
"""

from __future__ import annotations

import torch

from .recurrence import l2norm, repeat_heads, segment_resets

__all__ = ["chunked", "segment_masks", "decayed_scores", "solve_unit_lower", "simple_gla", "gla",
           "delta_rule", "gated_delta_rule", "kda"]

DEFAULT_CHUNK = 64
DEFAULT_SUB_CHUNK = 16


def _to_chunks(x: torch.Tensor, chunk: int) -> torch.Tensor:
    """``[B, T, H, ...]`` (``T % chunk == 0``) to ``[B, H, NC, C, ...]``."""
    b, t, h = x.shape[:3]
    x = x.reshape(b, t // chunk, chunk, h, *x.shape[3:])
    return x.movedim(3, 1)


def _from_chunks(x: torch.Tensor) -> torch.Tensor:
    """``[B, H, NC, C, ...]`` back to ``[B, T, H, ...]``."""
    x = x.movedim(1, 3)
    b, nc, c, h = x.shape[:4]
    return x.reshape(b, nc * c, h, *x.shape[4:])


def segment_masks(segment_ids: torch.Tensor, chunk: int, pad: int):
    """``(same [B,1,NC,C,C], carry_in [B,1,NC,C], tail [B,1,NC,C])`` bool (``chunked.py:108-121``)."""
    runs = torch.cumsum(segment_resets(segment_ids).to(torch.int64), dim=1)
    if pad:
        runs = torch.cat([runs, runs[:, -1:].expand(-1, pad)], dim=1)  # padding joins the last run
    b = runs.shape[0]
    runs = runs.reshape(b, 1, -1, chunk)
    entering = torch.cat([runs[:, :, :1, :1], runs[:, :, :-1, -1:]], dim=2)
    return runs[..., :, None] == runs[..., None, :], runs == entering, runs == runs[..., -1:]


def _masked_exp(exponent: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
    """``exp`` on the mask, exact zero elsewhere, never evaluating ``exp`` off the mask (``chunked.py:124-130``)."""
    neg_inf = torch.full((), float("-inf"), dtype=exponent.dtype)
    return torch.exp(torch.where(mask, exponent, neg_inf))


def decayed_scores(a, b, g_cum, *, inclusive: bool, sub_chunk: int = DEFAULT_SUB_CHUNK):
    """Causal ``P[i, j] = sum_c a_ic b_jc exp(G_ic - G_jc)`` per chunk (``chunked.py:133-182``)."""
    chunk = a.shape[-2]
    causal = torch.tril(torch.ones(chunk, chunk, dtype=torch.bool), 0 if inclusive else -1)
    if g_cum.ndim != a.ndim:  # one decay per head
        scores = torch.einsum("...ik,...jk->...ij", a, b)
        return scores * _masked_exp(g_cum[..., :, None] - g_cum[..., None, :], causal)
    if chunk % sub_chunk:
        raise ValueError(f"chunk size {chunk} must be a multiple of sub_chunk {sub_chunk}")
    lead, key_dim = a.shape[:-2], a.shape[-1]
    blocks = chunk // sub_chunk
    a_b, b_b, g_b = (x.reshape(*lead, blocks, sub_chunk, key_dim) for x in (a, b, g_cum))
    g_ref = g_b[..., :, 0, :]
    rows = a_b * torch.exp(g_b - g_ref[..., :, None, :])
    below = torch.tril(torch.ones(blocks, blocks, dtype=torch.bool), -1)[:, :, None, None]
    cols = b_b[..., None, :, :, :] * _masked_exp(g_ref[..., :, None, None, :] - g_b[..., None, :, :, :], below)
    off = torch.einsum("...ick,...ijdk->...ijcd", rows, cols)
    tri = torch.tril(torch.ones(sub_chunk, sub_chunk, dtype=torch.bool), 0 if inclusive else -1)[:, :, None]
    weights = _masked_exp(g_b[..., :, None, :] - g_b[..., None, :, :], tri)
    diag = torch.einsum("...ik,...jk,...ijk->...ij", a_b, b_b, weights)
    on_diag = torch.eye(blocks, dtype=torch.bool)[:, :, None, None]
    tiles = torch.where(on_diag, diag[..., :, None, :, :], off)
    return tiles.transpose(-3, -2).reshape(*lead, chunk, chunk)


def solve_unit_lower(a: torch.Tensor) -> torch.Tensor:
    """``(I + A)^-1`` for strictly lower ``A`` (``chunked.py:213-217``)."""
    eye = torch.eye(a.shape[-1], dtype=a.dtype).expand_as(a)
    return torch.linalg.solve_triangular(eye + a, eye, upper=False, unitriangular=True)


def _key_decay(g_cum, k):
    decay = torch.exp(g_cum)
    return decay if g_cum.ndim == k.ndim else decay[..., None]


def wy_factors(k, v, beta, g_cum, t, carry_in=None):
    """``w = T (beta exp(G) k)`` and ``u = T (beta v)`` (``chunked.py:226-252``)."""
    rhs = k * _key_decay(g_cum, k) * beta[..., None]
    if carry_in is not None:
        rhs = rhs * carry_in[..., None]
    return t @ rhs, t @ (v * beta[..., None])


def state_pass(k, w, u, g_cum, initial_state, tail=None, keep=None):
    """Serial pass over chunks (``chunked.py:255-307``): ``h [B,H,NC,K,V]``, ``v_new``, final state."""
    vector = g_cum.ndim == k.ndim
    state = initial_state
    hs, vns = [], []
    for n in range(k.shape[2]):
        k_n, u_n, g_n = k[:, :, n], u[:, :, n], g_cum[:, :, n]
        v_new = u_n if w is None else u_n - w[:, :, n] @ state
        if vector:
            g_last = g_n[..., -1, :]
            k_dec = k_n * torch.exp(g_last[..., None, :] - g_n)
            decayed = state * torch.exp(g_last)[..., :, None]
        else:
            g_last = g_n[..., -1]
            k_dec = k_n * torch.exp(g_last[..., None] - g_n)[..., None]
            decayed = state * torch.exp(g_last)[..., None, None]
        if tail is not None:
            k_dec = k_dec * tail[:, :, n][..., None]
            decayed = decayed * keep[:, :, n][..., None, None]
        hs.append(state)
        vns.append(v_new)
        state = decayed + k_dec.transpose(-1, -2) @ v_new
    return torch.stack(hs, dim=2), torch.stack(vns, dim=2), state


def chunk_output(q, k, v_new, h, g_cum, scale, same=None, carry_in=None, sub_chunk=DEFAULT_SUB_CHUNK):
    """``o = scale ((q exp(G)) h + P v_new)`` (``chunked.py:310-331``)."""
    q_dec = q * _key_decay(g_cum, q)
    if carry_in is not None:
        q_dec = q_dec * carry_in[..., None]
    scores = decayed_scores(q, k, g_cum, inclusive=True, sub_chunk=sub_chunk)
    if same is not None:
        scores = scores * same
    return scale * (q_dec @ h + scores @ v_new)


def chunked(q, k, v, g=None, beta=None, *, delta: bool, scale=None, initial_state=None,
            output_final_state=False, segment_ids=None, use_qk_l2norm=False, chunk_size=DEFAULT_CHUNK,
            sub_chunk=DEFAULT_SUB_CHUNK, dtype=torch.float32, return_stages=False):
    """The chunked op (``chunked.py:334-402``); ``g`` is ``[B,T,H]``, ``[B,T,H,K]`` or ``None``."""
    batch, seq_len, _, key_dim = q.shape
    heads, value_dim = v.shape[2], v.shape[3]
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    if scale is None:
        scale = key_dim ** -0.5
    q, k = repeat_heads(q, heads), repeat_heads(k, heads)
    if g is None:
        g = torch.zeros(batch, seq_len, heads, dtype=dtype)
    if initial_state is None:
        initial_state = torch.zeros(batch, heads, key_dim, value_dim, dtype=dtype)
    pad = (-seq_len) % chunk_size

    def prep(x):
        x = x.to(dtype)
        if pad:
            x = torch.cat([x, torch.zeros(batch, pad, *x.shape[2:], dtype=dtype)], dim=1)
        return _to_chunks(x, chunk_size)

    same = carry_in = tail = keep = None
    if segment_ids is not None:
        segment_ids = torch.as_tensor(segment_ids)
        if tuple(segment_ids.shape) != (batch, seq_len):
            raise ValueError(f"segment_ids must be [B, T] = {(batch, seq_len)}; got {tuple(segment_ids.shape)}")
        same, carry_in, tail = segment_masks(segment_ids, chunk_size, pad)
        keep = carry_in[..., -1]
    q_c, k_c, v_c = prep(q), prep(k), prep(v)
    g_cum = torch.cumsum(prep(g), dim=3)
    stages = {"g_cum": g_cum}
    if delta:
        beta_c = prep(beta)
        a = decayed_scores(k_c, k_c, g_cum, inclusive=False, sub_chunk=sub_chunk) * beta_c[..., :, None]
        if same is not None:
            a = a * same
        t = solve_unit_lower(a)
        w, u = wy_factors(k_c, v_c, beta_c, g_cum, t, carry_in)
        stages.update(a=a, t=t, w=w, u=u)
    else:
        w, u = None, v_c
    h, v_new, final = state_pass(k_c, w, u, g_cum, initial_state.to(dtype),
                                 None if tail is None else tail.to(dtype),
                                 None if keep is None else keep.to(dtype))
    o = chunk_output(q_c, k_c, v_new, h, g_cum, scale, same, None if carry_in is None else carry_in.to(dtype),
                     sub_chunk)
    o = _from_chunks(o)[:, :seq_len]
    stages.update(h=h, v_new=v_new)
    result = (o, final if output_final_state else None)
    return (*result, stages) if return_stages else result


def simple_gla(q, k, v, g, **kw):
    return chunked(q, k, v, g, None, delta=False, **kw)


def gla(q, k, v, g, **kw):
    return chunked(q, k, v, g, None, delta=False, **kw)


def delta_rule(q, k, v, beta, **kw):
    return chunked(q, k, v, None, beta, delta=True, **kw)


def gated_delta_rule(q, k, v, g, beta, **kw):
    return chunked(q, k, v, g, beta, delta=True, **kw)


def kda(q, k, v, g, beta, **kw):
    return chunked(q, k, v, g, beta, delta=True, **kw)


KIND_FUNCTIONS = {
    "simple_gla": (simple_gla, ("g",)),
    "gla": (gla, ("g",)),
    "deltanet": (delta_rule, ("beta",)),
    "gated_deltanet": (gated_delta_rule, ("g", "beta")),
    "kda": (kda, ("g", "beta")),
}
