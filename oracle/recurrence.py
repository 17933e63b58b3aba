"""CPU oracle: token-by-token recurrences of the linear-attention family.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module; it is the
checker used by ``tests/``, by ``__graft_entry__.smoke()`` and by the ``cpu_baseline`` /
``--impl reference`` legs of ``bench.py``.

It restates, in torch on the CPU (float64 by default, so that autograd provides the
gradients), the algorithm of the reference's ``src/jla/ops/reference.py``:

* ``l2norm``            follows ``reference.py:65-69``  (``x * rsqrt(sum x^2 + eps)``, eps 1e-6);
* ``segment_resets``    follows ``reference.py:72-75``  (True where the id changes, never at t = 0);
* ``recurrence``        follows ``reference.py:105-205`` (``_recurrence``: reset, decay, delta
  write, read; the ``cu_seqlens`` branch with per-sequence initial and final states, where an
  empty sequence keeps its initial state);
* ``simple_gla``, ``gla``, ``delta_rule``, ``gated_delta_rule``, ``kda`` follow the kind wrappers
  at ``reference.py:208-310``.

Parity pin: ``tests/test_oracle_golden.py`` checks these functions against fixtures made by the
reference's own JAX-free float64 oracles (``benchmarks/xcheck_scalar_gate_torch.py:71-171`` for the
scalar-gate kinds and Mamba-2, ``benchmarks/diff_vector_gate.py:209-250`` for KDA); the script
that wrote the fixtures is ``tests/golden/make_golden.py``.

Conventions (``reference.py:8-35``): ``q, k [B, T, Hk, K]``, ``v [B, T, H, V]`` with ``H % Hk == 0``
(value head ``h`` reads key head ``h // (H / Hk)``), ``g [B, T, H]`` or ``[B, T, H, K]`` natural-log
decay, ``beta [B, T, H]``, state ``[K, V]`` per head, ``o_t = scale * q_t S_t`` with ``S_t`` already
holding token ``t``.
"""

from __future__ import annotations

import torch

__all__ = [
    "delta_rule",
    "gated_delta_rule",
    "gla",
    "kda",
    "gdn2",
    "l2norm",
    "recurrence",
    "repeat_heads",
    "segment_resets",
    "simple_gla",
]


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Unit L2 norm over the last axis (``reference.py:65-69``)."""
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def segment_resets(segment_ids: torch.Tensor) -> torch.Tensor:
    """``[B, T]`` bool, True where a token starts a new document (``reference.py:72-75``)."""
    change = segment_ids[:, 1:] != segment_ids[:, :-1]
    return torch.cat([torch.zeros_like(change[:, :1]), change], dim=1)


def repeat_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    """``[B, T, Hk, D]`` to ``[B, T, H, D]``: value head ``h`` reads key head ``h // (H / Hk)``."""
    if x.shape[2] == heads:
        return x
    if heads % x.shape[2]:
        raise ValueError(f"value heads {heads} must be a multiple of key heads {x.shape[2]}")
    return x.repeat_interleave(heads // x.shape[2], dim=2)


def _step(state, q_t, k_t, v_t, g_t, beta_t, gate: str, delta: bool, erase_t=None, write_t=None):
    """One token for all rows and heads (``reference.py:140-157``). ``state [R, H, K, V]``. With an erase gate
    (Gated DeltaNet-2, ``reference.py:152-154``) the recall reads with ``erase_t * k_t`` and the write gate scales
    the value; ``beta_t`` is unused then."""
    if gate == "scalar":
        state = state * torch.exp(g_t)[..., None, None]
    elif gate == "vector":
        state = state * torch.exp(g_t)[..., None]
    if delta and erase_t is None:
        recalled = torch.einsum("rhk,rhkv->rhv", k_t, state)
        v_t = beta_t[..., None] * (v_t - recalled)
    elif delta:
        recalled = torch.einsum("rhk,rhkv->rhv", erase_t * k_t, state)
        v_t = write_t * v_t - recalled
    state = state + k_t[..., :, None] * v_t[..., None, :]
    return state, torch.einsum("rhk,rhkv->rhv", q_t, state)


def recurrence(q, k, v, g=None, beta=None, *, gate: str, delta: bool, scale=None, initial_state=None,
               output_final_state: bool = False, cu_seqlens=None, segment_ids=None,
               use_qk_l2norm: bool = False, dtype=torch.float64, erase=None, write=None):
    """Token loop of ``reference.py:105-205``; returns ``(o, final_state | None)`` in ``dtype``. ``erase [B, T, H, K]``
    and ``write [B, T, H, V]`` are the channel gates of Gated DeltaNet-2 (``beta`` is None then).

    Inputs are torch tensors (leaves that require grad keep their graph, so
    ``torch.autograd.grad`` of the outputs gives the oracle gradients).
    """
    if cu_seqlens is not None and segment_ids is not None:
        raise ValueError("pass cu_seqlens or segment_ids, not both")
    if q.ndim != 4 or k.shape != q.shape:
        raise ValueError(f"q and k must both be [B, T, H, K]; got {tuple(q.shape)} and {tuple(k.shape)}")
    if v.ndim != 4 or v.shape[:2] != q.shape[:2]:
        raise ValueError(f"v must be [B, T, H, V] matching q; got {tuple(v.shape)} for q {tuple(q.shape)}")
    batch, seq_len, _, key_dim = q.shape
    heads, value_dim = v.shape[2], v.shape[3]
    if cu_seqlens is not None and batch != 1:
        raise ValueError("cu_seqlens packs sequences along T and requires batch size 1")
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    if use_qk_l2norm:
        q, k = l2norm(q), l2norm(k)
    if scale is None:
        scale = key_dim ** -0.5
    q = repeat_heads(q, heads) * scale
    k = repeat_heads(k, heads)
    g = None if g is None else g.to(dtype)
    beta = None if beta is None else beta.to(dtype)
    if erase is not None:
        if tuple(erase.shape) != tuple(q.shape) or write is None or tuple(write.shape) != tuple(v.shape):
            raise ValueError(f"b must be [B, T, H, K] = {tuple(q.shape)} and w must be [B, T, H, V] = "
                             f"{tuple(v.shape)}; got {tuple(erase.shape)} and "
                             f"{None if write is None else tuple(write.shape)}")
        erase, write = erase.to(dtype), write.to(dtype)

    def tok(x, t):
        return None if x is None else x[:, t]

    outs = []
    if cu_seqlens is None:
        state = (torch.zeros(batch, heads, key_dim, value_dim, dtype=dtype) if initial_state is None
                 else initial_state.to(dtype))
        resets = None if segment_ids is None else segment_resets(torch.as_tensor(segment_ids))
        for t in range(seq_len):
            if resets is not None:
                state = state * (~resets[:, t]).to(dtype)[:, None, None, None]
            state, o_t = _step(state, q[:, t], k[:, t], v[:, t], tok(g, t), tok(beta, t), gate, delta, tok(erase, t),
                                 tok(write, t))
            outs.append(o_t)
        final = state
    else:
        cu = [int(c) for c in torch.as_tensor(cu_seqlens).tolist()]
        num_seqs = len(cu) - 1
        if cu[-1] != seq_len:
            raise ValueError(f"cu_seqlens[-1] must equal T = {seq_len}; got {cu[-1]}")
        state0 = (torch.zeros(num_seqs, heads, key_dim, value_dim, dtype=dtype) if initial_state is None
                  else initial_state.to(dtype))
        finals = [state0[n] for n in range(num_seqs)]  # empty sequences keep their initial state
        for n in range(num_seqs):
            state = state0[n][None]
            for t in range(cu[n], cu[n + 1]):
                state, o_t = _step(state, q[:, t], k[:, t], v[:, t], tok(g, t), tok(beta, t), gate, delta, tok(erase, t),
                                 tok(write, t))
                outs.append(o_t)
            if cu[n + 1] > cu[n]:
                finals[n] = state[0]
        final = torch.stack(finals)
    o = torch.stack(outs, dim=1) if outs else torch.zeros(batch, 0, heads, value_dim, dtype=dtype)
    return o, (final if output_final_state else None)


def simple_gla(q, k, v, g, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
               segment_ids=None, dtype=torch.float64):
    """``S_t = exp(g_t) S_{t-1} + k_t^T v_t`` (``reference.py:208-225``)."""
    return recurrence(q, k, v, g, None, gate="scalar", delta=False, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      dtype=dtype)


def gla(q, k, v, g, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
        segment_ids=None, dtype=torch.float64):
    """``S_t = diag(exp(g_t)) S_{t-1} + k_t^T v_t`` (``reference.py:228-245``)."""
    return recurrence(q, k, v, g, None, gate="vector", delta=False, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      dtype=dtype)


def delta_rule(q, k, v, beta, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
               segment_ids=None, use_qk_l2norm=False, dtype=torch.float64):
    """``S_t = S_{t-1} + beta_t k_t^T (v_t - k_t S_{t-1})`` (``reference.py:248-266``)."""
    return recurrence(q, k, v, None, beta, gate="none", delta=True, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      use_qk_l2norm=use_qk_l2norm, dtype=dtype)


def gated_delta_rule(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                     cu_seqlens=None, segment_ids=None, use_qk_l2norm=False, dtype=torch.float64):
    """``S' = exp(g_t) S_{t-1}; S_t = S' + beta_t k_t^T (v_t - k_t S')`` (``reference.py:269-288``)."""
    return recurrence(q, k, v, g, beta, gate="scalar", delta=True, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      use_qk_l2norm=use_qk_l2norm, dtype=dtype)


def kda(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
        segment_ids=None, use_qk_l2norm=False, dtype=torch.float64):
    """``S' = diag(exp(g_t)) S_{t-1}; S_t = S' + beta_t k_t^T (v_t - k_t S')`` (``reference.py:291-310``)."""
    return recurrence(q, k, v, g, beta, gate="vector", delta=True, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      use_qk_l2norm=use_qk_l2norm, dtype=dtype)


def gdn2(q, k, v, g, b, w, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
         segment_ids=None, use_qk_l2norm=False, dtype=torch.float64):
    """Gated DeltaNet-2 (``reference.py:313-343``): ``S_t = (I - k_t (b_t * k_t)^T) diag(exp g_t) S_{t-1} + k_t (w_t *
    v_t)^T`` with an erase gate ``b [B, T, H, K]`` and a write gate ``w [B, T, H, V]``; ``b = w = beta`` is KDA."""
    return recurrence(q, k, v, g, None, gate="vector", delta=True, scale=scale, initial_state=initial_state,
                      output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                      use_qk_l2norm=use_qk_l2norm, dtype=dtype, erase=b, write=w)


KIND_FUNCTIONS = {
    "simple_gla": (simple_gla, ("g",)),
    "gla": (gla, ("g",)),
    "deltanet": (delta_rule, ("beta",)),
    "gated_deltanet": (gated_delta_rule, ("g", "beta")),
    "kda": (kda, ("g", "beta")),
    "gdn2": (gdn2, ("g", "b", "w")),
}
