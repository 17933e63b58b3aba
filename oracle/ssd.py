"""CPU oracle: the Mamba-2 SSD scan and its mapping onto ``simple_gla``.

TEST INFRASTRUCTURE ONLY (see ``oracle/recurrence.py``).

* ``mamba2_ssd`` follows the reference's ``src/jla/layers/ssm.py:183-230``:
  ``v = (x * dt)`` rounded to the input dtype, ``g = dt * A`` (float32), ``q = C``, ``k = B`` (grouped
  ``[B, T, G, N]``, head ``h`` reads group ``h // (H / G)``), ``scale = 1``, ``y = o + D * x``; the
  state is presented as ``[B, H, N, P]``, which equals ``simple_gla``'s ``[B, H, K, V]`` with ``K = N``
  and ``V = P``.
* ``ssd_direct`` is the independent form ``h_t = exp(dt_t A) h_{t-1} + dt_t B_t^T x_t``,
  ``y_t = C_t h_t + D x_t`` written from the docstring at ``ssm.py:198-200`` (the role of
  ``_ssd_recurrence`` in the reference's ``tests/test_layers_ssm.py``).
"""

from __future__ import annotations

import torch

from . import recurrence


def mamba2_ssd(x, dt, a, b, c, *, d=None, segment_ids=None, initial_state=None, output_final_state=False,
               op=None, dtype=torch.float64, round_v_to=None):
    """SSD through ``simple_gla``; ``op`` defaults to the token recurrence."""
    op = op or recurrence.simple_gla
    v = x.to(dtype) * dt.to(dtype)[..., None]
    if round_v_to is not None:  # the reference rounds dt*x to the activation dtype before the op
        v = v.to(round_v_to).to(dtype)
    g = dt.to(dtype) * a.to(dtype)
    y, state = op(c, b, v, g, scale=1.0, segment_ids=segment_ids, initial_state=initial_state,
                  output_final_state=output_final_state, dtype=dtype)
    if d is not None:
        y = y + d.to(dtype)[:, None] * x.to(dtype)
    return y, state


def ssd_direct(x, dt, a, b, c, *, d=None, segment_ids=None, initial_state=None, dtype=torch.float64):
    """Direct SSD token loop; returns ``(y, final_state [B, H, N, P])``."""
    batch, seq_len, heads, p = x.shape
    groups, n = b.shape[2], b.shape[3]
    x, dt, a, b, c = (t.to(dtype) for t in (x, dt, a, b, c))
    b = recurrence.repeat_heads(b, heads)
    c = recurrence.repeat_heads(c, heads)
    state = (torch.zeros(batch, heads, n, p, dtype=dtype) if initial_state is None else initial_state.to(dtype))
    resets = None if segment_ids is None else recurrence.segment_resets(torch.as_tensor(segment_ids))
    ys = []
    for t in range(seq_len):
        if resets is not None:
            state = state * (~resets[:, t]).to(dtype)[:, None, None, None]
        decay = torch.exp(dt[:, t] * a)  # [B, H]
        state = state * decay[..., None, None] + (dt[:, t, :, None] * b[:, t])[..., :, None] * x[:, t][..., None, :]
        y = torch.einsum("bhn,bhnp->bhp", c[:, t], state)
        if d is not None:
            y = y + d[:, None] * x[:, t]
        ys.append(y)
    del groups
    return torch.stack(ys, dim=1), state
