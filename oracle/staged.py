"""CPU model of the chunk-64 kernels of the scalar-gate family, stage by stage, with a hand-written backward.

TEST INFRASTRUCTURE ONLY (see ``oracle/recurrence.py``). The CUDA kernels are checked against these
intermediates one stage at a time, the way the reference checks its kernels against ``chunked``
(``tests/test_mosaic_gpu_gated_delta_rule.py:104-146, 238-264``).

The stages are the gate-free formulation of the reference's kernels
(``src/jla/ops/mosaic_gpu/gated_delta_rule_kernels.py:351-370``, ``scalar_gate_fused.py:427-504``,
``gated_delta_rule_bwd.py:449-519, 557-841``), per head and chunk, ``S`` the state entering the chunk:

    A0 = strict_lower(beta_i k_i.k_j) * same      T0 = (I + A0)^-1
    Ag = T0 * D * beta_j                          D_ij = exp(G_i - G_j) * same  (i >= j)
    W  = V - (cin Gamma) * (K S)                  Vn = Ag W
    P  = (Q K^T) * D                              O  = scale [ (cin Gamma) * (Q S) + P Vn ]
    S+ = keep gamma S + ((tail Gamma_r) * K)^T Vn

and the backward (given dO and dS+):

    dVn = scale P^T dO + (tail Gamma_r) * (K dS+)         dW = Ag^T dVn = dV
    dS  = keep gamma dS+ + scale ((cin Gamma) Q)^T dO - ((cin Gamma) K)^T dW
    dP  = scale (dO Vn^T) * D                             dQ = scale (cin Gamma) * (dO S^T) + dP K
    dAg = tril(dVn W^T)       dT0 = dAg * D * beta_j      dA0 = -strict(T0^T dT0 T0^T) * same
    dK  = (tail Gamma_r)*(Vn dS+^T) - (cin Gamma)*(dW S^T) + dP^T Q + (dA0 beta_i) K + (dA0 beta_i)^T K
    dbeta_j = sum_i dAg_ij T0_ij D_ij + sum_m dA0_jm (k_j.k_m)
    dG_i = rowsum_i(E) - colsum_i(E) + rowsum_i(F) - colsum_i(F)           E = dP * (Q K^T) ,  F = dAg * Ag
           + cin_i Gamma_i [ scale (dO S^T)_i . q_i - (dW S^T)_i . k_i ]
           - tail_i Gamma_r,i (Vn dS+^T)_i . k_i
    dG_last += sum_i tail_i Gamma_r,i (Vn dS+^T)_i . k_i + keep gamma <S, dS+>
    dg = reverse cumulative sum of dG inside the chunk.

Without the delta rule (simple GLA): ``Ag = I``, ``W = Vn = V``. ``tests/test_staged.py`` checks this
backward against autograd of ``oracle/recurrence.py``.
"""

from __future__ import annotations

import torch

from .recurrence import l2norm, repeat_heads, segment_resets

C = 64


def _chunks(x, pad):
    """[B, T, H, ...] -> [B, H, NC, C, ...] with zero padding."""
    b, t, h = x.shape[:3]
    if pad:
        x = torch.cat([x, torch.zeros(b, pad, *x.shape[2:], dtype=x.dtype)], dim=1)
    x = x.reshape(b, (t + pad) // C, C, h, *x.shape[3:])
    return x.movedim(3, 1)


def _unchunk(x, seq_len):
    x = x.movedim(1, 3)
    b, nc, c, h = x.shape[:4]
    return x.reshape(b, nc * c, h, *x.shape[4:])[:, :seq_len]


def masks(segment_ids, batch, seq_len, pad, dtype):
    """same [B,1,NC,C,C], cin, tail [B,1,NC,C], keep [B,1,NC] as floats."""
    nc = (seq_len + pad) // C
    if segment_ids is None:
        one = torch.ones(batch, 1, nc, C, dtype=dtype)
        return torch.ones(batch, 1, nc, C, C, dtype=dtype), one, one, torch.ones(batch, 1, nc, dtype=dtype)
    runs = torch.cumsum(segment_resets(torch.as_tensor(segment_ids)).to(torch.int64), dim=1)
    if pad:
        runs = torch.cat([runs, runs[:, -1:].expand(-1, pad)], dim=1)
    runs = runs.reshape(batch, 1, nc, C)
    entering = torch.cat([runs[:, :, :1, :1], runs[:, :, :-1, -1:]], dim=2)
    same = (runs[..., :, None] == runs[..., None, :]).to(dtype)
    cin = (runs == entering).to(dtype)
    tail = (runs == runs[..., -1:]).to(dtype)
    return same, cin, tail, cin[..., -1]


def forward(q, k, v, g, beta, *, delta, scale, h0=None, segment_ids=None, dtype=torch.float64):
    """All forward stages; returns a dict of tensors in chunk layout [B, H, NC, ...]."""
    batch, seq_len, _, key_dim = q.shape
    heads, value_dim = v.shape[2], v.shape[3]
    pad = (-seq_len) % C
    q, k, v = (x.to(dtype) for x in (q, k, v))
    qc = _chunks(repeat_heads(q, heads), pad)
    kc = _chunks(repeat_heads(k, heads), pad)
    vc = _chunks(v, pad)
    gc = _chunks(torch.zeros(batch, seq_len, heads, dtype=dtype) if g is None else g.to(dtype), pad)
    G = torch.cumsum(gc, dim=-1)
    same, cin, tail, keep = masks(segment_ids, batch, seq_len, pad, dtype)
    lower = torch.tril(torch.ones(C, C, dtype=dtype))
    strict = torch.tril(torch.ones(C, C, dtype=dtype), -1)
    expo = G[..., :, None] - G[..., None, :]
    D = torch.exp(torch.where(lower.bool(), expo, torch.full((), -float("inf"), dtype=dtype))) * same
    Gam = torch.exp(G)
    gamma = Gam[..., -1]
    Gam_r = torch.exp(G[..., -1:] - G)
    st = dict(q=qc, k=kc, v=vc, G=G, D=D, same=same, cin=cin, tail=tail, keep=keep, Gam=Gam, gamma=gamma,
              Gam_r=Gam_r, scale=scale, delta=delta, seq_len=seq_len)
    if delta:
        bc = _chunks(beta.to(dtype), pad)
        kk = kc @ kc.transpose(-1, -2)
        A0 = bc[..., :, None] * kk * strict * same
        eye = torch.eye(C, dtype=dtype).expand_as(A0)
        T0 = torch.linalg.solve_triangular(eye + A0, eye, upper=False, unitriangular=True)
        Ag = T0 * D * bc[..., None, :]
        st.update(beta=bc, kk=kk, A0=A0, T0=T0, Ag=Ag)
    S = torch.zeros(batch, heads, key_dim, value_dim, dtype=dtype) if h0 is None else h0.to(dtype)
    nc = qc.shape[2]
    hs, Ws, Vns, Os = [], [], [], []
    P = (qc @ kc.transpose(-1, -2)) * D
    for n in range(nc):
        cg = (cin[:, :, n] * Gam[:, :, n])[..., None]
        KS = kc[:, :, n] @ S
        if delta:
            W = vc[:, :, n] - cg * KS
            Vn = Ag[:, :, n] @ W
        else:
            W = vc[:, :, n]
            Vn = W
        O = scale * (cg * (qc[:, :, n] @ S) + P[:, :, n] @ Vn)
        hs.append(S)
        Ws.append(W)
        Vns.append(Vn)
        Os.append(O)
        kd = (tail[:, :, n] * Gam_r[:, :, n])[..., None] * kc[:, :, n]
        S = (keep[:, :, n] * gamma[:, :, n])[..., None, None] * S + kd.transpose(-1, -2) @ Vn
    st.update(P=P, h=torch.stack(hs, 2), W=torch.stack(Ws, 2), Vn=torch.stack(Vns, 2), o_c=torch.stack(Os, 2),
              final=S)
    st["o"] = _unchunk(st["o_c"], seq_len)
    return st


def backward(st, do, dht=None):
    """Hand-written backward of :func:`forward`; returns gradients in the layouts of the inputs
    (per VALUE head for dq, dk) plus the per-chunk intermediates ``dh``, ``dVn``, ``dG``."""
    q, k, v, G, D = st["q"], st["k"], st["v"], st["G"], st["D"]
    same, cin, tail, keep = st["same"], st["cin"], st["tail"], st["keep"]
    Gam, gamma, Gam_r, scale, delta = st["Gam"], st["gamma"], st["Gam_r"], st["scale"], st["delta"]
    dtype = q.dtype
    batch, heads, nc = q.shape[:3]
    seq_len = st["seq_len"]
    pad = nc * C - seq_len
    doc = _chunks(do.to(dtype), pad)
    dS = torch.zeros_like(st["final"]) if dht is None else dht.to(dtype)
    strict = torch.tril(torch.ones(C, C, dtype=dtype), -1)
    lower = torch.tril(torch.ones(C, C, dtype=dtype))
    dq_, dk_, dv_, dG_, db_, dh_, dVn_ = [], [], [], [], [], [], []
    for n in reversed(range(nc)):
        S, Vn, W = st["h"][:, :, n], st["Vn"][:, :, n], st["W"][:, :, n]
        qn, kn, dO, Pn, Dn = q[:, :, n], k[:, :, n], doc[:, :, n], st["P"][:, :, n], D[:, :, n]
        cg = (cin[:, :, n] * Gam[:, :, n])[..., None]
        tg = (tail[:, :, n] * Gam_r[:, :, n])[..., None]
        kg = (keep[:, :, n] * gamma[:, :, n])[..., None, None]
        dh_.append(dS)
        dVn = scale * Pn.transpose(-1, -2) @ dO + tg * (kn @ dS)
        dVn_.append(dVn)
        dP = scale * (dO @ Vn.transpose(-1, -2)) * Dn
        dOS = dO @ S.transpose(-1, -2)
        dq = scale * cg * dOS + dP @ kn
        VdS = Vn @ dS.transpose(-1, -2)
        E = dP * (qn @ kn.transpose(-1, -2))
        dG = E.sum(-1) - E.sum(-2) + (scale * cg * dOS * qn).sum(-1) - (tg * VdS * kn).sum(-1)
        dk = tg * VdS + dP.transpose(-1, -2) @ qn
        if delta:
            Ag, T0, beta = st["Ag"][:, :, n], st["T0"][:, :, n], st["beta"][:, :, n]
            dW = Ag.transpose(-1, -2) @ dVn
            dAg = (dVn @ W.transpose(-1, -2)) * lower
            dT0 = dAg * Dn * beta[..., None, :]
            dA0 = -(T0.transpose(-1, -2) @ dT0 @ T0.transpose(-1, -2)) * strict * same[:, :, n]
            dA0b = dA0 * beta[..., :, None]
            dWS = dW @ S.transpose(-1, -2)
            dk = dk - cg * dWS + dA0b @ kn + dA0b.transpose(-1, -2) @ kn
            F = dAg * Ag
            dG = dG + F.sum(-1) - F.sum(-2) - (cg * dWS * kn).sum(-1)
            db = (dAg * T0 * Dn).sum(-2) + (dA0 * st["kk"][:, :, n]).sum(-1)
            db_.append(db)
            dS_new = kg * dS + scale * (cg * qn).transpose(-1, -2) @ dO - (cg * kn).transpose(-1, -2) @ dW
        else:
            dW = dVn
            dS_new = kg * dS + scale * (cg * qn).transpose(-1, -2) @ dO
        dG_last = (tg * VdS * kn).sum((-1, -2)) + kg[..., 0, 0] * (S * dS).sum((-1, -2))
        dG = dG.clone()
        dG[..., -1] = dG[..., -1] + dG_last
        dq_.append(dq)
        dk_.append(dk)
        dv_.append(dW)
        dG_.append(dG)
        dS = dS_new

    def stack(xs):
        return torch.stack(xs[::-1], 2)

    dGc = stack(dG_)
    dg = torch.flip(torch.cumsum(torch.flip(dGc, [-1]), -1), [-1])
    out = dict(dq=_unchunk(stack(dq_), seq_len), dk=_unchunk(stack(dk_), seq_len), dv=_unchunk(stack(dv_), seq_len),
               dg=_unchunk(dg, seq_len), dh0=dS, dh=stack(dh_), dVn=stack(dVn_), dG=dGc)
    if delta:
        out["dbeta"] = _unchunk(stack(db_), seq_len)
    return out


def group_sum(dx, key_heads):
    """[B, T, H, K] per value head -> [B, T, Hk, K] summed over each group."""
    b, t, h, d = dx.shape
    return dx.reshape(b, t, key_heads, h // key_heads, d).sum(3)
