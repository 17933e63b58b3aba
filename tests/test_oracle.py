"""Self-tests of the CPU oracle: the closed forms and cross-implementation identities that the reference's
``tests/test_reference_ops.py`` and ``tests/test_chunked_ops.py`` use to pin this path (float64 here)."""

import numpy as np
import pytest
import torch

from oracle import chunked, recurrence
from oracle.cases import make_case, max_rel, seg_to_cu

F64 = torch.float64


def tens(case, names, grad=False):
    return {n: torch.tensor(case[n], dtype=F64, requires_grad=grad) for n in names if n in case}


def call(mod, case, t, **extra):
    kind = case["meta"]["kind"]
    fn, gates = mod.KIND_FUNCTIONS[kind]
    opts = dict(scale=case["meta"]["scale"], initial_state=t.get("h0"), output_final_state=True, dtype=F64)
    if "seg" in case:
        opts["segment_ids"] = torch.tensor(case["seg"])
    opts.update(extra)
    return fn(t["q"], t["k"], t["v"], *[t[g] for g in gates], **opts)


@pytest.mark.parametrize("kind", ["simple_gla", "deltanet", "gated_deltanet", "kda"])
@pytest.mark.parametrize("chunk", [16, 64])
def test_chunked_matches_recurrence_values_and_grads(kind, chunk):
    case = make_case(kind, B=2, T=150, H=2, Hk=1, K=32, V=16, seed=3, docs="mixed", h0=True)
    names = ("q", "k", "v", "g", "beta", "h0")
    a, b = tens(case, names, True), tens(case, names, True)
    o1, s1 = call(recurrence, case, a)
    o2, s2 = call(chunked, case, b, chunk_size=chunk)
    do, dht = torch.tensor(case["do"], dtype=F64), torch.tensor(case["dht"], dtype=F64)
    g1 = torch.autograd.grad([o1, s1], list(a.values()), [do, dht])
    g2 = torch.autograd.grad([o2, s2], list(b.values()), [do, dht])
    assert max_rel(o2.detach(), o1.detach()) < 1e-9 and max_rel(s2.detach(), s1.detach()) < 1e-9
    for n, x, y in zip(a, g1, g2):
        assert max_rel(y, x) < 1e-8, n


def test_scalar_gates_are_broadcast_vector_gates():
    case = make_case("gated_deltanet", B=1, T=70, H=2, K=16, V=16, seed=1, h0=True)
    t = tens(case, ("q", "k", "v", "g", "beta", "h0"))
    o1, s1 = call(recurrence, case, t)
    gv = t["g"][..., None].expand(-1, -1, -1, 16)
    o2, s2 = recurrence.kda(t["q"], t["k"], t["v"], gv, t["beta"], scale=case["meta"]["scale"],
                            initial_state=t["h0"], output_final_state=True)
    assert max_rel(o2, o1) < 1e-12 and max_rel(s2, s1) < 1e-12


def test_gated_delta_rule_without_decay_is_delta_rule():
    case = make_case("gated_deltanet", B=1, T=50, H=2, K=16, V=16, seed=2)
    t = tens(case, ("q", "k", "v", "g", "beta"))
    o1, _ = recurrence.gated_delta_rule(t["q"], t["k"], t["v"], torch.zeros_like(t["g"]), t["beta"])
    o2, _ = recurrence.delta_rule(t["q"], t["k"], t["v"], t["beta"])
    assert max_rel(o2, o1) < 1e-13


def test_delta_rule_overwrites_the_value_of_a_repeated_key():
    k = torch.zeros(1, 2, 1, 4, dtype=F64)
    k[0, :, 0, 1] = 1.0
    v = torch.tensor([[[[1.0, 2.0, 3.0]], [[-4.0, 5.0, 6.0]]]], dtype=F64)
    beta = torch.ones(1, 2, 1, dtype=F64)
    o, s = recurrence.delta_rule(k, k, v, beta, scale=1.0, output_final_state=True)
    assert torch.allclose(o[0, 1, 0], v[0, 1, 0]) and torch.allclose(s[0, 0, 1], v[0, 1, 0])
    assert float(s[0, 0, [0, 2, 3]].abs().max()) == 0.0


@pytest.mark.parametrize("kind", ["simple_gla", "gated_deltanet", "kda"])
def test_final_state_chains_across_a_split(kind):
    case = make_case(kind, B=2, T=90, H=2, K=16, V=8, seed=4, h0=True)
    t = tens(case, ("q", "k", "v", "g", "beta", "h0"))
    o, s = call(recurrence, case, t)
    cut = 37
    first = {n: (x[:, :cut] if n != "h0" else x) for n, x in t.items()}
    o1, s1 = call(recurrence, case, first)
    second = {n: (x[:, cut:] if n != "h0" else s1) for n, x in t.items()}
    o2, s2 = call(recurrence, case, second)
    assert max_rel(torch.cat([o1, o2], 1), o) < 1e-12 and max_rel(s2, s) < 1e-12


@pytest.mark.parametrize("kind", ["simple_gla", "deltanet", "gated_deltanet", "kda"])
def test_packed_sequences_match_separate_runs(kind):
    """cu_seqlens incl. an empty sequence: per-sequence initial and final states (reference.py:170-203)."""
    case = make_case(kind, B=1, T=60, H=2, K=8, V=8, seed=5)
    t = tens(case, ("q", "k", "v", "g", "beta"))
    cu = [0, 13, 13, 40, 60]
    h0 = torch.randn(4, 2, 8, 8, dtype=F64, generator=torch.Generator().manual_seed(0))
    fn, gates = recurrence.KIND_FUNCTIONS[kind]
    o, s = fn(t["q"], t["k"], t["v"], *[t[g] for g in gates], scale=0.5, initial_state=h0,
              output_final_state=True, cu_seqlens=torch.tensor(cu))
    for n in range(4):
        lo, hi = cu[n], cu[n + 1]
        if lo == hi:
            assert torch.equal(s[n], h0[n])
            continue
        o_n, s_n = fn(t["q"][:, lo:hi], t["k"][:, lo:hi], t["v"][:, lo:hi], *[t[g][:, lo:hi] for g in gates],
                      scale=0.5, initial_state=h0[n:n + 1], output_final_state=True)
        assert max_rel(o[:, lo:hi], o_n) < 1e-12 and max_rel(s[n], s_n[0]) < 1e-12


def test_segment_ids_match_separate_runs_and_reused_ids_restart():
    case = make_case("gated_deltanet", B=1, T=50, H=2, K=8, V=8, seed=6, h0=True)
    t = tens(case, ("q", "k", "v", "g", "beta", "h0"))
    seg = torch.tensor([[0] * 20 + [1] * 5 + [0] * 25])  # id 0 comes back: still a new document
    o, s = recurrence.gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["beta"], initial_state=t["h0"],
                                       output_final_state=True, segment_ids=seg)
    bounds = [(0, 20), (20, 25), (25, 50)]
    for i, (lo, hi) in enumerate(bounds):
        o_n, s_n = recurrence.gated_delta_rule(*(t[n][:, lo:hi] for n in ("q", "k", "v", "g", "beta")),
                                               initial_state=t["h0"] if i == 0 else None, output_final_state=True)
        assert max_rel(o[:, lo:hi], o_n) < 1e-12
    assert max_rel(s, s_n) < 1e-12
    cu = torch.tensor(seg_to_cu(seg[0].numpy()))
    o_cu, _ = recurrence.gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["beta"], cu_seqlens=cu,
                                          initial_state=torch.cat([t["h0"], torch.zeros(2, 2, 8, 8, dtype=F64)]))
    assert max_rel(o_cu, o) < 1e-12


def test_qk_l2norm_option_matches_normalized_inputs():
    case = make_case("gated_deltanet", B=1, T=40, H=2, K=16, V=8, seed=7, l2norm=True)
    t = tens(case, ("q", "k", "v", "g", "beta"))
    o1, _ = recurrence.gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["beta"], use_qk_l2norm=True)
    o2, _ = recurrence.gated_delta_rule(recurrence.l2norm(t["q"]), recurrence.l2norm(t["k"]), t["v"], t["g"],
                                        t["beta"])
    assert max_rel(o1, o2) < 1e-13


def test_vector_gates_survive_huge_decays():
    case = make_case("kda", B=1, T=130, H=2, K=16, V=8, seed=8)
    t = tens(case, ("q", "k", "v", "g", "beta"), True)
    g = (t["g"].detach() * 0 - 60.0).requires_grad_(True)
    o, s = chunked.kda(t["q"], t["k"], t["v"], g, t["beta"], output_final_state=True, dtype=F64)
    grads = torch.autograd.grad([o.sum() + s.sum()], [t["q"], t["k"], t["v"], g, t["beta"]])
    assert all(bool(torch.isfinite(x).all()) for x in (o, s, *grads))
    o_ref, _ = recurrence.kda(t["q"], t["k"], t["v"], g, t["beta"])
    assert max_rel(o.detach(), o_ref.detach()) < 1e-9


def test_stage_identities():
    case = make_case("gated_deltanet", B=1, T=128, H=2, K=16, V=8, seed=9, docs="mixed")
    t = tens(case, ("q", "k", "v", "g", "beta"))
    _, _, st = chunked.gated_delta_rule(t["q"], t["k"], t["v"], t["g"], t["beta"], dtype=F64,
                                        segment_ids=torch.tensor(case["seg"]), return_stages=True)
    a, tt = st["a"], st["t"]
    assert float(torch.triu(a).abs().max()) == 0.0
    eye = torch.eye(64, dtype=F64)
    assert max_rel((eye + a) @ tt, eye.expand_as(a)) < 1e-12


def test_shape_errors():
    q = torch.zeros(2, 8, 2, 4)
    with pytest.raises(ValueError, match="cu_seqlens packs"):
        recurrence.simple_gla(q, q, q, torch.zeros(2, 8, 2), cu_seqlens=torch.tensor([0, 8]))
    with pytest.raises(ValueError, match="not both"):
        recurrence.simple_gla(q[:1], q[:1], q[:1], torch.zeros(1, 8, 2), cu_seqlens=torch.tensor([0, 8]),
                              segment_ids=torch.zeros(1, 8, dtype=torch.int32))
    with pytest.raises(ValueError, match="q and k"):
        recurrence.simple_gla(q, q[..., :2], q, torch.zeros(2, 8, 2))


def test_gate_activations_closed_form():
    """``_mamba_gate`` and ``_write_strength`` (linear_attention.py:84-86, 159-162) at points with known values."""
    import math

    from oracle import gates

    a = torch.tensor([[[0.0, 1.0], [-2.0, 30.0]]])           # [1, 2, 2]
    a_log = torch.tensor([0.0, math.log(2.0)], dtype=torch.float64)
    dt_bias = torch.tensor([0.0, -1.0])
    g = gates.mamba_gate(a, a_log, dt_bias)
    want = [[-math.log(2.0), -2 * math.log(2.0)], [-math.log1p(math.exp(-2.0)), -2 * (29.0 + math.log1p(math.exp(-29.0)))]]
    assert torch.allclose(g[0], torch.tensor(want, dtype=torch.float64), rtol=1e-12)
    b = torch.tensor([0.0, math.log(3.0)], dtype=torch.float64)
    assert torch.allclose(gates.write_strength(b), torch.tensor([0.5, 0.75], dtype=torch.float64))
    assert torch.allclose(gates.write_strength(b, True), torch.tensor([1.0, 1.5], dtype=torch.float64))
    k = gates.mamba_gate(torch.zeros(1, 1, 2, 3), a_log, torch.zeros(2, 3))  # per-channel form: A_log per head
    assert torch.allclose(k[0, 0], torch.tensor([[-math.log(2.0)] * 3, [-2 * math.log(2.0)] * 3], dtype=torch.float64))


def test_gated_rms_norm_closed_form():
    """``GatedRMSNorm`` (norm.py:96-109): a constant row has unit RMS; both gate placements; groups."""
    import math

    from oracle import gates

    x = torch.full((1, 4), 3.0, dtype=torch.float64)
    z = torch.zeros(1, 4, dtype=torch.float64)          # silu(0) = 0, sigmoid(0) = 0.5
    w = torch.tensor([1.0, 2.0, 3.0, 4.0], dtype=torch.float64)
    assert torch.allclose(gates.gated_rms_norm(x, z, w, eps=0.0, activation="sigmoid"), 0.5 * w[None])
    assert torch.allclose(gates.gated_rms_norm(x, z, w, eps=0.0, activation="sigmoid", norm_before_gate=False), w[None])
    assert torch.allclose(gates.gated_rms_norm(x, z, w, eps=0.0), torch.zeros(1, 4, dtype=torch.float64))
    x2 = torch.tensor([[1.0, 1.0, 3.0, 3.0]], dtype=torch.float64)
    z2 = torch.full((1, 4), 50.0, dtype=torch.float64)  # silu(50) = 50 to 1e-20
    got = gates.gated_rms_norm(x2, z2, torch.ones(4, dtype=torch.float64), eps=0.0, group_size=2)
    assert torch.allclose(got, torch.full((1, 4), 50.0, dtype=torch.float64), rtol=1e-12)
    whole = gates.gated_rms_norm(x2, z2, torch.ones(4, dtype=torch.float64), eps=0.0)
    assert torch.allclose(whole, 50.0 * x2 / math.sqrt(5.0), rtol=1e-12)


def test_short_conv_closed_form():
    """``ShortConv`` (conv.py:97-142): identity taps, the causal shift, document masking, the carried state."""
    from oracle import gates

    x = torch.arange(1.0, 7.0, dtype=torch.float64).reshape(1, 6, 1)          # tokens 1..6, one channel
    ident = torch.tensor([[0.0, 0.0, 0.0, 1.0]], dtype=torch.float64)
    y, st = gates.short_conv(x, ident, activation=False)
    assert torch.equal(y, x) and torch.equal(st[0, :, 0], torch.tensor([4.0, 5.0, 6.0], dtype=torch.float64))
    shift = torch.tensor([[0.0, 0.0, 1.0, 0.0]], dtype=torch.float64)         # y_t = x_{t-1}
    y, _ = gates.short_conv(x, shift, activation=False)
    assert torch.equal(y[0, :, 0], torch.tensor([0.0, 1.0, 2.0, 3.0, 4.0, 5.0], dtype=torch.float64))
    seg = torch.tensor([[0, 0, 0, 1, 1, 1]])
    y, st = gates.short_conv(x, shift, activation=False, segment_ids=seg)     # token 4 starts a document: no tap into 3
    assert torch.equal(y[0, :, 0], torch.tensor([0.0, 1.0, 2.0, 0.0, 4.0, 5.0], dtype=torch.float64))
    state = torch.tensor([[[7.0], [8.0], [9.0]]], dtype=torch.float64)
    y, _ = gates.short_conv(x, shift, activation=False, state=state)
    assert y[0, 0, 0] == 9.0
    two = torch.tensor([[3.0, 4.0]], dtype=torch.float64).reshape(1, 1, 2)    # head of two channels: unit norm
    y, _ = gates.short_conv(two, torch.tensor([[1.0], [1.0]], dtype=torch.float64), activation=False, head_dim=2)
    assert torch.allclose(y[0, 0], torch.tensor([0.6, 0.8], dtype=torch.float64), atol=1e-7)


def test_softplus_series_of_the_gate_kernel_is_accurate_everywhere():
    """The gate kernel's forward softplus is ``max(x, 0) + 2 atanh(s)``, ``s = e / (2 + e)``, ``e = exp(-|x|)``, with
    the odd series of ``atanh`` cut after ``s^13`` (``csrc/gate_prologue.cu``). Restated here in float32 arithmetic
    and held to float64 ``log1p(exp(x))``: the relative error stays below 4e-7 from x = -40 (result 4e-18) to +40,
    which is what lets the float32 gate path keep its 1e-5 parity bound without the library's ``log1pf``."""
    rng = np.random.default_rng(0)
    x = np.concatenate([np.linspace(-40, 40, 200001), rng.standard_normal(100000) * 3])
    f32 = np.float32
    e = np.exp(-np.abs(x)).astype(f32)
    s = (e / (f32(2) + e)).astype(f32)
    z = (s * s).astype(f32)
    poly = f32(1 / 13)
    for c in (1 / 11, 1 / 9, 1 / 7, 1 / 5, 1 / 3, 1.0):
        poly = (poly * z + f32(c)).astype(f32)
    got = (np.maximum(x, 0).astype(f32) + f32(2) * s * poly).astype(np.float64)
    want = np.logaddexp(0.0, x)
    assert np.max(np.abs(got - want) / want) < 4e-7
