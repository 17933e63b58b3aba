"""GPU parity of the callers around the op: the Mamba-2 SSD mapping (the op of the B8 T2048 H64 P64 N128 benchmark workload) and KDA through the
default dispatch. Tolerance: relative L2 <= 1e-2 against the float64 oracle (bf16 tensors, fp32 state)."""

import numpy as np
import pytest
import torch

from oracle import ssd as oracle_ssd
from oracle.cases import baseline_config, make_case, make_mamba2_case, rel_l2
from tests._util import compare, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


def _run_ssd_cuda(case, dtype=torch.bfloat16):
    from jax_linear_attention_b200.layers import mamba2_ssd

    dev = "cuda"
    half = ("x", "B", "C")
    t = {n: torch.tensor(case[n], device=dev, dtype=dtype if n in half else torch.float32, requires_grad=True)
         for n in ("x", "dt", "A", "B", "C", "D", "h0") if n in case}
    seg = torch.tensor(case["seg"], device=dev) if "seg" in case else None
    y, st = mamba2_ssd(t["x"], t["dt"], t["A"], t["B"], t["C"], d=t["D"], segment_ids=seg,
                       initial_state=t.get("h0"), output_final_state=True)
    names = list(t)
    grads = torch.autograd.grad([y, st], [t[n] for n in names],
                                [torch.tensor(case["do"], device=dev, dtype=dtype),
                                 torch.tensor(case["dht"], device=dev)])
    res = {"y": y.detach().float().cpu().numpy(), "state": st.detach().cpu().numpy()}
    res.update({"d" + n: g.detach().float().cpu().numpy() for n, g in zip(names, grads)})
    return res


def _run_ssd_oracle(case):
    f64 = torch.float64
    t = {n: torch.tensor(case[n], dtype=f64, requires_grad=True) for n in ("x", "dt", "A", "B", "C", "D", "h0")
         if n in case}
    seg = torch.tensor(case["seg"]) if "seg" in case else None
    y, st = oracle_ssd.mamba2_ssd(t["x"], t["dt"], t["A"], t["B"], t["C"], d=t["D"], segment_ids=seg,
                                  initial_state=t.get("h0"), output_final_state=True, round_v_to=torch.bfloat16)
    names = list(t)
    grads = torch.autograd.grad([y, st], [t[n] for n in names],
                                [torch.tensor(case["do"], dtype=f64),
                                 torch.tensor(case["dht"], dtype=f64)])
    res = {"y": y.detach().numpy(), "state": st.detach().numpy()}
    res.update({"d" + n: g.numpy() for n, g in zip(names, grads)})
    return res


@pytest.mark.parametrize("docs", [None, "mixed"])
def test_mamba2_ssd_shared_bc(docs):
    """Config 2's op at a reduced size: H = 8 heads sharing one B/C group, P = 64, N = 128, initial state."""
    case = make_mamba2_case(B=2, T=1000, H=8, P=64, N=128, G=1, seed=7, docs=docs, h0=True, baseline=True)
    want, got = _run_ssd_oracle(case), _run_ssd_cuda(case)
    tol = dict.fromkeys(want, 1e-2)
    tol["dA"] = 3e-2  # dA sums dg*dt over every token of a head: the reference reports the same loss of accuracy
    for name in want:  # (benchmarks/mamba2.md:107-114)
        assert compare({name: got[name]}, {name: want[name]}, tol[name], f"ssd {name}")


def test_mamba2_ssd_backward_routes_of_the_skip_term():
    """The layer's backward has three routes for dx: one fused pass when D is given and a gradient reaches y, the
    input side alone without D, and the input side alone when only the final state carries a gradient (then dD = 0).
    Each is held to the float64 oracle."""
    from jax_linear_attention_b200.layers import mamba2_ssd

    case = make_mamba2_case(B=1, T=300, H=4, P=64, N=128, G=1, seed=11, docs="mixed", h0=False, baseline=True)
    dev, f64 = "cuda", torch.float64
    half = ("x", "B", "C")
    for with_d, through_y in ((True, True), (False, True), (True, False)):
        names = ["x", "dt", "A", "B", "C"] + (["D"] if with_d else [])
        t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in half else torch.float32,
                             requires_grad=True) for n in names}
        r = {n: torch.tensor(case[n], dtype=f64, requires_grad=True) for n in names}
        seg = torch.tensor(case["seg"])
        y, st = mamba2_ssd(t["x"], t["dt"], t["A"], t["B"], t["C"], d=t.get("D"), segment_ids=seg.to(dev),
                           output_final_state=True)
        yr, sr = oracle_ssd.mamba2_ssd(r["x"], r["dt"], r["A"], r["B"], r["C"], d=r.get("D"), segment_ids=seg,
                                       output_final_state=True, round_v_to=torch.bfloat16)
        do = torch.tensor(case["do"]) * (1.0 if through_y else 0.0)
        dht = torch.tensor(case["dht"])
        outs, outs_r = ([y, st], [yr, sr]) if through_y else ([st], [sr])
        cot = [do.to(dev, torch.bfloat16), dht.to(dev)] if through_y else [dht.to(dev)]
        cot_r = [do.to(f64), dht.to(f64)] if through_y else [dht.to(f64)]
        got = torch.autograd.grad(outs, [t[n] for n in names], cot, allow_unused=True)
        want = torch.autograd.grad(outs_r, [r[n] for n in names], cot_r, allow_unused=True)
        for n, a, b in zip(names, got, want):
            if b is None:  # D and C reach only y
                assert not through_y and n in ("D", "C") and (a is None or float(a.abs().max()) == 0.0), n
                continue
            tol = 3e-2 if n == "A" else 1e-2
            assert rel_l2(a.detach().float().cpu().numpy(), b.numpy()) < tol, (with_d, through_y, n)


def test_mamba2_ssd_config2_full_size_runs_and_matches_a_slice():
    """The Mamba-2 benchmark workload at full size (B8 T2048 H64 P64 N128 G1): finite everywhere; batch row 0 against the oracle
    on a 4-head slice (heads are independent given B, C)."""
    from jax_linear_attention_b200.layers import mamba2_ssd

    case = baseline_config(2)
    dev = "cuda"
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in ("x", "B", "C") else torch.float32)
         for n in ("x", "dt", "A", "B", "C", "D")}
    y, _ = mamba2_ssd(t["x"], t["dt"], t["A"], t["B"], t["C"], d=t["D"])
    assert bool(torch.isfinite(y.float()).all())
    f64 = torch.float64
    s = {n: torch.tensor(case[n][:1], dtype=f64) for n in ("x", "dt", "B", "C")}
    want, _ = oracle_ssd.mamba2_ssd(s["x"][:, :, :4], s["dt"][:, :, :4], torch.tensor(case["A"][:4], dtype=f64),
                                    s["B"], s["C"], d=torch.tensor(case["D"][:4], dtype=f64),
                                    round_v_to=torch.bfloat16)
    compare({"y": y[:1, :, :4].float().cpu().numpy()}, {"y": want.numpy()}, 1e-2, "config2 slice")


@pytest.mark.parametrize("docs", [None, "uniform"])
def test_kda_default_dispatch_bf16(docs):
    """KDA (the op of the B4 T4096 H16 d128 benchmark workload at a reduced size) through impl='auto': bf16 tensors, per-channel gates, documents."""
    case = make_case("kda", B=2, T=600, H=4, K=128, V=128, seed=9, gates="kda_baseline", docs=docs, h0=True,
                     doc_range=(128, 600))
    want = run_oracle("kda", case, scale=case["meta"]["scale"], chunked=True)
    got = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="bfloat16")
    compare(got, want, 1e-2, "kda")


@pytest.mark.parametrize("width,dtype,neg", [(1, torch.bfloat16, False), (128, torch.bfloat16, True), (1, torch.float32, True)])
def test_gate_prologue_matches_the_cpu_restatement(width, dtype, neg):
    """g = -exp(A_log) softplus(a + dt_bias), beta = (2) sigmoid(b), and all their gradients."""
    from jax_linear_attention_b200.layers import gate_prologue
    from oracle import gates

    torch.manual_seed(3)
    B, T, H = 2, 300, 16
    shape = (B, T, H) if width == 1 else (B, T, H, width)
    dev = torch.device("cuda")
    a = (torch.randn(shape) * 2).to(dtype)
    b = torch.randn(B, T, H).to(dtype)
    a_log = torch.randn(H) * 0.5
    dt_bias = torch.randn(H * width).reshape(shape[2:]) - 1.0
    dg = torch.randn(shape)
    dbeta = torch.randn(B, T, H)
    leaves = [x.to(dev).requires_grad_(True) for x in (a, a_log, dt_bias, b)]
    g, beta = gate_prologue(leaves[0], leaves[1], leaves[2], leaves[3], allow_neg_eigval=neg)
    got = torch.autograd.grad([g, beta], leaves, [dg.to(dev), dbeta.to(dev)])
    ref = [x.double().requires_grad_(True) for x in (a, a_log, dt_bias, b)]
    g64, b64 = gates.mamba_gate(ref[0], ref[1], ref[2]), gates.write_strength(ref[3], neg)
    want = torch.autograd.grad([g64, b64], ref, [dg.double(), dbeta.double()])
    tol = 1e-5 if dtype == torch.float32 else 6e-3  # 16-bit: da, db are rounded to the activation dtype
    assert rel_l2(g.detach().cpu().numpy(), g64.detach().numpy()) < 1e-5
    assert rel_l2(beta.detach().cpu().numpy(), b64.detach().numpy()) < 1e-5
    for name, x, y in zip(("da", "dA_log", "ddt_bias", "db"), got, want):
        assert rel_l2(x.float().cpu().numpy(), y.numpy()) < (tol if name in ("da", "db") else 1e-4), name


@pytest.mark.parametrize("shape,group,act,nbg,dtype", [
    ((2, 300, 16, 128), None, "silu", True, torch.bfloat16),      # Gated DeltaNet output norm: one group per head
    ((2, 300, 16, 128), None, "sigmoid", True, torch.bfloat16),   # KDA
    ((3, 70, 4096), 4096, "silu", False, torch.bfloat16),         # Mamba-2, one group over d_inner (block-wide sum)
    ((3, 70, 1024), 64, "silu", False, torch.float32),            # grouped norm, float32
])
def test_gated_rms_norm_matches_the_cpu_restatement(shape, group, act, nbg, dtype):
    from jax_linear_attention_b200.layers import gated_rms_norm
    from oracle import gates

    torch.manual_seed(5)
    dev = torch.device("cuda")
    x = torch.randn(shape).to(dtype)
    z = torch.randn(shape).to(dtype)
    w = 1.0 + 0.1 * torch.randn(shape[-1])
    dy = torch.randn(shape).to(dtype)
    leaves = [t.to(dev).requires_grad_(True) for t in (x, z, w)]
    y = gated_rms_norm(leaves[0], leaves[1], leaves[2], eps=1e-5, activation=act, norm_before_gate=nbg, group_size=group)
    got = torch.autograd.grad([y], leaves, [dy.to(dev)])
    ref = [t.double().requires_grad_(True) for t in (x, z, w)]
    y64 = gates.gated_rms_norm(ref[0], ref[1], ref[2], eps=1e-5, activation=act, norm_before_gate=nbg, group_size=group)
    want = torch.autograd.grad([y64], ref, [dy.double()])
    tol = 1e-5 if dtype == torch.float32 else 6e-3  # 16-bit: y, dx, dz are rounded to the activation dtype
    assert rel_l2(y.detach().float().cpu().numpy(), y64.detach().numpy()) < tol
    for name, a, b in zip(("dx", "dz", "dweight"), got, want):
        assert rel_l2(a.float().cpu().numpy(), b.numpy()) < (tol if name != "dweight" else 1e-4), name


@pytest.mark.parametrize("K,head_dim,act,docs,with_state,bias,dtype", [
    (4, 128, True, True, True, False, torch.bfloat16),    # the q / k prologue of the mixers
    (4, 64, True, False, False, True, torch.bfloat16),
    (4, None, True, True, True, True, torch.float32),     # plain ShortConv
    (2, 128, False, True, True, False, torch.float32),
    (3, None, True, False, True, False, torch.bfloat16),
    (4, 256, True, True, True, True, torch.bfloat16),     # a head wider than 32 four-channel lanes: eight per thread
    (4, 256, True, True, False, False, torch.float32),
    (1, 128, True, True, False, True, torch.float16),     # no taps behind the token
])
def test_short_conv_matches_the_cpu_restatement(K, head_dim, act, docs, with_state, bias, dtype):
    from jax_linear_attention_b200.layers import short_conv
    from oracle import gates

    torch.manual_seed(11)
    B, T, Cn = 2, 333, 512
    dev = torch.device("cuda")
    x = torch.randn(B, T, Cn).to(dtype)
    w = torch.randn(Cn, K) * 0.5
    bb = torch.randn(Cn) * 0.3 if bias else None
    st = torch.randn(B, K - 1, Cn).to(dtype) if with_state else None
    seg = None
    if docs:  # documents of 1 .. 90 tokens, one starting at the first token after the state
        cuts = torch.sort(torch.randint(1, T, (B, 9)), dim=1).values
        seg = (torch.arange(T)[None, None] >= cuts[..., None]).sum(1).to(torch.int32)
    dy = torch.randn(B, T, Cn).to(dtype)
    names = ["x", "weight"] + (["bias"] if bias else []) + (["state"] if with_state else [])
    vals = {"x": x, "weight": w, "bias": bb, "state": st}
    leaves = {n: vals[n].to(dev).requires_grad_(True) for n in names}
    y, new_state = short_conv(leaves["x"], leaves["weight"], leaves.get("bias"), activation=act, head_dim=head_dim,
                              segment_ids=None if seg is None else seg.to(dev), state=leaves.get("state"))
    got = torch.autograd.grad([y], [leaves[n] for n in names], [dy.to(dev)])
    ref = {n: vals[n].double().requires_grad_(True) for n in names}
    y64, st64 = gates.short_conv(ref["x"], ref["weight"], ref.get("bias"), activation=act, head_dim=head_dim,
                                 segment_ids=seg, state=ref.get("state"))
    want = torch.autograd.grad([y64], [ref[n] for n in names], [dy.double()])
    tol = 1e-5 if dtype == torch.float32 else 6e-3
    assert rel_l2(y.detach().float().cpu().numpy(), y64.detach().numpy()) < tol
    assert torch.equal(new_state.detach().double().cpu(), st64.detach())
    for n, a, b in zip(names, got, want):
        assert rel_l2(a.float().cpu().numpy(), b.numpy()) < (tol if n in ("x", "state") else 2e-4), n


@pytest.mark.parametrize("T,Cn,head_dim", [(1, 264, None), (3, 264, 8), (33, 136, 136 // 17), (257, 1032, 8), (700, 128, 64)])
def test_short_conv_ragged_shapes(T, Cn, head_dim):
    """Sequences shorter than the kernel and than one walk, walks that end inside a group of tokens, and channel
    counts that fill neither a block nor a warp: forward, every gradient and the carried state against the oracle."""
    from jax_linear_attention_b200.layers import short_conv
    from oracle import gates

    torch.manual_seed(5)
    B, K = 3, 4
    dev = torch.device("cuda")
    x = torch.randn(B, T, Cn)
    w = torch.randn(Cn, K) * 0.5
    bb = torch.randn(Cn) * 0.3
    st = torch.randn(B, K - 1, Cn)
    seg = (torch.arange(T)[None] >= torch.randint(0, T + 1, (B, 1))).to(torch.int32) if T > 1 else None
    dy = torch.randn(B, T, Cn)
    vals = {"x": x, "weight": w, "bias": bb, "state": st}
    leaves = {n: v.to(dev).requires_grad_(True) for n, v in vals.items()}
    y, new_state = short_conv(leaves["x"], leaves["weight"], leaves["bias"], activation=True, head_dim=head_dim,
                              segment_ids=None if seg is None else seg.to(dev), state=leaves["state"])
    got = torch.autograd.grad([y], list(leaves.values()), [dy.to(dev)])
    ref = {n: v.double().requires_grad_(True) for n, v in vals.items()}
    y64, st64 = gates.short_conv(ref["x"], ref["weight"], ref["bias"], activation=True, head_dim=head_dim,
                                 segment_ids=seg, state=ref["state"])
    want = torch.autograd.grad([y64], list(ref.values()), [dy.double()])
    assert rel_l2(y.detach().cpu().numpy(), y64.detach().numpy()) < 1e-5
    assert torch.equal(new_state.detach().double().cpu(), st64.detach())
    for n, a, b in zip(vals, got, want):
        assert rel_l2(a.cpu().numpy(), b.numpy()) < 2e-4, n


def test_mamba2_ssd_config2_gradient_slice_against_the_oracle():
    """The Mamba-2 benchmark workload's shape (T2048 H64 P64 N128 G1 bf16), forward + backward: the full-size call is finite
    everywhere; batch row 0 restricted to 4 heads is run on its own through the kernels and held to the float64
    oracle for y and ALL gradients (dx, ddt, dA, dB, dC, dD) -- dB and dC sum over the heads that share them, so they
    are only comparable on a call that has exactly those heads; and the full-size call's dx and ddt of those heads
    equal the small call's (heads are independent given B and C)."""
    from jax_linear_attention_b200.layers import mamba2_ssd

    case = baseline_config(2)
    dev = "cuda"
    half = ("x", "B", "C")
    names = ("x", "dt", "A", "B", "C", "D")
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in half else torch.float32, requires_grad=True)
         for n in names}
    do = torch.tensor(case["do"], device=dev, dtype=torch.bfloat16)
    y, _ = mamba2_ssd(t["x"], t["dt"], t["A"], t["B"], t["C"], d=t["D"])
    full = dict(zip(names, torch.autograd.grad(y, [t[n] for n in names], do)))
    assert all(bool(torch.isfinite(g.float()).all()) for g in full.values())

    heads = slice(8, 12)
    small = {n: case[n][:1] for n in ("x", "dt", "B", "C", "do")}
    small = {n: (v[:, :, heads] if n in ("x", "dt", "do") else v) for n, v in small.items()}
    small["A"], small["D"] = case["A"][heads], case["D"][heads]
    small["dht"] = np.zeros((1, 4, 128, 64), np.float32)
    want, got = _run_ssd_oracle(small), _run_ssd_cuda(small)
    tol = dict.fromkeys(want, 1e-2)
    tol["dA"] = 3e-2  # dA sums dg * dt over every token of a head (the reference reports the same loss of accuracy)
    for name in want:
        if name != "state":
            compare({name: got[name]}, {name: want[name]}, tol[name], f"config2 slice {name}")
    for n in ("x", "dt"):
        a = full[n][:1, :, heads].float().cpu().numpy()
        assert rel_l2(a, got["d" + n]) < 4e-3, n  # same kernels; dB/dC partial sums differ in order only
