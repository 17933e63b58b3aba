"""GPU parity of the chunk-64 tensor-core kernels (bf16 / f16 operands, fp32 state and accumulation).

Tolerance of the path: relative L2 error <= 1e-2 for outputs and gradients against the float64 oracle on the
same (bf16-representable) inputs. Stage-level checks use the reference's own metric max|x - want| / max|want|
and thresholds (T0 4e-3, stages 1e-2: tests/test_mosaic_gpu_gated_delta_rule.py:104-146).
"""

import numpy as np
import pytest
import torch

from oracle import staged
from oracle.cases import baseline_config, make_case, max_rel, rel_l2, seg_to_cu
from tests._util import ChunkedLayout, cabi_fwd_bwd, compare, run_cuda, run_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2


@pytest.mark.parametrize("kind,K,V,Hk", [("gated_deltanet", 128, 128, 2), ("gated_deltanet", 64, 64, 1),
                                         ("deltanet", 64, 128, 2), ("simple_gla", 128, 64, 1)])
def test_stages_match_the_cpu_model(kind, K, V, Hk):
    case = make_case(kind, B=2, T=200, H=2, Hk=Hk, K=K, V=V, seed=5, docs="mixed", h0=True)
    scale = case["meta"]["scale"]
    delta = kind != "simple_gla"
    out = cabi_fwd_bwd(kind, case, scale=scale)
    f64 = torch.float64
    d = {n: torch.tensor(case[n], dtype=f64) for n in ("q", "k", "v", "g", "beta", "h0") if n in case}
    st = staged.forward(d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), delta=delta, scale=scale, h0=d["h0"],
                        segment_ids=torch.tensor(case["seg"]))
    bw = staged.backward(st, torch.tensor(case["do"], dtype=f64), torch.tensor(case["dht"], dtype=f64))
    lay = ChunkedLayout(out["problem"], out["residuals"], out["bwd_scratch"])
    G, beta = lay.gates()
    assert max_rel(G, st["G"]) < 1e-5
    if delta:
        assert max_rel(beta, st["beta"]) == 0.0
        assert max_rel(lay.t0(), st["T0"]) < 4e-3
        assert max_rel(lay.vn(), st["Vn"]) < 1e-2
        if lay.transposed:
            w = lay.w()
            w[:, :, 200 // 64, 200 % 64:] = 0.0  # rows past the end of the last chunk are never used
            assert max_rel(w, st["W"]) < 1e-2
        assert max_rel(lay.dvn(), bw["dVn"]) < 1e-2
    assert max_rel(lay.h(), st["h"]) < 1e-2
    assert max_rel(lay.dh(), bw["dh"]) < 1e-2


CASES = [
    # kind, kwargs
    ("gated_deltanet", dict(B=2, T=1000, H=4, K=128, V=128, docs=None, h0=True)),          # dense, odd T
    ("gated_deltanet", dict(B=2, T=1536, H=4, K=128, V=128, docs="mixed", h0=True)),       # random documents
    ("gated_deltanet", dict(B=2, T=777, H=4, K=64, V=64, docs="mixed", h0=True)),          # K = V = 64
    ("gated_deltanet", dict(B=1, T=1100, H=8, Hk=2, K=128, V=128, docs="mixed", h0=True)),  # grouped key heads
    ("gated_deltanet", dict(B=1, T=1024, H=4, K=128, V=128, docs="mixed", h0=True, gates="extreme")),
    ("gated_deltanet", dict(B=1, T=1000, H=4, K=128, V=128, docs="mixed", h0=True, beta_scale=2.0)),
    ("gated_deltanet", dict(B=2, T=1000, H=4, Hk=2, K=128, V=128, docs="mixed", h0=True, l2norm=True)),
    ("gated_deltanet", dict(B=4, T=700, H=8, K=128, V=128, docs="mixed", h0=True)),
    ("gated_deltanet", dict(B=1, T=17, H=2, K=128, V=64, docs=None, h0=False)),            # shorter than a chunk
    ("deltanet", dict(B=2, T=1000, H=4, K=128, V=128, docs=None, h0=True)),
    ("deltanet", dict(B=2, T=777, H=4, K=64, V=64, docs="mixed", h0=True)),
    ("deltanet", dict(B=2, T=1000, H=4, K=128, V=128, docs="mixed", h0=True, l2norm=True)),
    ("simple_gla", dict(B=2, T=1000, H=4, K=128, V=128, docs=None, h0=True)),
    ("simple_gla", dict(B=1, T=1100, H=8, Hk=2, K=128, V=64, docs="mixed", h0=True)),
    ("simple_gla", dict(B=2, T=1000, H=8, Hk=1, K=128, V=64, docs="mixed", h0=True)),      # Mamba-2 shared B/C
    ("simple_gla", dict(B=1, T=1024, H=4, K=128, V=128, docs="mixed", h0=True, gates="extreme")),
    ("simple_gla", dict(B=1, T=300, H=4, Hk=2, K=64, V=128, docs="mixed", h0=True)),  # output wider than the q tile
]


@pytest.mark.parametrize("kind,spec", CASES, ids=[f"{k}-{i}" for i, (k, _) in enumerate(CASES)])
def test_outputs_and_gradients_bf16(kind, spec):
    case = make_case(kind, seed=100 + len(str(spec)), **spec)
    scale, l2 = case["meta"]["scale"], bool(spec.get("l2norm"))
    want = run_oracle(kind, case, scale=scale, l2norm=l2, chunked=True)
    got = run_cuda(kind, case, scale=scale, dtype="bfloat16", l2norm=l2)
    table = compare(got, want, TOL, f"{kind} {spec}")
    assert all(np.isfinite(v).all() for v in got.values()), table


WIDE = [
    ("gated_deltanet", dict(B=2, T=300, H=2, K=128, V=256, docs="mixed", h0=True)),            # the usual expand_v = 2
    ("gated_deltanet", dict(B=1, T=200, H=4, Hk=2, K=128, V=512, docs="uniform", h0=True, l2norm=True)),
    ("simple_gla", dict(B=1, T=260, H=2, K=64, V=384, docs="mixed", h0=True)),
    ("kda", dict(B=1, T=200, H=2, K=128, V=256, docs="mixed", h0=True, gates="kda_baseline")),
]


@pytest.mark.parametrize("kind,spec", WIDE, ids=[f"{k}-V{s['V']}" for k, s in WIDE])
def test_wide_value_heads_run_as_blocks_of_128_channels(kind, spec):
    """V = 256, 384, 512: the chunk kernels run the head as V / 128 value heads that share its key and gates (the
    columns of the state are independent recurrences). Outputs, final state and every gradient -- the gates' are
    summed over the blocks, the states permuted back -- against the float64 oracle; and where the token scan can run
    the shape (V = 256) the two paths give different bits, i.e. the chunk kernels did run."""
    case = make_case(kind, seed=7 + spec["V"], **spec)
    scale, l2 = case["meta"]["scale"], bool(spec.get("l2norm"))
    want = run_oracle(kind, case, scale=scale, l2norm=l2)
    got = run_cuda(kind, case, scale=scale, dtype="bfloat16", l2norm=l2)
    compare(got, want, TOL, f"wide {kind} {spec}")
    if spec["V"] == 256:
        scan = run_cuda(kind, case, scale=scale, dtype="bfloat16", l2norm=l2, precision="highest")
        assert any(not np.array_equal(got[n], scan[n]) for n in got), "the chunk kernels did not run"


def test_float16():
    case = make_case("gated_deltanet", B=1, T=300, H=2, K=128, V=128, seed=3, dtype="float16", docs="mixed", h0=True)
    want = run_oracle("gated_deltanet", case, scale=case["meta"]["scale"], chunked=True)
    got = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="float16")
    compare(got, want, 3e-3, "float16")  # 11-bit mantissa: tighter than bf16


@pytest.mark.parametrize("kind", ["simple_gla", "gated_deltanet"])
def test_cu_seqlens_per_sequence_states_and_empty_sequence(kind):
    case = make_case(kind, B=1, T=700, H=2, K=128, V=64, seed=12)
    cu = [0, 13, 13, 77, 141, 500, 700]
    rng = np.random.default_rng(0)
    case["h0"] = (0.5 * rng.standard_normal((6, 2, 128, 64))).astype(np.float32)
    case["dht"] = (0.1 * rng.standard_normal((6, 2, 128, 64))).astype(np.float32)
    want = run_oracle(kind, case, scale=case["meta"]["scale"], cu_seqlens=cu)
    got = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="bfloat16", cu_seqlens=cu)
    compare(got, want, TOL, kind)
    assert np.array_equal(got["ht"][1], case["h0"][1])
    assert np.array_equal(got["dh0"][1], case["dht"][1])


def test_cu_seqlens_equals_segment_ids():
    """Packing with cu_seqlens or with segment ids gives the same outputs (zero initial states)."""
    case = make_case("gated_deltanet", B=1, T=900, H=2, K=128, V=128, seed=14, docs="mixed")
    cu = seg_to_cu(case["seg"][0])
    a = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16", grads=False)
    del case["seg"]
    b = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16", grads=False, cu_seqlens=cu)
    assert rel_l2(b["o"], a["o"]) < 4e-3  # chunk boundaries differ, so rounding differs
    assert rel_l2(b["ht"][-1], a["ht"][0]) < 4e-3


def test_final_state_chains_across_two_calls():
    from jax_linear_attention_b200 import ops

    case = make_case("gated_deltanet", B=2, T=1024, H=2, K=128, V=128, seed=15, h0=True)
    t = {n: torch.tensor(case[n], device="cuda", dtype=torch.bfloat16 if n in "qkv" else torch.float32)
         for n in ("q", "k", "v", "g", "beta", "h0")}
    o, s = ops.linear_attention("gated_deltanet", t["q"], t["k"], t["v"], g=t["g"], beta=t["beta"],
                                initial_state=t["h0"], output_final_state=True)
    h = 512  # chunk aligned: the two halves walk exactly the same chunks, so the results are identical
    o1, s1 = ops.linear_attention("gated_deltanet", t["q"][:, :h], t["k"][:, :h], t["v"][:, :h], g=t["g"][:, :h],
                                  beta=t["beta"][:, :h], initial_state=t["h0"], output_final_state=True)
    o2, s2 = ops.linear_attention("gated_deltanet", t["q"][:, h:], t["k"][:, h:], t["v"][:, h:], g=t["g"][:, h:],
                                  beta=t["beta"][:, h:], initial_state=s1, output_final_state=True)
    assert torch.equal(torch.cat([o1, o2], 1), o) and torch.equal(s2, s)


def test_baseline_config1_full_size_slices_and_properties():
    """The headline benchmark workload at full size (B8 T2048 H16 d128, bf16, packed documents): two (b, h) slices against the
    oracle, plus the size-independent property that every head of every batch row is independent (running a
    slice alone gives the same bits)."""
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.ops.cuda import no_pieces

    case = baseline_config(1)
    dev = "cuda"
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in ("q", "k", "v", "do") else torch.float32,
                         requires_grad=n in ("q", "k", "v", "g", "beta"))
         for n in ("q", "k", "v", "g", "beta", "do")}
    seg = torch.tensor(case["seg"], device=dev)
    o, s = ops.linear_attention("gated_deltanet", t["q"], t["k"], t["v"], g=t["g"], beta=t["beta"], segment_ids=seg,
                                output_final_state=True)
    grads = torch.autograd.grad(o, [t[n] for n in ("q", "k", "v", "g", "beta")], t["do"])
    assert all(bool(torch.isfinite(x).all()) for x in (o, s, *grads))
    for b, h in ((0, 0), (7, 15)):
        sl = {n: case[n][b:b + 1, :, h:h + 1] for n in ("q", "k", "v", "g", "beta", "do")}
        sl["seg"] = case["seg"][b:b + 1]
        sl["dht"] = np.zeros((1, 1, 128, 128), np.float32)
        want = run_oracle("gated_deltanet", sl, scale=128 ** -0.5, chunked=True)
        got = dict(o=o.detach()[b:b + 1, :, h:h + 1].float().cpu().numpy(),
                   ht=s.detach()[b:b + 1, h:h + 1].cpu().numpy())
        for n, gr in zip(("q", "k", "v", "g", "beta"), grads):
            got["d" + n] = gr[b:b + 1, :, h:h + 1].float().cpu().numpy()
        compare(got, want, TOL, f"config1 slice {b},{h}")
        with no_pieces():  # (one row of one head would otherwise be cut into pieces along T: same values to 1e-2, other bits)
            alone = run_cuda("gated_deltanet", sl, scale=128 ** -0.5, dtype="bfloat16")
        assert np.array_equal(alone["o"], got["o"]) and np.array_equal(alone["dk"], got["dk"])


@pytest.mark.parametrize("kind", ["gated_deltanet", "kda"])
def test_shared_prep_and_state_only_backward_match_the_plain_calls(kind):
    """Passes that share one chunk table (JLA_FLAG_PREP_DONE), the reverse-state-pass-only backward
    (JLA_FLAG_STATE_GRADS_ONLY) and the state-only forward (JLA_FLAG_STATE_ONLY) give the plain calls' results bit
    for bit; for KDA the shared buffer also carries the gate-folded operands."""
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.ops.cuda import final_state_only, shared_prep, state_grads_only

    case = make_case(kind, B=1, T=1500, H=4, K=128, V=128, seed=77, docs="mixed", h0=True,
                     gates="kda_baseline" if kind == "kda" else "plain")
    dev = torch.device("cuda")
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in "qkv" else torch.float32)
         for n in ("q", "k", "v", "g", "beta")}
    cu = torch.tensor([0, 300, 301, 900, 1500], dtype=torch.int32, device=dev)
    h0 = torch.randn(4, 4, 128, 128, device=dev) * 0.1
    do = torch.tensor(case["do"], device=dev, dtype=torch.bfloat16)

    kleaf = t["k"].clone().requires_grad_(True)

    def run(v, init, grad):
        leaf = init.clone().requires_grad_(grad)
        o, f = ops.linear_attention(kind, t["q"], kleaf if grad else t["k"], v, g=t["g"], beta=t["beta"], cu_seqlens=cu,
                                    initial_state=leaf, output_final_state=True)
        return o, f, leaf

    o1, f1, _ = run(t["v"], h0, False)
    o2, f2, leaf2 = run(t["v"] * 0.5, h0 * 2, True)
    want_dh0, want_dk = torch.autograd.grad([o2], [leaf2, kleaf], [do])
    with shared_prep():
        o1s, f1s, _ = run(t["v"], h0, False)
        o2s, f2s, leaf2s = run(t["v"] * 0.5, h0 * 2, True)  # second call: tables reused, residuals saved
    assert torch.equal(o1, o1s) and torch.equal(f1, f1s)
    assert torch.equal(o2, o2s) and torch.equal(f2, f2s)
    with state_grads_only():
        (got_dh0,) = torch.autograd.grad([o2s], [leaf2s], [do], retain_graph=True)
    assert torch.equal(got_dh0, want_dh0)
    full_dh0, full_dk = torch.autograd.grad([o2s], [leaf2s, kleaf], [do])
    assert torch.equal(full_dh0, want_dh0)
    # everything the backward reads from the shared prologue was written by its first (forward-only) call
    assert torch.equal(full_dk, want_dk)
    with final_state_only():  # JLA_FLAG_STATE_ONLY: the outputs are skipped, the state pass is the same
        _, f1o, _ = run(t["v"], h0, False)
    assert torch.equal(f1o, f1)


@pytest.mark.parametrize("kind", ["gated_deltanet", "kda"])
def test_a_call_without_tokens_passes_the_state_through(kind):
    """T = 0 (an empty shard): no chunk kernel runs; the final state is the initial state and its gradient is the
    upstream gradient of the final state."""
    from jax_linear_attention_b200 import ops

    dev = torch.device("cuda")
    B, H, K, V = 2, 2, 128, 128
    q = torch.zeros(B, 0, H, K, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(B, 0, H, V, device=dev, dtype=torch.bfloat16)
    g = torch.zeros((B, 0, H, K) if kind == "kda" else (B, 0, H), device=dev)
    beta = torch.zeros(B, 0, H, device=dev)
    h0 = torch.randn(B, H, K, V, device=dev, requires_grad=True)
    o, f = ops.linear_attention(kind, q, q, v, g=g, beta=beta, initial_state=h0, output_final_state=True)
    assert o.shape == v.shape and torch.equal(f, h0.detach())
    dht = torch.randn_like(f)
    (dh0,) = torch.autograd.grad([f], [h0], [dht])
    assert torch.equal(dh0, dht)
