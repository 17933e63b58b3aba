"""Gated DeltaNet-2 (``kind="gdn2"``: erase gate ``b`` per key channel, write gate ``w`` per value channel) on the
GPU -- the KDA token scan with a separate read key ``b * k`` -- against the reference's float64 fixtures, the CPU
oracle's autograd, and KDA itself where ``b = w = beta``. Tolerances: float32 tensors 2e-5 of the maximum (forward)
and relative L2 <= 1e-4 (gradients); bf16 tensors relative L2 <= 1e-2, the bound the reference holds its GDN-2
kernels to (tests/test_mosaic_gpu_gdn2.py of the reference)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle.cases import make_case, max_rel, rel_l2
from tests._util import compare, load_golden, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["gdn2_dense_h0", "gdn2_packed_l2norm", "gdn2_extreme", "gdn2_d128"])
def test_forward_matches_the_reference_fixtures(name):
    meta, ins, want = load_golden(name)
    ins = dict(ins)
    if "cu" in meta:
        cu = np.asarray(meta["cu"])
        ins["seg"] = np.searchsorted(cu[1:], np.arange(meta["T"]), side="right")[None].astype(np.int32)
    got = run_cuda("gdn2", ins, scale=meta["scale"], dtype="float32", l2norm=bool(meta.get("l2norm")), grads=False)
    assert max_rel(got["o"], want["o"]) < 2e-5, max_rel(got["o"], want["o"])
    assert max_rel(got["ht"], want["final"]) < 2e-5


@pytest.mark.parametrize("spec", [
    dict(B=2, T=150, H=2, K=32, V=16, docs="mixed", h0=True),
    dict(B=1, T=90, H=3, K=64, V=32, docs=None, h0=False, l2norm=True),
    dict(B=1, T=130, H=2, K=128, V=128, docs="uniform", doc_range=(10, 60), h0=True, gates="extreme"),
])
def test_float32_gradients_match_the_oracle_autograd(spec):
    case = make_case("gdn2", seed=71, dtype="float32", **spec)
    l2 = bool(spec.get("l2norm"))
    want = run_oracle("gdn2", case, scale=case["meta"]["scale"], l2norm=l2)
    got = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="float32", l2norm=l2)
    compare(got, want, 1e-4, f"gdn2 f32 {spec}")


@pytest.mark.parametrize("gates,docs,T", [("kda_baseline", "mixed", 300), ("plain", "uniform", 700),
                                          ("kda_baseline", None, 64)])
def test_bf16_head_128_runs_the_chunked_kernels_and_matches_the_oracle(gates, docs, T):
    """bf16 tensors with K = V = 128 take the KDA chunk kernels with the read key in tiles of its own: forward and
    every gradient (q, k, v, g, b, w, initial state) against the float64 oracle's autograd."""
    case = make_case("gdn2", B=2, T=T, H=4, K=128, V=128, seed=72 + T, gates=gates, docs=docs, h0=True,
                     doc_range=(40, 300))
    want = run_oracle("gdn2", case, scale=case["meta"]["scale"])
    got = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="bfloat16")
    compare(got, want, 1e-2, f"gdn2 bf16 d128 {gates} {docs}")
    scan = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="bfloat16", precision="highest")
    assert any(not np.array_equal(got[n], scan[n]) for n in got), "the chunked kernels did not run"
    compare(got, scan, 1e-2, "gdn2 chunked against the token scan")


def test_float16_head_128_runs_the_chunked_kernels():
    """f16 tensors take the same kernels (factored scores up to exp(+-6), the exact loop beyond)."""
    case = make_case("gdn2", B=1, T=300, H=2, K=128, V=128, seed=77, gates="plain", docs="mixed", h0=True,
                     dtype="float16")
    want = run_oracle("gdn2", case, scale=case["meta"]["scale"])
    got = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="float16")
    compare(got, want, 1e-2, "gdn2 f16 d128")
    scan = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="float16", precision="highest")
    assert any(not np.array_equal(got[n], scan[n]) for n in got), "the chunked kernels did not run"


def test_bf16_strong_decay_takes_the_exact_score_path():
    """Channels that decay by e^-80 at one token in ten (the factored scores would overflow) and gates at 0 and 1:
    the chunks run the exact fp32 loops, forward and backward, with the read key in its own role."""
    case = make_case("gdn2", B=1, T=320, H=2, K=128, V=128, seed=75, gates="extreme", docs="mixed", h0=True)
    assert float(np.abs(case["g"]).max()) >= 80.0
    want = run_oracle("gdn2", case, scale=case["meta"]["scale"])
    got = run_cuda("gdn2", case, scale=case["meta"]["scale"], dtype="bfloat16")
    assert all(np.isfinite(x).all() for x in got.values())
    compare(got, want, 1.5e-2, "gdn2 extreme gates")


def test_bf16_l2norm_and_packed_rows():
    """In-op unit norm (applied before the erase gate multiplies the key) and cu_seqlens rows with partial chunks."""
    from jax_linear_attention_b200 import ops

    case = make_case("gdn2", B=1, T=200, H=2, K=128, V=128, seed=76, gates="kda_baseline", l2norm=True)
    cu = [0, 64, 65, 192, 200]
    dev = "cuda"
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16) for n in ("q", "k", "v", "b", "w")}
    g = torch.tensor(case["g"], device=dev)
    h0 = torch.tensor(np.random.default_rng(1).standard_normal((4, 2, 128, 128)).astype(np.float32) * 0.5, device=dev)
    outs = []
    for precision in (None, "highest"):
        with torch.no_grad():
            outs.append(ops.linear_attention("gdn2", t["q"], t["k"], t["v"], g=g, b=t["b"], w=t["w"],
                                             cu_seqlens=torch.tensor(cu, device=dev, dtype=torch.int32),
                                             initial_state=h0, output_final_state=True, use_qk_l2norm=True,
                                             scale=case["meta"]["scale"], precision=precision))
    (o, f), (o_ref, f_ref) = outs
    assert rel_l2(o.float().cpu().numpy(), o_ref.float().cpu().numpy()) < 1e-2
    assert rel_l2(f.cpu().numpy(), f_ref.cpu().numpy()) < 1e-2


def test_equal_gates_are_kda():
    """``b = w = beta`` (reference.py:330-331): the same token scan, so float32 results agree to rounding."""
    case = make_case("kda", B=1, T=120, H=2, K=32, V=32, seed=73, dtype="float32", docs="mixed", h0=True)
    kda = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="float32", grads=False)
    two = dict(case)
    beta = two.pop("beta")[..., None]
    two["b"] = np.broadcast_to(beta, case["k"].shape).copy()
    two["w"] = np.broadcast_to(beta, case["v"].shape).copy()
    gdn2 = run_cuda("gdn2", two, scale=case["meta"]["scale"], dtype="float32", grads=False)
    assert rel_l2(gdn2["o"], kda["o"]) < 1e-6 and rel_l2(gdn2["ht"], kda["ht"]) < 1e-6


def test_bad_gate_shapes_are_rejected_on_the_host():
    from jax_linear_attention_b200 import ops

    q = torch.zeros(1, 8, 2, 32, device="cuda")
    v = torch.zeros(1, 8, 2, 16, device="cuda")
    with pytest.raises(ValueError, match="b must be"):
        ops.linear_attention("gdn2", q, q, v, g=q, b=v, w=v)
    with pytest.raises(ValueError, match="takes gates"):
        ops.linear_attention("gdn2", q, q, v, g=q, beta=q[..., 0])
