"""GPU parity of the fp32 token-scan kernels (JLA_PATH_RECURRENT) through the public API and the C ABI.

Tolerance: relative L2 error <= 1e-5 against the float64 oracle (the fp32 configuration's bar), on the
golden fixtures made by the reference's own oracles and on the fp32 benchmark workload (GDN forward, B1 T512 H4 d64).
"""

import numpy as np
import pytest
import torch

from oracle.cases import baseline_config, make_case, rel_l2
from tests._util import compare, load_golden, run_cuda, run_oracle

pytestmark = pytest.mark.gpu
TOL = 1e-5

SCALAR = ["gdn_dense_h0", "gdn_docs_gqa", "gdn_extreme", "gdn_l2norm", "gdn_beta2", "gdn_f32", "dn_docs",
          "dn_l2norm_dense", "sgla_docs_gqa", "sgla_extreme"]
KDA = ["kda_dense_h0", "kda_packed", "kda_packed_h0_l2norm", "kda_extreme", "kda_grouped", "kda_d128_packed_h0",
       "kda_d128_extreme"]


@pytest.mark.parametrize("name", SCALAR)
def test_golden_scalar_gate_fixtures(name):
    meta, ins, want = load_golden(name)
    got = run_cuda(meta["kind"], ins, scale=meta["scale"], dtype="float32", l2norm=bool(meta.get("l2norm")),
                   precision="highest")
    compare(got, want, TOL, name)


@pytest.mark.parametrize("name", KDA)
def test_golden_kda_fixtures(name):
    meta, ins, want = load_golden(name)
    if "cu" in meta:
        cu = np.asarray(meta["cu"])
        ins["seg"] = np.searchsorted(cu[1:], np.arange(meta["T"]), side="right")[None].astype(np.int32)
    got = run_cuda("kda", ins, scale=meta["scale"], dtype="float32", l2norm=bool(meta.get("l2norm")),
                   precision="highest", grads=False)
    compare(got, {"o": want["o"], "ht": want["final"]}, TOL, name)


def test_baseline_config0_forward_fp32():
    """The fp32 benchmark workload: GDN forward, fp32, B=1 T=512 H=4 d=64, zero initial state, one document."""
    case = baseline_config(0)
    want = run_oracle("gated_deltanet", case, scale=case["meta"]["scale"], grads=False, chunked=True)
    got = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="float32", grads=False)
    table = compare(got, want, TOL, "config0")
    print("config0 rel-L2:", table)


@pytest.mark.parametrize("kind", ["simple_gla", "deltanet", "gated_deltanet", "kda"])
def test_gradients_fp32_docs_h0(kind):
    case = make_case(kind, B=2, T=150, H=4, Hk=2, K=64, V=32, seed=11, dtype="float32", docs="mixed", h0=True)
    want = run_oracle(kind, case, scale=case["meta"]["scale"])
    got = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="float32")
    compare(got, want, TOL, kind)


@pytest.mark.parametrize("kind", ["simple_gla", "gated_deltanet", "kda"])
def test_cu_seqlens_per_sequence_states_and_empty_sequence(kind):
    case = make_case(kind, B=1, T=200, H=2, K=32, V=32, seed=12, dtype="float32")
    cu = [0, 13, 13, 77, 141, 200]
    rng = np.random.default_rng(0)
    case["h0"] = (0.5 * rng.standard_normal((5, 2, 32, 32))).astype(np.float32)
    case["dht"] = (0.1 * rng.standard_normal((5, 2, 32, 32))).astype(np.float32)
    want = run_oracle(kind, case, scale=case["meta"]["scale"], cu_seqlens=cu)
    got = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="float32", cu_seqlens=cu)
    compare(got, want, TOL, kind)
    assert np.array_equal(got["ht"][1], case["h0"][1])  # the empty sequence keeps its initial state


def test_bf16_storage_through_the_exact_path():
    case = make_case("gated_deltanet", B=1, T=130, H=2, K=128, V=128, seed=13, dtype="bfloat16", docs="mixed",
                     h0=True)
    want = run_oracle("gated_deltanet", case, scale=case["meta"]["scale"])
    got = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16", precision="highest")
    compare(got, want, 6e-3, "bf16 storage")  # outputs are rounded to bf16: 2^-9 relative per element


def test_rejected_calls_raise():
    from jax_linear_attention_b200 import ops

    q = torch.zeros(2, 8, 2, 64, device="cuda")
    g = torch.zeros(2, 8, 2, device="cuda")
    with pytest.raises(ValueError, match="takes gates"):
        ops.linear_attention("gated_deltanet", q, q, q, g=g)
    with pytest.raises(ValueError, match="cu_seqlens packs"):
        ops.linear_attention("simple_gla", q, q, q, g=g, cu_seqlens=torch.tensor([0, 8]))
    with pytest.raises(ValueError, match="unknown linear-attention kind"):
        ops.linear_attention("nope", q, q, q)
    with pytest.raises(ValueError, match="no CPU fallback"):
        ops.linear_attention("simple_gla", q.cpu(), q.cpu(), q.cpu(), g=g.cpu())


def test_head_size_256_runs_the_token_scan():
    """K = V = 256 (the head size of the reference's K-blocked kernels, ``mosaic_gpu/scalar_gate_kb.py``): no chunk
    kernel here, so 16-bit calls of that size take the fp32 token scan; forward and all gradients against the
    float64 oracle at the tolerance of bf16 tensors."""
    case = make_case("gated_deltanet", B=1, T=150, H=2, K=256, V=256, seed=31, docs="mixed", h0=True)
    want = run_oracle("gated_deltanet", case, scale=case["meta"]["scale"])
    got = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    compare(got, want, 1e-2, "gdn K = V = 256")
