"""Chunked KDA forward (per-channel gates) on the tensor cores against the CPU oracle and against the library's
own fp32 token scan, and the chunked backward (reverse state pass + chunk-parallel gradient kernels) against the
oracle's autograd. Tolerance: relative L2 <= 1e-2 (bf16 tensors, fp32 state); 1.5e-2 for the gradients under
extreme gates, the reference's own bound for KDA gradients (tests/test_mosaic_gpu_kda.py:98-130 of the reference)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

from oracle.cases import baseline_config, make_case, rel_l2
from tests._util import compare, load_golden, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


def _forward(case, *, precision=None, cu=None, l2norm=False, h0=True):
    from jax_linear_attention_b200 import ops

    dev = "cuda"
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16) for n in ("q", "k", "v")}
    g = torch.tensor(case["g"], device=dev)
    beta = torch.tensor(case["beta"], device=dev)
    opts = dict(scale=case["meta"]["scale"], output_final_state=True, precision=precision, use_qk_l2norm=l2norm)
    if h0 and "h0" in case:
        opts["initial_state"] = torch.tensor(case["h0"], device=dev)
    if "seg" in case and cu is None:
        opts["segment_ids"] = torch.tensor(case["seg"], device=dev)
    if cu is not None:
        opts["cu_seqlens"] = torch.tensor(cu, device=dev, dtype=torch.int32)
    with torch.no_grad():
        o, ht = ops.linear_attention("kda", t["q"], t["k"], t["v"], g=g, beta=beta, impl="cuda", **opts)
    torch.cuda.synchronize()
    return o.float().cpu().numpy(), ht.float().cpu().numpy()


def test_bf16_calls_take_the_chunked_path():
    from jax_linear_attention_b200 import _lib
    from jax_linear_attention_b200.ops.cuda import _problem

    import ctypes as C

    lib = _lib.load()
    p = _problem("kda", torch.bfloat16, 2, 256, 4, 4, 128, 128, 0, 1.0, _lib.FLAG_SAVE_RESIDUALS, None)
    assert lib.jla_residual_bytes(C.byref(p)) > 0         # only the chunked path keeps residuals
    p.flags = 0
    assert lib.jla_fwd_scratch_bytes(C.byref(p)) > 0      # and needs a forward scratch when it keeps none
    p16 = _problem("kda", torch.float16, 2, 256, 4, 4, 128, 128, 0, 1.0, _lib.FLAG_SAVE_RESIDUALS, None)
    assert lib.jla_residual_bytes(C.byref(p16)) > 0       # f16 tensors as well
    p64 = _problem("kda", torch.bfloat16, 2, 256, 4, 4, 64, 64, 0, 1.0, 0, None)
    assert lib.jla_fwd_scratch_bytes(C.byref(p64)) == 0   # other head sizes stay on the token scan


@pytest.mark.parametrize("docs", [None, "uniform", "mixed"])
@pytest.mark.parametrize("T", [64, 200, 1024])
def test_forward_matches_the_oracle(docs, T):
    case = make_case("kda", B=2, T=T, H=4, K=128, V=128, seed=21 + T, gates="kda_baseline", docs=docs, h0=True,
                     doc_range=(16, max(T // 2, 17)))
    want = run_oracle("kda", case, scale=case["meta"]["scale"], grads=False)
    o, ht = _forward(case)
    compare({"o": o, "ht": ht}, want, 1e-2, f"kda T={T} docs={docs}")


def test_plain_gates_and_grouped_key_heads():
    """Gates of the scalar-gate tests' size per channel (decay up to e^-5 per token in places) and Hk < H."""
    case = make_case("kda", B=1, T=500, H=4, Hk=2, K=128, V=128, seed=5, gates="plain", h0=True)
    want = run_oracle("kda", case, scale=case["meta"]["scale"], grads=False)
    o, ht = _forward(case)
    compare({"o": o, "ht": ht}, want, 1e-2, "kda plain gates")


def test_strong_decay_takes_the_exact_score_path():
    """Channels that decay by e^-80 at one token in ten: the factored tensor-core scores would overflow, so these
    chunks run the exact fp32 score loop; beta hits 0 and 1."""
    case = make_case("kda", B=1, T=320, H=2, K=128, V=128, seed=6, gates="extreme", docs="mixed", h0=True)
    assert float(np.abs(case["g"]).max()) >= 80.0
    want = run_oracle("kda", case, scale=case["meta"]["scale"], grads=False)
    o, ht = _forward(case)
    assert np.isfinite(o).all() and np.isfinite(ht).all()
    compare({"o": o, "ht": ht}, want, 1e-2, "kda extreme gates")


def test_packed_sequences_with_l2norm_match_the_token_scan():
    """cu_seqlens rows with ragged lengths (partial chunks in every row) and the in-op L2 norm: the chunked forward
    against the library's own fp32-arithmetic scan on the same bf16 tensors."""
    case = make_case("kda", B=1, T=1500, H=4, K=128, V=128, seed=8, gates="kda_baseline", l2norm=True)
    cu = [0, 1, 65, 300, 777, 1500]
    rng = np.random.default_rng(3)
    case["h0"] = (rng.standard_normal((len(cu) - 1, 4, 128, 128)) * 0.5).astype(np.float32)
    o, ht = _forward(case, cu=cu, l2norm=True)
    o_ref, ht_ref = _forward(case, cu=cu, l2norm=True, precision="highest")
    assert rel_l2(o, o_ref) <= 1e-2 and rel_l2(ht, ht_ref) <= 1e-2, (rel_l2(o, o_ref), rel_l2(ht, ht_ref))


@pytest.mark.parametrize("docs,T", [(None, 128), ("uniform", 300), ("mixed", 200)])
def test_gradients_match_the_oracle(docs, T):
    """All gradients (q, k, v, per-channel g, beta, initial state) of the chunked backward, with an upstream
    gradient on the final state as well."""
    case = make_case("kda", B=2, T=T, H=2, K=128, V=128, seed=12 + T, gates="kda_baseline", docs=docs, h0=True,
                     doc_range=(20, max(T // 2, 21)))
    want = run_oracle("kda", case, scale=case["meta"]["scale"])
    got = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="bfloat16")
    compare(got, want, 1e-2, f"kda fwd+bwd T={T} docs={docs}")


def test_gradients_with_l2norm_and_grouped_key_heads():
    case = make_case("kda", B=1, T=260, H=4, Hk=2, K=128, V=128, seed=31, gates="plain", l2norm=True, h0=True)
    want = run_oracle("kda", case, scale=case["meta"]["scale"], l2norm=True)
    got = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="bfloat16", l2norm=True)
    compare(got, want, 1e-2, "kda fwd+bwd l2norm grouped")


def test_gradients_under_strong_decay():
    """The exact fp32 score path of the backward (channels decaying by e^-80 at a token)."""
    case = make_case("kda", B=1, T=192, H=2, K=128, V=128, seed=33, gates="extreme", docs="mixed", h0=True)
    want = run_oracle("kda", case, scale=case["meta"]["scale"])
    got = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="bfloat16")
    for name, x in got.items():
        assert np.isfinite(x).all(), name
    compare(got, want, 1.5e-2, "kda fwd+bwd extreme gates")


@pytest.mark.parametrize("gates,tol", [("kda_baseline", 5e-3), ("plain", 1e-2), ("extreme", 1.5e-2)])
def test_float16_forward_and_gradients(gates, tol):
    """f16 tensors on the same kernels: the factored scores stop at exp(+-6) there (f16 ends at 65504), so "plain"
    gates (a chunk decays by up to e^-30 in places) mix factored and exact chunks and "extreme" ones are all exact."""
    case = make_case("kda", B=1, T=260, H=2, K=128, V=128, seed=41, gates=gates, docs="mixed", h0=True,
                     dtype="float16")
    want = run_oracle("kda", case, scale=case["meta"]["scale"])
    got = run_cuda("kda", case, scale=case["meta"]["scale"], dtype="float16")
    for name, x in got.items():
        assert np.isfinite(x).all(), name
    compare(got, want, tol, f"kda f16 {gates}")


def test_config3_full_size_matches_the_token_scan():
    """The KDA benchmark shape (B4 T4096 H16 d128, packed documents): chunked forward against the token scan."""
    case = baseline_config(3)
    o, ht = _forward(case, h0=False)
    o_ref, ht_ref = _forward(case, h0=False, precision="highest")
    assert np.isfinite(o).all()
    assert rel_l2(o, o_ref) <= 1e-2 and rel_l2(ht, ht_ref) <= 1e-2, (rel_l2(o, o_ref), rel_l2(ht, ht_ref))


@pytest.mark.parametrize("name", ["kda_d128_packed_h0", "kda_d128_extreme"])
def test_chunked_forward_against_the_reference_float64_oracle(name):
    """The committed outputs of the reference's own float64 KDA oracle (benchmarks/diff_vector_gate.py:209-250, run on
    bf16-representable inputs; tests/golden/make_golden.py) at the head size of the chunked kernels: packed rows with
    partial chunks and an initial state, and gates down to e^-1000 per token."""
    meta, ins, want = load_golden(name)
    if "cu" in meta:  # the reference's KDA harness turns cu into one row of segment ids
        cu = np.asarray(meta["cu"])
        ins["seg"] = np.searchsorted(cu[1:], np.arange(meta["T"]), side="right")[None].astype(np.int32)
    got = run_cuda("kda", ins, scale=meta["scale"], dtype="bfloat16", grads=False)
    assert np.isfinite(got["o"]).all() and np.isfinite(got["ht"]).all()
    compare(got, {"o": want["o"], "ht": want["final"]}, 1e-2, name)


def test_config3_full_size_gradient_slices_against_the_oracle():
    """The KDA benchmark shape (B4 T4096 H16 d128 bf16, documents U[128, 4096]) forward + backward at full size:
    everything finite, and two (batch row, head) slices of the output and of ALL gradients (q, k, v, the
    per-channel gate, beta) against the float64 chunked oracle run on that slice alone (heads and batch rows are
    independent). Tolerance of the path: relative L2 <= 1e-2."""
    from jax_linear_attention_b200 import ops

    case = baseline_config(3)
    dev = "cuda"
    names = ("q", "k", "v", "g", "beta")
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in ("q", "k", "v", "do") else torch.float32,
                         requires_grad=n in names) for n in (*names, "do")}
    seg = torch.tensor(case["seg"], device=dev)
    o, s = ops.linear_attention("kda", t["q"], t["k"], t["v"], g=t["g"], beta=t["beta"], segment_ids=seg,
                                output_final_state=True)
    grads = torch.autograd.grad(o, [t[n] for n in names], t["do"])
    assert all(bool(torch.isfinite(x.float()).all()) for x in (o, s, *grads))
    for b, h in ((0, 3), (3, 12)):
        sl = {n: case[n][b:b + 1, :, h:h + 1] for n in (*names, "do")}
        sl["seg"] = case["seg"][b:b + 1]
        sl["dht"] = np.zeros((1, 1, 128, 128), np.float32)
        want = run_oracle("kda", sl, scale=128 ** -0.5, chunked=True)
        got = dict(o=o.detach()[b:b + 1, :, h:h + 1].float().cpu().numpy(), ht=s.detach()[b:b + 1, h:h + 1].cpu().numpy())
        for n, gr in zip(names, grads):
            got["d" + n] = gr[b:b + 1, :, h:h + 1].float().cpu().numpy()
        compare(got, want, 1e-2, f"config3 slice {b},{h}")
