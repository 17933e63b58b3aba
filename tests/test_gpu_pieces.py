"""The sequence split inside one GPU: a call with few rows and heads is cut along T into pieces that run as
independent kernel rows, joined by affine maps and a device-side scan (the reference's intra-GPU split,
src/jla/ops/mosaic_gpu/scalar_gate.py:129-271, scalar_gate_scan.py:49-140). Checked here: the scan kernel against the
same recursion written with torch products, and the split call against the unsplit call (tolerance of the path,
relative L2 <= 1e-2: the pieces re-enter with an fp32 state and the maps come from passes with 16-bit operands) and
against the float64 oracle."""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle.cases import make_case, rel_l2
from tests._util import compare, run_cuda, run_oracle

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("K,V", [(128, 128), (64, 64), (128, 64)])
def test_scan_kernel_matches_the_recursion(K, V):
    from jax_linear_attention_b200.distributed.context_parallel import piece_scan

    torch.manual_seed(K + V)
    dev = torch.device("cuda")
    P, H = 9, 3
    cont = [False, True, True, False, True, False, False, True, True]
    cont_dev = torch.tensor([int(c) for c in cont], dtype=torch.int32, device=dev)
    maps = (torch.randn(P, H, K, K, device=dev) * K ** -0.5).contiguous()
    e = torch.randn(P, H, K, V, device=dev)
    boundary = torch.randn(H, K, V, device=dev)
    # forward, in two ranges as a rank does (tail first, then the head that depends on the received state)
    got = e.clone()
    piece_scan(maps, cont, cont_dev, boundary, got, 5, P)
    piece_scan(maps, cont, cont_dev, boundary, got, 0, 5)
    want = e.double().cpu()
    piece_scan(maps.double().cpu(), cont, None, boundary.double().cpu(), want, 0, P)
    assert rel_l2(got.cpu().numpy(), want.numpy()) < 1e-5
    # a piece that starts a document keeps its E
    assert torch.equal(got[3], e[3]) and torch.equal(got[0], e[0])
    # backward
    ds_in, ds_out = e.clone(), torch.zeros_like(e)
    piece_scan(maps, cont, cont_dev, boundary, ds_in, 3, P, ds_out=ds_out)
    piece_scan(maps, cont, cont_dev, boundary, ds_in, 0, 3, ds_out=ds_out)
    w_in, w_out = e.double().cpu(), torch.zeros(P, H, K, V, dtype=torch.float64)
    piece_scan(maps.double().cpu(), cont, None, boundary.double().cpu(), w_in, 0, P, ds_out=w_out)
    assert rel_l2(ds_in.cpu().numpy(), w_in.numpy()) < 1e-5
    assert rel_l2(ds_out.cpu().numpy(), w_out.numpy()) < 1e-5


def test_policy_follows_the_reference():
    from jax_linear_attention_b200.ops.cuda import pieces

    assert pieces(8, 16, 2048, delta=True) == 1          # 128 rows x heads fill the GPU
    assert pieces(1, 16, 2048, delta=True) == 1          # too short to pay for the split's own launches (measured)
    assert pieces(1, 16, 8192, delta=True) == 1
    assert pieces(1, 16, 16384, delta=True) == 8         # 32 chunks per piece: the most the delta rule takes
    assert pieces(1, 16, 12288, delta=True) == 4         # more than 4 pieces only with 32 chunks each
    assert pieces(1, 16, 1_064_960, delta=True) == 8     # at most 8 pieces with the delta rule
    assert pieces(1, 4, 16384, delta=False) == 32        # every piece keeps at least 8 chunks
    assert pieces(1, 2, 900, delta=True) == 1


@pytest.mark.parametrize("kind", ["gated_deltanet", "simple_gla", "kda"])
def test_split_call_matches_the_unsplit_call_and_the_oracle(kind, monkeypatch):
    from jax_linear_attention_b200.ops import cuda
    from jax_linear_attention_b200.ops.cuda import no_pieces, pieces

    monkeypatch.setattr(cuda, "MIN_SPLIT_CHUNKS", 8)  # the policy's length floor is a speed matter; 4096 tokens keep
    T, H = 4096, 4                                    # the float64 oracle of this test short
    assert pieces(1, H, T, delta=kind != "simple_gla") > 1
    case = make_case(kind, B=1, T=T, H=H, K=128, V=128, seed=71, h0=True, docs="uniform", doc_range=(300, 3000),
                     gates="kda_baseline" if kind == "kda" else "baseline")
    split = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="bfloat16")
    with no_pieces():
        plain = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="bfloat16")
    for name in plain:
        assert np.isfinite(split[name]).all(), name
        assert rel_l2(split[name], plain[name]) < 1e-2, (name, rel_l2(split[name], plain[name]))
    assert any(not np.array_equal(split[n], plain[n]) for n in plain), "the split did not run"
    want = run_oracle(kind, case, scale=case["meta"]["scale"], chunked=True)
    compare(split, want, 1e-2, f"{kind} split")


def test_documents_shorter_than_a_piece_run_as_plain_rows(monkeypatch):
    """When no document is longer than a piece nothing has to be joined: the split call is the plain call with the
    documents as rows (initial state into the first document, final state of the last), held to the unsplit packed
    row and to the oracle."""
    from jax_linear_attention_b200.distributed import context_parallel as cp_mod
    from jax_linear_attention_b200.ops import cuda
    from jax_linear_attention_b200.ops.cuda import no_pieces, pieces

    monkeypatch.setattr(cuda, "MIN_SPLIT_CHUNKS", 8)
    T, H = 4096, 4
    assert pieces(1, H, T, delta=True) == 4  # pieces of 1024 tokens
    case = make_case("gated_deltanet", B=1, T=T, H=H, K=128, V=128, seed=77, h0=True, docs="uniform",
                     doc_range=(100, 900), gates="baseline")
    calls = []
    real = cp_mod.context_parallel_linear_attention
    monkeypatch.setattr(cp_mod, "context_parallel_linear_attention", lambda *a, **k: calls.append(1) or real(*a, **k))
    split = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    assert not calls, "the piece machinery ran although no document needs joining"
    with no_pieces():
        plain = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    for name in plain:
        assert rel_l2(split[name], plain[name]) < 1e-2, (name, rel_l2(split[name], plain[name]))
    want = run_oracle("gated_deltanet", case, scale=case["meta"]["scale"], chunked=True)
    compare(split, want, 1e-2, "documents as rows")
