"""The stage-by-stage kernel model (``oracle/staged.py``) against autograd of the token recurrence."""

import pytest
import torch

from oracle import recurrence, staged
from oracle.cases import make_case, max_rel

F64 = torch.float64


@pytest.mark.parametrize("kind", ["simple_gla", "deltanet", "gated_deltanet"])
@pytest.mark.parametrize("docs", [None, "mixed"])
def test_staged_forward_and_hand_backward_match_autograd(kind, docs):
    case = make_case(kind, B=2, T=200, H=2, Hk=1, K=16, V=8, seed=21, docs=docs, h0=True, gates="extreme")
    names = [n for n in ("q", "k", "v", "g", "beta", "h0") if n in case]
    t = {n: torch.tensor(case[n], dtype=F64, requires_grad=True) for n in names}
    seg = None if docs is None else torch.tensor(case["seg"])
    fn, gates = recurrence.KIND_FUNCTIONS[kind]
    scale = case["meta"]["scale"]
    o, s = fn(t["q"], t["k"], t["v"], *[t[g] for g in gates], scale=scale, initial_state=t["h0"],
              output_final_state=True, segment_ids=seg)
    do, dht = torch.tensor(case["do"], dtype=F64), torch.tensor(case["dht"], dtype=F64)
    want = dict(zip(names, torch.autograd.grad([o, s], [t[n] for n in names], [do, dht])))
    d = {n: x.detach() for n, x in t.items()}
    st = staged.forward(d["q"], d["k"], d["v"], d.get("g"), d.get("beta"), delta=kind != "simple_gla", scale=scale,
                        h0=d["h0"], segment_ids=seg)
    assert max_rel(st["o"], o.detach()) < 1e-10 and max_rel(st["final"], s.detach()) < 1e-10
    got = staged.backward(st, do, dht)
    assert max_rel(staged.group_sum(got["dq"], 1), want["q"]) < 1e-9
    assert max_rel(staged.group_sum(got["dk"], 1), want["k"]) < 1e-9
    assert max_rel(got["dv"], want["v"]) < 1e-9
    assert max_rel(got["dh0"], want["h0"]) < 1e-9
    if "g" in want:
        assert max_rel(got["dg"], want["g"]) < 1e-9
    if "beta" in want:
        assert max_rel(got["dbeta"], want["beta"]) < 1e-9
