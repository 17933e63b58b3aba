"""Pin the CPU oracle to the fixtures written by the reference's own float64 oracles.

The fixtures under ``tests/golden`` were produced by ``tests/golden/make_golden.py`` from
``benchmarks/xcheck_scalar_gate_torch.py`` (``run_oracle``) and ``benchmarks/diff_vector_gate.py``
(``oracle64``) of the reference. Tolerances: the scalar-gate fixtures store float32, so 2e-6 of the
tensor's maximum; the KDA fixtures store float64, so 1e-10.
"""

import glob
import json
import os

import numpy as np
import pytest
import torch

from oracle import recurrence, ssd
from oracle.cases import max_rel

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
NAMES = sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN, "*.npz")))


def load(name):
    with np.load(os.path.join(GOLDEN, f"{name}.npz"), allow_pickle=False) as f:
        data = {k: f[k] for k in f.files}
    meta = json.loads(str(data.pop("meta")))
    ins = {k[3:]: v for k, v in data.items() if k.startswith("in_")}
    outs = {k[4:]: v for k, v in data.items() if k.startswith("out_")}
    return meta, ins, outs


def test_fixture_set_is_complete():
    with open(os.path.join(GOLDEN, "MANIFEST.json")) as f:
        manifest = json.load(f)
    assert sorted(manifest) == NAMES and len(NAMES) >= 17


@pytest.mark.parametrize("name", [n for n in NAMES if not n.startswith(("kda", "mamba2", "gdn2"))])
def test_scalar_gate_kinds_match_reference_oracle(name):
    meta, ins, want = load(name)
    f64 = torch.float64
    leaves = {n: torch.tensor(ins[n], dtype=f64, requires_grad=True) for n in ("q", "k", "v", "g", "beta", "h0")
              if n in ins}
    fn, gates = recurrence.KIND_FUNCTIONS[meta["kind"]]
    opts = dict(scale=meta["scale"], initial_state=leaves.get("h0"), output_final_state=True,
                segment_ids=None if "seg" not in ins else torch.tensor(ins["seg"]))
    if meta["kind"] != "simple_gla":
        opts["use_qk_l2norm"] = bool(meta.get("l2norm"))
    o, ht = fn(leaves["q"], leaves["k"], leaves["v"], *[leaves[g] for g in gates], **opts)
    names = list(leaves)
    grads = torch.autograd.grad([o, ht], [leaves[n] for n in names],
                                [torch.tensor(ins["do"], dtype=f64), torch.tensor(ins["dht"], dtype=f64)])
    assert max_rel(o.detach().numpy(), want["o"]) < 2e-6
    assert max_rel(ht.detach().numpy(), want["ht"]) < 2e-6
    for n, gr in zip(names, grads):
        assert max_rel(gr.numpy(), want["d" + n]) < 2e-6, n


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("mamba2")])
def test_mamba2_matches_reference_oracle(name):
    meta, ins, want = load(name)
    f64 = torch.float64
    leaves = {n: torch.tensor(ins[n], dtype=f64, requires_grad=True) for n in ("x", "dt", "A", "B", "C", "h0")}
    seg = None if "seg" not in ins else torch.tensor(ins["seg"])
    # the fixture keeps the state as [B, H, P, N] (the upstream Mamba-2 layout); ours is [B, H, N, P]
    y, state = ssd.mamba2_ssd(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], segment_ids=seg,
                              initial_state=leaves["h0"].transpose(-1, -2), output_final_state=True)
    ht = state.transpose(-1, -2)
    names = list(leaves)
    grads = torch.autograd.grad([y, ht], [leaves[n] for n in names],
                                [torch.tensor(ins["do"], dtype=f64), torch.tensor(ins["dht"], dtype=f64)])
    assert max_rel(y.detach().numpy(), want["o"]) < 2e-6
    assert max_rel(ht.detach().numpy(), want["ht"]) < 2e-6
    for n, gr in zip(names, grads):
        assert max_rel(gr.numpy(), want["d" + n]) < 3e-6, n
    y2, st2 = ssd.ssd_direct(leaves["x"], leaves["dt"], leaves["A"], leaves["B"], leaves["C"], segment_ids=seg,
                             initial_state=leaves["h0"].transpose(-1, -2))
    assert max_rel(y2.detach().numpy(), y.detach().numpy()) < 1e-12
    assert max_rel(st2.detach().numpy(), state.detach().numpy()) < 1e-12


def test_softplus_gate_and_write_strength_match_reference_oracle64():
    """The gate activations of the layers (oracle/gates.py) in front of the KDA recurrence, against the reference's
    float64 oracle run with its ``gate="softplus"`` branch (benchmarks/diff_vector_gate.py:215-225): raw gate
    activations, ``A_log`` in (log 1, log 16), a ``dt_bias`` per channel, beta before its sigmoid."""
    from oracle import gates

    meta, ins, want = load("kda_softplus")
    f64 = torch.float64
    t = {n: torch.tensor(v, dtype=f64) for n, v in ins.items()}
    g = gates.mamba_gate(t["g"], t["A_log"], t["dt_bias"])
    beta = gates.write_strength(t["beta"])
    assert float(g.min()) < -20.0  # strong decays: the activations matter
    o, final = recurrence.kda(t["q"], t["k"], t["v"], g, beta, scale=meta["scale"], initial_state=t["h0"],
                              output_final_state=True, use_qk_l2norm=True)
    assert max_rel(o.numpy(), want["o"]) < 1e-10
    assert max_rel(final.numpy(), want["final"]) < 1e-10


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("kda") and n != "kda_softplus"])
def test_kda_matches_reference_oracle64(name):
    meta, ins, want = load(name)
    f64 = torch.float64
    t = {n: torch.tensor(v, dtype=f64) for n, v in ins.items()}
    seg = None
    if "cu" in meta:  # the reference's KDA harness turns cu into one row of segment ids
        cu = np.asarray(meta["cu"])
        seg = torch.tensor(np.searchsorted(cu[1:], np.arange(meta["T"]), side="right")[None])
    o, final = recurrence.kda(t["q"], t["k"], t["v"], t["g"], t["beta"], scale=meta["scale"],
                              initial_state=t.get("h0"), output_final_state=True, segment_ids=seg,
                              use_qk_l2norm=bool(meta.get("l2norm")))
    assert max_rel(o.numpy(), want["o"]) < 1e-10
    assert max_rel(final.numpy(), want["final"]) < 1e-10


@pytest.mark.parametrize("name", [n for n in NAMES if n.startswith("gdn2")])
def test_gdn2_matches_reference_oracle64(name):
    """Gated DeltaNet-2 (erase gate b, write gate w) against ``diff_vector_gate.oracle64("gdn2", ...)``."""
    meta, ins, want = load(name)
    f64 = torch.float64
    t = {n: torch.tensor(v, dtype=f64) for n, v in ins.items()}
    seg = None
    if "cu" in meta:
        cu = np.asarray(meta["cu"])
        seg = torch.tensor(np.searchsorted(cu[1:], np.arange(meta["T"]), side="right")[None])
    o, final = recurrence.gdn2(t["q"], t["k"], t["v"], t["g"], t["b"], t["w"], scale=meta["scale"],
                               initial_state=t.get("h0"), output_final_state=True, segment_ids=seg,
                               use_qk_l2norm=bool(meta.get("l2norm")))
    assert max_rel(o.numpy(), want["o"]) < 1e-10
    assert max_rel(final.numpy(), want["final"]) < 1e-10


def test_gdn2_with_equal_gates_is_kda():
    """``b = w = beta`` recovers KDA (reference.py:330-331)."""
    meta, ins, _ = load("kda_dense_h0")
    f64 = torch.float64
    t = {n: torch.tensor(v, dtype=f64) for n, v in ins.items()}
    beta = t["beta"][..., None]
    kw = dict(scale=meta["scale"], initial_state=t.get("h0"), output_final_state=True)
    o1, f1 = recurrence.kda(t["q"], t["k"], t["v"], t["g"], t["beta"], **kw)
    o2, f2 = recurrence.gdn2(t["q"], t["k"], t["v"], t["g"], beta.expand_as(t["k"]), beta.expand_as(t["v"]), **kw)
    assert torch.allclose(o1, o2, rtol=0, atol=1e-12) and torch.allclose(f1, f2, rtol=0, atol=1e-12)
