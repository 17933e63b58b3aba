"""One call over a 1,064,960-token sequence (Gated DeltaNet, H = 16, K = V = 128, bf16, documents of 4 Ki - 128 Ki
tokens): every tensor passes 2**31 elements, so flat token offsets, TMA coordinates and buffer sizes are exercised
beyond 32 bits. The acceptance checks are those of the reference's long-context test
(tests/test_long_context.py:238-267 and :302-319 of the reference):

* the one call equals two chained calls over the halves (the second starts from the first's final state) -- bit for
  bit here, because the split (532,480 = 8,320 chunks) is chunk aligned and both runs walk the same chunks (with
  the library's own sequence split switched off: a call with one row of 16 heads is otherwise cut into pieces joined
  by affine maps, and then the one call and the halves cut at different places; the split call is held to the
  unsplit one at 1e-2, the tolerance of the path);
* 256-token windows of the one call's output agree with the float64 token loop of the oracle started from the state
  carried into the window (tolerance of the path: relative L2 <= 1e-2);
* gradients: one call (split into pieces by the library) against the two chained halves (each split on its own),
  <= 1e-2 relative L2 (the two runs cut the sequence at different places), and the last window against the
  oracle's autograd (<= 1e-2).

Inputs are drawn on the device (a host round trip of 4 x 8.7 GB of float32 would dominate the test).
"""

import numpy as np
import pytest
import torch

from oracle import recurrence
from oracle.cases import rel_l2, uniform_docs

pytestmark = pytest.mark.gpu

T_BIG, SPLIT, WINDOW = 1_064_960, 532_480, 256
H, D = 16, 128
KIND = "gated_deltanet"


def _enough_memory() -> bool:
    return torch.cuda.is_available() and torch.cuda.get_device_properties(0).total_memory > 120 * 2**30


needs_big_gpu = pytest.mark.skipif(not _enough_memory(), reason="needs one GPU with > 120 GB")


@pytest.fixture(scope="module")
def inputs():
    dev = torch.device("cuda")
    gen = torch.Generator(device=dev).manual_seed(1234)

    def randn(*shape):
        return torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32)

    def unit(x):
        return (x * torch.rsqrt((x * x).sum(-1, keepdim=True) + 1e-6)).to(torch.bfloat16)

    x = dict(q=unit(randn(1, T_BIG, H, D)), k=unit(randn(1, T_BIG, H, D)), v=randn(1, T_BIG, H, D).to(torch.bfloat16),
             do=randn(1, T_BIG, H, D).to(torch.bfloat16), beta=torch.sigmoid(randn(1, T_BIG, H)),
             g=torch.nn.functional.logsigmoid(randn(1, T_BIG, H) + 3.0))
    seg = uniform_docs(np.random.default_rng(4), 1, T_BIG, 4096, 131072)
    assert seg[0, SPLIT] == seg[0, SPLIT - 1], "the split must fall inside a document for the chained run to carry a state"
    x["seg_host"] = seg
    x["seg"] = torch.from_numpy(seg).to(device=dev, dtype=torch.int32)
    assert x["q"].numel() > 2**31
    yield x
    x.clear()
    torch.cuda.empty_cache()


def _call(x, lo, hi, state=None, grad=False):
    from jax_linear_attention_b200 import ops

    cut = {n: x[n][:, lo:hi] for n in ("q", "k", "v", "g", "beta", "seg")}
    if grad:
        cut = {n: (t.detach().requires_grad_(True) if n != "seg" else t) for n, t in cut.items()}
    o, s = ops.linear_attention(KIND, cut["q"], cut["k"], cut["v"], g=cut["g"], beta=cut["beta"],
                                segment_ids=cut["seg"], initial_state=state, output_final_state=True)
    return o, s, cut


def _state_before(x, start):
    """The state carried into token ``start`` (a CUDA pass over the prefix that skips scores and outputs)."""
    from jax_linear_attention_b200.ops.cuda import final_state_only, no_pieces

    if start == 0:
        return None
    assert x["seg_host"][0, start] == x["seg_host"][0, start - 1], "window must not begin at a document start"
    with torch.no_grad(), final_state_only(), no_pieces():
        return _call(x, 0, start)[1]


def _oracle_window(x, start, state, grads=False):
    f64 = torch.float64
    sl = slice(start, start + WINDOW)
    leaves = {n: x[n][:, sl].detach().to("cpu", f64).requires_grad_(grads) for n in ("q", "k", "v", "g", "beta")}
    seg = torch.from_numpy(x["seg_host"][:, sl].astype(np.int64))
    o, _ = recurrence.gated_delta_rule(leaves["q"], leaves["k"], leaves["v"], leaves["g"], leaves["beta"],
                                       scale=D ** -0.5, initial_state=None if state is None else state.cpu().to(f64),
                                       output_final_state=True, segment_ids=seg, dtype=f64)
    if not grads:
        return o.numpy(), None
    do = x["do"][:, sl].to("cpu", f64)
    gr = torch.autograd.grad(o, [leaves[n] for n in leaves], do)
    return o.detach().numpy(), {n: g.numpy() for n, g in zip(leaves, gr)}


def _windows(seg_row):
    """Window starts: the beginning, one straddling a document start, one across the split, the end."""
    starts = np.nonzero(seg_row[1:] != seg_row[:-1])[0] + 1
    mid = int(starts[len(starts) // 2])
    return [0, mid - WINDOW // 2, SPLIT - WINDOW // 2, T_BIG - WINDOW]


@needs_big_gpu
def test_one_call_equals_chained_halves_and_float64_windows(inputs):
    from jax_linear_attention_b200.ops.cuda import no_pieces

    x = inputs
    with torch.no_grad():
        o_split, final_split, _ = _call(x, 0, T_BIG)  # the default: one row of 16 heads is split into pieces
    with torch.no_grad(), no_pieces():
        o, final, _ = _call(x, 0, T_BIG)
        num = float((o_split[:, ::7].float() - o[:, ::7].float()).norm())
        assert 0 < num <= 1e-2 * float(o[:, ::7].float().norm())
        assert float((final_split - final).norm()) <= 1e-2 * float(final.norm())
        del o_split, final_split
        o1, s1, _ = _call(x, 0, SPLIT)
        assert torch.equal(o[:, :SPLIT], o1)
        del o1
        o2, s2, _ = _call(x, SPLIT, T_BIG, state=s1)
        assert torch.equal(o[:, SPLIT:], o2)
        assert torch.equal(final, s2)
        del o2
    assert bool(torch.isfinite(o[:, ::4097].float()).all())
    for start in _windows(x["seg_host"][0]):
        want, _ = _oracle_window(x, start, _state_before(x, start))
        got = o[:, start:start + WINDOW].float().cpu().numpy()
        assert rel_l2(got, want) <= 1e-2, (start, rel_l2(got, want))


@needs_big_gpu
def test_gradients_of_one_call_equal_chained_halves_and_a_float64_window(inputs):
    from jax_linear_attention_b200.ops.cuda import no_pieces

    x = inputs
    names = ("q", "k", "v", "g", "beta")
    o, _, leaves = _call(x, 0, T_BIG, grad=True)  # the default call: split into pieces
    one = torch.autograd.grad(o, [leaves[n] for n in names], x["do"])
    del o, leaves
    assert all(bool(torch.isfinite(t[:, ::4097].float()).all()) for t in one)

    o1, s1, a = _call(x, 0, SPLIT, grad=True)
    o2, _, b = _call(x, SPLIT, T_BIG, state=s1, grad=True)
    chained = torch.autograd.grad([o1, o2], [a[n] for n in names] + [b[n] for n in names],
                                  [x["do"][:, :SPLIT], x["do"][:, SPLIT:]])
    del o1, o2, s1, a, b
    for i, n in enumerate(names):
        for label, got, want in (("half 1", one[i][:, :SPLIT], chained[i]), ("half 2", one[i][:, SPLIT:], chained[5 + i])):
            num = float((got.float() - want.float()).norm())
            den = float(want.float().norm())
            assert num <= 1e-2 * den, (n, label, num / den)
    del chained
    # the last window's gradients depend on nothing after it: float64 autograd of the token loop, started from the
    # state the kernels carried into the window
    start = T_BIG - WINDOW
    _, want = _oracle_window(x, start, _state_before(x, start), grads=True)
    for i, n in enumerate(names):
        got = one[i][:, start:].float().cpu().numpy()
        assert rel_l2(got, want[n]) <= 1e-2, (n, rel_l2(got, want[n]))
