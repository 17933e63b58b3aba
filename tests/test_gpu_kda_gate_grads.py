"""Gradients of the softplus gate's parameters through the chunked KDA kernels, the property the reference guards
with tests/test_vector_gate_gate_grads.py: the layers' gate is g = -exp(A_log) softplus(raw + dt_bias), so
dA_log = sum(dg * g) multiplies every per-token error of dG by the cumulative log decay. With A_log = log U(1, 16)
the mean log decay is near -11 per token, and chunks decay by e^-10 ... e^-700: the regime where the two
contributions of a token pair to dG (row and column direction of the score gradients) must cancel to rounding.

Chain under test: gate_prologue (CUDA) -> kda (CUDA, bf16, in-op L2 norm, initial state) -> cotangents on o and on
the final state, against the float64 oracle (oracle/gates.py in front of oracle/recurrence.py, both pinned to the
reference's float64 oracle by tests/test_oracle_golden.py). Bounds are the reference's: dA_log <= 1.5e-2 relative L2
and <= 3 % per head, ddt_bias <= 6e-3, every other gradient <= 1e-2. (With the row and column copies of a pair's
term rounded differently -- bf16 factors on one side, fp32 on the other -- the decay 0.5 and 0.9 cases of the sweep
below miss these bounds.)
"""

import numpy as np
import pytest
import torch

from oracle import gates as oracle_gates
from oracle import recurrence
from oracle.cases import rel_l2

pytestmark = pytest.mark.gpu


def _inputs(T, H, K, a_lo, a_hi, seed=0):
    rng = np.random.default_rng(seed)
    bf = lambda a: torch.tensor(a, dtype=torch.float32).to(torch.bfloat16).to(torch.float32)  # noqa: E731
    x = dict(q=bf(rng.standard_normal((1, T, H, K))), k=bf(rng.standard_normal((1, T, H, K))),
             v=bf(rng.standard_normal((1, T, H, K))), raw=bf(rng.standard_normal((1, T, H, K))),
             A_log=torch.tensor(np.log(rng.uniform(a_lo, a_hi, H)), dtype=torch.float32),
             dt_bias=torch.tensor(0.1 * rng.standard_normal(H * K), dtype=torch.float32),
             beta=bf(rng.standard_normal((1, T, H))),
             h0=torch.tensor(0.5 * rng.standard_normal((1, H, K, K)), dtype=torch.float32))
    do = bf(rng.standard_normal((1, T, H, K)))
    dht = torch.tensor(rng.standard_normal((1, H, K, K)), dtype=torch.float32)
    return x, do, dht


def _grads_cuda(x, do, dht):
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.layers import gate_prologue

    dev = torch.device("cuda")
    half = ("q", "k", "v", "raw", "beta")
    t = {n: v.to(dev, torch.bfloat16 if n in half else torch.float32).requires_grad_(True) for n, v in x.items()}
    H, K = x["q"].shape[2:]
    g, beta = gate_prologue(t["raw"], t["A_log"], t["dt_bias"].reshape(H, K), t["beta"])
    o, final = ops.linear_attention("kda", t["q"], t["k"], t["v"], g=g, beta=beta, scale=K ** -0.5,
                                    initial_state=t["h0"], output_final_state=True, use_qk_l2norm=True)
    names = list(t)
    gr = torch.autograd.grad([o, final], [t[n] for n in names], [do.to(dev, torch.bfloat16), dht.to(dev)])
    return {n: g_.detach().double().cpu().numpy() for n, g_ in zip(names, gr)}, float(g.detach().min())


def _grads_oracle(x, do, dht):
    f64 = torch.float64
    t = {n: v.to(f64).requires_grad_(True) for n, v in x.items()}
    H, K = x["q"].shape[2:]
    g = oracle_gates.mamba_gate(t["raw"], t["A_log"], t["dt_bias"].reshape(H, K))
    beta = oracle_gates.write_strength(t["beta"])
    o, final = recurrence.kda(t["q"], t["k"], t["v"], g, beta, scale=K ** -0.5, initial_state=t["h0"],
                              output_final_state=True, use_qk_l2norm=True)
    names = list(t)
    gr = torch.autograd.grad([o, final], [t[n] for n in names], [do.to(f64), dht.to(f64)])
    return {n: g_.numpy() for n, g_ in zip(names, gr)}


def _check(got, want, label):
    assert rel_l2(got["A_log"], want["A_log"]) < 1.5e-2, (label, rel_l2(got["A_log"], want["A_log"]))
    # per head, as the reference asserts -- but a head whose gradient nearly cancels (the sum over tokens changes sign
    # from head to head) is measured against a tenth of the largest head's gradient, not against its own near-zero
    floor = 0.1 * np.abs(want["A_log"]).max()
    per_head = np.max(np.abs(got["A_log"] - want["A_log"]) / np.maximum(np.abs(want["A_log"]), floor))
    assert per_head < 3e-2, (label, per_head, got["A_log"], want["A_log"])
    assert rel_l2(got["dt_bias"].ravel(), want["dt_bias"].ravel()) < 6e-3, (label, rel_l2(got["dt_bias"].ravel(), want["dt_bias"].ravel()))
    for name in set(want) - {"A_log", "dt_bias"}:
        assert rel_l2(got[name], want[name]) < 1e-2, (label, name, rel_l2(got[name], want[name]))


def test_softplus_gate_parameter_grads_under_strong_decays():
    """The reference's case: T = 1000, H = 4, K = V = 128, A = exp(A_log) ~ U(1, 16)."""
    x, do, dht = _inputs(1000, 4, 128, 1.0, 16.0)
    got, g_min = _grads_cuda(x, do, dht)
    assert g_min < -20.0
    _check(got, _grads_oracle(x, do, dht), "A in U(1,16)")


@pytest.mark.parametrize("decay", [0.01, 0.1, 0.5, 0.9])
def test_gate_parameter_grads_across_decay_strengths(decay):
    """Mean log decay per token about -decay (A = decay / E[softplus] with a 20 % spread per head), T = 512: chunks
    decay by e^-0.6 (0.01), e^-6 (0.1), e^-32 (0.5) and e^-58 (0.9) -- from the fully tensor-core factored scores to
    the edge where the factored form hands over to the exact fp32 loop."""
    mean_softplus = 0.806  # E[softplus(N(0, 1))]
    x, do, dht = _inputs(512, 4, 128, 0.8 * decay / mean_softplus, 1.2 * decay / mean_softplus, seed=int(decay * 100))
    got, _ = _grads_cuda(x, do, dht)
    _check(got, _grads_oracle(x, do, dht), f"decay {decay}")
