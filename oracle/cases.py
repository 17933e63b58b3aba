"""Seeded synthetic inputs for the parity tests and the benchmark (NumPy, host side).

TEST / BENCH INFRASTRUCTURE ONLY. The reference benches this path on synthetic tensors
(``benchmarks/harness.py:140-155``) and differential-tests it on NumPy-drawn cases
(``benchmarks/xcheck_scalar_gate.py:119-179``); these generators draw from the same distributions
with ``numpy.random.default_rng(seed)``. Values of bf16 cases are rounded to bf16-representable
float32 so every implementation sees identical numbers.
"""

from __future__ import annotations

import numpy as np
import torch


def round_to(x: np.ndarray, dtype: str) -> np.ndarray:
    """float32 array holding values representable in ``dtype`` ("bfloat16" | "float16" | "float32")."""
    t = torch.from_numpy(np.ascontiguousarray(x, dtype=np.float32))
    if dtype in ("bfloat16", "float16"):
        t = t.to(getattr(torch, dtype)).to(torch.float32)
    return t.numpy()


def logsigmoid(x):
    return -np.logaddexp(0.0, -x)


def softplus(x):
    return np.logaddexp(0.0, x)


def l2normalize(x):
    return x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)


def uniform_docs(rng, batch: int, seq_len: int, lo: int, hi: int) -> np.ndarray:
    """``segment_ids [B, T]``: per row, lengths uniform in ``[lo, hi]`` until the row is full (last one cut)."""
    seg = np.zeros((batch, seq_len), np.int32)
    for b in range(batch):
        t, idx = 0, 0
        while t < seq_len:
            n = int(rng.integers(lo, hi + 1))
            seg[b, t:t + n] = idx
            t += n
            idx += 1
    return seg


def mixed_docs(rng, batch: int, seq_len: int, chunk: int = 64) -> np.ndarray:
    """Adversarial document mix: 1-token documents, chunk-multiple lengths, documents ending exactly
    on a chunk edge, and long documents (the mix the reference's differential harness stresses)."""
    seg = np.zeros((batch, seq_len), np.int32)
    for b in range(batch):
        t, idx = 0, 0
        while t < seq_len:
            r = rng.random()
            if r < 0.15:
                n = 1
            elif r < 0.35:
                n = chunk * int(rng.integers(1, 6))
            elif r < 0.5:
                n = (chunk - t % chunk) or chunk
            else:
                n = int(rng.integers(2, max(3, seq_len // 3)))
            seg[b, t:t + n] = idx
            t += n
            idx += 1
    return seg


def seg_to_cu(seg_row: np.ndarray) -> np.ndarray:
    """One row of segment ids to ``cu_seqlens [N + 1]``."""
    starts = [0] + [t for t in range(1, len(seg_row)) if seg_row[t] != seg_row[t - 1]]
    return np.asarray(starts + [len(seg_row)], np.int32)


def make_case(kind: str, *, B: int, T: int, H: int, K: int, V: int, Hk: int | None = None, seed: int = 0,
              dtype: str = "bfloat16", docs: str | None = None, h0: bool = False, gates: str = "plain",
              l2norm: bool = False, beta_scale: float = 1.0, doc_range=(64, 2048)) -> dict:
    """Inputs and cotangents for one linear-attention call.

    ``kind``: simple_gla | deltanet | gated_deltanet | kda. ``docs``: None | "uniform" | "mixed".
    ``gates``: "plain" (g = logsigmoid(N(3, 1.5))), "baseline" (g = logsigmoid(N(0,1)+3), the
    benchmark workloads), "extreme" (10 % of tokens forget everything, 20 % keep everything; beta hits 0 and 1),
    "kda_baseline" (per channel logsigmoid(N(0,1)+4)/8).
    """
    rng = np.random.default_rng(seed)
    Hk = Hk or H
    out: dict = {}
    q = rng.standard_normal((B, T, Hk, K))
    k = rng.standard_normal((B, T, Hk, K))
    if kind == "simple_gla":
        q, k, scale = q * 0.25, k * 0.25, 1.0
    elif l2norm:
        scale = K ** -0.5  # raw q, k: the op normalises them
    elif gates in ("baseline", "kda_baseline"):
        q, k, scale = l2normalize(q), l2normalize(k), K ** -0.5
    else:
        k = k / np.linalg.norm(k, axis=-1, keepdims=True)
        q = q / np.linalg.norm(q, axis=-1, keepdims=True) * np.sqrt(K) * 0.5
        scale = K ** -0.5
    out["q"], out["k"] = round_to(q, dtype), round_to(k, dtype)
    out["v"] = round_to(rng.standard_normal((B, T, H, V)), dtype)
    if kind != "deltanet":
        gshape = (B, T, H, K) if kind in ("kda", "gdn2") else (B, T, H)
        if gates == "baseline":
            g = logsigmoid(rng.standard_normal(gshape) + 3.0)
        elif gates == "kda_baseline":
            g = logsigmoid(rng.standard_normal(gshape) + 4.0) / 8.0
        else:
            g = logsigmoid(rng.normal(3.0, 1.5, gshape))
        if gates == "extreme":
            mask = rng.random(gshape)
            g = np.where(mask < 0.1, -80.0, np.where(mask < 0.3, -1e-7, g))
        out["g"] = g.astype(np.float32)
    if kind == "gdn2":  # erase gate per key channel, write gate per value channel (both in (0, 1), as sigmoids)
        for name, shape in (("b", (B, T, H, K)), ("w", (B, T, H, V))):
            gate = 1.0 / (1.0 + np.exp(-rng.standard_normal(shape)))
            if gates == "extreme":
                mask = rng.random(shape)
                gate = np.where(mask < 0.1, 0.0, np.where(mask < 0.2, 1.0, gate))
            out[name] = round_to(gate * beta_scale, dtype)  # the kernels take them in the tensors' dtype
    elif kind != "simple_gla":
        beta = 1.0 / (1.0 + np.exp(-rng.standard_normal((B, T, H))))
        if gates == "extreme":
            mask = rng.random((B, T, H))
            beta = np.where(mask < 0.1, 0.0, np.where(mask < 0.2, 1.0, beta))
        out["beta"] = (beta * beta_scale).astype(np.float32)
    if h0:
        out["h0"] = (rng.standard_normal((B, H, K, V)) * 0.5).astype(np.float32)
    out["do"] = round_to(rng.standard_normal((B, T, H, V)), dtype)
    out["dht"] = (rng.standard_normal((B, H, K, V)) * 0.1).astype(np.float32)
    if docs == "uniform":
        out["seg"] = uniform_docs(rng, B, T, *doc_range)
    elif docs == "mixed":
        out["seg"] = mixed_docs(rng, B, T)
    out["meta"] = dict(kind=kind, B=B, T=T, H=H, Hk=Hk, K=K, V=V, dtype=dtype, scale=scale, l2norm=l2norm,
                       seed=seed)
    return out


def make_mamba2_case(*, B: int, T: int, H: int, P: int, N: int, G: int = 1, seed: int = 0,
                     dtype: str = "bfloat16", docs: str | None = None, h0: bool = False,
                     baseline: bool = False) -> dict:
    """Mamba-2 SSD inputs. ``baseline=True`` draws the distributions of the Mamba-2 benchmark workload (B, C ~ N(0,1)/sqrt(N),
    dt = softplus(N(0,1) + log(expm1(U[0.001, 0.1]))), A = -exp(log U[1, 16]), D ~ N(0,1)); otherwise the
    differential-harness style (B, C ~ 0.5 N(0,1), dt = softplus(N(0,1) - 3), A = -U[0.5, 4])."""
    rng = np.random.default_rng(seed)
    out: dict = {}
    out["x"] = round_to(rng.standard_normal((B, T, H, P)), dtype)
    bc_scale = N ** -0.5 if baseline else 0.5
    out["B"] = round_to(rng.standard_normal((B, T, G, N)) * bc_scale, dtype)
    out["C"] = round_to(rng.standard_normal((B, T, G, N)) * bc_scale, dtype)
    if baseline:
        dt0 = rng.uniform(0.001, 0.1, (H,))
        dt = softplus(rng.standard_normal((B, T, H)) + np.log(np.expm1(dt0)))
        a = -np.exp(np.log(rng.uniform(1.0, 16.0, H)))
    else:
        dt = softplus(rng.standard_normal((B, T, H)) - 3.0)
        a = -rng.uniform(0.5, 4.0, H)
    out["dt"] = dt.astype(np.float32)
    out["A"] = a.astype(np.float32)
    out["D"] = rng.standard_normal(H).astype(np.float32)
    if h0:
        out["h0"] = (rng.standard_normal((B, H, N, P)) * 0.5).astype(np.float32)
    out["do"] = round_to(rng.standard_normal((B, T, H, P)), dtype)
    out["dht"] = (rng.standard_normal((B, H, N, P)) * 0.1).astype(np.float32)
    if docs == "uniform":
        out["seg"] = uniform_docs(rng, B, T, 64, T)
    elif docs == "mixed":
        out["seg"] = mixed_docs(rng, B, T)
    out["meta"] = dict(kind="mamba2", B=B, T=T, H=H, P=P, N=N, G=G, dtype=dtype, seed=seed)
    return out


# The five benchmark workloads (0: GDN fp32 B1 T512 H4 d64; 1: GDN bf16 B8 T2048 H16 d128; 2: Mamba-2 SSD B8 T2048 H64
# P64 N128; 3: KDA bf16 B4 T4096 H16 d128; 4: GDN on one 1,064,960-token sequence); ``shrink`` overrides sizes for tests that must finish on a CPU.
def baseline_config(index: int, seed: int = 0, **shrink) -> dict:
    if index == 0:
        spec = dict(B=1, T=512, H=4, K=64, V=64, dtype="float32", gates="baseline")
        spec.update(shrink)
        return make_case("gated_deltanet", seed=seed, **spec)
    if index == 1:
        spec = dict(B=8, T=2048, H=16, K=128, V=128, dtype="bfloat16", gates="baseline", docs="uniform",
                    doc_range=(64, 2048))
        spec.update(shrink)
        return make_case("gated_deltanet", seed=seed, **spec)
    if index == 2:
        spec = dict(B=8, T=2048, H=64, P=64, N=128, G=1, dtype="bfloat16", baseline=True)
        spec.update(shrink)
        return make_mamba2_case(seed=seed, **spec)
    if index == 3:
        spec = dict(B=4, T=4096, H=16, K=128, V=128, dtype="bfloat16", gates="kda_baseline", docs="uniform",
                    doc_range=(128, 4096))
        spec.update(shrink)
        return make_case("kda", seed=seed, **spec)
    if index == 4:
        spec = dict(B=1, T=1_064_960, H=16, K=128, V=128, dtype="bfloat16", gates="baseline", docs="uniform",
                    doc_range=(4096, 131072))
        spec.update(shrink)
        return make_case("gated_deltanet", seed=seed, **spec)
    raise ValueError(f"no benchmark workload {index}")


def rel_l2(x, want) -> float:
    x, want = np.asarray(x, np.float64), np.asarray(want, np.float64)
    return float(np.linalg.norm(x - want) / max(np.linalg.norm(want), 1e-30))


def max_rel(x, want) -> float:
    """The reference's report metric ``max|x - want| / max|want|`` (``xcheck_scalar_gate.py:257-268``)."""
    x, want = np.asarray(x, np.float64), np.asarray(want, np.float64)
    return float(np.abs(x - want).max() / max(np.abs(want).max(), 1e-30))
