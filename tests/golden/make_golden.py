"""Write the golden fixtures of ``tests/golden/*.npz`` from the reference's own float64 oracles.

Run once in a checkout that has the reference tree (it is NOT needed to run the tests):

    python tests/golden/make_golden.py --reference /path/to/jax-linear-attention

What it imports from the reference (read-only, nothing is copied):

* ``benchmarks/xcheck_scalar_gate.py``: ``gen_case`` (NumPy inputs, seed = crc32 of the case name),
* ``benchmarks/xcheck_scalar_gate_torch.py``: ``run_oracle`` (float64 token loop + autograd VJP) for
  Gated DeltaNet, DeltaNet, simple GLA and Mamba-2 SSD,
* ``benchmarks/diff_vector_gate.py``: ``oracle64`` (NumPy float64 token loop, forward only) for KDA and Gated
  DeltaNet-2.

Shims, because those modules were written for a CUDA torch / JAX environment: a no-op
``torch.cuda.set_per_process_memory_fraction`` and ``DEV = "cpu"`` for the torch module; empty stand-in
modules named ``jax``, ``jax.numpy``, ``harness`` and ``jla`` so that ``diff_vector_gate`` imports (only its
NumPy function ``oracle64`` is called; the KDA inputs are drawn here with NumPy because the module's own
``draw`` needs ``jax.random``).

The specs below are the reference's differential cases reduced in size so that each fixture is a
few hundred KB; every feature of the full-size cases is kept (documents incl. 1-token documents and
chunk-edge boundaries, initial state, grouped key heads, extreme gates, beta in (0, 2), in-op L2 norm,
float32, Mamba-2 shared B/C).
"""

from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

SCALAR_SPECS = {
    "gdn_dense_h0": dict(kind="gated_deltanet", B=2, T=100, Hk=2, H=2, K=32, V=32, docs=None, h0=True),
    "gdn_docs_gqa": dict(kind="gated_deltanet", B=1, T=200, Hk=1, H=2, K=32, V=16, docs="random", h0=True),
    "gdn_extreme": dict(kind="gated_deltanet", B=1, T=160, Hk=2, H=2, K=32, V=32, docs="random", h0=True,
                        gates="extreme"),
    "gdn_l2norm": dict(kind="gated_deltanet", B=1, T=130, Hk=1, H=2, K=32, V=32, docs="random", h0=True,
                       l2norm=True),
    "gdn_beta2": dict(kind="gated_deltanet", B=1, T=130, Hk=2, H=2, K=32, V=32, docs="random", h0=True,
                      beta_scale=2.0),
    "gdn_f32": dict(kind="gated_deltanet", B=1, T=140, Hk=2, H=2, K=16, V=16, docs="random", h0=True,
                    dtype="float32"),
    "dn_docs": dict(kind="deltanet", B=2, T=130, Hk=2, H=2, K=32, V=32, docs="random", h0=True),
    "dn_l2norm_dense": dict(kind="deltanet", B=1, T=100, Hk=2, H=2, K=32, V=32, docs=None, h0=False,
                            l2norm=True),
    "sgla_docs_gqa": dict(kind="simple_gla", B=1, T=200, Hk=1, H=4, K=32, V=16, docs="random", h0=True),
    "sgla_extreme": dict(kind="simple_gla", B=1, T=160, Hk=2, H=2, K=32, V=32, docs="random", h0=True,
                         gates="extreme"),
    "mamba2_docs": dict(kind="mamba2", B=2, T=130, G=1, H=4, N=32, P=16, docs="random", h0=True),
    "mamba2_extreme": dict(kind="mamba2", B=1, T=160, G=1, H=4, N=32, P=16, docs="random", h0=True,
                           gates="extreme"),
}

# KDA: config dicts in the vocabulary of diff_vector_gate.oracle64 (B, T, H, HV, K, V, gate, cu, h0, l2norm).
KDA_SPECS = {
    "kda_dense_h0": dict(B=2, T=100, H=2, K=32, V=32, gate="plain", h0=True),
    "kda_packed": dict(B=1, T=200, H=2, K=32, V=16, gate="plain", cu=(0, 37, 100, 101, 128, 170, 200)),
    "kda_packed_h0_l2norm": dict(B=1, T=200, H=2, K=32, V=32, gate="plain", cu=(0, 64, 65, 192, 200), h0=True,
                                 l2norm=True),
    "kda_extreme": dict(B=1, T=160, H=2, K=32, V=32, gate="extreme", h0=True),
    "kda_grouped": dict(B=1, T=100, H=1, HV=2, K=32, V=32, gate="plain", h0=True),
    # the head size of the chunked tensor-core kernels (K = V = 128): packed rows with partial chunks, and extreme gates
    "kda_d128_packed_h0": dict(B=1, T=200, H=2, K=128, V=128, gate="plain", cu=(0, 64, 65, 192, 200), h0=True),
    "kda_d128_extreme": dict(B=1, T=160, H=2, K=128, V=128, gate="extreme", h0=True),
    # the layers' softplus gate inside the oracle (g = -exp(A_log) softplus(raw + dt_bias), beta = sigmoid(raw)):
    # pins the CPU restatement of the gate activations together with the recurrence (strong decays: A in (1, 16))
    "kda_softplus": dict(B=1, T=120, H=2, K=32, V=32, gate="softplus", h0=True, l2norm=True),
}

# Gated DeltaNet-2 (erase gate b [B, T, H, K], write gate w [B, T, H, V]) through the same float64 loop
# (diff_vector_gate.oracle64("gdn2", ...)).
GDN2_SPECS = {
    "gdn2_dense_h0": dict(B=2, T=100, H=2, K=32, V=32, gate="plain", h0=True),
    "gdn2_packed_l2norm": dict(B=1, T=200, H=2, K=32, V=16, gate="plain", cu=(0, 37, 100, 101, 128, 170, 200),
                               l2norm=True),
    "gdn2_extreme": dict(B=1, T=160, H=2, K=32, V=32, gate="extreme", h0=True),
    "gdn2_d128": dict(B=1, T=200, H=2, K=128, V=128, gate="plain", cu=(0, 64, 65, 192, 200), h0=True),
}


def bf16(x):
    return torch.from_numpy(np.asarray(x, np.float32)).to(torch.bfloat16).to(torch.float32).numpy()


def draw_kda(c: dict, seed: int) -> dict:
    """KDA inputs with NumPy (float32 arrays of bf16-representable values), in oracle64's vocabulary."""
    rng = np.random.default_rng(seed)
    B, T, Hk, K, V = c["B"], c["T"], c["H"], c["K"], c["V"]
    H = c.get("HV", Hk)
    q = rng.standard_normal((B, T, Hk, K))
    k = rng.standard_normal((B, T, Hk, K))
    if not c.get("l2norm"):
        k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    x = dict(q=bf16(q), k=bf16(k), v=bf16(rng.standard_normal((B, T, H, V))))
    g = -np.logaddexp(0.0, -rng.standard_normal((B, T, H, K)))
    if c["gate"] == "extreme":
        u = rng.random((B, T, H, K))
        strong = -rng.uniform(10.0, 60.0, (B, T, H, K))
        none = -rng.uniform(0.0, 1e-4, (B, T, H, K))
        g = np.where(u < 0.15, strong, np.where(u < 0.5, none, g))
        g[:, 64:96] = -30.0
        g[:, 100:103] = -1000.0
        g[:, 120:150] = 0.0
    if c["gate"] == "softplus":  # raw gate activations and the gate's parameters; beta is drawn before its sigmoid
        x["g"] = bf16(rng.standard_normal((B, T, H, K)))
        x["A_log"] = np.log(rng.uniform(1.0, 16.0, (H,))).astype(np.float32)
        x["dt_bias"] = (0.1 * rng.standard_normal((H * K,))).astype(np.float32)
        x["beta"] = bf16(rng.standard_normal((B, T, H)))
        if c.get("h0"):
            x["h0"] = (0.5 * rng.standard_normal((B, H, K, V))).astype(np.float32)
        return x
    x["g"] = g.astype(np.float32)
    sharp = 6.0 if c["gate"] == "extreme" else 1.0
    if c.get("gdn2"):  # channel gates in (0, 1), bf16-representable (the kernels take them in the tensors' dtype)
        x["b"] = bf16(1.0 / (1.0 + np.exp(-sharp * rng.standard_normal((B, T, H, K)))))
        x["w"] = bf16(1.0 / (1.0 + np.exp(-sharp * rng.standard_normal((B, T, H, V)))))
    x["beta"] = (1.0 / (1.0 + np.exp(-sharp * rng.standard_normal((B, T, H))))).astype(np.float32)
    if c.get("h0"):
        x["h0"] = (0.5 * rng.standard_normal((B, H, K, V))).astype(np.float32)
    return x


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of jla-org/jax-linear-attention")
    ap.add_argument("--out", default=HERE)
    ap.add_argument("--only", nargs="*", default=None, help="fixture names to (re)write; the manifest keeps the others")
    args = ap.parse_args()
    bench_dir = os.path.join(args.reference, "benchmarks")
    sys.path.insert(0, bench_dir)

    torch.cuda.set_per_process_memory_fraction = lambda *a, **k: None  # shim 1 (module line 38)
    gen = importlib.import_module("xcheck_scalar_gate")
    tor = importlib.import_module("xcheck_scalar_gate_torch")
    tor.DEV = "cpu"  # shim 2 (module line 39)

    manifest = {}
    manifest_path = os.path.join(args.out, "MANIFEST.json")
    if args.only is not None and os.path.exists(manifest_path):
        with open(manifest_path) as f:
            manifest = json.load(f)
    for name, spec in SCALAR_SPECS.items():
        if args.only is not None and name not in args.only:
            continue
        case = gen.gen_case(name, spec)
        meta = json.loads(str(case["meta"]))
        res = tor.run_oracle(case, meta)
        arrays = {f"in_{k}": v for k, v in case.items() if k != "meta"}
        arrays.update({f"out_{k}": np.asarray(v, np.float32) for k, v in res.items()})
        arrays["meta"] = case["meta"]
        path = os.path.join(args.out, f"{name}.npz")
        np.savez_compressed(path, **arrays)
        manifest[name] = dict(spec=spec, source="xcheck_scalar_gate_torch.run_oracle", bytes=os.path.getsize(path))
        print(name, manifest[name]["bytes"])

    for mod in ("jax", "jax.numpy", "harness", "jla", "jla.ops", "jla.ops.reference"):  # stand-ins
        sys.modules.setdefault(mod, types.ModuleType(mod))
    sys.modules["jax"].numpy = sys.modules["jax.numpy"]
    sys.modules["jax.numpy"].float32 = np.float32
    sys.modules["jax.numpy"].bfloat16 = np.float32
    sys.modules["jla"].ops = sys.modules["jla.ops"]
    sys.modules["jla.ops"].reference = sys.modules["jla.ops.reference"]
    dvg = importlib.import_module("diff_vector_gate")
    for i, (name, c) in enumerate(KDA_SPECS.items()):
        if args.only is not None and name not in args.only:
            continue
        x = draw_kda(c, seed=1000 + i)
        res = dvg.oracle64("kda", c, x)
        arrays = {f"in_{k}": v for k, v in x.items()}
        arrays["out_o"] = np.asarray(res["o"], np.float64)
        arrays["out_final"] = np.asarray(res["final"], np.float64)
        arrays["meta"] = np.array(json.dumps(dict(c, kind="kda", name=name, scale=c["K"] ** -0.5)))
        path = os.path.join(args.out, f"{name}.npz")
        np.savez_compressed(path, **arrays)
        manifest[name] = dict(spec=c, source="diff_vector_gate.oracle64", bytes=os.path.getsize(path))
        print(name, manifest[name]["bytes"])
    for i, (name, c) in enumerate(GDN2_SPECS.items()):
        if args.only is not None and name not in args.only:
            continue
        x = draw_kda(dict(c, gdn2=True), seed=2000 + i)
        del x["beta"]
        res = dvg.oracle64("gdn2", c, x)
        arrays = {f"in_{k}": v for k, v in x.items()}
        arrays["out_o"] = np.asarray(res["o"], np.float64)
        arrays["out_final"] = np.asarray(res["final"], np.float64)
        arrays["meta"] = np.array(json.dumps(dict(c, kind="gdn2", name=name, scale=c["K"] ** -0.5)))
        path = os.path.join(args.out, f"{name}.npz")
        np.savez_compressed(path, **arrays)
        manifest[name] = dict(spec=c, source="diff_vector_gate.oracle64", bytes=os.path.getsize(path))
        print(name, manifest[name]["bytes"])
    with open(manifest_path, "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True, default=list)


if __name__ == "__main__":
    main()
