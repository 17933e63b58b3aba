"""Helpers shared by the GPU parity tests: run the CUDA op and the CPU oracle on the same case."""

from __future__ import annotations

import json
import os

import numpy as np
import torch

from oracle import chunked as oracle_chunked
from oracle import recurrence as oracle_rec
from oracle.cases import max_rel, rel_l2

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TORCH_DTYPE = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}
GATES = {"simple_gla": ("g",), "deltanet": ("beta",), "gated_deltanet": ("g", "beta"), "kda": ("g", "beta")}


def load_golden(name):
    with np.load(os.path.join(GOLDEN, f"{name}.npz"), allow_pickle=False) as f:
        data = {k: f[k] for k in f.files}
    meta = json.loads(str(data.pop("meta")))
    ins = {k[3:]: v for k, v in data.items() if k.startswith("in_")}
    outs = {k[4:]: v for k, v in data.items() if k.startswith("out_")}
    return meta, ins, outs


def run_cuda(kind, ins, *, scale, dtype, l2norm=False, precision=None, grads=True, cu_seqlens=None, device="cuda:0"):
    """Run ``ops.linear_attention(kind, ..., impl='cuda')``; returns dict of float32 numpy arrays."""
    from jax_linear_attention_b200 import ops

    td = TORCH_DTYPE[dtype]
    leaves = {}
    for n in ("q", "k", "v"):
        leaves[n] = torch.tensor(ins[n], dtype=td, device=device, requires_grad=grads)
    for n in ("g", "beta", "h0"):
        if n in ins:
            leaves[n] = torch.tensor(ins[n], dtype=torch.float32, device=device, requires_grad=grads)
    opts = dict(scale=scale, initial_state=leaves.get("h0"), output_final_state=True, precision=precision)
    if "seg" in ins:
        opts["segment_ids"] = torch.tensor(ins["seg"], device=device)
    if cu_seqlens is not None:
        opts["cu_seqlens"] = torch.tensor(cu_seqlens, device=device)
    if kind != "simple_gla":
        opts["use_qk_l2norm"] = l2norm
    gates = {g: leaves[g] for g in GATES[kind]}
    o, ht = ops.linear_attention(kind, leaves["q"], leaves["k"], leaves["v"], impl="cuda", **gates, **opts)
    res = {"o": o.detach().float().cpu().numpy(), "ht": ht.detach().float().cpu().numpy()}
    if grads:
        do = torch.tensor(ins["do"], dtype=td, device=device)
        dht = torch.tensor(ins["dht"], dtype=torch.float32, device=device)
        names = list(leaves)
        gr = torch.autograd.grad([o, ht], [leaves[n] for n in names], [do, dht])
        for n, x in zip(names, gr):
            res["d" + n] = x.detach().float().cpu().numpy()
    torch.cuda.synchronize()
    return res


def run_oracle(kind, ins, *, scale, l2norm=False, grads=True, cu_seqlens=None, chunked=False, dtype=torch.float64):
    """The CPU oracle on the same inputs (float64 token loop, or the chunked form when ``chunked``)."""
    leaves = {n: torch.tensor(ins[n], dtype=dtype, requires_grad=grads) for n in ("q", "k", "v", "g", "beta", "h0")
              if n in ins}
    mod = oracle_chunked if chunked else oracle_rec
    fn, gate_names = mod.KIND_FUNCTIONS[kind]
    opts = dict(scale=scale, initial_state=leaves.get("h0"), output_final_state=True, dtype=dtype)
    if "seg" in ins:
        opts["segment_ids"] = torch.tensor(ins["seg"])
    if cu_seqlens is not None:
        opts["cu_seqlens"] = torch.tensor(cu_seqlens)
    if kind != "simple_gla":
        opts["use_qk_l2norm"] = l2norm
    o, ht = fn(leaves["q"], leaves["k"], leaves["v"], *[leaves[g] for g in gate_names], **opts)
    res = {"o": o.detach().numpy(), "ht": ht.detach().numpy()}
    if grads:
        names = list(leaves)
        gr = torch.autograd.grad([o, ht], [leaves[n] for n in names],
                                 [torch.tensor(ins["do"], dtype=dtype), torch.tensor(ins["dht"], dtype=dtype)])
        for n, x in zip(names, gr):
            res["d" + n] = x.numpy()
    return res


def compare(got: dict, want: dict, tol: float, label: str = "", metric=rel_l2) -> dict:
    """Assert every tensor of ``want`` present in ``got`` is within ``tol``; returns the error table."""
    table = {}
    for name, w in want.items():
        if name not in got:
            continue
        table[name] = metric(got[name], w)
    bad = {n: e for n, e in table.items() if not (e <= tol)}
    assert not bad, f"{label}: over tolerance {tol}: {bad} (all: {table})"
    return table
