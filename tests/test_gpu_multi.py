"""Two-GPU tests (skipped on a single-GPU box): sequence parallelism over NCCL against the single-GPU result, and
batch x heads sharding (``shard_kernel_call``, no collective) against the unsharded run. Ranks are child processes,
one per GPU."""

import os
import socket

import numpy as np
import pytest
import torch

from oracle.cases import make_case, rel_l2

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _cp_worker(rank, world, port, out, piece_len=None, kind="gated_deltanet"):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from jax_linear_attention_b200.distributed import context_parallel_linear_attention

    T = 4096
    case = make_case(kind, B=2 if piece_len is None else 1, T=T, H=4, K=128, V=128, seed=50, h0=True,
                     docs="uniform", doc_range=(300, 3000), gates="kda_baseline" if kind == "kda" else "plain")
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    dev = torch.device("cuda", rank)
    loc = {n: torch.tensor(case[n][:, sl], device=dev, dtype=torch.bfloat16 if n in "qkv" else torch.float32,
                           requires_grad=True) for n in ("q", "k", "v", "g", "beta")}
    h0 = torch.tensor(case["h0"], device=dev, requires_grad=True)
    seg = torch.tensor(case["seg"][:, sl], device=dev)
    o, f = context_parallel_linear_attention(kind, loc["q"], loc["k"], loc["v"], g=loc["g"],
                                             beta=loc["beta"], segment_ids=seg, piece_len=piece_len,
                                             initial_state=h0 if rank == 0 else None, output_final_state=True)
    do = torch.tensor(case["do"][:, sl], device=dev, dtype=torch.bfloat16)
    outs, cots = [o], [do]
    if f is not None:
        outs.append(f)
        cots.append(torch.tensor(case["dht"], device=dev))
    wrt = [loc[n] for n in loc] + ([h0] if rank == 0 else [])
    grads = torch.autograd.grad(outs, wrt, cots, allow_unused=True)
    res = {"o": o.detach().float().cpu().numpy()}
    for n, gr in zip(list(loc) + (["h0"] if rank == 0 else []), grads):
        res["d" + n] = gr.detach().float().cpu().numpy()
    if f is not None:
        res["f"] = f.detach().cpu().numpy()
    np.savez(os.path.join(out, f"rank{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_context_parallel_two_gpus_matches_one_gpu(tmp_path):
    import torch.multiprocessing as mp

    from tests._util import run_cuda

    world = 2
    mp.spawn(_cp_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = make_case("gated_deltanet", B=2, T=4096, H=4, K=128, V=128, seed=50, h0=True, docs="uniform",
                     doc_range=(300, 3000))
    want = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    parts = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    for key in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        got = np.concatenate([p[key] for p in parts], axis=1)
        # same kernels, same chunk grid (the shard edge is a multiple of 64): the split is exact up to the order of
        # bf16 roundings in the correction pass
        assert rel_l2(got, want[key]) < 4e-3, key
    assert rel_l2(parts[-1]["f"], want["ht"]) < 4e-3
    assert rel_l2(parts[0]["dh0"], want["dh0"]) < 4e-3


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("kind", ["gated_deltanet", "kda"])
def test_pieces_two_gpus_match_one_gpu(tmp_path, kind):
    """Documents cut into 512-token pieces joined by affine maps, over two ranks, against the plain one-GPU call."""
    import torch.multiprocessing as mp

    from tests._util import run_cuda

    world = 2
    mp.spawn(_cp_worker, args=(world, _free_port(), str(tmp_path), 512, kind), nprocs=world, join=True)
    case = make_case(kind, B=1, T=4096, H=4, K=128, V=128, seed=50, h0=True, docs="uniform",
                     doc_range=(300, 3000), gates="kda_baseline" if kind == "kda" else "plain")
    want = run_cuda(kind, case, scale=case["meta"]["scale"], dtype="bfloat16")
    parts = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    for key in ("o", "dq", "dk", "dv", "dg", "dbeta"):
        got = np.concatenate([p[key] for p in parts], axis=1)
        # the pieces re-enter with an fp32 state where the plain run carries it unrounded through the chunks; the
        # map M itself comes from a pass with 16-bit operands
        assert rel_l2(got, want[key]) < 1e-2, key
    assert rel_l2(parts[-1]["f"], want["ht"]) < 1e-2
    assert rel_l2(parts[0]["dh0"], want["dh0"]) < 1e-2


def _shard_worker(rank, world, out, spec):
    """One rank of the batch x heads sharded call: slices its shard out of the global case, runs forward and
    backward through ``shard_kernel_call`` on its own GPU (no process group: the path has no collective)."""
    torch.cuda.set_device(rank)
    from jax_linear_attention_b200 import ops
    from jax_linear_attention_b200.distributed import plan_shards, shard_kernel_call, shard_slices

    case = make_case("gated_deltanet", seed=61, **spec)
    dev = torch.device("cuda", rank)
    t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16 if n in "qkv" else torch.float32,
                         requires_grad=True) for n in ("q", "k", "v", "g", "beta", "h0")}
    seg = torch.tensor(case["seg"], device=dev)

    def fn(q, k, v, g, beta, **opts):
        return ops.linear_attention("gated_deltanet", q, k, v, g=g, beta=beta, **opts)

    o, f = shard_kernel_call(fn, t["q"], t["k"], t["v"], [t["g"], t["beta"]],
                             dict(initial_state=t["h0"], segment_ids=seg, output_final_state=True,
                                  scale=case["meta"]["scale"]),
                             rank=rank, world=world, supports=ops.cuda.SUPPORTS["gated_deltanet"])
    B, H, Hk = spec["B"], spec["H"], spec.get("Hk", spec["H"])
    bs, hs, ks = shard_slices(plan_shards(B, H, Hk, world), rank, B, H, Hk)
    do = torch.tensor(case["do"], device=dev, dtype=torch.bfloat16)[bs][:, :, hs]
    dht = torch.tensor(case["dht"], device=dev)[bs][:, hs]
    names = list(t)
    grads = torch.autograd.grad([o, f], [t[n] for n in names], [do, dht])
    res = {"o": o.detach().float().cpu().numpy(), "ht": f.detach().cpu().numpy()}
    # the gradient of a global leaf is zero outside this rank's shard: save only the shard
    cut = {"q": lambda x: x[bs][:, :, ks], "k": lambda x: x[bs][:, :, ks], "v": lambda x: x[bs][:, :, hs],
           "g": lambda x: x[bs][:, :, hs], "beta": lambda x: x[bs][:, :, hs], "h0": lambda x: x[bs][:, hs]}
    for n, gr in zip(names, grads):
        res["d" + n] = cut[n](gr).detach().float().cpu().numpy()
    np.savez(os.path.join(out, f"rank{rank}.npz"), **res)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("spec,axis", [
    (dict(B=2, T=700, H=4, K=128, V=128, docs="mixed", h0=True), "batch"),           # the batch splits first
    (dict(B=1, T=700, H=4, Hk=2, K=128, V=128, docs="mixed", h0=True), "heads"),     # heads, in whole key groups
    (dict(B=1, T=500, H=8, Hk=2, K=64, V=64, docs="mixed", h0=True), "heads"),       # the mma.sync head size
])
def test_batch_x_heads_sharding_two_gpus_matches_one_gpu(tmp_path, spec, axis):
    """The reference's check for its kernel sharding (tests/test_kernel_sharding.py:310-354: 2 GPUs = 1 GPU,
    bf16-close): every (batch row, head) recurrence is independent, so the shards of a two-rank call put side by
    side are the unsharded call -- same kernels on the same rows, hence equal bits for everything except the key
    gradients of heads whose group sums run in a different launch geometry."""
    import torch.multiprocessing as mp

    from tests._util import run_cuda

    world = 2
    mp.spawn(_shard_worker, args=(world, str(tmp_path), spec), nprocs=world, join=True)
    case = make_case("gated_deltanet", seed=61, **spec)
    want = run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    parts = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    cat_axis = {"batch": dict.fromkeys(("o", "ht", "dq", "dk", "dv", "dg", "dbeta", "dh0"), 0),
                "heads": dict(o=2, ht=1, dq=2, dk=2, dv=2, dg=2, dbeta=2, dh0=1)}[axis]
    for key, ax in cat_axis.items():
        got = np.concatenate([p[key] for p in parts], axis=ax)
        assert got.shape == want[key].shape, key
        assert rel_l2(got, want[key]) < 1e-6, (key, rel_l2(got, want[key]))
