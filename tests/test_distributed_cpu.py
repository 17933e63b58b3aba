"""Host logic of the multi-GPU forms on CPU ranks (gloo, world_size 2 and 3): batch x heads sharding and the
sequence-parallel state hand-off, with the CPU oracle standing in for the kernels (the orchestration, the
messages and the gradients are what is tested here; the kernels themselves are tested on the GPU).

Mirrors the reference's ``tests/test_context_parallel.py`` (document boundaries inside shards and exactly on
shard edges, a document spanning every shard, values and all gradients against the unsharded run, plus the
sensitivity check that dropping the carried state changes the answer) and ``tests/test_kernel_sharding.py``.
"""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import recurrence
from oracle.cases import make_case, max_rel

F64 = torch.float64


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _oracle_call(kind, leaves, state, seg, tslice, row):
    q, k, v, *gates = leaves
    rows = slice(None) if row is None else slice(row, row + 1)
    fn, names = recurrence.KIND_FUNCTIONS[kind]
    return fn(q[rows, tslice], k[rows, tslice], v[rows, tslice], *[g[rows, tslice] for g in gates],
              initial_state=None if state is None else state[rows], output_final_state=True,
              segment_ids=None if seg is None else seg[rows, tslice], dtype=F64)


def _cp_worker(rank, world, port, kind, seg_np, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from jax_linear_attention_b200.distributed import context_parallel_linear_attention

    T = 96
    case = make_case(kind, B=2, T=T, H=2, K=8, V=8, seed=40, h0=True)
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    names = [n for n in ("q", "k", "v", "g", "beta") if n in case]
    loc = {n: torch.tensor(case[n][:, sl], dtype=F64, requires_grad=True) for n in names}
    h0 = torch.tensor(case["h0"], dtype=F64, requires_grad=True)
    seg = None if seg_np is None else torch.tensor(seg_np[:, sl])
    gates = {n: loc[n] for n in ("g", "beta") if n in loc}
    o, f = context_parallel_linear_attention(kind, loc["q"], loc["k"], loc["v"], call=_oracle_call, segment_ids=seg,
                                             initial_state=h0 if rank == 0 else None, output_final_state=True, **gates)
    do = torch.tensor(case["do"][:, sl], dtype=F64)
    outs, cots = [o], [do]
    if f is not None:
        outs.append(f)
        cots.append(torch.tensor(case["dht"], dtype=F64))
    wrt = [loc[n] for n in names] + ([h0] if rank == 0 else [])
    grads = torch.autograd.grad(outs, wrt, cots, allow_unused=True)
    res = {"o": o.detach().numpy()}
    for n, gr in zip(names + (["h0"] if rank == 0 else []), grads):
        res["d" + n] = gr.numpy()
    if f is not None:
        res["f"] = f.detach().numpy()
    np.savez(os.path.join(out, f"rank{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


def _seg(kind_of_docs, T=96):
    if kind_of_docs == "none":
        return None
    if kind_of_docs == "inside":      # starts inside every shard (world 2 and 3), one row starts late
        return np.stack([np.repeat(np.arange(8), 12), np.concatenate([np.zeros(40), np.ones(30), 2 * np.ones(26)])]).astype(np.int32)
    if kind_of_docs == "on_edges":    # starts exactly on the shard edges of world 2 (48) and 3 (32, 64)
        a = np.concatenate([np.zeros(32), np.ones(16), 2 * np.ones(16), 3 * np.ones(32)])
        return np.stack([a, a]).astype(np.int32)
    if kind_of_docs == "spanning":    # row 0: one document over everything; row 1: a single start in the last shard
        return np.stack([np.zeros(T), np.concatenate([np.zeros(90), np.ones(6)])]).astype(np.int32)
    raise ValueError(kind_of_docs)


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("docs", ["none", "inside", "on_edges", "spanning"])
@pytest.mark.parametrize("kind", ["gated_deltanet", "simple_gla"])
def test_context_parallel_matches_the_unsharded_run(tmp_path, world, docs, kind):
    seg = _seg(docs)
    mp.spawn(_cp_worker, args=(world, _free_port(), kind, seg, str(tmp_path)), nprocs=world, join=True)
    T = 96
    case = make_case(kind, B=2, T=T, H=2, K=8, V=8, seed=40, h0=True)
    names = [n for n in ("q", "k", "v", "g", "beta") if n in case]
    full = {n: torch.tensor(case[n], dtype=F64, requires_grad=True) for n in names + ["h0"]}
    fn, gate_names = recurrence.KIND_FUNCTIONS[kind]
    o, f = fn(full["q"], full["k"], full["v"], *[full[g] for g in gate_names], initial_state=full["h0"],
              output_final_state=True, segment_ids=None if seg is None else torch.tensor(seg))
    grads = torch.autograd.grad([o, f], [full[n] for n in names + ["h0"]],
                                [torch.tensor(case["do"], dtype=F64), torch.tensor(case["dht"], dtype=F64)])
    want = {"o": o.detach().numpy(), "f": f.detach().numpy()}
    want.update({"d" + n: g.numpy() for n, g in zip(names + ["h0"], grads)})
    parts = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    for key in ["o"] + ["d" + n for n in names]:
        got = np.concatenate([p[key] for p in parts], axis=1)
        assert max_rel(got, want[key]) < 1e-9, key
    assert max_rel(parts[-1]["f"], want["f"]) < 1e-9
    assert max_rel(parts[0]["dh0"], want["dh0"]) < 1e-9
    if docs == "none":  # sensitivity: cutting the state at the shard edge must change the answer
        cut = torch.tensor(np.repeat(np.arange(world), T // world)[None].repeat(2, 0))
        o_cut, _ = fn(full["q"], full["k"], full["v"], *[full[g] for g in gate_names], initial_state=full["h0"],
                      segment_ids=cut)
        assert max_rel(o_cut.detach().numpy(), want["o"]) > 1e-3


def _oracle_piece_call(kind, leaves, cu, init):
    q, k, v, *gates = leaves
    fn, _ = recurrence.KIND_FUNCTIONS[kind]
    return fn(q, k, v, *gates, initial_state=init, output_final_state=True, cu_seqlens=cu, dtype=F64)


def _piece_worker(rank, world, port, kind, seg_np, piece_len, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from jax_linear_attention_b200.distributed import context_parallel_linear_attention

    T = 96
    case = make_case(kind, B=1, T=T, H=2, K=8, V=8, seed=43, h0=True)
    tl = T // world
    sl = slice(rank * tl, (rank + 1) * tl)
    names = [n for n in ("q", "k", "v", "g", "beta") if n in case]
    loc = {n: torch.tensor(case[n][:, sl], dtype=F64, requires_grad=True) for n in names}
    h0 = torch.tensor(case["h0"], dtype=F64, requires_grad=True)
    seg = None if seg_np is None else torch.tensor(seg_np[:1, sl])
    gates = {n: loc[n] for n in ("g", "beta") if n in loc}
    o, f = context_parallel_linear_attention(kind, loc["q"], loc["k"], loc["v"], piece_call=_oracle_piece_call,
                                             piece_len=piece_len, segment_ids=seg,
                                             initial_state=h0 if rank == 0 else None, output_final_state=True, **gates)
    do = torch.tensor(case["do"][:, sl], dtype=F64)
    outs, cots = [o], [do]
    if f is not None:
        outs.append(f)
        cots.append(torch.tensor(case["dht"], dtype=F64))
    wrt = [loc[n] for n in names] + ([h0] if rank == 0 else [])
    grads = torch.autograd.grad(outs, wrt, cots, allow_unused=True)
    res = {"o": o.detach().numpy()}
    for n, gr in zip(names + (["h0"] if rank == 0 else []), grads):
        res["d" + n] = gr.numpy()
    if f is not None:
        res["f"] = f.detach().numpy()
    np.savez(os.path.join(out, f"rank{rank}.npz"), **res)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,piece_len", [(2, 8), (3, 16)])
@pytest.mark.parametrize("docs", ["none", "inside", "spanning_then_start"])
@pytest.mark.parametrize("kind", ["gated_deltanet", "simple_gla"])
def test_pieces_joined_by_affine_maps_match_the_unsharded_run(tmp_path, world, piece_len, docs, kind):
    """Documents cut into independent pieces (``piece_len``): values and every gradient equal the plain run."""
    T = 96
    if docs == "none":
        seg = None
    elif docs == "inside":
        seg = np.concatenate([np.zeros(20), np.ones(37), 2 * np.ones(3), 3 * np.ones(36)])[None].astype(np.int32)
    else:  # one document over the first shards, a start only near the very end
        seg = np.concatenate([np.zeros(90), np.ones(6)])[None].astype(np.int32)
    mp.spawn(_piece_worker, args=(world, _free_port(), kind, seg, piece_len, str(tmp_path)), nprocs=world, join=True)
    case = make_case(kind, B=1, T=T, H=2, K=8, V=8, seed=43, h0=True)
    names = [n for n in ("q", "k", "v", "g", "beta") if n in case]
    full = {n: torch.tensor(case[n], dtype=F64, requires_grad=True) for n in names + ["h0"]}
    fn, gate_names = recurrence.KIND_FUNCTIONS[kind]
    o, f = fn(full["q"], full["k"], full["v"], *[full[g] for g in gate_names], initial_state=full["h0"],
              output_final_state=True, segment_ids=None if seg is None else torch.tensor(seg))
    grads = torch.autograd.grad([o, f], [full[n] for n in names + ["h0"]],
                                [torch.tensor(case["do"], dtype=F64), torch.tensor(case["dht"], dtype=F64)])
    want = {"o": o.detach().numpy(), "f": f.detach().numpy()}
    want.update({"d" + n: g.numpy() for n, g in zip(names + ["h0"], grads)})
    parts = [dict(np.load(tmp_path / f"rank{r}.npz")) for r in range(world)]
    for key in ["o"] + ["d" + n for n in names]:
        got = np.concatenate([p[key] for p in parts], axis=1)
        assert max_rel(got, want[key]) < 1e-9, key
    assert max_rel(parts[-1]["f"], want["f"]) < 1e-9
    assert max_rel(parts[0]["dh0"], want["dh0"]) < 1e-9


def _shard_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from jax_linear_attention_b200.distributed import shard_kernel_call

    case = make_case("simple_gla", B=2, T=40, H=4, Hk=2, K=8, V=8, seed=41, h0=True, docs="mixed")
    t = {n: torch.tensor(case[n], dtype=F64) for n in ("q", "k", "v", "g", "h0")}
    shapes = []

    def fn(q, k, v, g, **kw):
        shapes.append((tuple(q.shape), tuple(v.shape)))
        return recurrence.simple_gla(q, k, v, g, dtype=F64, **kw)

    o, f = shard_kernel_call(fn, t["q"], t["k"], t["v"], [t["g"]],
                             dict(initial_state=t["h0"], output_final_state=True, scale=1.0,
                                  segment_ids=torch.tensor(case["seg"])),
                             rank=rank, world=world, gather_group=dist.group.WORLD)
    if rank == 0:
        np.savez(os.path.join(out, "sharded.npz"), o=o.numpy(), f=f.numpy(), q_shape=np.array(shapes[0][0]))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_batch_heads_sharding_matches_unsharded(tmp_path, world):
    mp.spawn(_shard_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    case = make_case("simple_gla", B=2, T=40, H=4, Hk=2, K=8, V=8, seed=41, h0=True, docs="mixed")
    t = {n: torch.tensor(case[n], dtype=F64) for n in ("q", "k", "v", "g", "h0")}
    o, f = recurrence.simple_gla(t["q"], t["k"], t["v"], t["g"], initial_state=t["h0"], output_final_state=True,
                                 scale=1.0, segment_ids=torch.tensor(case["seg"]))
    got = np.load(tmp_path / "sharded.npz")
    assert np.array_equal(got["o"], o.numpy()) and np.array_equal(got["f"], f.numpy())
    assert tuple(got["q_shape"]) == ((1, 40, 2, 8) if world == 2 else (1, 40, 1, 8))


def test_shard_plans():
    from jax_linear_attention_b200.distributed import plan_shards, shard_slices

    p = plan_shards(8, 16, 16, 8)
    assert (p.batch_parts, p.head_parts) == (8, 1)
    p = plan_shards(1, 16, 16, 8)
    assert (p.batch_parts, p.head_parts) == (1, 8)
    p = plan_shards(2, 64, 1, 8)  # Mamba-2, one shared B/C group: heads split, the key head is replicated
    assert (p.batch_parts, p.head_parts) == (2, 4)
    assert shard_slices(p, 5, 2, 64, 1) == (slice(1, 2), slice(16, 32), slice(0, 1))
    p = plan_shards(1, 8, 2, 4)   # two heads per shard inside a group of four
    assert shard_slices(p, 3, 1, 8, 2) == (slice(0, 1), slice(6, 8), slice(1, 2))
    with pytest.raises(ValueError, match="cannot split"):
        plan_shards(3, 5, 5, 4)


def test_piece_table_cuts_documents_and_marks_continuations():
    from jax_linear_attention_b200.distributed.context_parallel import _piece_table

    ids = torch.tensor([0] * 10 + [1] * 3 + [2] * 9)
    cu, cont = _piece_table(ids, cont0=True, piece_len=4)
    assert cu == [0, 4, 8, 10, 13, 17, 21, 22]
    assert cont == [True, True, True, False, False, True, True]      # piece 0 continues the previous rank's document
    cu, cont = _piece_table(ids, cont0=False, piece_len=100)          # nothing longer than a piece: one per document
    assert cu == [0, 10, 13, 22] and cont == [False, False, False]
    cu, cont = _piece_table(torch.zeros(7, dtype=torch.int64), cont0=True, piece_len=7)
    assert cu == [0, 7] and cont == [True]


# ---------------------------------------------------------------------------------------------------------------
# Failure detection on the host: a neighbour that never sends, and a message that is not the tensor expected.
# The failures are made on the CPU ranks themselves (no kernel runs, nothing hangs): every hand-off is announced
# by a small header and every receive ends with the process group's timeout at the latest.
def _fault_worker(rank, world, port, out, fault):
    import datetime

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    from jax_linear_attention_b200.distributed import context_parallel as cp

    result = "no error"
    try:
        if fault == "never_sends":
            if rank == 0:
                pass  # rank 0 leaves the step out: its neighbour waits for a state that is never sent
            else:
                case = make_case("simple_gla", B=1, T=32, H=1, K=8, V=8, seed=3)
                t = {n: torch.tensor(case[n][:, 16:], dtype=F64) for n in ("q", "k", "v", "g")}
                cp.context_parallel_linear_attention("simple_gla", t["q"], t["k"], t["v"], g=t["g"], call=_oracle_call)
        elif fault == "wrong_shape":
            if rank == 0:
                cp.send_state(torch.zeros(1, 1, 8, 4, dtype=F64), 1, dist.group.WORLD).wait()  # V = 4 instead of 8
            else:
                cp.recv_state(torch.empty(1, 1, 8, 8, dtype=F64), 0, dist.group.WORLD)
        elif fault == "wrong_dtype":
            if rank == 0:
                cp.send_state(torch.zeros(1, 1, 8, 8, dtype=torch.float32), 1, dist.group.WORLD).wait()
            else:
                cp.recv_state(torch.empty(1, 1, 8, 8, dtype=F64), 0, dist.group.WORLD)
    except cp.StateMessageError as err:
        result = f"StateMessageError: {err}"
    except Exception as err:  # anything else is a test failure, reported by the parent
        result = f"{type(err).__name__}: {err}"
    with open(os.path.join(out, f"rank{rank}.txt"), "w") as f:
        f.write(result)
    # no barrier here: after a failed hand-off the group is not in a state to run one; the ranks just leave
    try:
        dist.destroy_process_group()
    except Exception:
        pass


@pytest.mark.parametrize("fault,needle", [("never_sends", "arrived from rank 0"), ("wrong_shape", "expected"),
                                          ("wrong_dtype", "expected")])
def test_a_failed_state_hand_off_is_an_error_on_the_host_not_a_hang(tmp_path, fault, needle):
    import time

    t0 = time.time()
    mp.spawn(_fault_worker, args=(2, _free_port(), str(tmp_path), fault), nprocs=2, join=True)
    assert time.time() - t0 < 60, "the receiver must give up at the group's timeout"
    got = (tmp_path / "rank1.txt").read_text()
    assert got.startswith("StateMessageError") and needle in got, got
    if fault == "never_sends":
        assert (tmp_path / "rank0.txt").read_text() == "no error"
    # (after a refused message the sender may see its payload's connection closed by the receiver: also an error on
    # the host, also no hang)
