"""Run the kernels per shard of batch x heads: every (batch row, head) recurrence is independent, so a group of
ranks splits the batch first and then the heads in whole key groups, and no collective is needed.

Mirror of the reference's ``src/jla/distributed/kernel_sharding.py`` (``shard_kernel_call`` :210-312, ``_splits``
:142-193), restated for one process per GPU: where the reference wraps the kernels in a ``shard_map`` over the
context mesh, a rank here slices its shard out of the (replicated or host-resident) global tensors, runs the op
locally and, if asked, all-gathers the shards (tests only; a training step keeps activations sharded).
The split is chosen so that the local shapes are accepted by the op's ``supports`` predicate, like the reference
(``kernel_sharding.py:268-293``).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch


@dataclass(frozen=True)
class ShardPlan:
    world: int
    batch_parts: int  # ranks along the batch axis
    head_parts: int   # ranks along the (value) head axis; batch_parts * head_parts == world

    def coords(self, rank: int) -> tuple[int, int]:
        return rank // self.head_parts, rank % self.head_parts


def plan_shards(batch: int, heads: int, key_heads: int, world: int) -> ShardPlan:
    """Batch first (the largest divisor of ``world`` that divides ``batch``), the rest over heads.

    A head shard holds whole key groups, or a part of one group (its key head is then replicated to the
    shards that share it, e.g. Mamba-2's single B/C group).
    """
    if world < 1:
        raise ValueError("world must be >= 1")
    group = heads // key_heads
    for bp in range(min(world, max(batch, 1)), 0, -1):
        if world % bp or batch % bp:
            continue
        hp = world // bp
        if heads % hp:
            continue
        hsz = heads // hp
        if hsz % group == 0 or group % hsz == 0:
            return ShardPlan(world, bp, hp)
    raise ValueError(f"cannot split batch {batch} x heads {heads} (key heads {key_heads}) over {world} ranks")


def shard_slices(plan: ShardPlan, rank: int, batch: int, heads: int, key_heads: int):
    """``(batch slice, value-head slice, key-head slice)`` of ``rank``."""
    bi, hi = plan.coords(rank)
    bsz, hsz = batch // plan.batch_parts, heads // plan.head_parts
    group = heads // key_heads
    k_lo = (hi * hsz) // group
    k_hi = ((hi + 1) * hsz - 1) // group + 1
    return slice(bi * bsz, (bi + 1) * bsz), slice(hi * hsz, (hi + 1) * hsz), slice(k_lo, k_hi)


def shard_kernel_call(fn, q, k, v, gates, options, *, rank: int, world: int, supports=None, gather_group=None):
    """Run ``fn(q, k, v, *gates, **options)`` on this rank's shard of the global tensors.

    ``gates`` are ``[B, T, H]`` or ``[B, T, H, K]``; ``options`` may hold ``initial_state [B, H, K, V]`` and
    ``segment_ids [B, T]`` (sliced along the batch) — ``cu_seqlens`` packs one row and is sharded over heads only.
    Returns the local ``(o, final_state)``; with ``gather_group`` the shards are all-gathered back to global shape.
    """
    batch, _, key_heads, _ = q.shape
    heads = v.shape[2]
    plan = plan_shards(batch, heads, key_heads, world)
    bs, hs, ks = shard_slices(plan, rank, batch, heads, key_heads)
    def cut(x, dim: int, sl: slice):
        """``x`` restricted to ``sl`` along ``dim``; the tensor itself when the slice is the whole axis (a view would
        cost an autograd node forward and a zero-filled copy of the gradient backward)."""
        if (sl.start or 0) == 0 and (sl.stop is None or sl.stop >= x.shape[dim]):
            return x
        return x.narrow(dim, sl.start or 0, sl.stop - (sl.start or 0))

    lq, lk, lv = cut(cut(q, 0, bs), 2, ks), cut(cut(k, 0, bs), 2, ks), cut(cut(v, 0, bs), 2, hs)
    lgates = [cut(cut(g, 0, bs), 2, hs) for g in gates]
    lopts = dict(options)
    if lopts.get("initial_state") is not None:
        st = lopts["initial_state"]
        lopts["initial_state"] = cut(st, 1, hs) if lopts.get("cu_seqlens") is not None else cut(cut(st, 0, bs), 1, hs)
    if lopts.get("segment_ids") is not None:
        lopts["segment_ids"] = cut(lopts["segment_ids"], 0, bs)
    if supports is not None and not supports(lq, lk, lv, *lgates, **lopts):
        raise ValueError(f"the kernels do not accept the per-shard call of plan {plan} (local q {tuple(lq.shape)}, "
                         f"v {tuple(lv.shape)})")
    o, final = fn(lq.contiguous(), lk.contiguous(), lv.contiguous(), *[g.contiguous() for g in lgates], **lopts)
    if gather_group is None:
        return o, final
    import torch.distributed as dist

    def gather(x, batch_dim, head_dim):
        parts = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(parts, x.contiguous(), group=gather_group)
        rows = [torch.cat(parts[b * plan.head_parts:(b + 1) * plan.head_parts], dim=head_dim)
                for b in range(plan.batch_parts)]
        return torch.cat(rows, dim=batch_dim)

    return gather(o, 0, 2), (None if final is None else gather(final, 0, 1))
