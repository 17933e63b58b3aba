"""Sequence (context) parallel linear attention: one sequence split over the ranks of a group along T.

Role of the reference's ``src/jla/distributed/context_parallel.py:113-182``, redesigned for one process per GPU
with point-to-point hand-offs instead of all-gathered affine maps. Rank ``r`` holds tokens
``[r * T/P, (r + 1) * T/P)`` of every batch row. The recurrent state is the only thing that crosses a shard edge:

1. every rank runs the op on its whole shard from a zero state (rank 0: from ``initial_state``); this is already
   exact for every token at or after the shard's first document start, because a document start discards the
   carried state (the observation the reference's intra-GPU split uses: ``scalar_gate_docs.py:16-27``);
2. the fp32 chunk-final state ``[B, H, K, V]`` goes to the next rank with ``send``/``recv`` (NCCL over NVLink on GPUs,
   gloo in the CPU tests). A rank whose rows all contain a document start sends right after step 1, so no serial
   chain forms across ranks; otherwise it first applies the correction of step 3 and then sends;
3. the correction: the op is re-run on the prefix of each row up to its first document start, now from the received
   state, and replaces those outputs (and the final state if the row has no document start at all).

The backward mirrors this with ``dS`` flowing right to left: the prefix pass is differentiated first (its result,
the gradient of the received state, goes to the previous rank at once unless the row's prefix reaches the shard
end), then the gradient of the sent state is received and the full-shard pass is differentiated. This is exact for
every kind, including the delta rule, where the entering state acts through a K x K transition and cannot be
applied as a decayed additive term.

Document boundaries are read on the host (one small device-to-host copy per call) to size the prefixes.

**Pieces** (``piece_len``, single packed row). The state passes of the kernels walk one document's chunks in order,
so a long document is a long serial chain however many ranks there are. With ``piece_len`` set, every document is
cut into pieces of at most that many tokens and each piece becomes an independent kernel row (``cu_seqlens``), the
form of the reference's intra-GPU split (``src/jla/ops/mosaic_gpu/scalar_gate.py:129-148``, pieces joined by affine
maps). A piece maps the state entering it affinely, ``S_out = M S_in + E``: ``E`` is the final state of the piece run
from a zero state, and ``M`` (K x K per head) is the final state of the same piece run with zero values from an
identity state of value width K (the recurrence is linear in the state, so its response to the identity is the map).
Forward: pass E and pass M over all pieces in parallel, a scan of small matrix products over the pieces of each
document (across ranks: one state hand-off, sent early when the shard's last document starts inside the shard), then
the real pass with every piece's true entering state. Backward: the state gradients obey the transposed recursion
``dS_in = e + M^T dS_out`` with ``e`` the entering-state gradient for a zero final-state cotangent, so one backward
pass yields ``e``, a reverse scan yields every piece's ``dS_out``, and a second backward pass gives the gradients.
Three forward and two backward passes instead of one each, but none of them is longer than a piece.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from .. import ops
from ..ops.cuda import final_state_only, shared_prep, state_grads_only

_GATES = {"simple_gla": ("g",), "deltanet": ("beta",), "gated_deltanet": ("g", "beta"), "kda": ("g", "beta")}

_DTYPE_CODES = {torch.float32: 1, torch.float64: 2, torch.int32: 3, torch.int64: 4, torch.bfloat16: 5, torch.float16: 6}
_MAGIC = 0x4A4C41  # "JLA"


class StateMessageError(RuntimeError):
    """A hand-off between neighbouring ranks failed: the peer never sent (the group's timeout ran out), or what it
    announced is not the tensor this rank expects. Raised on the host before any kernel consumes the message."""


def _checked(group) -> bool:
    """Announce every message with a small header (shape, dtype) and compare it on arrival? Always on gloo groups
    (the CPU tests); on NCCL only with ``JLA_B200_CP_CHECK=1``, because reading the header costs a device
    synchronisation per hand-off."""
    import os

    return dist.get_backend(group) == "gloo" or os.environ.get("JLA_B200_CP_CHECK", "0") == "1"


def _header(t: torch.Tensor) -> torch.Tensor:
    fields = [_MAGIC, _DTYPE_CODES.get(t.dtype, 0), t.dim(), *t.shape]
    return torch.tensor(fields + [0] * (8 - len(fields)), dtype=torch.int64, device=t.device)


class _Requests:
    """The requests of one batched point-to-point call, waited on together."""

    def __init__(self, works):
        self.works = works

    def wait(self):
        for w in self.works:
            w.wait()


def _p2p(op, t: torch.Tensor, peer: int, group) -> _Requests:
    """One point-to-point transfer as a batched op: NCCL then runs it as a grouped send/recv of its own instead of
    serialising it with every other operation of the process group (what an unbatched ``send``/``recv`` does on a
    group that was initialised eagerly)."""
    return _Requests(dist.batch_isend_irecv([dist.P2POp(op, t, peer, group=group)]))


def _exchange_with_neighbours(send: torch.Tensor, recv: torch.Tensor, prev_rank, next_rank, group) -> None:
    """``send`` goes to the next rank and ``recv`` is filled by the previous one (either may be absent), as one batch."""
    ops = []
    if next_rank is not None:
        ops.append(dist.P2POp(dist.isend, send, next_rank, group=group))
    if prev_rank is not None:
        ops.append(dist.P2POp(dist.irecv, recv, prev_rank, group=group))
    if ops:
        _Requests(dist.batch_isend_irecv(ops)).wait()


def send_state(t: torch.Tensor, dst: int, group, what: str = "state"):
    """``isend`` of a hand-off tensor (preceded by its header when checks are on); returns the request to wait on."""
    t = t.contiguous()
    try:
        if _checked(group):
            _p2p(dist.isend, _header(t), dst, group).wait()
        return _p2p(dist.isend, t, dst, group)
    except RuntimeError as err:
        raise StateMessageError(f"context parallel: sending the {what} to rank {dst} failed: {err}") from err


def recv_state(t: torch.Tensor, src: int, group, what: str = "state") -> torch.Tensor:
    """Blocking receive of a hand-off tensor into ``t``. With checks on, the peer's header is compared with ``t``
    first, so a message of another shape or dtype is refused instead of being reinterpreted; a peer that never
    sends surfaces as ``StateMessageError`` when the process group's timeout runs out (never a hang: every group
    this module is used with is created with a finite timeout)."""
    try:
        if _checked(group):
            got = torch.zeros(8, dtype=torch.int64, device=t.device)
            _p2p(dist.irecv, got, src, group).wait()
            want = _header(t)
            if not torch.equal(got.cpu(), want.cpu()):
                g = got.cpu().tolist()
                raise StateMessageError(
                    f"context parallel: rank {src} announced a {what} message with header {g} (magic, dtype code, ndim, "
                    f"shape); expected {want.cpu().tolist()} = {tuple(t.shape)} {t.dtype}")
        _p2p(dist.irecv, t, src, group).wait()
    except StateMessageError:
        raise
    except RuntimeError as err:
        raise StateMessageError(f"context parallel: no {what} arrived from rank {src}: {err}") from err
    return t


def _first_starts(seg_local, prev_last, t_local: int) -> list[int]:
    """Per row, the index of the first token that starts a new document (``t_local`` if none)."""
    if seg_local is None:
        return None
    seg = seg_local.cpu()
    starts = []
    for b in range(seg.shape[0]):
        row = seg[b]
        change = torch.zeros(t_local, dtype=torch.bool)
        change[1:] = row[1:] != row[:-1]
        if prev_last is not None:
            change[0] = bool(row[0] != prev_last[b])
        idx = torch.nonzero(change)
        starts.append(int(idx[0]) if idx.numel() else t_local)
    return starts


class _ContextParallel(torch.autograd.Function):
    @staticmethod
    def forward(ctx, call, kind, group, seg, want_final, *tensors):
        # tensors = (q, k, v, *gates, h0 or None)
        rank, world, prev_rank, next_rank = _group_info(group)
        *xs, h0 = tensors
        q = xs[0]
        batch, t_local = q.shape[:2]
        dev = q.device
        sdt = torch.float64 if q.dtype == torch.float64 else torch.float32  # dtype of the carried state

        prev_last = None
        if seg is not None and world > 1:  # the previous rank's last segment id decides whether token 0 is a start
            last = seg[:, -1].contiguous()
            recv = torch.empty_like(last)
            _exchange_with_neighbours(last, recv, prev_rank, next_rank, group)
            prev_last = recv.cpu() if prev_rank is not None else None

        leaves = [x.detach().requires_grad_(True) for x in xs]
        h0_leaf = None if (h0 is None or rank > 0) else h0.detach().requires_grad_(True)
        if rank == 0:
            starts = [0] * batch
        elif seg is None:
            starts = [t_local] * batch
        else:
            starts = _first_starts(seg, prev_last, t_local)
        early = all(s < t_local for s in starts)
        # a shard without any document start is covered entirely by the correction pass: skip the zero-state pass
        skip_a = rank > 0 and all(s == t_local for s in starts)
        o_a = f_a = None
        if not skip_a:
            with torch.enable_grad():
                o_a, f_a = call(kind, leaves, h0_leaf, seg, slice(None), None)
            o = o_a.detach().clone()
            f = f_a.detach().clone()
        else:
            o = torch.empty(batch, t_local, xs[2].shape[2], xs[2].shape[3], dtype=xs[2].dtype, device=dev)
            f = torch.empty(batch, xs[2].shape[2], q.shape[3], xs[2].shape[3], dtype=sdt, device=dev)
        send_req = None
        if next_rank is not None and early:
            send_req = send_state(f, next_rank, group)
        s_in_leaf, prefix = None, []
        if rank > 0:
            s_in = torch.empty_like(f)
            recv_state(s_in, prev_rank, group)
            s_in_leaf = s_in.requires_grad_(True)
            with torch.enable_grad():
                for b, length in enumerate(starts):
                    if length == 0:
                        prefix.append(None)
                        continue
                    o_p, f_p = call(kind, leaves, s_in_leaf, seg, slice(0, length), b)
                    prefix.append((o_p, f_p))
                    o[b, :length] = o_p.detach()[0]
                    if length == t_local:
                        f[b] = f_p.detach()[0]
        if send_req is not None:
            send_req.wait()
        if next_rank is not None and not early:
            send_state(f, next_rank, group).wait()

        ctx.state = dict(leaves=leaves, h0_leaf=h0_leaf, o_a=o_a, f_a=f_a, s_in_leaf=s_in_leaf, prefix=prefix,
                         starts=starts, t_local=t_local, group=group, prev_rank=prev_rank, next_rank=next_rank,
                         n_in=len(xs), has_h0=h0 is not None, dev=dev, f_shape=tuple(f.shape), sdt=sdt)
        return o, f

    @staticmethod
    def backward(ctx, d_o, d_f):
        st = ctx.state
        leaves, starts, t_local, group = st["leaves"], st["starts"], st["t_local"], st["group"]
        grads = [torch.zeros_like(x) for x in leaves]
        d_o = d_o.contiguous()
        # gradient of the state this rank sent on (last rank: the caller's cotangent of the final state)
        g_f = None

        def recv_gf():
            nonlocal g_f
            if st["next_rank"] is not None:
                g_f = torch.empty(st["f_shape"], dtype=st["sdt"], device=st["dev"])
                recv_state(g_f, st["next_rank"], group, "state gradient")
            else:
                g_f = (d_f.contiguous() if d_f is not None
                       else torch.zeros(st["f_shape"], dtype=st["sdt"], device=st["dev"]))

        d_s_in = None
        if st["s_in_leaf"] is not None:
            needs_gf = any(s == t_local for s in starts)
            if needs_gf:
                recv_gf()
            d_s_in = torch.zeros_like(st["s_in_leaf"])
            for b, item in enumerate(st["prefix"]):
                if item is None:
                    continue
                o_p, f_p = item
                cot_f = g_f[b:b + 1] if starts[b] == t_local else torch.zeros_like(f_p)
                got = torch.autograd.grad([o_p, f_p], [*leaves, st["s_in_leaf"]], [d_o[b:b + 1, :starts[b]], cot_f],
                                          allow_unused=True)
                for acc, x in zip(grads, got[:-1]):
                    if x is not None:
                        acc += x
                if got[-1] is not None:
                    d_s_in += got[-1]
            send_state(d_s_in, st["prev_rank"], group, "state gradient").wait()
        if g_f is None:
            recv_gf()
        if st["o_a"] is None:  # the whole shard was handled by the correction pass
            return (None, None, None, None, None, *grads, None)
        cot_o = d_o.clone()
        cot_f = g_f.clone()
        for b, s in enumerate(starts):
            if st["s_in_leaf"] is not None:
                cot_o[b, :s] = 0  # those outputs came from the prefix pass
                if s == t_local:
                    cot_f[b] = 0
        wrt = leaves + ([st["h0_leaf"]] if st["h0_leaf"] is not None else [])
        got = torch.autograd.grad([st["o_a"], st["f_a"]], wrt, [cot_o, cot_f], allow_unused=True)
        for acc, x in zip(grads, got[:len(leaves)]):
            if x is not None:
                acc += x
        d_h0 = None
        if st["has_h0"]:
            d_h0 = got[-1] if st["h0_leaf"] is not None else None
        return (None, None, None, None, None, *grads, d_h0)


def _group_info(group):
    """``(rank, world, prev_rank, next_rank)`` of this process in ``group``; ``group=False`` means a single process
    with no process group at all (the intra-GPU split: nothing is sent anywhere)."""
    if group is False:
        return 0, 1, None, None
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    ranks = dist.get_process_group_ranks(group)
    return rank, world, (ranks[rank - 1] if rank > 0 else None), (ranks[rank + 1] if rank < world - 1 else None)


def piece_scan(maps, cont, cont_device, boundary, states, p_lo: int, p_hi: int, *, ds_out=None):
    """The scan over pieces ``p_lo .. p_hi - 1`` (forward: ``states`` holds E and becomes S_out) or, with ``ds_out``,
    ``p_hi - 1`` down to ``p_lo`` of the transposed recursion (``states`` holds dS_in). CUDA float32 tensors run the
    library's scan kernel (``jla_piece_scan``); anything else (the CPU ranks of the tests, float64) takes the same
    recursion written with torch products."""
    if p_lo >= p_hi:
        return
    pieces, heads, kd, vd = states.shape
    backward = ds_out is not None
    if states.is_cuda:
        if maps is None:  # no piece continues another: only the last piece's cotangent has to be placed
            if backward and p_hi == pieces:
                ds_out[-1] = 0 if boundary is None else boundary
            return
        if states.dtype != torch.float32 or maps.dtype != torch.float32:
            raise ValueError("the piece scan kernel takes float32 states and maps")
        import ctypes as C

        from .. import _lib

        lib = _lib.load()
        for t in (maps, states, boundary, ds_out):
            if t is not None and not t.is_contiguous():
                raise ValueError("the piece scan kernel takes contiguous tensors")
        with torch.cuda.device(states.device):
            stream = torch.cuda.current_stream(states.device).cuda_stream
            _lib.check(lib.jla_piece_scan(1 if backward else 0, pieces, heads, kd, vd, maps.data_ptr(),
                                          cont_device.data_ptr(), None if boundary is None else boundary.data_ptr(),
                                          states.data_ptr(), None if ds_out is None else ds_out.data_ptr(),
                                          p_lo, p_hi, C.c_void_p(stream)), "piece scan")
        return
    if not backward:
        for p in range(p_lo, p_hi):
            if cont[p]:
                prev = states[p - 1] if p > 0 else (boundary if boundary is not None else torch.zeros_like(states[0]))
                states[p] += maps[p] @ prev
        return
    for p in range(p_hi - 1, p_lo - 1, -1):
        if p == pieces - 1:
            ds_out[p] = 0 if boundary is None else boundary
        elif cont[p + 1]:
            ds_out[p] = states[p + 1]
        else:
            continue
        if cont[p] and maps is not None:
            states[p] += maps[p].transpose(-1, -2) @ ds_out[p]


def _piece_table(ids, cont0: bool, piece_len: int):
    """Cut points of the local row: document starts plus every ``piece_len`` tokens inside a document.
    Returns (cu, cont): ``cu`` has P + 1 entries; ``cont[p]`` says piece p continues the document of piece p - 1
    (for p = 0: of the previous rank's last token)."""
    t_local = ids.numel()
    change = torch.zeros(t_local, dtype=torch.bool)
    change[1:] = ids[1:] != ids[:-1]
    doc_starts = [0] + torch.nonzero(change).flatten().tolist() + [t_local]
    cu, cont = [], []
    for a, b in zip(doc_starts[:-1], doc_starts[1:]):
        for s in range(a, b, piece_len):
            cu.append(s)
            cont.append(s != a)
    cont[0] = cont0
    cu.append(t_local)
    return cu, cont


class PiecePlan:
    """The piece table of one rank's shard: cut points ``cu`` (P + 1 entries, also on the device as int32) and, per
    piece, whether it continues the previous piece's document."""

    def __init__(self, cu, cont, cu_device):
        self.cu, self.cont, self.cu_device = cu, cont, cu_device
        self.buffers = {}  # constant operands of the map pass (identity states, zero values), kept between calls
        # pieces (other than the first) that continue a document, as a device index: building it per call would
        # cost a synchronous host-to-device copy in the middle of the step
        self.cont_index = torch.tensor([p for p in range(1, len(cont)) if cont[p]], dtype=torch.long,
                                       device=cu_device.device)
        self.cont_device = torch.tensor([1 if c else 0 for c in cont], dtype=torch.int32, device=cu_device.device)


def plan_pieces(segment_ids, piece_len: int, *, group=None, t_local: int | None = None, device=None) -> PiecePlan:
    """Builds the piece table of this rank's shard (collective: neighbouring ranks exchange one document id, and the
    ids are read on the host). A caller whose document layout stays the same over many calls builds the plan once and
    passes it as ``piece_len=plan``; that also keeps the device-to-host copy out of the step. ``group=False``: a single
    process without a process group (the split inside one GPU)."""
    if group is not False:
        group = group if group is not None else dist.group.WORLD
    rank, world, prev_rank, next_rank = _group_info(group)
    if segment_ids is None:
        ids = torch.zeros(t_local, dtype=torch.int64)
        cont0 = rank > 0
    else:
        if segment_ids.shape[0] != 1:
            raise ValueError(f"pieces need a single packed row (batch 1); got batch {segment_ids.shape[0]}")
        device = segment_ids.device
        ids = segment_ids[0].cpu().to(torch.int64)
        cont0 = False
        if world > 1:  # does this shard's first token continue the previous rank's document?
            last = segment_ids[:, -1].contiguous()
            recv = torch.empty_like(last)
            _exchange_with_neighbours(last, recv, prev_rank, next_rank, group)
            cont0 = prev_rank is not None and int(recv.cpu()[0]) == int(ids[0])
    cu, cont = _piece_table(ids, cont0, int(piece_len))
    return PiecePlan(cu, cont, torch.tensor(cu, dtype=torch.int32, device=device))


class _PiecewiseContextParallel(torch.autograd.Function):
    """One packed row per rank, cut into pieces joined by affine maps (see the module docstring)."""

    @staticmethod
    def forward(ctx, pcall, kind, group, seg, piece_len, *tensors):
        rank, world, prev_rank, next_rank = _group_info(group)
        *xs, h0 = tensors
        q, k, v, *gates = xs
        t_local, heads, kd, vd = q.shape[1], v.shape[2], q.shape[3], v.shape[3]
        dev = q.device
        sdt = torch.float64 if q.dtype == torch.float64 else torch.float32

        plan = piece_len if isinstance(piece_len, PiecePlan) else plan_pieces(seg, piece_len, group=group,
                                                                               t_local=t_local, device=dev)
        cont, cu_t = plan.cont, plan.cu_device
        pieces = len(cont)
        plain = [x.detach() for x in xs]
        has_h0 = rank == 0 and h0 is not None

        share = shared_prep()  # the three passes read the same keys and gates: one chunk table, one set of inverses
        share.__enter__()
        try:
            with torch.no_grad(), final_state_only():
                init_e = None
                if has_h0:
                    init_e = torch.zeros(pieces, heads, kd, vd, dtype=sdt, device=dev)
                    init_e[0] = h0[0].to(sdt)
                _, e_state = pcall(kind, plain, cu_t, init_e)
                m_map = None
                if any(cont):
                    bkey = (pieces, heads, kd, t_local, v.dtype, sdt)
                    if plan.buffers.get("key") != bkey:
                        plan.buffers.update(
                            key=bkey, eye=torch.eye(kd, dtype=sdt, device=dev).expand(pieces, heads, kd, kd).contiguous(),
                            vz=torch.zeros(1, t_local, heads, kd, dtype=v.dtype, device=dev))
                    eye, vz = plan.buffers["eye"], plan.buffers["vz"]
                    _, m_map = pcall(kind, [plain[0], plain[1], vz, *plain[3:]], cu_t, eye)
                    m_map = m_map.to(sdt).contiguous()
                s_out = e_state.to(sdt).clone().contiguous()
                s_recv = torch.zeros(1, heads, kd, vd, dtype=sdt, device=dev)

                def scan(p0, p1):  # S_out[p] = E[p] + M[p] S_out[p - 1] along a document's pieces
                    piece_scan(m_map, cont, plan.cont_device, s_recv[0], s_out, p0, p1)

                # the shard's last document starts at piece `tail`: its states do not depend on the received state
                tail = max((p for p in range(pieces) if not cont[p]), default=0)
                send_req = None
                if not cont[tail]:
                    scan(tail, pieces)
                    if next_rank is not None:
                        send_req = send_state(s_out[-1:], next_rank, group)
                if prev_rank is not None:
                    recv_state(s_recv, prev_rank, group)
                if cont[tail]:  # one document fills the whole shard
                    scan(0, pieces)
                    if next_rank is not None:
                        send_req = send_state(s_out[-1:], next_rank, group)
                else:
                    scan(0, tail)
                if send_req is not None:
                    send_req.wait()
                # entering states: the previous piece's final state where the document continues, else zero
                s_in = torch.zeros(pieces, heads, kd, vd, dtype=sdt, device=dev)
                idx = plan.cont_index
                if idx.numel():
                    s_in[idx] = s_out[idx - 1]
                if cont[0]:
                    s_in[0] = s_recv[0]
                if has_h0:
                    s_in[0] = h0[0].to(sdt)

            leaves = [x.detach().requires_grad_(True) for x in xs]
            s_in_leaf = s_in.requires_grad_(True)
            with torch.enable_grad():
                o, f = pcall(kind, leaves, cu_t, s_in_leaf)
        finally:
            share.__exit__(None, None, None)
        ctx.state = dict(leaves=leaves, s_in_leaf=s_in_leaf, o=o, f=f, m_map=m_map, cont=cont, group=group, plan=plan,
                         prev_rank=prev_rank, next_rank=next_rank, has_h0=has_h0, h0_given=h0 is not None, sdt=sdt)
        return o.detach(), f.detach()[-1:].to(sdt)

    @staticmethod
    def backward(ctx, d_o, d_f):
        st = ctx.state
        cont, m_map, group, sdt = st["cont"], st["m_map"], st["group"], st["sdt"]
        leaves, s_in_leaf, o, f = st["leaves"], st["s_in_leaf"], st["o"], st["f"]
        pieces = len(cont)
        d_o = d_o.contiguous()
        # entering-state gradients for a zero final-state cotangent
        with state_grads_only():
            (e_grad,) = torch.autograd.grad([o], [s_in_leaf], [d_o], retain_graph=True)
        ds_in = e_grad.to(sdt).clone().contiguous()
        ds_out = torch.zeros_like(ds_in)
        g_next = torch.zeros_like(ds_in[:1])
        plan = st["plan"]

        def scan(p_hi, p_lo):  # pieces p_hi - 1 down to p_lo: dS_in[p] = e[p] + M[p]^T dS_out[p]
            piece_scan(m_map, cont, plan.cont_device, g_next[0], ds_in, p_lo, p_hi, ds_out=ds_out)

        # the shard's first document ends before piece `head`: its gradients do not depend on the received one
        head = min((p for p in range(1, pieces) if not cont[p]), default=pieces)
        send_req = None
        if head < pieces:
            scan(head, 0)
            if st["prev_rank"] is not None:
                send_req = send_state(ds_in[:1] if cont[0] else torch.zeros_like(ds_in[:1]), st["prev_rank"], group,
                                      "state gradient")
        if st["next_rank"] is not None:
            recv_state(g_next, st["next_rank"], group, "state gradient")
        elif d_f is not None:
            g_next = d_f.to(sdt).contiguous().clone()
        if head < pieces:
            scan(pieces, head)
        else:
            scan(pieces, 0)
            if st["prev_rank"] is not None:
                send_req = send_state(ds_in[:1] if cont[0] else torch.zeros_like(ds_in[:1]), st["prev_rank"], group,
                                      "state gradient")
        got = torch.autograd.grad([o, f], [*leaves, s_in_leaf], [d_o, ds_out.to(f.dtype)], allow_unused=True)
        if send_req is not None:
            send_req.wait()
        grads = [x if x is not None else torch.zeros_like(l) for x, l in zip(got[:-1], leaves)]
        d_h0 = got[-1][:1].to(sdt) if st["has_h0"] else None
        return (None, None, None, None, None, *grads, d_h0)


def _default_call(impl, options):
    """The op on (a slice of) the local shard. A single packed row is handed over as ``cu_seqlens`` (the document
    boundaries are on the host anyway), so that every document is an independent row for the kernels instead of
    one long serial chain; the carried state goes to the first document, the state after the last one comes back."""
    def call(kind, leaves, state, seg, tslice, row):
        q, k, v, *gates = leaves
        rows = slice(None) if row is None else slice(row, row + 1)
        names = _GATES[kind]
        kw = dict(options)
        kw.update({n: g[rows, tslice] for n, g in zip(names, gates)})
        ql, kl, vl = q[rows, tslice], k[rows, tslice], v[rows, tslice]
        init = None if state is None else state[rows]
        if seg is not None and ql.shape[0] == 1 and ql.shape[1] > 0:
            ids = seg[rows, tslice][0]
            starts = torch.nonzero(ids[1:] != ids[:-1]).flatten() + 1
            if starts.numel() > 0:
                cu = torch.cat([starts.new_zeros(1), starts, starts.new_full((1,), ids.numel())]).to(torch.int32)
                nseq = cu.numel() - 1
                init_all = None
                if init is not None:
                    init_all = torch.cat([init, init.new_zeros(nseq - 1, *init.shape[1:])], dim=0)
                o, final = ops.linear_attention(kind, ql, kl, vl, impl=impl, initial_state=init_all,
                                                output_final_state=True, cu_seqlens=cu, **kw)
                return o, final[-1:]
        if seg is not None:
            kw["segment_ids"] = seg[rows, tslice]
        return ops.linear_attention(kind, ql, kl, vl, impl=impl, initial_state=init, output_final_state=True, **kw)
    return call


def _default_piece_call(impl, options):
    """The op over the local row cut into ``cu_seqlens`` pieces, each with its own entering state."""
    def pcall(kind, leaves, cu, init):
        q, k, v, *gates = leaves
        kw = dict(options)
        kw.update(dict(zip(_GATES[kind], gates)))
        return ops.linear_attention(kind, q, k, v, impl=impl, initial_state=init, output_final_state=True,
                                    cu_seqlens=cu, **kw)
    return pcall


def context_parallel_linear_attention(kind: str, q, k, v, *, group=None, impl: str = "auto", call=None,
                                      piece_len=None, piece_call=None, **inputs):
    """``(o_local, final_state)`` for this rank's T-shard ``q, k, v [B, T/P, ...]`` (gates and ``segment_ids``
    sharded the same way). ``initial_state`` is read on the first rank; the final state of the whole sequence is
    returned on the last rank when ``output_final_state`` is set (``None`` elsewhere). ``cu_seqlens`` is not
    supported: pass ``segment_ids``, as in the reference's sequence-parallel op.

    ``piece_len`` (tokens, or a ``PiecePlan`` from ``plan_pieces``; batch 1 only) cuts documents into independent
    pieces joined by affine maps, which is what lets a long document use more than one SM per head and more than
    one rank. With ``group=False`` and a ``piece_len`` the call involves no process group at all: it is the split of
    one sequence inside one GPU (``ops.cuda`` applies it by itself when a call would leave most SMs idle).

    ``call(kind, leaves, state, seg, tslice, row)`` or, with pieces, ``piece_call(kind, leaves, cu, init)`` may
    replace the op (tests inject the CPU oracle).
    """
    if kind not in _GATES:
        raise ValueError(f"unknown linear-attention kind {kind!r}; expected one of {sorted(_GATES)}")
    if inputs.get("cu_seqlens") is not None:
        raise NotImplementedError("context parallelism does not support cu_seqlens; pass segment_ids")
    group = group if group is not None else dist.group.WORLD
    names = _GATES[kind]
    missing = [n for n in names if inputs.get(n) is None]
    if missing:
        raise ValueError(f"{kind} takes gates {names}; missing {missing}")
    gates = [inputs.pop(n) for n in names]
    h0 = inputs.pop("initial_state", None)
    want_final = bool(inputs.pop("output_final_state", False))
    seg = inputs.pop("segment_ids", None)
    if piece_len is not None:
        if q.shape[0] != 1:
            raise ValueError(f"piece_len needs a single packed row (batch 1); got batch {q.shape[0]}")
        if not isinstance(piece_len, PiecePlan) and piece_len <= 0:
            raise ValueError(f"piece_len must be positive; got {piece_len}")
        pcall = piece_call or _default_piece_call(impl, inputs)
        o, f = _PiecewiseContextParallel.apply(pcall, kind, group, seg, piece_len, q, k, v, *gates, h0)
    else:
        call = call or _default_call(impl, inputs)
        o, f = _ContextParallel.apply(call, kind, group, seg, want_final, q, k, v, *gates, h0)
    last = group is False or dist.get_rank(group) == dist.get_world_size(group) - 1
    return o, (f if (want_final and last) else None)
