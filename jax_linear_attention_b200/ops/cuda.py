"""The ``"cuda"`` implementation of the linear-attention kinds: host side of ``libjla_b200.so``.

One function per kind with the signatures of the reference's kernel entry points
(``src/jla/ops/mosaic_gpu/gated_delta_rule.py:24-37``, ``mosaic_gpu/kda.py:23-37``,
``mosaic_gpu/scalar_gate.py:591-603``) and the semantics of ``src/jla/ops/reference.py``:
``(o, final_state | None)``, ``o`` in ``q``'s dtype, the state float32. Differences from the
reference's kernels, all widening: ``cu_seqlens`` is supported (per-sequence initial and final
states, ``reference.py:170-203``), any ``T`` runs without padding copies, and ``precision="highest"``
selects the fp32 token-scan kernels for any dtype.

Gradients flow through a ``torch.autograd.Function`` (the role ``jax.custom_vjp`` has in
``mosaic_gpu/scalar_gate.py:455-469``): the forward saves the residuals the C ABI asks for and the
backward is one ``jla_linear_attention_bwd`` call. There is no fallback path.
"""

from __future__ import annotations

import ctypes as C
from typing import Any

import torch

from .. import _lib

CHUNK = 64
SUPPORTED_HEAD_DIMS = (64, 128)
_DTYPES = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}
_COMMON_OPTIONS = frozenset({"scale", "initial_state", "output_final_state", "cu_seqlens", "segment_ids",
                             "chunk_size", "precision"})


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _shape(x) -> tuple:
    return tuple(x.shape)


def _path(precision) -> str:
    if precision in (None, "default", "auto"):
        return "auto"
    if precision in ("highest", "recurrent", "float32"):
        return "recurrent"
    if precision == "chunked":
        return "chunked"
    raise ValueError(f"unknown precision {precision!r}; expected None, 'highest' or 'chunked'")


def _problem(kind: str, dtype, B, T, H, Hk, K, V, num_seqs, scale, flags, precision) -> _lib.Problem:
    p = _lib.Problem()
    p.kind, p.dtype, p.path, p.flags = _lib.KIND[kind], _DTYPES[dtype], _lib.PATH[_path(precision)], flags
    p.B, p.T, p.H, p.Hk, p.K, p.V, p.num_seqs, p.scale = B, T, H, Hk, K, V, num_seqs, float(scale)
    return p


VALUE_BLOCK = 128  # value channels per head of the chunk kernels


def _value_blocks(kind, dtype, key_dim, value_dim, path, read_key) -> int:
    """How many 128-channel blocks a wide value head is cut into for the chunk kernels, 1 if the call runs as it is.

    The columns of the state are independent recurrences (``S[:, j]`` only ever meets ``v[j]``), so a head with
    ``V = n * 128`` value channels is exactly ``n`` value heads of 128 that share the head's key and gates: grouped
    heads, which the kernels have anyway. Without this a 16-bit call with ``V`` in (256, 384, 512) -- the reference's
    wide heads, ``src/jla/ops/mosaic_gpu/scalar_gate_kb.py`` -- would run the fp32 token scan (256) or not at all."""
    if dtype == torch.float32 or read_key or path == "recurrent":
        return 1
    if value_dim <= VALUE_BLOCK or value_dim % VALUE_BLOCK:
        return 1
    if key_dim != 128 and (kind == "kda" or key_dim != 64):
        return 1
    return value_dim // VALUE_BLOCK


def unsupported_reason(kind: str, q, k, v, gates: tuple, options: dict, *, read_key: bool = False) -> str | None:
    """Why the CUDA kernels cannot run this call (``None`` if they can); ``read_key``: the call passes a separate
    read key (Gated DeltaNet-2), which only the KDA chunk kernels and the token scan take.

    Works on anything with ``.shape`` and ``.dtype`` (tensors or shape structs), so it can be evaluated
    on per-shard shapes; mirrors ``unsupported_reason`` of ``mosaic_gpu/scalar_gate.py:476-515``.
    """
    if kind == "gdn2":  # KDA kernels with a read key; the erase and write gates are shaped like k and v
        if len(gates) != 3 or _shape(gates[1]) != _shape(q) or _shape(gates[2]) != _shape(v) or \
                _shape(q)[2:3] != _shape(v)[2:3]:
            return (f"b must be [B, T, H, K] = {_shape(q)} and w must be [B, T, H, V] = {_shape(v)} with as many key "
                    f"heads as value heads; got {[_shape(x) for x in gates[1:]]}")
        kind, gates, read_key = "kda", gates[:1], True
    delta = kind != "simple_gla"
    allowed = _COMMON_OPTIONS | ({"use_qk_l2norm"} if delta else set()) | ({"sub_chunk"} if kind == "kda" else set())
    extra = sorted(set(options) - allowed)
    if extra:
        return f"unsupported options {extra}"
    if options.get("chunk_size", CHUNK) not in (None, CHUNK):
        return f"chunk_size must be {CHUNK}"
    if len(_shape(q)) != 4 or _shape(k) != _shape(q) or len(_shape(v)) != 4 or _shape(v)[:2] != _shape(q)[:2]:
        return f"expected q, k [B, T, Hk, K] and v [B, T, H, V]; got {_shape(q)}, {_shape(k)}, {_shape(v)}"
    batch, seq_len, kv_heads, key_dim = _shape(q)
    heads, value_dim = _shape(v)[2:]
    if kv_heads == 0 or heads % kv_heads:
        return f"value heads {heads} must be a multiple of key heads {kv_heads}"
    dtypes = {q.dtype, k.dtype, v.dtype}
    if len(dtypes) != 1 or q.dtype not in _DTYPES:
        return f"q, k, v must share a dtype in {tuple(_DTYPES)}; got {q.dtype}, {k.dtype}, {v.dtype}"
    gate_shape = (batch, seq_len, heads)
    names = {"simple_gla": ("g",), "deltanet": ("beta",), "gated_deltanet": ("g", "beta"), "kda": ("g", "beta")}[kind]
    for name, gate in zip(names, gates):
        want = (*gate_shape, key_dim) if (kind == "kda" and name == "g") else gate_shape
        if _shape(gate) != want:
            return f"{name} must be {want}; got {_shape(gate)}"
    cu, seg = options.get("cu_seqlens"), options.get("segment_ids")
    if cu is not None and seg is not None:
        return "pass cu_seqlens or segment_ids, not both"
    if cu is not None and batch != 1:
        return "cu_seqlens packs sequences along T and requires batch size 1"
    rows = batch if cu is None else _shape(cu)[0] - 1
    state = options.get("initial_state")
    if state is not None and _shape(state) != (rows, heads, key_dim, value_dim):
        return (f"initial_state must be [{'N' if cu is not None else 'B'}, H, K, V] = "
                f"{(rows, heads, key_dim, value_dim)}; got {_shape(state)}")
    if seg is not None and (_shape(seg) != (batch, seq_len) or seg.dtype in (torch.float16, torch.bfloat16,
                                                                                torch.float32, torch.float64)):
        return f"segment_ids must be integer [B, T] = {(batch, seq_len)}; got {seg.dtype}{_shape(seg)}"
    try:
        precision = _path(options.get("precision"))
    except ValueError as err:
        return str(err)
    blocks = _value_blocks(kind, q.dtype, key_dim, value_dim, precision, read_key)  # wide value heads run in blocks
    p = _problem(kind, q.dtype, batch, seq_len, heads * blocks, kv_heads, key_dim, value_dim // blocks,
                 0 if cu is None else max(rows, 0), 1.0, 0, precision)
    if read_key:
        p.k_read = 1  # only looked at for being non-NULL
    return _lib.unsupported_reason(p)


def _supports(kind: str):
    def supports(q, k, v, *gates, **options) -> bool:
        return unsupported_reason(kind, q, k, v, gates, options) is None
    return supports


class _PassOptions:
    """Process-wide switches for callers that run several passes over the same tokens (the piecewise
    sequence-parallel form). Plain module state, not thread-local: autograd runs backward on its own thread."""
    share = None              # dict(key=..., buffer=...) while shared_prep() is active
    state_grads_only = False  # backward runs the reverse state pass only (dh0, dv)
    final_state_only = False  # forward computes the final state only (o is left unwritten)


class shared_prep:
    """``with shared_prep():`` lets successive forward calls on the same ``k``, gates and document layout (and, with
    the in-op L2 norm, the same ``q``) share one residual-layout buffer, so that only the first of them computes the
    chunk table, the gate cumsums and the triangular inverses. Every call overwrites the buffer's state residuals:
    only the last call inside the block may be differentiated."""

    def __enter__(self):
        self._outer = _PassOptions.share
        _PassOptions.share = dict(key=None, buffer=None)
        return self

    def __exit__(self, *exc):
        _PassOptions.share = self._outer


class final_state_only:
    """``with final_state_only():`` forward calls return a valid final state and an ``o`` that must be ignored
    (the kernels skip the score and output products)."""

    def __enter__(self):
        self._outer = _PassOptions.final_state_only
        _PassOptions.final_state_only = True
        return self

    def __exit__(self, *exc):
        _PassOptions.final_state_only = self._outer


class state_grads_only:
    """``with state_grads_only():`` backward calls compute only the gradient of the initial state (and ``dv``);
    the gradients of q, k and the gates come back as zeros-shaped garbage and must be ignored."""

    def __enter__(self):
        self._outer = _PassOptions.state_grads_only
        _PassOptions.state_grads_only = True
        return self

    def __exit__(self, *exc):
        _PassOptions.state_grads_only = self._outer


class _LinearAttention(torch.autograd.Function):
    """``(o, final) = op(q, k, v, g, beta, h0, k_read)``; the config rides in ``cfg``."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, h0, k_read, cfg: dict):
        lib = _lib.load()
        B, T, Hk, K = q.shape
        H, V = v.shape[2:]
        needs_grad = any(x is not None and x.requires_grad for x in (q, k, v, g, beta, h0, k_read))
        flags = (_lib.FLAG_QK_L2NORM if cfg["l2norm"] else 0) | (_lib.FLAG_SAVE_RESIDUALS if needs_grad else 0)
        if _PassOptions.final_state_only and not needs_grad:
            flags |= _lib.FLAG_STATE_ONLY
        cu, seg = cfg["cu_seqlens"], cfg["segment_ids"]
        rows = B if cu is None else cu.numel() - 1
        p = _problem(cfg["kind"], q.dtype, B, T, H, Hk, K, V, 0 if cu is None else rows, cfg["scale"], flags,
                     cfg["precision"])
        p.q, p.k, p.v, p.g, p.beta, p.h0 = (_ptr(x) for x in (q, k, v, g, beta, h0))
        p.segment_ids, p.cu_seqlens, p.k_read = _ptr(seg), _ptr(cu), _ptr(k_read)
        dev = q.device
        o = torch.empty_like(v)
        final = torch.empty(rows, H, K, V, dtype=torch.float32, device=dev) if cfg["output_final_state"] else None
        res_bytes = lib.jla_residual_bytes(C.byref(p)) if needs_grad else 0
        share = _PassOptions.share
        if share is not None:  # one residual-layout buffer for a run of calls; the first one fills its tables
            # identity and version of the tensors the CALLER passed (not of the float32 / int32 / contiguous copies
            # made on the way here, whose addresses can be reused by the allocator inside one shared_prep block)
            key = (cfg["prep_identity"], tuple(q.shape), tuple(v.shape[2:3]), q.dtype, cfg["kind"], cfg["l2norm"],
                   cfg["precision"])
            p.flags = flags | _lib.FLAG_SAVE_RESIDUALS
            full = lib.jla_residual_bytes(C.byref(p))
            as_residuals = needs_grad and full > 0
            if full == 0:  # a forward that keeps no residuals (KDA with the token-scan backward): the buffer is its scratch
                full = lib.jla_fwd_scratch_bytes(C.byref(p))
            if share["key"] == key and share["buffer"] is not None and share["buffer"].numel() >= full:
                flags |= _lib.FLAG_PREP_DONE
            else:
                share["key"], share["buffer"] = key, torch.empty(full, dtype=torch.uint8, device=dev)
                share["keep"] = cfg["prep_owners"]  # the keyed objects stay alive, so their ids stay theirs
            p.flags = flags
            residuals = share["buffer"] if as_residuals else None
            scratch = None if as_residuals else share["buffer"]
            res_bytes = full if as_residuals else 0
            scr_bytes = 0 if as_residuals else full
        else:
            residuals = torch.empty(res_bytes, dtype=torch.uint8, device=dev) if res_bytes else None
            scr_bytes = lib.jla_fwd_scratch_bytes(C.byref(p))
            scratch = torch.empty(scr_bytes, dtype=torch.uint8, device=dev) if scr_bytes else None
        io = _lib.FwdIO(_ptr(o), _ptr(final), _ptr(residuals), res_bytes, _ptr(scratch), scr_bytes)
        stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            _lib.check(lib.jla_linear_attention_fwd(C.byref(p), C.byref(io), C.c_void_p(stream)),
                       f"{cfg['kind']} forward")
        ctx.cfg, ctx.flags, ctx.rows = cfg, flags, rows
        ctx.save_for_backward(q, k, v, g, beta, h0, k_read, residuals)
        return o, final

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, d_o, d_final):
        lib = _lib.load()
        q, k, v, g, beta, h0, k_read, residuals = ctx.saved_tensors
        cfg = ctx.cfg
        B, T, Hk, K = q.shape
        H, V = v.shape[2:]
        cu, seg = cfg["cu_seqlens"], cfg["segment_ids"]
        flags = (ctx.flags & ~_lib.FLAG_PREP_DONE) | (_lib.FLAG_STATE_GRADS_ONLY if _PassOptions.state_grads_only else 0)
        p = _problem(cfg["kind"], q.dtype, B, T, H, Hk, K, V, 0 if cu is None else ctx.rows, cfg["scale"], flags,
                     cfg["precision"])
        p.q, p.k, p.v, p.g, p.beta, p.h0 = (_ptr(x) for x in (q, k, v, g, beta, h0))
        p.segment_ids, p.cu_seqlens, p.k_read = _ptr(seg), _ptr(cu), _ptr(k_read)
        dev = q.device
        d_o = d_o.contiguous() if d_o is not None else torch.zeros_like(v)
        d_final = None if d_final is None else d_final.contiguous().float()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        dg = None if g is None else torch.empty_like(g)
        dbeta = None if beta is None else torch.empty_like(beta)
        dh0 = None if h0 is None else torch.empty_like(h0)
        dk_read = None if k_read is None else torch.empty_like(k_read)
        scr_bytes = lib.jla_bwd_scratch_bytes(C.byref(p))
        scratch = torch.empty(scr_bytes, dtype=torch.uint8, device=dev) if scr_bytes else None
        io = _lib.BwdIO(_ptr(d_o), _ptr(d_final), _ptr(dq), _ptr(dk), _ptr(dv), _ptr(dg), _ptr(dbeta), _ptr(dh0),
                        _ptr(residuals), 0 if residuals is None else residuals.numel(), _ptr(scratch), scr_bytes,
                        _ptr(dk_read))
        stream = torch.cuda.current_stream(dev).cuda_stream
        with torch.cuda.device(dev):
            _lib.check(lib.jla_linear_attention_bwd(C.byref(p), C.byref(io), C.c_void_p(stream)),
                       f"{cfg['kind']} backward")
        return dq, dk, dv, dg, dbeta, dh0, dk_read, None


# Sequence split policy for the serial state passes, after ``pieces()`` of the reference
# (``src/jla/ops/mosaic_gpu/scalar_gate.py:98-148``): a state pass runs one CTA per (row, head), so a call with few
# rows and heads leaves most SMs idle while each CTA walks a long chain of chunks. Such a call is cut along T into
# pieces that run as independent rows, joined by affine maps (``distributed.context_parallel``, ``group=False``).
MAX_SPLIT_CTAS = 32          # split only when rows * heads is at most this
MIN_PIECE_CHUNKS = 8         # every piece keeps at least this many chunks
MAX_DELTA_PIECES = 8         # the delta rule pays an extra state pass for the maps and their scan
DELTA_PIECE_CHUNKS_ABOVE_4 = 32
# Not in the reference (whose split runs inside one jitted graph): here the split is a sequence of calls driven from
# the host -- two state-only passes, the scan, the real pass, and their mirror images backward -- and costs about
# 1.2 ms of launches whatever the length. Measured on a B200 (one row, 4 and 16 heads, d = 128, forward + backward):
# 8 Ki tokens 1.29 ms unsplit = 1.30 ms split; 16 Ki 2.50 against 1.67 ms; 128 Ki 19.4 against 9.3 ms.
MIN_SPLIT_CHUNKS = 192       # shorter sequences run unsplit


def pieces(batch: int, heads: int, seq_len: int, *, delta: bool, sm_count: int = 148) -> int:
    """Pieces per sequence for the serial state passes (a power of two; 1 = no split)."""
    ctas = max(batch * heads, 1)
    if ctas > MAX_SPLIT_CTAS:
        return 1
    chunks = -(-seq_len // CHUNK)
    if chunks < MIN_SPLIT_CHUNKS:
        return 1
    limit = min(MAX_DELTA_PIECES, sm_count // ctas) if delta else sm_count // ctas
    cp = 1
    while 2 * cp <= limit and chunks // (2 * cp) >= MIN_PIECE_CHUNKS:
        if delta and 2 * cp > 4 and chunks // (2 * cp) < DELTA_PIECE_CHUNKS_ABOVE_4:
            break
        cp *= 2
    return cp


class no_pieces:
    """``with no_pieces():`` calls run unsplit whatever the policy says (the split's own passes, A/B timing)."""
    active = False

    def __enter__(self):
        self._outer = no_pieces.active
        no_pieces.active = True
        return self

    def __exit__(self, *exc):
        no_pieces.active = self._outer


def _split_applies(kind, q, v, cu_seqlens, initial_state, precision) -> int:
    """Pieces per sequence for this call, 1 if it runs unsplit. The split needs the chunked tensor-core path (16-bit
    tensors with K = V = 128), one packed row, and no cu_seqlens (the pieces themselves are passed that way)."""
    if no_pieces.active or _PassOptions.share is not None or cu_seqlens is not None or q.shape[0] != 1:
        return 1
    if q.dtype == torch.float32 or q.shape[-1] != 128 or v.shape[-1] != 128 or _path(precision) == "recurrent":
        return 1
    sms = torch.cuda.get_device_properties(q.device).multi_processor_count
    return pieces(1, v.shape[2], q.shape[1], delta=kind != "simple_gla", sm_count=sms)


def _run_value_blocks(n, kind, q, k, v, g, beta, *, initial_state, output_final_state, **options):
    """The call with every value head cut into ``n`` heads of 128 channels (see ``_value_blocks``): ``v`` and ``o``
    are views, the gates are repeated per block (autograd sums their gradients back), the states are permuted."""
    batch, seq_len, heads, width = v.shape

    def per_block(x):  # [B, T, H(, K)] -> [B, T, H * n(, K)]
        return None if x is None else x.repeat_interleave(n, dim=2)

    def split_state(s):  # [R, H, K, V] -> [R, H * n, K, 128]
        if s is None:
            return None
        r, _, kd, _ = s.shape
        return s.reshape(r, heads, kd, n, VALUE_BLOCK).permute(0, 1, 3, 2, 4).reshape(r, heads * n, kd, VALUE_BLOCK)

    o, final = _run(kind, q, k, v.reshape(batch, seq_len, heads * n, VALUE_BLOCK), per_block(g), per_block(beta),
                    initial_state=split_state(initial_state), output_final_state=output_final_state, **options)
    if final is not None:
        r, _, kd, _ = final.shape
        final = final.reshape(r, heads, n, kd, VALUE_BLOCK).permute(0, 1, 3, 2, 4).reshape(r, heads, kd, width)
    return o.reshape(batch, seq_len, heads, width), final


def _run(kind: str, q, k, v, g, beta, *, scale, initial_state, output_final_state, cu_seqlens, segment_ids,
         use_qk_l2norm=False, chunk_size=CHUNK, precision=None, sub_chunk=None, k_read=None):
    del sub_chunk  # the kernels choose their own sub-blocking
    for name, x in (("q", q), ("k", k), ("v", v)):
        if not isinstance(x, torch.Tensor) or not x.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor: the 'cuda' implementation has no CPU fallback")
    options: dict[str, Any] = dict(scale=scale, initial_state=initial_state, output_final_state=output_final_state,
                                   cu_seqlens=cu_seqlens, segment_ids=segment_ids, chunk_size=chunk_size,
                                   precision=precision)
    gates = tuple(x for x in (g, beta) if x is not None)
    why = unsupported_reason(kind, q, k, v, gates, options, read_key=k_read is not None)
    if why is not None:
        raise ValueError(f"the CUDA kernels cannot run this {kind} call: {why}")
    dev = q.device
    if scale is None:
        scale = q.shape[-1] ** -0.5
    blocks = _value_blocks(kind, q.dtype, q.shape[-1], v.shape[-1], _path(precision), k_read is not None)
    if blocks > 1:
        return _run_value_blocks(blocks, kind, q, k, v, g, beta, scale=scale, initial_state=initial_state,
                                 output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                                 use_qk_l2norm=use_qk_l2norm, chunk_size=chunk_size, precision=precision)
    cp = 1 if k_read is not None else _split_applies(kind, q, v, cu_seqlens, initial_state, precision)
    if cp > 1:
        from ..distributed.context_parallel import context_parallel_linear_attention, plan_pieces

        piece_len = -(-(-(-q.shape[1] // CHUNK)) // cp) * CHUNK  # whole chunks per piece
        plan = plan_pieces(segment_ids, piece_len, group=False, t_local=q.shape[1], device=dev)
        if not any(plan.cont):
            # No document is longer than a piece: the pieces are the documents, nothing has to be joined, and the call
            # is the plain one with the documents as rows (one state pass instead of three forward and two backward).
            rows = len(plan.cu) - 1
            state = None
            if initial_state is not None:  # it enters the first document only
                state = torch.cat([initial_state.to(device=dev, dtype=torch.float32),
                                   torch.zeros(rows - 1, *initial_state.shape[1:], dtype=torch.float32, device=dev)])
            with no_pieces():
                o, final = _run(kind, q, k, v, g, beta, scale=scale, initial_state=state,
                                output_final_state=output_final_state, cu_seqlens=plan.cu_device, segment_ids=None,
                                use_qk_l2norm=use_qk_l2norm, chunk_size=chunk_size, precision=precision)
            return o, (final[-1:] if output_final_state else None)
        gates = {n: x for n, x in (("g", g), ("beta", beta)) if x is not None}
        extra = dict(use_qk_l2norm=use_qk_l2norm) if kind != "simple_gla" else {}
        with no_pieces():
            o, final = context_parallel_linear_attention(
                kind, q, k, v, group=False, impl="cuda", piece_len=plan, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, segment_ids=segment_ids, precision=precision, **gates, **extra)
        return o, (final if output_final_state else None)

    def f32(x):
        return None if x is None else x.to(device=dev, dtype=torch.float32).contiguous()

    def i32(x):
        return None if x is None else torch.as_tensor(x).to(device=dev, dtype=torch.int32).contiguous()

    if cu_seqlens is not None and not (isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda):
        # a table that is still on the host is checked here (reference.py:170-203 takes it on trust); one that
        # already lives on the device is clamped by the kernels instead (a bad row then counts as empty)
        cu_host = torch.as_tensor(cu_seqlens).to(torch.int64).flatten()
        if cu_host.numel() < 1 or int(cu_host[0]) != 0 or int(cu_host[-1]) != q.shape[1] or \
                bool((cu_host[1:] < cu_host[:-1]).any()):
            raise ValueError(f"cu_seqlens must start at 0, end at T = {q.shape[1]} and never decrease; got "
                             f"{cu_host.tolist()[:8]}{'...' if cu_host.numel() > 8 else ''}")
    cfg = dict(kind=kind, scale=float(scale), l2norm=bool(use_qk_l2norm), precision=precision,
               output_final_state=bool(output_final_state), cu_seqlens=i32(cu_seqlens), segment_ids=i32(segment_ids),
               prep_owners=(k, g, beta, segment_ids, cu_seqlens, q if use_qk_l2norm else None),
               prep_identity=tuple((id(x), getattr(x, "_version", 0)) for x in (k, g, beta, segment_ids, cu_seqlens,
                                                                                q if use_qk_l2norm else None)))
    o, final = _LinearAttention.apply(q.contiguous(), k.contiguous(), v.contiguous(), f32(g), f32(beta),
                                      f32(initial_state), None if k_read is None else k_read.contiguous(), cfg)
    return o, (final if output_final_state else None)


def simple_gla(q, k, v, g, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
               segment_ids=None, chunk_size=CHUNK, precision=None):
    """Linear attention with one log-decay per head (Mamba-2 SSD core: ``scale=1``); ``q``/``k`` may have
    fewer heads than ``v`` (value head ``h`` reads key head ``h // (H / Hk)``)."""
    return _run("simple_gla", q, k, v, g, None, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                chunk_size=chunk_size, precision=precision)


def delta_rule(q, k, v, beta, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
               segment_ids=None, use_qk_l2norm=False, chunk_size=CHUNK, precision=None):
    """DeltaNet: the delta-rule write with no decay."""
    return _run("deltanet", q, k, v, None, beta, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                use_qk_l2norm=use_qk_l2norm, chunk_size=chunk_size, precision=precision)


def gated_delta_rule(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False,
                     cu_seqlens=None, segment_ids=None, use_qk_l2norm=False, chunk_size=CHUNK, precision=None):
    """Gated DeltaNet: delta rule with one log-decay per head."""
    return _run("gated_deltanet", q, k, v, g, beta, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                use_qk_l2norm=use_qk_l2norm, chunk_size=chunk_size, precision=precision)


def kda(q, k, v, g, beta, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
        segment_ids=None, use_qk_l2norm=False, chunk_size=CHUNK, sub_chunk=16, precision=None):
    """Kimi Delta Attention: delta rule with a log-decay per key channel (``g [B, T, H, K]``)."""
    return _run("kda", q, k, v, g, beta, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                use_qk_l2norm=use_qk_l2norm, chunk_size=chunk_size, precision=precision, sub_chunk=sub_chunk)


class _Gdn2Inputs(torch.autograd.Function):
    """``(k_read, v_gated) = (k * b, v * w)`` and its gradient, one fused kernel each way (``jla_gdn2_inputs_*``):
    fp32 products rounded once to the tensors' dtype."""

    @staticmethod
    def forward(ctx, k, b, v, w):
        lib = _lib.load()
        k, b, v, w = (x.contiguous() for x in (k, b, v, w))
        k_read, v_gated = torch.empty_like(k), torch.empty_like(v)
        stream = torch.cuda.current_stream(k.device).cuda_stream
        with torch.cuda.device(k.device):
            _lib.check(lib.jla_gdn2_inputs_fwd(_DTYPES[k.dtype], k.numel(), v.numel(), *(_ptr(x) for x in (k, b, v, w)),
                                               _ptr(k_read), _ptr(v_gated), C.c_void_p(stream)), "gdn2 inputs")
        ctx.save_for_backward(k, b, v, w)
        return k_read, v_gated

    @staticmethod
    @torch.autograd.function.once_differentiable
    def backward(ctx, dk_read, dv_gated):
        lib = _lib.load()
        k, b, v, w = ctx.saved_tensors
        dk_read = torch.zeros_like(k) if dk_read is None else dk_read.contiguous()
        dv_gated = torch.zeros_like(v) if dv_gated is None else dv_gated.contiguous()
        dk, db, dv, dw = torch.empty_like(k), torch.empty_like(k), torch.empty_like(v), torch.empty_like(v)
        stream = torch.cuda.current_stream(k.device).cuda_stream
        with torch.cuda.device(k.device):
            _lib.check(lib.jla_gdn2_inputs_bwd(_DTYPES[k.dtype], k.numel(), v.numel(), *(_ptr(x) for x in (k, b, v, w)),
                                               _ptr(dk_read), _ptr(dv_gated), *(_ptr(x) for x in (dk, db, dv, dw)),
                                               C.c_void_p(stream)), "gdn2 inputs backward")
        return dk, db, dv, dw


def gdn2(q, k, v, g, b, w, *, scale=None, initial_state=None, output_final_state=False, cu_seqlens=None,
         segment_ids=None, use_qk_l2norm=False, chunk_size=CHUNK, sub_chunk=16, precision=None):
    """Gated DeltaNet-2 (``gdn2`` of ``src/jla/ops/reference.py:313-343`` in the reference): ``S_t = (I - k_t (b_t *
    k_t)^T) diag(exp g_t) S_{t-1} + k_t (w_t * v_t)^T`` with an erase gate ``b [B, T, H, K]`` and a write gate
    ``w [B, T, H, V]`` in the tensors' dtype; ``b = w = beta`` is KDA.

    The kernels see it as KDA with ``beta = 1``, the values ``w * v`` and a separate read key ``b * k`` (the key the
    recall reads the state with; ``k`` still writes). The two products and their gradients are one fused kernel each
    way (``jla_gdn2_inputs_*``): fp32 products rounded once to the tensors' dtype, as the reference's kernels round
    the gates (``mosaic_gpu/gdn2.py:11-12``); the read side's and the write side's key gradients are added by
    autograd. The unit norm of ``use_qk_l2norm`` is applied first (the gate multiplies the normalised key,
    reference.py:118-119). bf16 and f16 tensors with ``K = V = 128`` run the KDA chunk kernels (the read key in tiles of its
    own); every other call with a read key runs the fp32 token scan.
    """
    for name, x in (("q", q), ("k", k), ("v", v), ("b", b), ("w", w)):
        if not isinstance(x, torch.Tensor) or not x.is_cuda:
            raise ValueError(f"{name} must be a CUDA tensor: the 'cuda' implementation has no CPU fallback")
    if _shape(b) != _shape(q) or _shape(w) != _shape(v) or _shape(k) != _shape(q):
        raise ValueError(f"b must be [B, T, H, K] = {_shape(q)} and w must be [B, T, H, V] = {_shape(v)} (q and k "
                         f"with as many heads as v); got {_shape(b)} and {_shape(w)} with k {_shape(k)}")
    if _shape(q)[2] != _shape(v)[2]:
        raise ValueError(f"gdn2 needs as many key heads as value heads; got {_shape(q)[2]} and {_shape(v)[2]}")
    if k.dtype not in _DTYPES or len({k.dtype, v.dtype}) != 1 or k.shape[-1] % 8 or v.shape[-1] % 8:
        raise ValueError(f"k and v must share a dtype in {tuple(_DTYPES)} and have head sizes that are multiples of 8; "
                         f"got {k.dtype} {_shape(k)}, {v.dtype} {_shape(v)}")
    if use_qk_l2norm:
        def unit(x):
            x32 = x.float()
            return (x32 * torch.rsqrt((x32 * x32).sum(-1, keepdim=True) + 1e-6)).to(x.dtype)
        q, k = unit(q), unit(k)
    k_read, values = _Gdn2Inputs.apply(k, b.to(k.dtype), v, w.to(v.dtype))
    ones = torch.ones(_shape(v)[:3], dtype=torch.float32, device=v.device)
    return _run("kda", q, k, values, g, ones, scale=scale, initial_state=initial_state,
                output_final_state=output_final_state, cu_seqlens=cu_seqlens, segment_ids=segment_ids,
                chunk_size=chunk_size, precision=precision, sub_chunk=sub_chunk, k_read=k_read)


def device_status(device=None) -> int:
    """Synchronises ``device``'s current stream and returns (and clears) its failure status word: non-zero when a
    bounded wait inside one of the tensor-core kernels ran out since the last query, in which case the outputs of
    that call must be discarded. The reference's kernels have no such word (their waits are unbounded)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    with torch.cuda.device(dev):
        return _lib.device_status(torch.cuda.current_stream(dev).cuda_stream)


FUNCTIONS = {
    "simple_gla": simple_gla,
    "deltanet": delta_rule,
    "gated_deltanet": gated_delta_rule,
    "kda": kda,
    "gdn2": gdn2,
}
SUPPORTS = {kind: _supports(kind) for kind in FUNCTIONS}
