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
GATES = {"simple_gla": ("g",), "deltanet": ("beta",), "gated_deltanet": ("g", "beta"), "kda": ("g", "beta"),
         "gdn2": ("g", "b", "w")}


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
    for n in ("q", "k", "v", "b", "w"):  # (b, w: the channel gates of Gated DeltaNet-2, in the tensors' dtype)
        if n in ins:
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
    leaves = {n: torch.tensor(ins[n], dtype=dtype, requires_grad=grads) for n in ("q", "k", "v", "b", "w", "g", "beta",
                                                                                       "h0") if n in ins}
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


# ---------------------------------------------------------------------------------------------------------
# direct C-ABI calls (ctypes), keeping the residual and scratch buffers for stage-level checks
def cabi_fwd_bwd(kind, ins, *, scale, dtype="bfloat16", l2norm=False, path="chunked", device="cuda:0",
                 backward=True):
    import ctypes as C

    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    td = TORCH_DTYPE[dtype]
    dev = torch.device(device)
    t = {n: torch.tensor(ins[n], dtype=td, device=dev).contiguous() for n in ("q", "k", "v", "do")}
    for n in ("g", "beta", "h0", "dht"):
        if n in ins:
            t[n] = torch.tensor(ins[n], dtype=torch.float32, device=dev).contiguous()
    if "seg" in ins:
        t["seg"] = torch.tensor(ins["seg"], dtype=torch.int32, device=dev).contiguous()
    B, T, Hk, K = t["q"].shape
    H, V = t["v"].shape[2:]
    p = _lib.Problem()
    p.kind, p.dtype, p.path = _lib.KIND[kind], {"bfloat16": 0, "float16": 1, "float32": 2}[dtype], _lib.PATH[path]
    p.flags = (_lib.FLAG_QK_L2NORM if l2norm else 0) | _lib.FLAG_SAVE_RESIDUALS
    p.B, p.T, p.H, p.Hk, p.K, p.V, p.num_seqs, p.scale = B, T, H, Hk, K, V, 0, scale

    def ptr(name):
        return t[name].data_ptr() if name in t else None

    p.q, p.k, p.v, p.g, p.beta, p.h0, p.segment_ids = (ptr(n) for n in ("q", "k", "v", "g", "beta", "h0", "seg"))
    why = lib.jla_unsupported_reason(C.byref(p))
    assert why is None, why
    o = torch.empty_like(t["v"])
    final = torch.empty(B, H, K, V, dtype=torch.float32, device=dev)
    rbytes = lib.jla_residual_bytes(C.byref(p))
    res = torch.zeros(max(rbytes, 1), dtype=torch.uint8, device=dev)
    sbytes = lib.jla_fwd_scratch_bytes(C.byref(p))
    scr = torch.zeros(max(sbytes, 1), dtype=torch.uint8, device=dev)
    io = _lib.FwdIO(o.data_ptr(), final.data_ptr(), res.data_ptr(), rbytes, scr.data_ptr(), sbytes)
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(lib.jla_linear_attention_fwd(C.byref(p), C.byref(io), C.c_void_p(stream)), "fwd")
    torch.cuda.synchronize()
    out = dict(o=o, ht=final, residuals=res, problem=p, tensors=t)
    if backward:
        dq, dk, dv = torch.empty_like(t["q"]), torch.empty_like(t["k"]), torch.empty_like(t["v"])
        dg = torch.empty_like(t["g"]) if "g" in t else None
        dbeta = torch.empty_like(t["beta"]) if "beta" in t else None
        dh0 = torch.empty_like(final)
        bbytes = lib.jla_bwd_scratch_bytes(C.byref(p))
        bscr = torch.zeros(max(bbytes, 1), dtype=torch.uint8, device=dev)
        bio = _lib.BwdIO(t["do"].data_ptr(), ptr("dht"), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                         None if dg is None else dg.data_ptr(), None if dbeta is None else dbeta.data_ptr(),
                         dh0.data_ptr(), res.data_ptr(), rbytes, bscr.data_ptr(), bbytes)
        _lib.check(lib.jla_linear_attention_bwd(C.byref(p), C.byref(bio), C.c_void_p(stream)), "bwd")
        torch.cuda.synchronize()
        out.update(dq=dq, dk=dk, dv=dv, dg=dg, dbeta=dbeta, dh0=dh0, bwd_scratch=bscr)
    return out


class ChunkedLayout:
    """Views into the residual / scratch buffers of a dense (no cu_seqlens) chunked call."""

    def __init__(self, problem, residuals, bwd_scratch=None, dtype=torch.bfloat16):
        import ctypes as C

        from jax_linear_attention_b200 import _lib

        class Layout(C.Structure):
            _fields_ = [("num_chunk_slots", C.c_int32)] + [(n, C.c_size_t) for n in (
                "meta", "row_chunks", "gates", "runs", "t0", "ag", "qn", "kn", "h", "vn", "w", "residual_bytes", "dh", "dvn",
                "dq_acc", "dk_acc", "dp", "dga", "bwd_scratch_bytes")]

        lay = Layout()
        lib = _lib.load()
        lib.jla_chunked_get_layout.argtypes = [C.POINTER(_lib.Problem), C.POINTER(Layout)]
        assert lib.jla_chunked_get_layout(C.byref(problem), C.byref(lay)) == 0
        self.lay, self.p, self.res, self.scr, self.dtype = lay, problem, residuals, bwd_scratch, dtype
        self.nc = lay.num_chunk_slots
        self.per_row = self.nc // problem.B

    def _view(self, buf, off, shape, dtype):
        n = int(np.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        return buf[off:off + n].view(dtype).reshape(shape)

    def chunked(self, x):
        """[nc, H, ...] -> [B, H, NC, ...] float64 numpy."""
        B = self.p.B
        x = x.reshape(B, self.per_row, *x.shape[1:]).movedim(2, 1)
        return x.double().cpu().numpy()

    def gates(self):
        g = self._view(self.res, self.lay.gates, (self.nc, self.p.H, 2, 64), torch.float32)
        return self.chunked(g[:, :, 0]), self.chunked(g[:, :, 1])

    def t0(self):
        return self.chunked(self._view(self.res, self.lay.t0, (self.nc, self.p.H, 64, 64), self.dtype))

    @property
    def transposed(self):
        """K = V = 128 runs the tcgen05 kernels, which keep h and Vn transposed ([V][K], [V][64])."""
        import os

        return self.p.K == 128 and self.p.V == 128 and os.environ.get("JLA_B200_LEGACY", "0") != "1"

    def h(self):
        if self.transposed:
            x = self._view(self.res, self.lay.h, (self.nc, self.p.H, self.p.V, self.p.K), self.dtype)
            return self.chunked(x.transpose(-1, -2))
        return self.chunked(self._view(self.res, self.lay.h, (self.nc, self.p.H, self.p.K, self.p.V), self.dtype))

    def vn(self):
        if self.transposed:
            x = self._view(self.res, self.lay.vn, (self.nc, self.p.H, self.p.V, 64), self.dtype)
            return self.chunked(x.transpose(-1, -2))
        return self.chunked(self._view(self.res, self.lay.vn, (self.nc, self.p.H, 64, self.p.V), self.dtype))

    def w(self):
        """W = V - cin Gamma (K S) per chunk; only the tcgen05 path keeps it (transposed)."""
        assert self.transposed
        x = self._view(self.res, self.lay.w, (self.nc, self.p.H, self.p.V, 64), self.dtype)
        return self.chunked(x.transpose(-1, -2))

    def dh(self):
        if self.transposed:
            x = self._view(self.scr, self.lay.dh, (self.nc, self.p.H, self.p.V, self.p.K), self.dtype)
            return self.chunked(x.transpose(-1, -2))
        return self.chunked(self._view(self.scr, self.lay.dh, (self.nc, self.p.H, self.p.K, self.p.V), self.dtype))

    def dvn(self):
        if self.transposed:
            x = self._view(self.scr, self.lay.dvn, (self.nc, self.p.H, self.p.V, 64), self.dtype)
            return self.chunked(x.transpose(-1, -2))
        return self.chunked(self._view(self.scr, self.lay.dvn, (self.nc, self.p.H, 64, self.p.V), self.dtype))
