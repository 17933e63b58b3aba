"""The forward entry point that brings its own scratch memory (``jla_linear_attention_fwd_noalloc``).

Some hosts of this library cannot allocate while they run: a custom call executing inside another runtime's
stream (the runtime owns the memory pool, and ``cudaMalloc`` would stall the whole device), or a serving process
that fixes its memory map at start-up. For them the library keeps a 32 MiB scratch array of its own on each GPU.
This test calls that entry point through the C ABI twice in a row -- the second call finds the first one's
leftovers in the shared array -- and checks both results against the ordinary entry point, which gets a fresh
caller-provided scratch buffer. The kernels and the order of operations are the same, so the comparison is
bit for bit (tighter than the 1e-2 relative-L2 bound the bf16 tests use).

Collected last on purpose (file name), so that a run that stops at the first failure has already run every
other test; it also passes when run alone in a fresh process.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from oracle.cases import make_case

pytestmark = pytest.mark.gpu


def _problem(lib_mod, case, t, flags=0):
    p = lib_mod.Problem()
    B, T, Hk, K = t["q"].shape
    H, V = t["v"].shape[2:]
    p.kind, p.dtype, p.path, p.flags = lib_mod.KIND[case["meta"]["kind"]], 0, lib_mod.PATH["auto"], flags
    p.B, p.T, p.H, p.Hk, p.K, p.V, p.num_seqs, p.scale = B, T, H, Hk, K, V, 0, case["meta"]["scale"]
    p.q, p.k, p.v = (t[n].data_ptr() for n in ("q", "k", "v"))
    p.g, p.beta, p.h0 = t["g"].data_ptr(), t["beta"].data_ptr(), t["h0"].data_ptr()
    p.segment_ids = t["seg"].data_ptr()
    return p


def test_noalloc_forward_matches_the_regular_entry_point_twice():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    lib.jla_noalloc_scratch_limit.restype = C.c_size_t
    lib.jla_linear_attention_fwd_noalloc.restype = C.c_int
    lib.jla_linear_attention_fwd_noalloc.argtypes = [C.POINTER(_lib.Problem), C.c_void_p, C.c_void_p, C.c_void_p]
    limit = lib.jla_noalloc_scratch_limit()
    assert limit == 32 << 20

    dev = torch.device("cuda:0")
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    outs = []
    # two different problems back to back: the second call sees the first one's scratch contents
    for seed, T in ((31, 1000), (32, 640)):
        case = make_case("gated_deltanet", B=2, T=T, H=4, Hk=2, K=128, V=128, seed=seed, docs="mixed", h0=True)
        t = {n: torch.tensor(case[n], device=dev, dtype=torch.bfloat16) for n in ("q", "k", "v")}
        t.update({n: torch.tensor(case[n], device=dev, dtype=torch.float32) for n in ("g", "beta", "h0")})
        t["seg"] = torch.tensor(case["seg"], device=dev, dtype=torch.int32)
        p = _problem(_lib, case, t)
        need = lib.jla_fwd_scratch_bytes(C.byref(p))
        assert 0 < need <= limit

        o_ref = torch.empty_like(t["v"])
        s_ref = torch.empty(2, 4, 128, 128, device=dev)
        scratch = torch.empty(need, dtype=torch.uint8, device=dev)
        io = _lib.FwdIO(o_ref.data_ptr(), s_ref.data_ptr(), None, 0, scratch.data_ptr(), need)
        _lib.check(lib.jla_linear_attention_fwd(C.byref(p), C.byref(io), stream), "regular forward")

        o = torch.full_like(t["v"], float("nan"))
        s = torch.full_like(s_ref, float("nan"))
        rc = lib.jla_linear_attention_fwd_noalloc(C.byref(p), C.c_void_p(o.data_ptr()), C.c_void_p(s.data_ptr()), stream)
        assert rc == 0, lib.jla_last_error()
        torch.cuda.synchronize()
        assert torch.equal(o, o_ref) and torch.equal(s, s_ref)
        assert bool(torch.isfinite(o.float()).all())
        outs.append(o)
    assert outs[0].shape != outs[1].shape


def test_noalloc_rejects_what_does_not_fit_or_needs_residuals():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    lib.jla_linear_attention_fwd_noalloc.restype = C.c_int
    lib.jla_linear_attention_fwd_noalloc.argtypes = [C.POINTER(_lib.Problem), C.c_void_p, C.c_void_p, C.c_void_p]
    p = _lib.Problem()
    p.kind, p.dtype, p.path, p.flags = _lib.KIND["gated_deltanet"], 0, 0, 0
    p.B, p.T, p.H, p.Hk, p.K, p.V, p.num_seqs, p.scale = 8, 2048, 16, 16, 128, 128, 0, 0.1
    dummy = torch.zeros(16, device="cuda")
    assert lib.jla_fwd_scratch_bytes(C.byref(p)) > (32 << 20)
    rc = lib.jla_linear_attention_fwd_noalloc(C.byref(p), C.c_void_p(dummy.data_ptr()), None, None)
    assert rc == _lib.ERR_WORKSPACE and b"more than" in lib.jla_last_error()
    p.B, p.T, p.flags = 1, 256, _lib.FLAG_SAVE_RESIDUALS
    rc = lib.jla_linear_attention_fwd_noalloc(C.byref(p), C.c_void_p(dummy.data_ptr()), None, None)
    assert rc == _lib.ERR_BAD_ARGUMENT and b"forward only" in lib.jla_last_error()
    # the array is shared by every call on the device: nobody can promise that an earlier call's tables are still there
    p.flags = _lib.FLAG_PREP_DONE
    rc = lib.jla_linear_attention_fwd_noalloc(C.byref(p), C.c_void_p(dummy.data_ptr()), None, None)
    assert rc == _lib.ERR_BAD_ARGUMENT and b"PREP_DONE" in lib.jla_last_error()
