"""ctypes binding of ``libjla_b200.so`` (C ABI: ``include/jla_b200.h``).

There is no fallback: if the library is missing or a call is rejected, an exception is raised.
"""

from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# The in-tree build's output; JLA_B200_LIB names another build of the same library (e.g. the CMake build's).
LIB_PATH = os.environ.get("JLA_B200_LIB") or os.path.join(HERE, "libjla_b200.so")

KIND = {"simple_gla": 0, "deltanet": 1, "gated_deltanet": 2, "kda": 3}  # (gdn2: KDA with a read key, ops.cuda.gdn2)
PATH = {"auto": 0, "recurrent": 1, "chunked": 2}
FLAG_QK_L2NORM = 1
FLAG_SAVE_RESIDUALS = 2
FLAG_PREP_DONE = 4
FLAG_STATE_GRADS_ONLY = 8
FLAG_STATE_ONLY = 16
OK, ERR_BAD_ARGUMENT, ERR_UNSUPPORTED, ERR_WORKSPACE, ERR_CUDA = 0, -1, -2, -3, -4

EXPORTS = (
    "jla_abi_version", "jla_last_error", "jla_unsupported_reason", "jla_residual_bytes",
    "jla_fwd_scratch_bytes", "jla_bwd_scratch_bytes", "jla_linear_attention_fwd", "jla_linear_attention_bwd",
)


class Problem(C.Structure):
    _fields_ = [
        ("kind", C.c_int32), ("dtype", C.c_int32), ("path", C.c_int32), ("flags", C.c_int32),
        ("B", C.c_int32), ("T", C.c_int32), ("H", C.c_int32), ("Hk", C.c_int32), ("K", C.c_int32), ("V", C.c_int32),
        ("num_seqs", C.c_int32), ("scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("g", C.c_void_p), ("beta", C.c_void_p),
        ("h0", C.c_void_p), ("segment_ids", C.c_void_p), ("cu_seqlens", C.c_void_p), ("k_read", C.c_void_p),
    ]


class FwdIO(C.Structure):
    _fields_ = [
        ("o", C.c_void_p), ("final_state", C.c_void_p), ("residuals", C.c_void_p), ("residual_bytes", C.c_size_t),
        ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t),
    ]


class BwdIO(C.Structure):
    _fields_ = [
        ("d_o", C.c_void_p), ("d_final", C.c_void_p), ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p),
        ("dg", C.c_void_p), ("dbeta", C.c_void_p), ("dh0", C.c_void_p), ("residuals", C.c_void_p),
        ("residual_bytes", C.c_size_t), ("scratch", C.c_void_p), ("scratch_bytes", C.c_size_t), ("dk_read", C.c_void_p),
    ]


_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build the CUDA kernels with `python -m jax_linear_attention_b200.build` "
            "(there is no CPU or eager fallback)")
    lib = C.CDLL(LIB_PATH)
    lib.jla_abi_version.restype = C.c_int
    lib.jla_last_error.restype = C.c_char_p
    lib.jla_unsupported_reason.restype = C.c_char_p
    lib.jla_unsupported_reason.argtypes = [C.POINTER(Problem)]
    for name in ("jla_residual_bytes", "jla_fwd_scratch_bytes", "jla_bwd_scratch_bytes"):
        fn = getattr(lib, name)
        fn.restype = C.c_size_t
        fn.argtypes = [C.POINTER(Problem)]
    lib.jla_linear_attention_fwd.restype = C.c_int
    lib.jla_linear_attention_fwd.argtypes = [C.POINTER(Problem), C.POINTER(FwdIO), C.c_void_p]
    lib.jla_linear_attention_bwd.restype = C.c_int
    lib.jla_linear_attention_bwd.argtypes = [C.POINTER(Problem), C.POINTER(BwdIO), C.c_void_p]
    lib.jla_piece_scan.restype = C.c_int
    lib.jla_piece_scan.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    lib.jla_gdn2_inputs_fwd.restype = C.c_int
    lib.jla_gdn2_inputs_fwd.argtypes = [C.c_int, C.c_int64, C.c_int64] + [C.c_void_p] * 7
    lib.jla_gdn2_inputs_bwd.restype = C.c_int
    lib.jla_gdn2_inputs_bwd.argtypes = [C.c_int, C.c_int64, C.c_int64] + [C.c_void_p] * 11
    lib.jla_device_status.restype = C.c_int
    lib.jla_device_status.argtypes = [C.POINTER(C.c_int), C.c_void_p]
    lib.jla_selftest_bounded_wait.restype = C.c_int
    lib.jla_selftest_bounded_wait.argtypes = [C.c_uint32, C.c_void_p]
    _lib = lib
    return lib


def device_status(stream: int | None = None) -> int:
    """Waits for ``stream`` (the default stream if None), returns the current device's status word and clears it:
    0 unless a bounded wait inside a tensor-core kernel gave up since the last query (then that launch's results
    are undefined; the codes are listed at ``jla_device_status`` in the header)."""
    out = C.c_int(0)
    check(load().jla_device_status(C.byref(out), C.c_void_p(stream)), "device status")
    return out.value


def unsupported_reason(problem: Problem) -> str | None:
    why = load().jla_unsupported_reason(C.byref(problem))
    return None if why is None else why.decode()


def check(rc: int, what: str) -> None:
    if rc == OK:
        return
    text = load().jla_last_error().decode()
    if rc == ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {text}")
    if rc in (ERR_BAD_ARGUMENT, ERR_WORKSPACE):
        raise ValueError(f"{what}: {text}")
    raise RuntimeError(f"{what}: {text} (status {rc})")
