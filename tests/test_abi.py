"""CPU checks of the boundary: the library loads, exports every symbol the header declares, and the host
dispatcher validates calls like the reference's (no kernel is launched here)."""

import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "jla_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(jla_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    names = _declared()
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), name
    assert set(_lib.EXPORTS) <= set(names)
    assert lib.jla_abi_version() >= 1000


def test_struct_layout_matches_header():
    """Field order and count of the ctypes mirrors follow the header (a reorder would silently corrupt calls)."""
    from jax_linear_attention_b200 import _lib

    text = open(os.path.join(ROOT, "include", "jla_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)

    def fields(struct):
        body = re.search(r"typedef struct %s \{(.*?)\} %s;" % (struct, struct), text, re.S).group(1)
        out = []
        for decl in body.split(";"):
            decl = decl.strip()
            if not decl:
                continue
            names = re.sub(r"^(const\s+)?\w+\s*\*?", "", decl, count=1)
            out += [n.strip(" *") for n in names.split(",")]
        return out

    assert fields("jla_problem") == [f[0] for f in _lib.Problem._fields_]
    assert fields("jla_fwd_io") == [f[0] for f in _lib.FwdIO._fields_]
    assert fields("jla_bwd_io") == [f[0] for f in _lib.BwdIO._fields_]


def test_unsupported_reason_and_sizes_without_a_gpu():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    p = _lib.Problem()
    p.kind, p.dtype, p.path, p.flags = _lib.KIND["gated_deltanet"], 2, 0, 0
    p.B, p.T, p.H, p.Hk, p.K, p.V, p.num_seqs, p.scale = 1, 512, 4, 4, 64, 64, 0, 0.125
    assert _lib.unsupported_reason(p) is None
    assert lib.jla_residual_bytes(ctypes.byref(p)) == 0
    assert lib.jla_bwd_scratch_bytes(ctypes.byref(p)) > 2 * 512 * 4 * 64 * 4
    p.Hk = 3
    assert "multiple of key heads" in _lib.unsupported_reason(p)
    p.Hk, p.num_seqs, p.B = 4, 2, 2
    assert "batch size 1" in _lib.unsupported_reason(p)
    rc = lib.jla_linear_attention_fwd(ctypes.byref(p), None, None)
    assert rc == _lib.ERR_BAD_ARGUMENT and b"batch size 1" in lib.jla_last_error()


def test_dispatcher_mirrors_reference_errors():
    from jax_linear_attention_b200 import ops

    assert set(ops.KINDS) == {"simple_gla", "deltanet", "gated_deltanet", "kda", "gdn2"}
    assert ops.available("kda") == ("cuda",)
    q = torch.zeros(1, 8, 2, 64)
    g = torch.zeros(1, 8, 2)
    with pytest.raises(ValueError, match="unknown linear-attention kind"):
        ops.linear_attention("gla2", q, q, q)
    with pytest.raises(ValueError, match=r"missing \['beta'\]"):
        ops.linear_attention("gated_deltanet", q, q, q, g=g)
    with pytest.raises(ValueError, match=r"unexpected \['beta'\]"):
        ops.linear_attention("simple_gla", q, q, q, g=g, beta=g)
    with pytest.raises(ValueError, match="no 'mosaic_gpu' implementation"):
        ops.linear_attention("simple_gla", q, q, q, g=g, impl="mosaic_gpu")
    with pytest.raises(ValueError, match="no CPU fallback"):
        ops.linear_attention("simple_gla", q, q, q, g=g, impl="cuda")
    # supports() works on shape structs (it is evaluated on per-shard shapes by the sharding layer)
    class Spec:
        def __init__(self, shape, dtype):
            self.shape, self.dtype = shape, dtype
    qs, gs = Spec((2, 100, 2, 64), torch.float32), Spec((2, 100, 4), torch.float32)
    vs = Spec((2, 100, 4, 64), torch.float32)
    assert ops.cuda.SUPPORTS["simple_gla"](qs, qs, vs, gs)
    assert not ops.cuda.SUPPORTS["simple_gla"](qs, qs, vs, gs, chunk_size=32)
    assert "g must be" in ops.cuda.unsupported_reason("kda", qs, qs, vs, (gs, gs), {})
    # Gated DeltaNet-2: gates shaped like k and v, as many key heads as value heads
    q4 = Spec((2, 100, 4, 64), torch.float32)
    assert ops.cuda.SUPPORTS["gdn2"](q4, q4, vs, q4, q4, vs)
    assert "b must be" in ops.cuda.unsupported_reason("gdn2", q4, q4, vs, (q4, gs, vs), {})
    assert "b must be" in ops.cuda.unsupported_reason("gdn2", qs, qs, vs, (qs, qs, vs), {})
    # wide value heads: 16-bit calls with V = 256, 384, 512 are answered for their blocks of 128 channels (K = 128, or
    # 64 for the scalar-gate kinds); other widths, the token scan asked for by name, and read keys are not
    bf = torch.bfloat16
    qb, gb = Spec((1, 300, 2, 128), bf), Spec((1, 300, 2), torch.float32)
    for width, ok in ((256, True), (384, True), (512, True), (320, False), (640, True)):
        assert ops.cuda.SUPPORTS["gated_deltanet"](qb, qb, Spec((1, 300, 2, width), bf), gb, gb) is ok, width
    v512 = Spec((1, 300, 2, 512), bf)
    assert not ops.cuda.SUPPORTS["gated_deltanet"](qb, qb, v512, gb, gb, precision="highest")
    assert ops.cuda.SUPPORTS["simple_gla"](Spec((1, 300, 2, 64), bf), Spec((1, 300, 2, 64), bf), v512, gb)
    assert not ops.cuda.SUPPORTS["kda"](Spec((1, 300, 2, 64), bf), Spec((1, 300, 2, 64), bf), v512,
                                        Spec((1, 300, 2, 64), torch.float32), gb)
    assert ops.cuda._value_blocks("kda", bf, 128, 256, "auto", True) == 1


def test_register_adds_an_implementation():
    from jax_linear_attention_b200 import ops

    calls = []
    ops.register("probe", "simple_gla", lambda q, k, v, g, **kw: calls.append(kw) or ("o", None))
    try:
        assert ops.available("simple_gla") == ("cuda", "probe")
        out = ops.linear_attention("simple_gla", 1, 2, 3, g=4, impl="probe", scale=2.0)
        assert out == ("o", None) and calls == [dict(scale=2.0)]
    finally:
        ops._REGISTRY.pop("probe")
    with pytest.raises(ValueError, match="unknown linear-attention kind"):
        ops.register("probe", "nope", lambda *a: None)
