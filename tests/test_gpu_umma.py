"""The tcgen05 primitive layer (descriptors, 128-byte swizzle, TMEM loads) against a plain matmul."""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,kd", [(64, 128, 128), (64, 64, 64), (64, 64, 128), (128, 128, 64)])
@pytest.mark.parametrize("a_mn", [0, 1])
@pytest.mark.parametrize("b_mn", [0, 1])
def test_umma_product(m, n, kd, a_mn, b_mn):
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(m * 7 + n * 3 + kd + 2 * a_mn + b_mn)
    a = torch.randn(m, kd, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(kd, n, generator=gen).to(torch.bfloat16).cuda()
    a_in = a.t().contiguous() if a_mn else a.contiguous()
    b_in = b.contiguous() if b_mn else b.t().contiguous()
    c = torch.full((m, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.jla_selftest_umma(m, n, kd, a_mn, b_mn, C.c_void_p(a_in.data_ptr()), C.c_void_p(b_in.data_ptr()),
                               C.c_void_p(c.data_ptr()), C.c_void_p(status.data_ptr()), C.c_void_p(stream))
    assert rc == 0, lib.jla_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "the MMA completion never arrived"
    want = a.float() @ b.float()
    err = (c - want).abs().max().item()
    assert err < 1e-3 * max(1.0, want.abs().max().item()), err


@pytest.mark.parametrize("n,kd", [(64, 128), (128, 64), (64, 64)])
@pytest.mark.parametrize("b_mn", [0, 1])
def test_umma_product_with_a_in_tmem(n, kd, b_mn):
    """A [128 x kd] written to TMEM as packed bf16 pairs by tcgen05.st (a_mn_major = 2 selects this mode)."""
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    gen = torch.Generator().manual_seed(n * 3 + kd + b_mn)
    a = torch.randn(128, kd, generator=gen).to(torch.bfloat16).cuda()
    b = torch.randn(kd, n, generator=gen).to(torch.bfloat16).cuda()
    b_in = b.contiguous() if b_mn else b.t().contiguous()
    c = torch.full((128, n), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.jla_selftest_umma(128, n, kd, 2, b_mn, C.c_void_p(a.data_ptr()), C.c_void_p(b_in.data_ptr()),
                               C.c_void_p(c.data_ptr()), C.c_void_p(status.data_ptr()), C.c_void_p(stream))
    assert rc == 0, lib.jla_last_error()
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    want = a.float() @ b.float()
    assert (c - want).abs().max().item() < 1e-3 * max(1.0, want.abs().max().item())
