"""The failure path of the tensor-core kernels, exercised without hanging or faulting anything: a bounded wait that
runs out makes the kernel return normally with a code in the device status word, which the host reads and clears."""

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.expects_status]


def test_a_wait_that_runs_out_sets_the_status_word_and_the_context_stays_usable():
    from jax_linear_attention_b200 import _lib
    from jax_linear_attention_b200.ops import cuda as ops_cuda

    lib = _lib.load()
    assert ops_cuda.device_status() == 0  # also clears whatever an earlier test left
    # a barrier nobody arrives on, polled 2000 times: the kernel gives up, records code 9 and exits normally
    _lib.check(lib.jla_selftest_bounded_wait(2000, None), "selftest")
    assert ops_cuda.device_status() == 9
    assert ops_cuda.device_status() == 0  # the query cleared it
    # the context is intact: ordinary work still runs and gives the right answer
    x = torch.arange(1024, device="cuda", dtype=torch.float32)
    assert float((x * 2).sum()) == 1023 * 1024
    # and a real kernel run afterwards leaves the word at zero
    from oracle.cases import make_case
    from tests._util import run_cuda

    case = make_case("gated_deltanet", B=1, T=256, H=2, K=128, V=128, seed=2)
    run_cuda("gated_deltanet", case, scale=case["meta"]["scale"], dtype="bfloat16")
    assert ops_cuda.device_status() == 0


def test_selftest_rejects_an_unbounded_limit():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    assert lib.jla_selftest_bounded_wait(0, None) == _lib.ERR_BAD_ARGUMENT
    assert lib.jla_selftest_bounded_wait((1 << 20) + 1, None) == _lib.ERR_BAD_ARGUMENT


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_every_gpu_has_its_own_status_word():
    from jax_linear_attention_b200 import _lib

    lib = _lib.load()
    with torch.cuda.device(1):
        assert _lib.device_status() == 0
        _lib.check(lib.jla_selftest_bounded_wait(500, None), "selftest on cuda:1")
    with torch.cuda.device(0):
        assert _lib.device_status() == 0  # cuda:0's word is untouched
    with torch.cuda.device(1):
        assert _lib.device_status() == 9
