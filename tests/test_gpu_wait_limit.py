"""A bounded device-side wait that runs out: the kernel returns, the status block says where, the context lives on.

``nq_row_reduce_p2p`` polls its inbox for the words its peers push.  Here it is called as rank 0 of a group of
two whose second member does not exist: ``inbox[1]`` is a second allocation on the same GPU that nobody reads
and no kernel ever pushes into ``inbox[0]``, so the poll can only end by its time limit (set to 2 ms for the
test).  Nothing faults, traps or spins without bound; the call must complete, report
``NQ_ERR_DEVICE_TIMEOUT`` with the site of the wait, and leave the device usable.
"""
import ctypes
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

NQ_ERR_DEVICE_TIMEOUT = -5
SITE_ROW_REDUCE = 64


@pytest.fixture(scope="module")
def lib(built_library):
    from nano_qwen_b200 import _cabi, ops
    ops.init()
    return _cabi.lib()


def test_row_reduce_poll_gives_up_and_reports(lib):
    from nano_qwen_b200 import _cabi, ops
    from oracle import fp8_spec as S
    torch.cuda.synchronize()
    assert _cabi.device_status(reset=True)["code"] in (0, NQ_ERR_DEVICE_TIMEOUT)
    slot = 4096
    ptrs = []

    def alloc(nbytes):
        p = ctypes.c_void_p()
        _cabi.check(lib.nq_p2p_alloc(nbytes, ctypes.byref(p)), "nq_p2p_alloc")
        ptrs.append(p)
        return p.value

    try:
        mine, absent_peer, state = alloc(2 * 2 * 2 * slot), alloc(2 * 2 * 2 * slot), alloc(256)
        inbox = (ctypes.c_void_p * 2)(mine, absent_peer)
        y = torch.ones(1024, dtype=torch.bfloat16, device="cuda")
        _cabi.check(lib.nq_set_wait_limit_ns(2_000_000), "nq_set_wait_limit_ns")
        t0 = time.perf_counter()
        st = lib.nq_row_reduce_p2p(y.data_ptr(), y.data_ptr(), y.numel(), inbox, 0, 2, slot, state,
                                   torch.cuda.current_stream().cuda_stream)
        assert st == 0                                     # the call itself is accepted and enqueued
        torch.cuda.synchronize()                           # ... and it ends, although no peer ever answers
        waited = time.perf_counter() - t0
        assert waited < 1.0, f"the poll should give up after about 2 ms, took {waited:.3f} s"
        status = _cabi.device_status()
        assert status["code"] == NQ_ERR_DEVICE_TIMEOUT
        assert status["where"] == SITE_ROW_REDUCE and status["aux"] == 1        # waiting for rank 1
        with pytest.raises(_cabi.NqError):
            ops.check_device_status()                      # what a host loop calls at its synchronisation points
    finally:
        lib.nq_set_wait_limit_ns(2_000_000_000)
        _cabi.device_status(reset=True)
        torch.cuda.synchronize()
        for p in ptrs:
            lib.nq_p2p_free(p)
    # the device and the library are still usable: an ordinary linear passes against the oracle
    g = torch.Generator().manual_seed(3)
    x = torch.randn(40, 512, generator=g).to(torch.bfloat16)
    w = (torch.randn(256, 512, generator=g) * 0.02).to(torch.bfloat16)
    wq, sw = S.quantize_weight_block128(w)
    yy = ops.fp8_linear(x.cuda(), wq.cuda(), sw.cuda())
    torch.cuda.synchronize()
    xq, sx = S.quantize_act_group128(x)
    assert S.max_rel_err(yy.cpu(), S.linear_dequant_matmul(xq, sx, wq, sw)) <= 2e-2
    assert _cabi.device_status()["code"] == 0
    ops.check_device_status()
