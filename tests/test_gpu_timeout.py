"""The give-up path of the kernels' bounded waits, exercised without faulting the GPU: a host-set test option
shortens the wait limit of one A8W8 launch to a few milliseconds and leaves out the loads of one K block, so the
tensor-core warp's wait for that block runs out.  The kernel must record its code, drain and free what it holds and
return; the host must read FNN_ERR_DEVICE_TIMEOUT once, and the next call must run clean on the same context."""
import ctypes

import pytest
import torch

from oracle import quant_oracle as O

pytestmark = pytest.mark.gpu

DEV_TIMEOUT_MMA, DEV_TIMEOUT_EPILOGUE = 2, 3


def _a8w8(a, b, row, col):
    import flashnn_b200
    return flashnn_b200.GemmA8W8(torch.bfloat16)(a, b, row, col)


def test_a_wait_that_runs_out_returns_an_error_code_and_leaves_the_context_usable():
    from flashnn_b200 import _lib
    L = _lib.lib()
    g = torch.Generator().manual_seed(0)
    a = torch.randint(-127, 128, (64, 2048), generator=g, dtype=torch.int8)
    b = torch.randint(-127, 128, (64, 2048), generator=g, dtype=torch.int8)
    row = (torch.rand(64, generator=g) * 0.015 + 0.005)
    col = (torch.rand(64, generator=g) * 0.009 + 0.001)
    dev = [t.cuda() for t in (a, b, row, col)]
    want = O.gemm_a8w8_from_acc(O.gemm_a8w8_acc_i32(a, b), row, col, torch.bfloat16)
    assert torch.equal(_a8w8(*dev).cpu().view(torch.int16), want.view(torch.int16))  # one tile, one CTA
    assert _lib.device_status() == 0

    _lib.set_option(_lib.OPT_TEST_STALL_US, 20000)  # every wait of the next launch gives up after 20 ms
    try:
        assert L.fnn_get_option(_lib.OPT_TEST_STALL_US) == 20000
        _a8w8(*dev)  # the launch itself succeeds; the kernel gives up on the missing K block and returns
        code = ctypes.c_int(0)
        st = L.fnn_device_status(ctypes.byref(code))
    finally:
        _lib.set_option(_lib.OPT_TEST_STALL_US, 0)
    assert st == 8, L.fnn_last_error_string()  # FNN_ERR_DEVICE_TIMEOUT
    # the tensor-core warp waits for the missing block; the epilogue warps wait for that warp and may be the first
    # to notice, a few microseconds apart
    assert code.value in (DEV_TIMEOUT_MMA, DEV_TIMEOUT_EPILOGUE)
    assert b"bounded wait" in L.fnn_last_error_string()

    # the status word was cleared by the read, the context is intact, and the same call now gives the right answer
    assert _lib.device_status() == 0
    assert torch.equal(_a8w8(*dev).cpu().view(torch.int16), want.view(torch.int16))
    assert torch.cuda.is_available() and float(torch.ones(4, device="cuda").sum()) == 4.0
    assert _lib.device_status() == 0


def test_the_option_rejects_out_of_range_values():
    from flashnn_b200 import _lib
    with pytest.raises(_lib.FlashNNError):
        _lib.set_option(_lib.OPT_TEST_STALL_US, -1)
    with pytest.raises(_lib.FlashNNError):
        _lib.set_option(_lib.OPT_TEST_STALL_US, 2000000)
    assert _lib.lib().fnn_get_option(_lib.OPT_TEST_STALL_US) == 0
