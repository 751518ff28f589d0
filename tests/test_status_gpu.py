"""What happens when a bounded wait inside a kernel runs out: the kernel must return (no hang, no trap) with a
code in the per-device status word, the C ABI must report and clear it, and the PyTorch operators -- which do
not synchronise per call -- must raise at the next operator call instead of handing out incomplete tensors
silently.  The time-out is produced by the library's own self-test kernel: a wait, limited to a few polls,
on a barrier that nothing ever arrives on."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def test_bounded_wait_gives_up_and_reports_through_the_c_abi():
    from tvdcn_b200 import cabi
    L = cabi.lib()
    assert L.tvdcn_b200_device_status() == 0
    cabi.check(L.tvdcn_b200_selftest_bounded_wait(8, _stream()))
    torch.cuda.synchronize()                       # the kernel returned: the context is alive
    assert L.tvdcn_b200_device_status() == 900     # the give-up code of the self test
    assert L.tvdcn_b200_device_status() == 0       # reading clears it
    assert L.tvdcn_b200_device_status_address() is not None
    # limits of the knob
    assert L.tvdcn_b200_selftest_bounded_wait(0, _stream()) != 0
    assert L.tvdcn_b200_selftest_bounded_wait(1 << 20, _stream()) != 0
    # the device still computes
    x = torch.arange(8, device='cuda', dtype=torch.float32)
    assert float((x * 2).sum()) == 56.0


def test_operators_raise_at_the_next_call_after_a_timed_out_wait():
    import tvdcn_b200
    from tvdcn_b200 import cabi
    L = cabi.lib()
    assert L.tvdcn_b200_device_status() == 0
    x = torch.randn(2, 8, 6, 6, device='cuda')
    w = torch.randn(4, 8, 3, 3, device='cuda')
    off = torch.randn(2, 18, 4, 4, device='cuda')
    good = tvdcn_b200.ops.deform_conv2d(x, w, off)
    torch.cuda.synchronize()

    cabi.check(L.tvdcn_b200_selftest_bounded_wait(8, _stream()))
    # this call's own kernels are fine; behind them the status word is copied to the host
    out = tvdcn_b200.ops.deform_conv2d(x, w, off)
    torch.cuda.synchronize()
    assert torch.equal(out, good)
    with pytest.raises(RuntimeError, match='gave up on a bounded wait .code 900'):
        tvdcn_b200.ops.deform_conv2d(x, w, off)
    # raised once, cleared: the next call works again
    assert L.tvdcn_b200_device_status() == 0
    out = tvdcn_b200.ops.deform_conv2d(x, w, off)
    torch.cuda.synchronize()
    assert torch.equal(out, good)
    assert L.tvdcn_b200_device_status() == 0
