"""Tensor-core (tcgen05) kernels against the CPU oracle, through the C ABI.  Shapes here satisfy the
64-channel granularity the tensor path needs; ENGINE_TENSOR makes the call fail instead of silently
using the SIMT kernels, and the device status word must stay clean (no bounded wait ran out)."""
import ctypes

import pytest
import torch

import cases
from cases import Case, make_inputs, nerr, run_cabi, run_oracle

pytestmark = pytest.mark.gpu

TC_CASES = [
    Case('tc2d_c64', 2, False, 3, 64, 64, (10, 10), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 1.5),
    Case('tc2d_c128_256', 2, False, 2, 128, 256, (8, 7), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 2, 1, True, 2.0),
    Case('tc2d_groups', 2, False, 2, 128, 128, (8, 8), (3, 2), (2, 1), (1, 0), (1, 2), (), 2, 2, 2, True, 1.0),
    Case('tc2d_plain', 2, False, 2, 64, 64, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 0, 0, False, 1.0),
    Case('tc2d_nomask', 2, False, 2, 64, 128, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 0, True, 1.0),
    Case('tc1d', 1, False, 2, 128, 128, (304,), (5,), (1,), (4,), (2,), (), 2, 2, 1, True, 3.0),
    Case('tc3d', 3, False, 1, 64, 64, (4, 6, 6), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (), 1, 1, 1, True, 1.0),
]


def forward_tensor(case, x, w, off, mask, bias):
    from tvdcn_b200 import cabi
    L = cabi.lib()
    L.tvdcn_b200_device_status.restype = ctypes.c_int
    aux = torch.float32
    p = cases.cabi_problem(case, x.dtype, aux, cabi.ENGINE_TENSOR)
    assert L.tvdcn_b200_engine_name(ctypes.byref(p), 0) == b'tcgen05'
    out = torch.full((case.batch, case.out_channels, *case.out_size), float('nan'), dtype=x.dtype, device='cuda')
    n = L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(p))
    ws = torch.empty(max(n, 1), dtype=torch.uint8, device='cuda')
    vp = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    cabi.check(L.tvdcn_b200_deform_conv_forward(ctypes.byref(p), vp(x), vp(w), vp(off), vp(mask), vp(bias), vp(out),
                                                vp(ws), ws.numel(),
                                                ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    assert L.tvdcn_b200_device_status() == 0
    return out


@pytest.mark.parametrize('case', TC_CASES, ids=[c.name for c in TC_CASES])
@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 2e-2), (torch.float16, 5e-3)],
                         ids=['f32split', 'bf16', 'f16'])
def test_forward_tensor(case, dtype, tol):
    x, w, off, mask, bias, go = make_inputs(case, seed=41)
    q = lambda t, d: None if t is None else t.to(d)
    dev = (q(x, dtype), q(w, dtype), q(off, torch.float32), q(mask, torch.float32), q(bias, torch.float32))
    ref = run_oracle(case, *(None if t is None else t.double() for t in dev), go)[0]
    got = forward_tensor(case, *(None if t is None else t.cuda() for t in dev))
    e = nerr(got, ref)
    assert e <= tol, f'{case.name}: normalised max error {e:.3e}'


def kernels_launched(fn):
    """Runs fn() with per-kernel timing on and returns ({kernel name: launches}, fn's result)."""
    from tvdcn_b200 import cabi
    L = cabi.lib()
    L.tvdcn_b200_timing_enable.argtypes = [ctypes.c_int]
    L.tvdcn_b200_timing_report.argtypes = [ctypes.c_char_p, ctypes.c_size_t]
    L.tvdcn_b200_timing_report.restype = ctypes.c_size_t
    buf = ctypes.create_string_buffer(1 << 14)
    L.tvdcn_b200_timing_report(buf, len(buf))  # drop anything recorded earlier
    L.tvdcn_b200_timing_enable(1)
    try:
        out = fn()
        torch.cuda.synchronize()
    finally:
        L.tvdcn_b200_timing_enable(0)
    L.tvdcn_b200_timing_report(buf, len(buf))
    names = {}
    for line in buf.value.decode().splitlines():
        n, c, _ = line.split()
        names[n] = int(c)
    return names, out


@pytest.mark.parametrize('case', TC_CASES, ids=[c.name for c in TC_CASES])
@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)], ids=['f32split', 'bf16'])
def test_forward_backward_all_tensor(case, dtype, tol):
    x, w, off, mask, bias, go = make_inputs(case, seed=43)
    q = lambda t, d: None if t is None else t.to(d)
    dev = (q(x, dtype), q(w, dtype), q(off, torch.float32), q(mask, torch.float32), q(bias, torch.float32),
           q(go, dtype))
    ref = run_oracle(case, *(None if t is None else t.double() for t in dev))
    names, got = kernels_launched(lambda: cases.run_cabi(case, *(None if t is None else t.cuda() for t in dev)))
    assert names.get('dcn_fwd_tc', 0) == 1 and names.get('dcn_dgrad_tc', 0) == 1, names
    assert 'sample_gemm' not in names and 'gemm_scatter' not in names, names
    import math
    if math.prod(case.out_size) % 8 == 0:  # row pitch of grad_output must be TMA-loadable
        assert names.get('dcn_wgrad_tc', 0) == 1 and 'sample_wgrad' not in names, names
    cases.assert_parity(got, ref, tol, case.name)
    from tvdcn_b200 import cabi
    assert cabi.lib().tvdcn_b200_device_status() == 0


@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 2e-2)], ids=['f32split', 'bf16'])
def test_transposed_all_tensor(dtype, tol):
    case = Case('tcT', 2, True, 2, 128, 64, (6, 8), (4, 4), (2, 2), (1, 1), (1, 1), (1, 0), 1, 1, 1, True, 1.5)
    x, w, off, mask, bias, go = make_inputs(case, seed=44)
    q = lambda t, d: None if t is None else t.to(d)
    dev = (q(x, dtype), q(w, dtype), q(off, torch.float32), q(mask, torch.float32), q(bias, torch.float32),
           q(go, dtype))
    ref = run_oracle(case, *(None if t is None else t.double() for t in dev))
    names, got = kernels_launched(lambda: cases.run_cabi(case, *(None if t is None else t.cuda() for t in dev)))
    # forward scatter + backward coordinate gradients, grad_input as sample -> GEMM, sampled weight gradient
    assert names.get('dcn_dgrad_tc', 0) == 2 and names.get('dcn_fwd_tc', 0) == 1 and names.get('dcn_wgrad_tc', 0) == 1, names
    cases.assert_parity(got, ref, tol, case.name)
    from tvdcn_b200 import cabi
    assert cabi.lib().tvdcn_b200_device_status() == 0


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16], ids=['f32split', 'bf16'])
def test_non_finite_pixel_does_not_leak_through_out_of_image_corners(dtype):
    """An Inf at pixel 0 of the image must reach only the results that sample that pixel, as in the reference,
    which never reads an out-of-image corner: the tensor-core kernels read a row of zeros there instead of
    multiplying whatever pixel 0 holds by a zero weight."""
    from oracle import build_ref
    if not build_ref.load():
        pytest.skip('oracle/_ref is not built')
    case = Case('inf_pixel', 2, False, 2, 64, 64, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 3.0)
    x, w, off, mask, bias, go = make_inputs(case, seed=9, dtype=torch.float32)
    x[0, :, 0, 0] = float('inf')
    q = lambda t: t.to(dtype)
    ref = cases.run_reference(case, q(x).float(), q(w).float(), off, mask, bias, q(go).float())
    got = run_cabi(case, q(x).cuda(), q(w).cuda(), off.cuda(), mask.cuda(), bias.cuda(), q(go).cuda(),
                   engine=2)
    tol = 1e-4 if dtype == torch.float32 else 2e-2
    for name, a, r in zip(cases.NAMES, got, ref):
        a = a.float().cpu()
        fin = torch.isfinite(r)
        assert fin.any(), name
        assert torch.equal(torch.isfinite(a), fin), f'{name}: non-finite values in different places'
        scale = float(r[fin].abs().max())
        err = float((a[fin] - r[fin]).abs().max()) / max(scale, 1e-30)
        assert err <= tol, f'{name}: {err:.3e}'


@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16], ids=['f32split', 'bf16'])
def test_backward_reuses_the_forward_staging(dtype):
    """TVDCN_FLAG_REUSE_STAGED_INPUT: a backward call on the forward call's workspace gives the same gradients as
    one that stages the input itself, with one launch less."""
    from tvdcn_b200 import cabi
    L = cabi.lib()
    case = Case('reuse', 2, False, 3, 128, 64, (9, 10), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 2, 1, True, 1.5)
    x, w, off, mask, bias, go = (None if t is None else t.cuda() for t in make_inputs(case, seed=5, dtype=torch.float32))
    x, w, go = x.to(dtype), w.to(dtype), go.to(dtype)
    p = cases.cabi_problem(case, dtype, torch.float32, cabi.ENGINE_TENSOR)
    q = cabi.Problem.from_buffer_copy(p)
    q.flags = cabi.FLAG_REUSE_STAGED_INPUT
    n = max(L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(p)), L.tvdcn_b200_backward_workspace_bytes(ctypes.byref(p)))
    ws = torch.empty(n, dtype=torch.uint8, device='cuda')
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.empty(case.batch, case.out_channels, *case.out_size, dtype=dtype, device='cuda')

    def backward(prob):
        g = [torch.full_like(t, float('nan')) for t in (x, w, off, mask, bias)]
        cabi.check(L.tvdcn_b200_deform_conv_backward(ctypes.byref(prob), vp(go), vp(x), vp(w), vp(off), vp(mask),
                                                     vp(g[0]), vp(g[1]), vp(g[2]), vp(g[3]), vp(g[4]), vp(ws), n, st))
        return g

    base = backward(p)                       # stages the input itself
    ws.fill_(0xff)                           # nothing useful left in the workspace
    cabi.check(L.tvdcn_b200_deform_conv_forward(ctypes.byref(p), vp(x), vp(w), vp(off), vp(mask), vp(bias), vp(out),
                                                vp(ws), n, st))
    names, got = kernels_launched(lambda: backward(q))
    # the input staging was reused, and grad_output is read in the caller's layout: nothing is re-laid out
    assert names.get('to_channels_last', 0) == 0, names
    # same arithmetic, but the f32 atomics land in another order: a bf16 result may round the other way
    tol = 1e-5 if dtype == torch.float32 else 4e-3
    for a, b in zip(got, base):
        assert torch.isfinite(a.float()).all()
        assert nerr(a, b) < tol
    assert L.tvdcn_b200_device_status() == 0


def test_misaligned_16bit_grad_output_still_computes():
    """A contiguous bf16 grad_output whose storage offset leaves it off a 16-byte boundary cannot be read by TMA:
    the weight gradient must fall back to the SIMT kernel instead of failing the whole backward call."""
    case = Case('misaligned', 2, False, 2, 64, 64, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 1.0)
    x, w, off, mask, bias, go = make_inputs(case, seed=47)
    dev = [x.bfloat16().cuda(), w.bfloat16().cuda(), off.float().cuda(), mask.float().cuda(), bias.float().cuda()]
    go16 = go.bfloat16()
    base = torch.empty(go16.numel() + 1, dtype=torch.bfloat16, device='cuda')
    go_dev = base[1:].view(go16.shape)
    go_dev.copy_(go16)
    assert go_dev.data_ptr() % 16 != 0 and go_dev.is_contiguous()
    ref = run_oracle(case, *(t.double().cpu() for t in dev), go16.double())
    names, got = kernels_launched(lambda: cases.run_cabi(case, *dev, go_dev))
    assert names.get('sample_wgrad', 0) == 1 and 'dcn_wgrad_tc' not in names, names
    assert names.get('dcn_dgrad_tc', 0) == 1, names
    cases.assert_parity(got, ref, 2e-2, case.name)


@pytest.mark.parametrize('shift', [0, 1], ids=['aligned', 'off_16_bytes'])
def test_f32_bias_gradient_comes_from_the_split_pass(shift):
    """f32 data, conv: grad_bias is taken in the pass that splits grad_output into bf16 parts (no channel_sum
    launch) when grad_output allows 16-byte loads; a grad_output that starts 4 bytes off such a boundary takes the
    plain split and the separate sum.  Both must match the oracle."""
    case = Case('bias_in_split', 2, False, 3, 64, 64, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 1.0)
    x, w, off, mask, bias, go = make_inputs(case, seed=53)
    dev = [x.float().cuda(), w.float().cuda(), off.float().cuda(), mask.float().cuda(), bias.float().cuda()]
    base = torch.empty(go.numel() + 4, dtype=torch.float32, device='cuda')
    go_dev = base[shift:shift + go.numel()].view(go.shape)
    go_dev.copy_(go.float())
    assert go_dev.is_contiguous() and (go_dev.data_ptr() % 16 != 0) == bool(shift)
    ref = run_oracle(case, *(t.double().cpu() for t in dev), go.double())
    names, got = kernels_launched(lambda: cases.run_cabi(case, *dev, go_dev))
    assert names.get('dcn_wgrad_tc', 0) == 1, names
    if shift:
        assert names.get('split_f32', 0) == 1 and names.get('channel_sum', 0) == 1, names
    else:
        assert names.get('split_f32_channel_sum', 0) == 1 and 'channel_sum' not in names, names
    cases.assert_parity(got, ref, 1e-4, case.name)
