"""Parity of the CUDA path with the CPU oracle, through the C ABI (ctypes -> libtvdcn_b200.so).

Tolerances (normalised max error, max|a-b| / max|ref|): 1e-4 for f32 and f64 as the task states (f64 is
held to 1e-10 here), 2e-2 for 16-bit inputs with f32 accumulation.
"""
import ctypes
import glob
import os

import pytest
import torch
import torch.nn.functional as F

import cases
from cases import Case, assert_parity, make_inputs, nerr, run_cabi, run_oracle

pytestmark = pytest.mark.gpu

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', '*.pt')))
ENGINES = {'simt': 1}


def cuda(ts, dtype=None):
    return tuple(None if t is None else t.to('cuda', dtype or t.dtype) for t in ts)


def load_golden(path):
    blob = torch.load(path)
    case = Case(**{k: tuple(v) if isinstance(v, list) else v for k, v in blob['case'].items()})
    return case, blob['inputs'], blob['results']


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[:-3] for p in GOLDEN])
def test_golden_f64(path):
    case, inputs, results = load_golden(path)
    assert_parity(run_cabi(case, *cuda(inputs)), results, 1e-10, case.name)


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[:-3] for p in GOLDEN])
def test_golden_f32(path):
    case, inputs, results = load_golden(path)
    assert_parity(run_cabi(case, *cuda(inputs, torch.float32)), results, 1e-4, case.name)


# Down-scaled versions of the five benchmark configurations (same operator, grouping and hyper-parameters).
SCALED = [
    Case('cfg1_small', 2, False, 2, 16, 16, (14, 14), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 1.5),
    Case('cfg2_small', 2, False, 3, 32, 32, (14, 14), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 4, 1, True, 2.0),
    Case('cfg3_small', 1, False, 2, 32, 32, (200,), (5,), (1,), (4,), (2,), (), 4, 4, 1, True, 3.0),
    Case('cfg4_small', 3, False, 1, 8, 8, (4, 10, 10), (3, 3, 3), (1, 1, 1), (1, 1, 1), (1, 1, 1), (), 1, 1, 1, True, 1.0),
    Case('cfg5_small', 2, True, 2, 16, 8, (8, 8), (4, 4), (2, 2), (1, 1), (1, 1), (), 1, 2, 1, True, 1.5),
    # ragged: nothing is a multiple of a tile extent
    Case('ragged2d', 2, False, 3, 5, 7, (9, 11), (3, 2), (2, 1), (1, 0), (1, 2), (), 1, 5, 1, True, 2.0),
    Case('ragged1dT', 1, True, 3, 6, 9, (13,), (3,), (2,), (1,), (1,), (1,), 3, 3, 3, False, 2.0),
    Case('far_offsets', 2, False, 2, 4, 4, (6, 6), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 2, 2, True, 50.0),
    Case('wide_channels', 2, False, 1, 96, 80, (6, 5), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 3, 2, True, 1.0),
]


@pytest.mark.parametrize('case', SCALED, ids=[c.name for c in SCALED])
def test_scaled_f32(case):
    inputs = make_inputs(case, seed=11)
    ref = run_oracle(case, *inputs)
    assert_parity(run_cabi(case, *cuda(inputs, torch.float32)), ref, 1e-4, case.name)


@pytest.mark.parametrize('case', SCALED[:5], ids=[c.name for c in SCALED[:5]])
@pytest.mark.parametrize('dtype', [torch.bfloat16, torch.float16], ids=['bf16', 'f16'])
@pytest.mark.parametrize('aux_f32', [True, False], ids=['aux32', 'aux16'])
def test_scaled_16bit(case, dtype, aux_f32):
    x, w, off, mask, bias, go = make_inputs(case, seed=12)
    aux = torch.float32 if aux_f32 else dtype
    q = lambda t, d: None if t is None else t.to(d)
    dev_in = (q(x, dtype), q(w, dtype), q(off, aux), q(mask, aux), q(bias, aux), q(go, dtype))
    # the oracle sees exactly the rounded inputs, so only the arithmetic is compared
    ref = run_oracle(case, *(None if t is None else t.double() for t in dev_in))
    assert_parity(run_cabi(case, *cuda(dev_in)), ref, 2e-2, f'{case.name}/{dtype}')


def test_exact_boundary_offsets():
    case = Case('edge', 1, False, 1, 1, 1, (4,), (1,), (1,), (0,), (1,), (), 1, 1, 0, False)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]])
    w = torch.ones(1, 1, 1)
    off = torch.tensor([[[-1.0, 3.0, 0.5, -0.25]]])
    go = torch.ones(1, 1, 4)
    out, gx, gw, goff, _, _ = run_cabi(case, *cuda((x, w, off, None, None, go)))
    assert torch.equal(out.cpu(), torch.tensor([[[0.0, 0.0, 3.5, 3.75]]]))
    assert torch.equal(goff.cpu(), torch.tensor([[[1.0, 0.0, 1.0, 1.0]]]))
    assert torch.equal(gx.cpu(), torch.tensor([[[0.0, 0.0, 0.75, 1.25]]]))


def test_empty_batch():
    case = Case('empty', 2, False, 0, 4, 4, (6, 6), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True)
    inputs = cuda(make_inputs(case, seed=1, dtype=torch.float32))
    out, gx, gw, goff, gmask, gb = run_cabi(case, *inputs, poison=True)
    assert out.numel() == 0 and gx.numel() == 0
    assert torch.count_nonzero(gw) == 0 and torch.count_nonzero(gb) == 0


def test_backward_skips_null_gradients():
    from tvdcn_b200 import cabi
    case = SCALED[0]
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=2, dtype=torch.float32))
    L = cabi.lib()
    p = cases.cabi_problem(case, torch.float32)
    gw = torch.full_like(w, float('nan'))
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    cabi.check(L.tvdcn_b200_deform_conv_backward(ctypes.byref(p), vp(go), vp(x), vp(w), vp(off), vp(mask), None,
                                                 vp(gw), None, None, None, None, 0,
                                                 ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)))
    torch.cuda.synchronize()
    full = run_cabi(case, x, w, off, mask, bias, go)
    assert nerr(gw, full[2]) < 1e-5


def test_repeatability():
    """Atomics reorder sums; two runs must still agree to rounding (the reference tests with nondet_tol=1e-5)."""
    case = SCALED[1]
    inputs = cuda(make_inputs(case, seed=3, dtype=torch.float32))
    a = run_cabi(case, *inputs)
    b = run_cabi(case, *inputs)
    assert torch.equal(a[0], b[0])
    for u, v in zip(a[1:], b[1:]):
        assert nerr(u, v) < 1e-5


# ---- size-independent properties at the benchmark's full sizes -------------------------------------
def test_full_size_zero_offset_equals_convolution():
    """deform_conv2d N=128 256->256 28x28: with zero offsets and a unit mask the operator is an ordinary
    convolution, forward and backward (checked against cuDNN in f32, TF32 off)."""
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    case = Case('cfg2_full', 2, False, 128, 256, 256, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 4, 1, True)
    g = torch.Generator(device='cuda').manual_seed(5)
    x = torch.randn(128, 256, 28, 28, device='cuda', generator=g)
    w = torch.randn(256, 256, 3, 3, device='cuda', generator=g) * 0.02
    bias = torch.randn(256, device='cuda', generator=g) * 0.1
    off = torch.zeros(128, 72, 28, 28, device='cuda')
    mask = torch.ones(128, 9, 28, 28, device='cuda')
    go = torch.randn(128, 256, 28, 28, device='cuda', generator=g)
    out, gx, gw, goff, gmask, gb = run_cabi(case, x, w, off, mask, bias, go, poison=False)
    xr, wr, br = x.clone().requires_grad_(True), w.clone().requires_grad_(True), bias.clone().requires_grad_(True)
    ref = F.conv2d(xr, wr, br, 1, 1)
    ref.backward(go)
    assert nerr(out, ref) < 1e-4
    assert nerr(gx, xr.grad) < 1e-4
    assert nerr(gw, wr.grad) < 1e-4
    assert nerr(gb, br.grad) < 1e-4
    # grad_mask[b, tap, p] = sum_c G * x shifted; its total equals <grad_out, conv without bias>
    total = (go * (ref.detach() - bias.view(1, -1, 1, 1))).sum().double()
    assert abs(gmask.double().sum() - total) / abs(total) < 1e-3


def test_full_size_linearity_transposed():
    """deform_conv_transpose2d N=64 256->128 32x32->64x64: the output is linear in the input and
    grad_bias is the plain sum of grad_output."""
    case = Case('cfg5_full', 2, True, 64, 256, 128, (32, 32), (4, 4), (2, 2), (1, 1), (1, 1), (), 1, 2, 1, False)
    g = torch.Generator(device='cuda').manual_seed(6)
    x1 = torch.randn(64, 256, 32, 32, device='cuda', generator=g)
    x2 = torch.randn(64, 256, 32, 32, device='cuda', generator=g)
    w = torch.randn(256, 128, 4, 4, device='cuda', generator=g) * 0.02
    off = torch.randn(64, 64, 32, 32, device='cuda', generator=g) * 1.5
    mask = torch.rand(64, 16, 32, 32, device='cuda', generator=g)
    go = torch.randn(64, 128, 64, 64, device='cuda', generator=g)
    o1 = run_cabi(case, x1, w, off, mask, None, go, poison=False)[0]
    o2 = run_cabi(case, x2, w, off, mask, None, go, poison=False)[0]
    o12 = run_cabi(case, x1 + 2 * x2, w, off, mask, None, go, poison=False)[0]
    assert nerr(o12, o1 + 2 * o2) < 1e-4


# ---- mask softmax ------------------------------------------------------------------------------------
@pytest.mark.parametrize('taps,spatial', [(9, (28, 28)), (27, (3, 5, 7)), (5, (4096,)), (16, (6, 6)), (40, (5, 3)),
                                          (9, (7, 3))])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64, torch.bfloat16])
def test_mask_softmax(taps, spatial, dtype):
    from tvdcn_b200 import cabi
    L = cabi.lib()
    g = torch.Generator().manual_seed(taps)
    B, MG = 3, 2
    logits = torch.randn(B, MG * taps, *spatial, generator=g, dtype=torch.float64).to(dtype)
    gy = torch.randn(B, MG * taps, *spatial, generator=g, dtype=torch.float64).to(dtype)
    ref_in = logits.double().requires_grad_(True)
    ref = torch.softmax(ref_in.view(B, MG, taps, -1), 2).view_as(ref_in)
    ref.backward(gy.double())
    x, gyd = logits.cuda(), gy.cuda()
    y = torch.full_like(x, float('nan'))
    gx = torch.full_like(x, float('nan'))
    sp = 1
    for s in spatial:
        sp *= s
    dt = cases._DT[dtype]
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    cabi.check(L.tvdcn_b200_mask_softmax_forward(dt, B, MG, taps, sp, vp(x), vp(y), st))
    cabi.check(L.tvdcn_b200_mask_softmax_backward(dt, B, MG, taps, sp, vp(gyd), vp(y), vp(gx), st))
    torch.cuda.synchronize()
    tol = 1e-2 if dtype == torch.bfloat16 else (1e-12 if dtype == torch.float64 else 1e-5)
    assert nerr(y, ref) < tol
    # backward is checked against the formula applied to the kernel's own (rounded) forward result
    yd = y.double().cpu().view(B, MG, taps, -1)
    gd = gy.double().view(B, MG, taps, -1)
    gref = (yd * (gd - (gd * yd).sum(2, keepdim=True))).view_as(ref)
    assert nerr(gx, gref) < tol
    assert torch.allclose(y.double().view(B, MG, taps, -1).sum(2).cpu(), torch.ones(B, MG, sp, dtype=torch.float64),
                          atol=5e-2 if dtype == torch.bfloat16 else 1e-5)
