"""The torch.ops.tvdcn.* operators and the nn.Module wrappers on a CUDA device: autograd, optional
tensors, unbatched / non-contiguous inputs, autocast, error behaviour."""
import pytest
import torch
import torch.nn.functional as F

import cases
from cases import Case, assert_parity, make_inputs, nerr, run_oracle
import tvdcn_b200 as tvdcn
from tvdcn_b200 import ops

pytestmark = pytest.mark.gpu


def op_fwd_bwd(case, x, w, off, mask, bias, go):
    leaves = [None if t is None else t.clone().requires_grad_(True) for t in (x, w, off, mask, bias)]
    if not case.transposed:
        f = getattr(ops, f'deform_conv{case.dim}d')
        out = f(*leaves, case.stride, case.padding, case.dilation, case.groups)
    else:
        f = getattr(ops, f'deform_conv_transpose{case.dim}d')
        out = f(*leaves, case.stride, case.padding, case.opad, case.dilation, case.groups)
    out.backward(go)
    return (out.detach(),) + tuple(None if l is None else l.grad for l in leaves)


def cuda(ts, dtype=None):
    return tuple(None if t is None else t.to('cuda', dtype or t.dtype) for t in ts)


ALL = [cases.reference_fixture(d, t, o, m, groups=2, offset_groups=4, mask_groups=2)
       for d in (1, 2, 3) for t in (False, True) for (o, m) in ((True, True), (True, False), (False, True),
                                                                (False, False))]


@pytest.mark.parametrize('case', ALL, ids=[c.name for c in ALL])
def test_autograd_matches_oracle_f64(case):
    inputs = make_inputs(case, seed=21)
    assert_parity(op_fwd_bwd(case, *cuda(inputs)), run_oracle(case, *inputs), 1e-10, case.name)


@pytest.mark.parametrize('dim,tr', [(1, False), (2, False), (3, False), (1, True), (2, True), (3, True)])
def test_gradcheck(dim, tr):
    """fp64 numerical-vs-analytic gradients, as tests/test_grad.py:8-81 of the tvdcn project does."""
    case = cases.reference_fixture(dim, tr, True, True, batch=1)
    x, w, off, mask, bias, _ = cuda(make_inputs(case, seed=22))
    # keep sample points away from integer coordinates, where the interpolant has a kink
    off = (off * 0.2).round() + 0.37
    leaves = [t.clone().requires_grad_(True) for t in (x, w, off, mask, bias)]
    if not tr:
        fn = lambda *a: getattr(ops, f'deform_conv{dim}d')(*a, case.stride, case.padding, case.dilation, 1)
    else:
        fn = lambda *a: getattr(ops, f'deform_conv_transpose{dim}d')(*a, case.stride, case.padding, case.opad,
                                                                     case.dilation, 1)
    assert torch.autograd.gradcheck(fn, leaves, nondet_tol=1e-5, eps=1e-6, atol=1e-6, rtol=1e-4)


def test_torchvision_equivalence_on_cuda():
    tv = pytest.importorskip('torchvision')
    case = cases.reference_fixture(2, False, True, True, offset_groups=1, mask_groups=1)
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=12))
    got = op_fwd_bwd(case, x, w, off, mask, bias, go)
    leaves = [t.clone().requires_grad_(True) for t in (x, w, off, mask, bias)]
    try:
        out = tv.ops.deform_conv2d(leaves[0], leaves[2], leaves[1], leaves[4], case.stride, case.padding,
                                   case.dilation, leaves[3])
    except (RuntimeError, NotImplementedError) as e:  # torchvision built without its CUDA ops
        pytest.skip(f'torchvision CUDA op unavailable: {e}')
    out.backward(go)
    assert_parity(got, (out.detach(),) + tuple(l.grad for l in leaves), 1e-10, 'torchvision')


def test_unbatched_and_noncontiguous():
    case = cases.reference_fixture(2, False, True, True, batch=1)
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=23))
    ref = op_fwd_bwd(case, x, w, off, mask, bias, go)
    got = op_fwd_bwd(case, x[0], w, off[0], mask[0], bias, go[0])
    for a, b in zip(got, ref):
        assert nerr(a.reshape(b.shape) if a.dim() != b.dim() else a, b) < 1e-12
    assert got[0].dim() == 3 and got[1].dim() == 3 and got[3].dim() == 3
    # permuted storage
    nc = lambda t: t.transpose(-1, -2).contiguous().transpose(-1, -2)
    got = op_fwd_bwd(case, nc(x), nc(w), nc(off), nc(mask), bias, nc(go))
    assert not nc(x).is_contiguous()
    assert_parity(got, ref, 1e-12, 'non-contiguous')


def test_absent_tensors_give_none_gradients():
    case = cases.reference_fixture(2, False, False, False)
    x, w, _, _, _, go = cuda(make_inputs(case, seed=24))
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    out = ops.deform_conv2d(xr, wr, None, None, None, case.stride, case.padding, case.dilation)
    out.backward(go)
    ref = F.conv2d(x, w, None, case.stride, case.padding, case.dilation)
    assert nerr(out, ref) < 1e-12
    grads = torch.ops.tvdcn._deform_conv2d_backward(go, x, w, None, None, None, list(case.stride),
                                                   list(case.padding), list(case.dilation), 1)
    assert grads[2] is None and grads[3] is None and grads[4] is None


def test_double_backward_raises():
    case = cases.reference_fixture(2, False, True, True)
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=25))
    xr = x.clone().requires_grad_(True)
    out = ops.deform_conv2d(xr, w, off, mask, bias, case.stride, case.padding, case.dilation)
    (g,) = torch.autograd.grad(out, xr, go, create_graph=True)
    with pytest.raises(RuntimeError, match='double backwards'):
        g.sum().backward()


def test_error_messages():
    x = torch.randn(2, 4, 8, 8, device='cuda')
    w = torch.randn(4, 4, 3, 3, device='cuda')
    with pytest.raises(RuntimeError, match='offset.shape\\[1\\] is not valid|multiple of'):
        ops.deform_conv2d(x, w, torch.randn(2, 17, 6, 6, device='cuda'))
    with pytest.raises(RuntimeError, match='computed output dims'):
        ops.deform_conv2d(x, w, torch.randn(2, 18, 5, 6, device='cuda'))
    with pytest.raises(RuntimeError, match='invalid batch size of mask'):
        ops.deform_conv2d(x, w, None, torch.rand(1, 9, 6, 6, device='cuda'))
    with pytest.raises(RuntimeError, match='same type'):
        ops.deform_conv2d(x, w.double())
    with pytest.raises(RuntimeError, match='Expected a sequence of 2'):
        torch.ops.tvdcn.deform_conv2d(x, w, None, None, None, [1, 1, 1], [0, 0], [1, 1], 1)
    with pytest.raises(RuntimeError, match='too small'):
        ops.deform_conv2d(x[:, :, :2, :2], w)
    with pytest.raises(RuntimeError, match='same device'):
        ops.deform_conv2d(x, w.cpu())


def test_mixed_precision_and_autocast():
    case = Case('amp', 2, False, 2, 16, 16, (10, 10), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 2, 1, True, 1.5)
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=26, dtype=torch.float32))
    ref = op_fwd_bwd(case, x, w, off, mask, bias, go)
    # bf16 input / weight, f32 offset / mask / bias
    got = op_fwd_bwd(case, x.bfloat16(), w.bfloat16(), off, mask, bias, go.bfloat16())
    assert got[0].dtype == torch.bfloat16 and got[3].dtype == torch.float32
    assert_parity(got, ref, 2e-2, 'bf16 in/weight')
    with torch.autocast('cuda', dtype=torch.bfloat16):
        out = ops.deform_conv2d(x, w, off, mask, bias, case.stride, case.padding, case.dilation)
    assert out.dtype == torch.bfloat16 and nerr(out, ref[0]) < 2e-2


@pytest.mark.parametrize('dim', [1, 2, 3])
def test_packed_modules_train_step(dim):
    torch.manual_seed(0)
    torch.backends.cudnn.allow_tf32 = False  # the cuDNN convolutions below are the f32 yardstick
    torch.backends.cuda.matmul.allow_tf32 = False
    size = (12,) * dim
    m = getattr(ops, f'PackedDeformConv{dim}d')(8, 8, 3, padding=1, offset_groups=2, mask_groups=2, modulated=True,
                                                mask_activation='softmax').cuda()
    x = torch.randn(2, 8, *size, device='cuda')
    conv = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[dim]
    # zero-initialised generators: offsets are 0 and the softmax mask is 1 / taps
    assert nerr(m(x), conv(x, m.weight / 3 ** dim, None, 1, 1) * 1.0 + m.bias.view(1, -1, *([1] * dim))) < 1e-4
    torch.nn.init.normal_(m.offset_generator.weight, std=0.1)
    torch.nn.init.normal_(m.mask_generator.weight, std=0.1)
    m(x).square().mean().backward()
    for n, p in m.named_parameters():
        assert p.grad is not None and torch.isfinite(p.grad).all() and p.grad.abs().sum() > 0, n
    t = getattr(ops, f'PackedDeformConvTranspose{dim}d')(8, 4, 3, stride=2, padding=1, offset_groups=2,
                                                         modulated=True).cuda()
    y = t(x, output_size=[24] * dim)
    assert y.shape == (2, 4) + (24,) * dim
    convt = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[dim]
    assert nerr(y, convt(x, t.weight, t.bias, 2, 1, 1)) < 1e-4  # zero offsets, mask = 2 * sigmoid(0) = 1
    y.mean().backward()
    assert t.weight.grad.abs().sum() > 0


def test_reflect_padding_mode():
    m = ops.DeformConv2d(4, 4, 3, padding=1, padding_mode='reflect').cuda().double()
    x = torch.randn(1, 4, 6, 6, device='cuda', dtype=torch.float64)
    off = torch.zeros(1, 18, 6, 6, device='cuda', dtype=torch.float64)
    ref = F.conv2d(F.pad(x, (1, 1, 1, 1), mode='reflect'), m.weight, m.bias)
    assert nerr(m(x, off), ref) < 1e-12


def test_mask_softmax_operator_autograd():
    m = torch.randn(2, 18, 5, 6, device='cuda', dtype=torch.float64, requires_grad=True)
    y = ops.mask_softmax2d(m, (3, 3))
    gy = torch.randn_like(y)
    y.backward(gy)
    mr = m.detach().clone().requires_grad_(True)
    yr = torch.softmax(mr.view(2, 2, 9, 5, 6), 2).view(2, 18, 5, 6)
    yr.backward(gy)
    assert nerr(y, yr) < 1e-12 and nerr(m.grad, mr.grad) < 1e-12
    assert torch.autograd.gradcheck(lambda t: ops.mask_softmax1d(t, (5,)),
                                    [torch.randn(1, 10, 7, device='cuda', dtype=torch.float64, requires_grad=True)])


def test_current_stream_is_used():
    case = cases.reference_fixture(2, False, True, True)
    x, w, off, mask, bias, go = cuda(make_inputs(case, seed=27))
    ref = ops.deform_conv2d(x, w, off, mask, bias, case.stride, case.padding, case.dilation)
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        out = ops.deform_conv2d(x, w, off, mask, bias, case.stride, case.padding, case.dilation)
    s.synchronize()
    assert torch.equal(out, ref)
    before = torch.ops.tvdcn._launch_count()
    ops.deform_conv2d(x, w, off, mask, bias, case.stride, case.padding, case.dilation)
    assert torch.ops.tvdcn._launch_count() > before


@pytest.mark.parametrize('dim', [1, 2, 3])
def test_scripted_modules_run_like_eager(dim):
    """torch.jit.script of the packed modules (conv and transposed): same output and gradients as eager."""
    torch.manual_seed(3)
    size = (9, 8, 7)[:dim]
    for name, kw in ((f'PackedDeformConv{dim}d', dict(padding=1)), (f'PackedDeformConvTranspose{dim}d', dict(stride=2))):
        m = getattr(ops, name)(4, 6, 3, modulated=True, mask_activation='softmax', offset_groups=2, **kw).cuda()
        for gen in (m.offset_generator, m.mask_generator):
            torch.nn.init.normal_(gen.weight, std=0.3)
        sm = torch.jit.script(m)
        x = torch.randn(2, 4, *size, device='cuda', requires_grad=True)
        y0 = m(x)
        g0, = torch.autograd.grad(y0.square().sum(), x)
        y1 = sm(x)
        g1, = torch.autograd.grad(y1.square().sum(), x)
        assert nerr(y1, y0) < 1e-6 and nerr(g1, g0) < 1e-5, name
