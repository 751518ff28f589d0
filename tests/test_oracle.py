"""Pins the CPU oracle (oracle/restate.py) before anything is compared with it.

1. against the golden vectors the reference's own CPU kernels produced (tests/golden/*.pt);
2. live against the built reference (oracle/_ref) where that exists, on fresh seeds and extra shapes;
3. against torchvision.ops.deform_conv2d -- the check the reference's own test-suite makes
   (tests/test_compatibility_with_torchvision.py:8-65 in the tvdcn project);
4. explicit gradient formulas against torch.autograd of the restated forward;
5. both-None equals an ordinary (transposed) convolution (README.md:216 of the tvdcn project).
"""
import glob
import os

import pytest
import torch
import torch.nn.functional as F

import cases
from cases import Case, assert_parity, make_inputs, run_oracle
from oracle import build_ref, restate

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), 'golden', '*.pt')))


def test_golden_files_present():
    assert len(GOLDEN) == 30


@pytest.mark.parametrize('path', GOLDEN, ids=[os.path.basename(p)[:-3] for p in GOLDEN])
def test_restatement_matches_golden(path):
    blob = torch.load(path)
    case = Case(**{k: tuple(v) if isinstance(v, list) else v for k, v in blob['case'].items()})
    # the stored inputs are reproducible from the seed
    regenerated = make_inputs(case, blob['seed'])
    for a, b in zip(regenerated, blob['inputs']):
        assert (a is None) == (b is None)
        if a is not None:
            assert torch.equal(a, b)
    got = run_oracle(case, *blob['inputs'])
    assert_parity(got, blob['results'], 1e-12, case.name)


LIVE = [
    Case('live2d_border', 2, False, 2, 6, 4, (7, 5), (3, 3), (1, 1), (1, 1), (1, 1), (), 2, 3, 2, True, 3.0),
    Case('live2d_stride', 2, False, 1, 4, 4, (9, 8), (3, 2), (2, 3), (2, 0), (2, 1), (), 1, 1, 4, False, 0.5),
    Case('live1d', 1, False, 3, 8, 8, (17,), (5,), (1,), (4,), (2,), (), 4, 2, 1, True, 3.0),
    Case('live3d', 3, False, 1, 4, 2, (4, 5, 6), (2, 2, 3), (1, 1, 2), (1, 0, 1), (1, 2, 1), (), 1, 2, 2, True, 1.0),
    Case('live2dT', 2, True, 2, 6, 6, (4, 5), (4, 4), (2, 2), (1, 1), (1, 1), (1, 0), 2, 3, 1, True, 1.5),
    Case('live1dT', 1, True, 2, 6, 4, (9,), (3,), (3,), (1,), (2,), (2,), 2, 2, 2, True, 2.0),
    Case('live3dT', 3, True, 1, 4, 4, (3, 3, 4), (2, 3, 2), (2, 1, 2), (0, 1, 0), (1, 1, 2), (1, 0, 1), 1, 4, 1, False, 1.0),
]


@pytest.mark.parametrize('case', LIVE, ids=[c.name for c in LIVE])
def test_restatement_matches_reference_build(case):
    if not build_ref.load():
        pytest.skip('oracle/_ref not built (python oracle/build_ref.py)')
    inputs = make_inputs(case, seed=7)
    assert_parity(run_oracle(case, *inputs), cases.run_reference(case, *inputs), 1e-12, case.name)


def test_reference_build_matches_golden():
    """The live reference build reproduces the committed vectors (guards against a stale build)."""
    if not build_ref.load():
        pytest.skip('oracle/_ref not built')
    blob = torch.load(GOLDEN[0])
    case = Case(**{k: tuple(v) if isinstance(v, list) else v for k, v in blob['case'].items()})
    assert_parity(cases.run_reference(case, *blob['inputs']), blob['results'], 1e-14, case.name)


@pytest.mark.parametrize('with_mask', [True, False])
def test_torchvision_equivalence(with_mask):
    tv = pytest.importorskip('torchvision')
    case = cases.reference_fixture(2, False, True, with_mask, offset_groups=1, mask_groups=1)
    x, w, off, mask, bias, go = make_inputs(case, seed=12)
    leaves = [t.clone().requires_grad_(True) for t in (x, w, off, bias)]
    m = mask.clone().requires_grad_(True) if with_mask else None
    out = tv.ops.deform_conv2d(leaves[0], leaves[2], leaves[1], leaves[3], case.stride, case.padding,
                               case.dilation, m)
    out.backward(go)
    ref = (out.detach(), leaves[0].grad, leaves[1].grad, leaves[2].grad, m.grad if with_mask else None,
           leaves[3].grad)
    assert_parity(run_oracle(case, x, w, off, mask, bias, go), ref, 1e-12, 'torchvision')


@pytest.mark.parametrize('dim,transposed', [(1, False), (2, False), (3, False), (1, True), (2, True), (3, True)])
def test_explicit_gradients_match_autograd(dim, transposed):
    case = cases.reference_fixture(dim, transposed, True, True, groups=2, offset_groups=4, mask_groups=2, batch=1)
    x, w, off, mask, bias, go = make_inputs(case, seed=3)
    leaves = [t.clone().requires_grad_(True) for t in (x, w, off, mask, bias)]
    if not transposed:
        out = restate.deform_conv(*leaves, case.stride, case.padding, case.dilation, case.groups)
    else:
        out = restate.deform_conv_transpose(*leaves, case.stride, case.padding, case.opad, case.dilation,
                                            case.groups)
    out.backward(go)
    ref = (out.detach(),) + tuple(l.grad for l in leaves)
    assert_parity(run_oracle(case, x, w, off, mask, bias, go), ref, 1e-12, case.name)


@pytest.mark.parametrize('dim', [1, 2, 3])
def test_no_offset_no_mask_is_plain_convolution(dim):
    case = cases.reference_fixture(dim, False, False, False, groups=2)
    x, w, _, _, bias, go = make_inputs(case, seed=5)
    conv = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}[dim]
    ref = conv(x, w, bias, case.stride, case.padding, case.dilation, case.groups)
    assert cases.nerr(run_oracle(case, x, w, None, None, bias, go)[0], ref) < 1e-12
    caset = cases.reference_fixture(dim, True, False, False, groups=2)
    x, w, _, _, bias, go = make_inputs(caset, seed=5)
    convt = {1: F.conv_transpose1d, 2: F.conv_transpose2d, 3: F.conv_transpose3d}[dim]
    ref = convt(x, w, bias, caset.stride, caset.padding, caset.opad, caset.groups, caset.dilation)
    assert cases.nerr(run_oracle(caset, x, w, None, None, bias, go)[0], ref) < 1e-12


def test_boundary_semantics():
    """Samples exactly at -1 and at H contribute nothing; the derivative at -1 sees the valid corner
    (tvdcn/csrc/ops/cpu/deform_conv2d_common_kernels.cpp:33-34 versus :104-135)."""
    case = Case('edge', 1, False, 1, 1, 1, (4,), (1,), (1,), (0,), (1,), (), 1, 1, 0, False)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0]]], dtype=torch.float64)
    w = torch.ones(1, 1, 1, dtype=torch.float64)
    # positions: 0 + (-1) = -1 ; 1 + 3 = 4 (== H) ; 2 + 0.5 = 2.5 ; 3 - 0.25 = 2.75
    off = torch.tensor([[[-1.0, 3.0, 0.5, -0.25]]], dtype=torch.float64)
    go = torch.ones(1, 1, 4, dtype=torch.float64)
    out, gx, gw, goff, _, _ = run_oracle(case, x, w, off, None, None, go)
    assert torch.allclose(out, torch.tensor([[[0.0, 0.0, 3.5, 3.75]]], dtype=torch.float64))
    # d/dpos at -1: (-1)*invalid + (+1)*x[0] = 1 ; at 4: both corners out of range -> 0
    assert torch.allclose(goff, torch.tensor([[[1.0, 0.0, 1.0, 1.0]]], dtype=torch.float64))
    if build_ref.load():
        ref = cases.run_reference(case, x, w, off, None, None, go)
        assert torch.equal(ref[0], out) and torch.allclose(ref[3], goff)


def test_mask_softmax_restatement():
    g = torch.Generator().manual_seed(0)
    m = torch.randn(2, 18, 3, 4, generator=g, dtype=torch.float64, requires_grad=True)
    y = restate.mask_softmax(m, (3, 3))
    assert torch.allclose(y.view(2, 2, 9, 3, 4).sum(2), torch.ones(2, 2, 3, 4, dtype=torch.float64))
    gy = torch.randn(2, 18, 3, 4, generator=g, dtype=torch.float64)
    y.backward(gy)
    assert torch.allclose(restate.mask_softmax_backward(gy, y.detach(), (3, 3)), m.grad, atol=1e-14)
