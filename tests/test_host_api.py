"""CPU-only checks of the Python surface: names, module construction, error behaviour, no CPU fallback."""
import pytest
import torch

import tvdcn_b200 as tvdcn
from tvdcn_b200 import ops

REFERENCE_NAMES = [
    'deform_conv1d', 'deform_conv2d', 'deform_conv3d', 'DeformConv1d', 'DeformConv2d', 'DeformConv3d',
    'PackedDeformConv1d', 'PackedDeformConv2d', 'PackedDeformConv3d',
    'deform_conv_transpose1d', 'deform_conv_transpose2d', 'deform_conv_transpose3d',
    'DeformConvTranspose1d', 'DeformConvTranspose2d', 'DeformConvTranspose3d',
    'PackedDeformConvTranspose1d', 'PackedDeformConvTranspose2d', 'PackedDeformConvTranspose3d',
    'mask_softmax1d', 'mask_softmax2d', 'mask_softmax3d', 'MaskSoftmax1d', 'MaskSoftmax2d', 'MaskSoftmax3d',
    'mask_sigmoid', 'MaskSigmoid',
]


def test_public_names():
    for n in REFERENCE_NAMES:
        assert hasattr(ops, n) and hasattr(tvdcn, n), n
    assert tvdcn.has_ops() and tvdcn.with_cuda()
    assert tvdcn.cuda_version() >= 12000
    assert tvdcn.cuda_arch_list() == ['sm_100a']


def test_schemas_are_the_reference_ones():
    s = str(torch.ops.tvdcn.deform_conv2d.default._schema)
    assert s == ('tvdcn::deform_conv2d(Tensor input, Tensor weight, Tensor? offset=None, Tensor? mask=None, '
                 'Tensor? bias=None, SymInt[2] stride=[1, 1], SymInt[2] padding=[0, 0], SymInt[2] dilation=[1, 1], '
                 'SymInt groups=1) -> Tensor')
    s = str(torch.ops.tvdcn._deform_conv_transpose1d_backward.default._schema)
    assert 'SymInt[1] output_padding=[0]' in s and s.endswith('-> (Tensor, Tensor, Tensor, Tensor, Tensor)')
    for d in (1, 2, 3):
        for n in (f'deform_conv{d}d', f'_deform_conv{d}d_backward', f'deform_conv_transpose{d}d',
                  f'_deform_conv_transpose{d}d_backward', f'mask_softmax{d}d'):
            assert hasattr(torch.ops.tvdcn, n)


def test_no_cpu_fallback():
    x, w = torch.randn(1, 4, 5, 5), torch.randn(2, 4, 3, 3)
    with pytest.raises(NotImplementedError):
        ops.deform_conv2d(x, w)
    with pytest.raises(NotImplementedError):
        ops.deform_conv_transpose2d(x, torch.randn(4, 2, 3, 3))


@pytest.mark.parametrize('dim', [1, 2, 3])
def test_modules_construct_like_the_reference(dim):
    conv = getattr(ops, f'PackedDeformConv{dim}d')(8, 16, 3, padding=1, groups=2, offset_groups=2, mask_groups=4,
                                                   modulated=True, mask_activation='softmax')
    assert conv.weight.shape == (16, 4) + (3,) * dim
    assert conv.offset_generator.out_channels == dim * 3 ** dim * 2
    assert conv.mask_generator.out_channels == 3 ** dim * 4
    assert conv.offset_generator.weight.abs().sum() == 0 and conv.mask_generator.weight.abs().sum() == 0
    assert sorted(conv.state_dict()) == ['bias', 'mask_generator.weight', 'offset_generator.weight', 'weight']
    tr = getattr(ops, f'PackedDeformConvTranspose{dim}d')(8, 4, 3, stride=2, padding=1, output_padding=1,
                                                          offset_groups=2, modulated=True)
    assert tr.weight.shape == (8, 4) + (3,) * dim
    assert tr.offset_generator.kernel_size == (1,) * dim
    assert isinstance(tr.mask_activation, ops.MaskSigmoid)
    plain = getattr(ops, f'DeformConv{dim}d')(4, 4, 3, bias=False)
    assert plain.bias is None and 'bias=False' in repr(plain)


def test_module_argument_errors():
    with pytest.raises(ValueError, match='offset_groups'):
        ops.PackedDeformConv2d(6, 8, 3, offset_groups=4)
    with pytest.raises(ValueError, match='mask_groups'):
        ops.PackedDeformConv2d(8, 6, 3, mask_groups=4)
    with pytest.raises(ValueError, match='activation'):
        ops.PackedDeformConv2d(8, 8, 3, mask_activation='tanh')
    with pytest.raises(ValueError, match='offset'):
        ops.PackedDeformConv2d(8, 8, 3, offset_activation='tanh')
    with pytest.raises(ValueError, match='scale'):
        ops.mask_sigmoid(torch.zeros(1), scale=0.)
    m = ops.DeformConvTranspose2d(4, 4, 3, stride=2)
    geom = (m.stride, m.padding, m.kernel_size, 2, m.dilation)
    with pytest.raises(ValueError, match='output size'):
        m._output_padding(torch.zeros(1, 4, 5, 5), [20, 20], *geom)
    assert list(m._output_padding(torch.zeros(1, 4, 5, 5), [12, 11], *geom)) == [1, 0]
    with pytest.raises(ValueError, match='zeros'):
        ops.DeformConvTranspose2d(4, 4, 3, padding_mode='reflect')


def test_everything_compiles_under_torchscript():
    """The reference advertises that all of its functions and modules are torch.jit.script-able; so are these.
    The graphs must call the tvdcn:: operators (checked on the scripted code, nothing runs on a GPU here)."""
    fns = [ops.deform_conv1d, ops.deform_conv2d, ops.deform_conv3d, ops.deform_conv_transpose1d,
           ops.deform_conv_transpose2d, ops.deform_conv_transpose3d, ops.mask_softmax1d, ops.mask_softmax2d,
           ops.mask_softmax3d, ops.mask_sigmoid]
    for f in fns:
        torch.jit.script(f)
    for dim in (1, 2, 3):
        mods = [
            getattr(ops, f'DeformConv{dim}d')(4, 8, 3, padding=1),
            getattr(ops, f'DeformConv{dim}d')(4, 8, 3, padding=1, padding_mode='reflect'),
            getattr(ops, f'PackedDeformConv{dim}d')(4, 8, 3, modulated=True, mask_activation='softmax'),
            getattr(ops, f'PackedDeformConv{dim}d')(4, 8, 3, deformable=False, modulated=True),
            getattr(ops, f'DeformConvTranspose{dim}d')(4, 8, 3, stride=2),
            getattr(ops, f'PackedDeformConvTranspose{dim}d')(4, 8, 3, stride=2, modulated=True),
            getattr(ops, f'MaskSoftmax{dim}d')(3),
        ]
        for m in mods:
            scripted = torch.jit.script(m)
            code = scripted.code
            if 'Deform' in type(m).__name__:
                name = 'deform_conv_transpose' if 'Transpose' in type(m).__name__ else 'deform_conv'
                inlined = str(scripted.inlined_graph)
                assert f'tvdcn::{name}{dim}d' in inlined, type(m).__name__
            assert code
    assert 'tvdcn::mask_softmax2d' in str(torch.jit.script(ops.MaskSoftmax2d(3)).inlined_graph)


def test_mask_softmax_has_no_cpu_path():
    """mask_softmax validates its arguments like the reference and then calls the CUDA operator; a CPU tensor is
    refused by the dispatcher (no silent torch.softmax fallback)."""
    m = torch.randn(2, 18, 5, 4)
    with pytest.raises((NotImplementedError, RuntimeError), match='mask_softmax2d|CPU'):
        ops.mask_softmax2d(m, (3, 3))
    with pytest.raises((NotImplementedError, RuntimeError), match='mask_softmax2d|CPU'):
        ops.MaskSoftmax2d(3)(m)
    with pytest.raises(RuntimeError, match='not valid'):
        ops.mask_softmax2d(torch.randn(1, 5, 2, 2), (3, 3))
    assert torch.allclose(ops.mask_sigmoid(torch.zeros(3)), torch.ones(3))


