"""CPU-only checks of the C ABI: the library loads, exports what the header declares, and its host-side
logic (validation, output extents, workspace sizing) behaves.  No kernel is launched."""
import ctypes
import os
import re

import pytest

import cases
from tvdcn_b200 import cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'tvdcn_b200.h')).read()
    return sorted(set(re.findall(r'\b(tvdcn_b200_[a-z0-9_]+)\s*\(', text)))


def test_library_exports_every_declared_symbol():
    L = cabi.lib()
    names = declared_symbols()
    assert len(names) >= 12
    for n in names:
        assert hasattr(L, n), f'{n} declared in include/tvdcn_b200.h but not exported'


def test_version_and_arch():
    L = cabi.lib()
    assert L.tvdcn_b200_cuda_version() >= 12000
    assert L.tvdcn_b200_cuda_arch_flags().decode() == 'sm_100a'
    assert isinstance(L.tvdcn_b200_launch_count(), int)


def test_struct_layout_matches_header():
    # 4 int32 + 3 int64 + 6 int64 + 15 int32 + 4 int32
    assert ctypes.sizeof(cabi.Problem) == 168  # 164 bytes of fields, padded to the int64 alignment


@pytest.mark.parametrize('dim,tr', [(1, False), (2, False), (3, False), (1, True), (2, True), (3, True)])
def test_output_extent(dim, tr):
    c = cases.reference_fixture(dim, tr)
    p = cases.cabi_problem(c, __import__('torch').float32)
    assert tuple(p.out_size[a] for a in range(dim)) == c.out_size
    assert all(p.out_size[a] == 1 for a in range(dim, 3))


def test_config_extents():
    # deform_conv2d N=128 256->256 28x28 k3 p1 and deform_conv_transpose2d 32x32 -> 64x64 k4 s2 p1
    p = cabi.make_problem(2, False, cabi.F32, 128, 256, 256, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1), 1, 4, 1)
    assert (p.out_size[0], p.out_size[1]) == (28, 28)
    p = cabi.make_problem(2, True, cabi.F32, 64, 256, 128, (32, 32), (4, 4), (2, 2), (1, 1), (1, 1), 1, 2, 1)
    assert (p.out_size[0], p.out_size[1]) == (64, 64)
    p = cabi.make_problem(1, False, cabi.F32, 64, 512, 512, (4096,), (5,), (1,), (4,), (2,), 8, 8, 1)
    assert p.out_size[0] == 4096


@pytest.mark.parametrize('kw,msg', [
    (dict(dim=4), 'dim'),
    (dict(groups=3), 'divisible by groups'),
    (dict(offset_groups=3), 'offset_groups'),
    (dict(mask_groups=3), 'mask_groups'),
    (dict(stride=(0, 1)), 'stride'),
    (dict(in_size=(1, 1), kernel=(3, 3), padding=(0, 0)), 'too small'),
    (dict(dtype=cabi.F64, aux_dtype=cabi.F32), 'aux_dtype'),
])
def test_invalid_problems_are_rejected(kw, msg):
    base = dict(dim=2, transposed=False, dtype=cabi.F32, batch=2, in_channels=4, out_channels=4, in_size=(8, 8),
                kernel=(3, 3), stride=(1, 1), padding=(1, 1), dilation=(1, 1), groups=1, offset_groups=2,
                mask_groups=1)
    base.update(kw)
    with pytest.raises(cabi.TvdcnError) as e:
        cabi.make_problem(**base)
    assert msg in str(e.value)


def test_workspace_sizes():
    L = cabi.lib()
    simt = dict(engine=cabi.ENGINE_SIMT)
    p32 = cabi.make_problem(2, False, cabi.F32, 2, 8, 8, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, 1, **simt)
    assert L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(p32)) == 0
    assert L.tvdcn_b200_backward_workspace_bytes(ctypes.byref(p32)) == 0
    p16 = cabi.make_problem(2, False, cabi.BF16, 2, 8, 8, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), 1, 1, 1, **simt)
    # f32 accumulators for grad_input, grad_weight, grad_offset, grad_mask
    need = 2 * 8 * 64 * 4 + 8 * 8 * 9 * 4 + 2 * 18 * 64 * 4 + 2 * 9 * 64 * 4
    got = L.tvdcn_b200_backward_workspace_bytes(ctypes.byref(p16))
    assert need <= got <= need + 4 * 256
    assert L.tvdcn_b200_engine_name(ctypes.byref(p32), 0).decode() == 'simt'


def test_null_pointer_is_an_error_not_a_crash():
    L = cabi.lib()
    p = cabi.make_problem(2, False, cabi.F32, 2, 8, 8, (8, 8), (3, 3), (1, 1), (1, 1), (1, 1), 1, 0, 0)
    rc = L.tvdcn_b200_deform_conv_forward(ctypes.byref(p), None, None, None, None, None, None, None, 0, None)
    assert rc == 1 and b'NULL' in L.tvdcn_b200_last_error()
