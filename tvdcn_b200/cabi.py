"""ctypes binding of the C ABI (include/tvdcn_b200.h) for callers that hold raw device pointers.

The torch operators do not go through this module (they call the same entry points from C++); it exists
for the parity tests, the benchmark and for embedding the kernels in hosts that are not PyTorch programs.
Pointers are plain integers (``tensor.data_ptr()``, ``cudaMalloc`` results, ...).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

from .extension import c_abi

F32, F64, F16, BF16 = 0, 1, 2, 3
ENGINE_AUTO, ENGINE_SIMT, ENGINE_TENSOR = 0, 1, 2
FLAG_REUSE_STAGED_INPUT = 1   # backward: the workspace still holds the forward call's staging of `input`


class Problem(C.Structure):
    """Mirror of ``tvdcn_problem``."""
    _fields_ = [
        ('dim', C.c_int32), ('transposed', C.c_int32), ('dtype', C.c_int32), ('aux_dtype', C.c_int32),
        ('batch', C.c_int64), ('in_channels', C.c_int64), ('out_channels', C.c_int64),
        ('in_size', C.c_int64 * 3), ('out_size', C.c_int64 * 3),
        ('kernel', C.c_int32 * 3), ('stride', C.c_int32 * 3), ('padding', C.c_int32 * 3),
        ('dilation', C.c_int32 * 3), ('output_padding', C.c_int32 * 3),
        ('groups', C.c_int32), ('offset_groups', C.c_int32), ('mask_groups', C.c_int32), ('engine', C.c_int32),
        ('flags', C.c_int32),
    ]


class TvdcnError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f'tvdcn_b200 status {code}: {message}')
        self.code = code


_proto_done = False


def lib() -> C.CDLL:
    global _proto_done
    L = c_abi()
    if not _proto_done:
        vp, sz, i32, i64 = C.c_void_p, C.c_size_t, C.c_int32, C.c_int64
        pp = C.POINTER(Problem)
        L.tvdcn_b200_problem_finalize.argtypes = [pp]
        L.tvdcn_b200_problem_finalize.restype = C.c_int
        for n in ('tvdcn_b200_forward_workspace_bytes', 'tvdcn_b200_backward_workspace_bytes'):
            getattr(L, n).argtypes = [pp]
            getattr(L, n).restype = sz
        L.tvdcn_b200_deform_conv_forward.argtypes = [pp, vp, vp, vp, vp, vp, vp, vp, sz, vp]
        L.tvdcn_b200_deform_conv_forward.restype = C.c_int
        L.tvdcn_b200_deform_conv_backward.argtypes = [pp] + [vp] * 11 + [sz, vp]
        L.tvdcn_b200_deform_conv_backward.restype = C.c_int
        L.tvdcn_b200_deform_conv_backward_ex.argtypes = [pp] + [vp] * 11 + [sz, vp, vp]
        L.tvdcn_b200_deform_conv_backward_ex.restype = C.c_int
        L.tvdcn_b200_mask_softmax_forward.argtypes = [i32, i64, i64, i64, i64, vp, vp, vp]
        L.tvdcn_b200_mask_softmax_forward.restype = C.c_int
        L.tvdcn_b200_mask_softmax_backward.argtypes = [i32, i64, i64, i64, i64, vp, vp, vp, vp]
        L.tvdcn_b200_mask_softmax_backward.restype = C.c_int
        L.tvdcn_b200_cuda_version.restype = C.c_int
        L.tvdcn_b200_cuda_arch_flags.restype = C.c_char_p
        L.tvdcn_b200_last_error.restype = C.c_char_p
        L.tvdcn_b200_launch_count.restype = C.c_uint64
        L.tvdcn_b200_engine_name.argtypes = [pp, C.c_int]
        L.tvdcn_b200_engine_name.restype = C.c_char_p
        L.tvdcn_b200_device_status.restype = C.c_int
        L.tvdcn_b200_device_status_address.restype = vp
        L.tvdcn_b200_publish_status.argtypes = [vp, vp]
        L.tvdcn_b200_publish_status.restype = C.c_int
        L.tvdcn_b200_selftest_bounded_wait.argtypes = [C.c_int, vp]
        L.tvdcn_b200_selftest_bounded_wait.restype = C.c_int
        _proto_done = True
    return L


def check(rc: int) -> None:
    if rc != 0:
        raise TvdcnError(rc, lib().tvdcn_b200_last_error().decode())


def make_problem(dim: int, transposed: bool, dtype: int, batch: int, in_channels: int, out_channels: int,
                 in_size: Sequence[int], kernel: Sequence[int], stride: Sequence[int], padding: Sequence[int],
                 dilation: Sequence[int], groups: int = 1, offset_groups: int = 0, mask_groups: int = 0,
                 output_padding: Optional[Sequence[int]] = None, aux_dtype: Optional[int] = None,
                 engine: int = ENGINE_AUTO) -> Problem:
    """Fill and finalize a problem description (raises :class:`TvdcnError` when it is inconsistent)."""
    p = Problem()
    p.dim, p.transposed, p.dtype = dim, int(transposed), dtype
    p.aux_dtype = dtype if aux_dtype is None else aux_dtype
    p.batch, p.in_channels, p.out_channels = batch, in_channels, out_channels
    for a in range(min(dim, 3, len(in_size))):
        p.in_size[a] = in_size[a]
        p.kernel[a], p.stride[a], p.padding[a], p.dilation[a] = kernel[a], stride[a], padding[a], dilation[a]
        p.output_padding[a] = output_padding[a] if output_padding is not None else 0
    p.groups, p.offset_groups, p.mask_groups, p.engine = groups, offset_groups, mask_groups, engine
    check(lib().tvdcn_b200_problem_finalize(C.byref(p)))
    return p
