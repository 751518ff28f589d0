"""The workspace-free forward (tvdcn_b200_deform_conv_forward_static) against the ordinary forward and against
the CPU oracle (the two forwards share every kernel, so agreement between them alone would not catch a fault
common to both).

That entry point is for embedders that may not allocate device memory when the operator runs (plugins that
only receive tensor pointers, arena runtimes that forbid cudaMalloc after start-up): it borrows a fixed
16 MiB array inside the library instead of a caller workspace.  The array is shared by all calls and keeps
its contents, so the check is made twice in a row, with different inputs, to catch anything stale leaking
from the first call into the second.  The file name sorts last on purpose: if this addition breaks, a run
that stops at the first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

import cases
from cases import Case, make_inputs, nerr, run_oracle

pytestmark = pytest.mark.gpu

# f32 through the tensor-core kernels (staged image + packed weights live in the scratch) and a transposed
# problem whose scatter accumulator lives there too
CASES = [
    Case('static_conv', 2, False, 3, 64, 128, (12, 10), (3, 3), (1, 1), (1, 1), (1, 1), (), 1, 1, 1, True, 1.5),
    Case('static_transposed', 2, True, 2, 64, 64, (6, 8), (4, 4), (2, 2), (1, 1), (1, 1), (), 1, 1, 1, True, 1.0),
]


def _lib():
    from tvdcn_b200 import cabi
    L = cabi.lib()
    vp = ctypes.c_void_p
    L.tvdcn_b200_deform_conv_forward_static.argtypes = [ctypes.POINTER(cabi.Problem)] + [vp] * 7
    L.tvdcn_b200_deform_conv_forward_static.restype = ctypes.c_int
    L.tvdcn_b200_static_scratch_bytes.restype = ctypes.c_size_t
    L.tvdcn_b200_device_status.restype = ctypes.c_int
    return cabi, L


def _forward_both(case, seed):
    cabi, L = _lib()
    x, w, off, mask, bias, _ = (None if t is None else t.to('cuda', torch.float32)
                                for t in make_inputs(case, seed=seed))
    p = cases.cabi_problem(case, torch.float32)
    vp = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    shape = (case.batch, case.out_channels, *case.out_size)
    n = L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(p))
    assert 0 < n <= L.tvdcn_b200_static_scratch_bytes()
    ws = torch.empty(n, dtype=torch.uint8, device='cuda')
    ref = torch.full(shape, float('nan'), device='cuda')
    cabi.check(L.tvdcn_b200_deform_conv_forward(ctypes.byref(p), vp(x), vp(w), vp(off), vp(mask), vp(bias), vp(ref),
                                                vp(ws), n, stream))
    got = torch.full(shape, float('nan'), device='cuda')
    cabi.check(L.tvdcn_b200_deform_conv_forward_static(ctypes.byref(p), vp(x), vp(w), vp(off), vp(mask), vp(bias),
                                                       vp(got), stream))
    torch.cuda.synchronize()
    assert L.tvdcn_b200_device_status() == 0
    # the CPU oracle on the same f32 values, in f64
    dbl = lambda t: None if t is None else t.double().cpu()
    go = torch.zeros(shape, dtype=torch.float64)
    oracle = run_oracle(case, dbl(x), dbl(w), dbl(off), dbl(mask), dbl(bias), go)[0]
    return got, ref, oracle


@pytest.mark.parametrize('case', CASES, ids=[c.name for c in CASES])
def test_static_forward_matches_workspace_forward_twice(case):
    for seed in (71, 72):  # second call reuses the scratch the first one dirtied
        got, ref, oracle = _forward_both(case, seed)
        assert torch.isfinite(ref).all()
        assert nerr(got, ref) <= 1e-4     # the f32 tolerance of the parity tests; in practice the two are equal
        assert nerr(got, oracle) <= 1e-4  # and against the oracle, which shares no code with either


def test_static_forward_refuses_problems_larger_than_its_scratch():
    cabi, L = _lib()
    big = cabi.make_problem(2, False, cabi.F32, 64, 256, 256, (28, 28), (3, 3), (1, 1), (1, 1), (1, 1), 1, 4, 1)
    assert L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(big)) > L.tvdcn_b200_static_scratch_bytes()
    dummy = torch.zeros(1, device='cuda')
    vp = ctypes.c_void_p(dummy.data_ptr())
    rc = L.tvdcn_b200_deform_conv_forward_static(ctypes.byref(big), vp, vp, vp, vp, vp, vp, None)
    assert rc == 3  # TVDCN_ERR_WORKSPACE, before anything is launched
    msg = L.tvdcn_b200_last_error().decode()
    assert 'scratch' in msg and str(L.tvdcn_b200_static_scratch_bytes()) in msg
