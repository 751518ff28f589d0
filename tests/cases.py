"""Shared fixtures of the parity tests: case descriptions, seeded inputs, oracle and C-ABI runners."""
from __future__ import annotations

import ctypes
import math
import os
import sys
from dataclasses import dataclass, field, asdict
from typing import Optional, Tuple

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@dataclass(frozen=True)
class Case:
    name: str
    dim: int
    transposed: bool = False
    batch: int = 2
    in_channels: int = 4
    out_channels: int = 2
    in_size: Tuple[int, ...] = (5, 6)
    kernel: Tuple[int, ...] = (2, 3)
    stride: Tuple[int, ...] = (1, 2)
    padding: Tuple[int, ...] = (0, 1)
    dilation: Tuple[int, ...] = (1, 2)
    output_padding: Tuple[int, ...] = ()
    groups: int = 1
    offset_groups: int = 2   # 0: no offset
    mask_groups: int = 1     # 0: no mask
    bias: bool = True
    offset_std: float = 1.0

    @property
    def taps(self) -> int:
        return math.prod(self.kernel)

    @property
    def opad(self):
        return self.output_padding if self.output_padding else (0,) * self.dim

    @property
    def out_size(self):
        if not self.transposed:
            return tuple((i + 2 * p - (d * (k - 1) + 1)) // s + 1 for i, k, s, p, d in
                         zip(self.in_size, self.kernel, self.stride, self.padding, self.dilation))
        return tuple((i - 1) * s - 2 * p + d * (k - 1) + 1 + op for i, k, s, p, d, op in
                     zip(self.in_size, self.kernel, self.stride, self.padding, self.dilation, self.opad))

    @property
    def grid(self):
        return self.in_size if self.transposed else self.out_size


def reference_fixture(dim: int, transposed: bool, offset: bool = True, mask: bool = True, groups: int = 1,
                      offset_groups: int = 2, mask_groups: int = 1, batch: int = 2) -> Case:
    """The anisotropic toy problem of the reference's own tests
    (tests/utils/deform_conv_test_args.py:31-52 in the tvdcn project): kernel (2,3,..), stride (1,2,..),
    padding (0,1,..), dilation (1,2,..), spatial extent (5,6,..), 4 -> 2 channels."""
    rng = lambda a: tuple(range(a, a + dim))
    name = f"ref{dim}d{'T' if transposed else ''}_o{int(offset)}m{int(mask)}_g{groups}og{offset_groups}mg{mask_groups}"
    if not transposed:
        return Case(name, dim, False, batch, 4, 2 * groups if groups > 1 else 2, rng(5), rng(2), rng(1), rng(0),
                    rng(1), (), groups, offset_groups if offset else 0, mask_groups if mask else 0)
    # transposed: channels of the sampled image (= out_channels) carry the offset / mask groups
    opad = tuple(min(a, max(s, d) - 1) for a, s, d in zip(rng(0), rng(1), rng(1)))
    return Case(name, dim, True, batch, 2 * groups if groups > 1 else 2, 4, rng(4), rng(2), rng(1), rng(0),
                rng(1), opad, groups, offset_groups if offset else 0, mask_groups if mask else 0)


def make_inputs(case: Case, seed: int = 0, dtype=torch.float64):
    """Seeded CPU tensors: input, weight, offset, mask, bias, grad_output (absent ones are None)."""
    g = torch.Generator().manual_seed(seed)
    d = case.dim
    x = torch.randn(case.batch, case.in_channels, *case.in_size, generator=g, dtype=torch.float64)
    if not case.transposed:
        wshape = (case.out_channels, case.in_channels // case.groups, *case.kernel)
        fan_in = case.in_channels // case.groups * case.taps
    else:
        wshape = (case.in_channels, case.out_channels // case.groups, *case.kernel)
        fan_in = case.out_channels // case.groups * case.taps
    bound = 1.0 / math.sqrt(fan_in)
    w = (torch.rand(*wshape, generator=g, dtype=torch.float64) * 2 - 1) * bound
    off = (torch.randn(case.batch, case.offset_groups * case.taps * d, *case.grid, generator=g,
                       dtype=torch.float64) * case.offset_std) if case.offset_groups else None
    mask = torch.rand(case.batch, case.mask_groups * case.taps, *case.grid, generator=g,
                      dtype=torch.float64) if case.mask_groups else None
    bias = torch.randn(case.out_channels, generator=g, dtype=torch.float64) * 0.1 if case.bias else None
    go = torch.randn(case.batch, case.out_channels, *case.out_size, generator=g, dtype=torch.float64)
    cast = lambda t: None if t is None else t.to(dtype)
    return tuple(cast(t) for t in (x, w, off, mask, bias, go))


def run_oracle(case: Case, x, w, off, mask, bias, go):
    """(output, grad_input, grad_weight, grad_offset, grad_mask, grad_bias) from the CPU restatement."""
    from oracle import restate
    if not case.transposed:
        args = (case.stride, case.padding, case.dilation, case.groups)
        out = restate.deform_conv(x, w, off, mask, bias, *args)
        grads = restate.deform_conv_backward(go, x, w, off, mask, bias, *args)
    else:
        args = (case.stride, case.padding, case.opad, case.dilation, case.groups)
        out = restate.deform_conv_transpose(x, w, off, mask, bias, *args)
        grads = restate.deform_conv_transpose_backward(go, x, w, off, mask, bias, *args)
    return (out,) + tuple(grads)


def run_reference(case: Case, x, w, off, mask, bias, go):
    """Same, from the reference's own CPU build (oracle/_ref); requires build_ref.load() == True."""
    name = f"deform_conv{'_transpose' if case.transposed else ''}{case.dim}d"
    op = getattr(torch.ops.tvdcn_ref, name)
    bop = getattr(torch.ops.tvdcn_ref, '_' + name + '_backward')
    if not case.transposed:
        args = (case.stride, case.padding, case.dilation, case.groups)
    else:
        args = (case.stride, case.padding, case.opad, case.dilation, case.groups)
    out = op(x, w, off, mask, bias, *args)
    grads = bop(go, x, w, off, mask, bias, *args)
    fix = lambda t: None if (t is None or t.numel() == 0 and t.dim() <= 1) else t
    return (out,) + tuple(fix(t) for t in grads)


_DT = {torch.float32: 0, torch.float64: 1, torch.float16: 2, torch.bfloat16: 3}


def cabi_problem(case: Case, dtype, aux_dtype=None, engine: int = 0):
    from tvdcn_b200 import cabi
    return cabi.make_problem(case.dim, case.transposed, _DT[dtype], case.batch, case.in_channels,
                             case.out_channels, case.in_size, case.kernel, case.stride, case.padding,
                             case.dilation, case.groups, case.offset_groups, case.mask_groups, case.opad,
                             None if aux_dtype is None else _DT[aux_dtype], engine)


def run_cabi(case: Case, x, w, off, mask, bias, go, engine: int = 0, poison: bool = True):
    """Forward + backward through the C ABI on CUDA tensors; returns the same 6-tuple as run_oracle.

    Outputs are pre-filled with NaN so that an element a kernel forgot to write shows up."""
    from tvdcn_b200 import cabi
    L = cabi.lib()
    aux = None
    for t in (off, mask, bias):
        if t is not None:
            aux = t.dtype
    if aux is None and x.dtype in (torch.float16, torch.bfloat16):
        aux = torch.float32  # no offset / mask / bias: nothing constrains it, and f32 keeps the tensor path open
    p = cabi_problem(case, x.dtype, aux, engine)
    dev = x.device
    stream = torch.cuda.current_stream(dev).cuda_stream
    ptr = lambda t: None if t is None else ctypes.c_void_p(t.data_ptr())
    new = (lambda like: torch.full_like(like, float('nan'))) if poison else torch.empty_like
    out = new(go)
    ws_f = L.tvdcn_b200_forward_workspace_bytes(ctypes.byref(p))
    ws_b = L.tvdcn_b200_backward_workspace_bytes(ctypes.byref(p))
    ws = torch.empty(max(ws_f, ws_b, 1), dtype=torch.uint8, device=dev)
    cabi.check(L.tvdcn_b200_deform_conv_forward(ctypes.byref(p), ptr(x), ptr(w), ptr(off), ptr(mask), ptr(bias),
                                                ptr(out), ptr(ws), ws.numel(), ctypes.c_void_p(stream)))
    gx, gw = new(x), new(w)
    goff = new(off) if off is not None else None
    gmask = new(mask) if mask is not None else None
    gb = new(bias) if bias is not None else None
    cabi.check(L.tvdcn_b200_deform_conv_backward(ctypes.byref(p), ptr(go), ptr(x), ptr(w), ptr(off), ptr(mask),
                                                 ptr(gx), ptr(gw), ptr(goff), ptr(gmask), ptr(gb), ptr(ws),
                                                 ws.numel(), ctypes.c_void_p(stream)))
    torch.cuda.synchronize(dev)
    return out, gx, gw, goff, gmask, gb


NAMES = ('output', 'grad_input', 'grad_weight', 'grad_offset', 'grad_mask', 'grad_bias')


def nerr(a: torch.Tensor, ref: torch.Tensor) -> float:
    """max|a - ref| / max|ref| in float64 (the parity metric used throughout)."""
    a64, r64 = a.detach().double().cpu(), ref.detach().double().cpu()
    if not torch.isfinite(a64).all():
        return float('inf')
    denom = r64.abs().max().clamp_min(1e-30)
    return ((a64 - r64).abs().max() / denom).item()


def assert_parity(got, ref, tol: float, what: str = ''):
    for name, a, r in zip(NAMES, got, ref):
        if r is None:
            assert a is None, f'{what} {name}: expected None'
            continue
        assert a is not None, f'{what} {name}: missing'
        assert tuple(a.shape) == tuple(r.shape), f'{what} {name}: shape {tuple(a.shape)} vs {tuple(r.shape)}'
        e = nerr(a, r)
        assert e <= tol, f'{what} {name}: normalised max error {e:.3e} > {tol:.1e}'
