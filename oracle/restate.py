"""CPU restatement of the reference's deformable-convolution arithmetic (all dims, fwd + bwd).

TEST INFRASTRUCTURE ONLY.  This module is the checker the CUDA path is compared with; it is
never imported by the product package and never timed as the product.

Parity of this restatement is pinned two ways (see tests/test_oracle.py): against golden
vectors produced by the reference's own CPU build (tests/golden/*.pt, made by
tests/golden/make_golden.py) and, when oracle/_ref has been built, live against
``torch.ops.tvdcn_ref.*``.

Everything is expressed with dense torch tensor algebra in the dtype of the inputs (tests use
float64).  The formulas follow the reference (paths are inside the tvdcn project):

* sampling position and tap / channel-group layout:
  tvdcn/csrc/ops/cpu/deform_conv2d_common_kernels.cpp:161-187 (1d: deform_conv1d_common_kernels.cpp,
  3d: deform_conv3d_common_kernels.cpp, same structure)
* bilinear sample with per-corner validity: ...2d_common_kernels.cpp:24-57
* scatter of a value onto the 2^dim corners: ...:73-102
* derivative of the sample w.r.t. one coordinate: ...:104-135
* offset gradient and mask gradient reductions over the channels of a group: ...:387-425, :511-543
* host loops (which GEMM multiplies what): tvdcn/csrc/ops/cpu/deform_conv2d_kernel.cpp:341-380, 518-627
  and tvdcn/csrc/ops/cpu/deform_conv_transpose2d_kernel.cpp:333-363, 529-614
* softmax over the taps of one mask group: tvdcn/ops/activations/mask_softmax.py:78-88

Vocabulary used below (shared by the conv and the transposed op):
  "dense" tensor   - the one that enters the GEMM unsampled (conv: output / grad_output,
                     transposed: input), laid out on the *grid* the offsets live on;
  "sampled" image  - the one that is read or written at fractional positions (conv: input,
                     transposed: output / grad_output); channel groups for offset and mask are
                     taken over ITS channel count;
  weight           - always [dense_channels, sampled_channels / groups, *kernel].
"""
from __future__ import annotations

import itertools
import math
from typing import Optional, Sequence, Tuple

import torch
from torch import Tensor


def _ntuple(v, n: int) -> Tuple[int, ...]:
    if isinstance(v, int):
        return (v,) * n
    v = tuple(int(e) for e in v)
    if len(v) == 1:
        return v * n
    if len(v) != n:
        raise ValueError(f"expected {n} values, got {len(v)}")
    return v


class _Plan:
    """Corner indices / weights of every (batch, offset group, tap, grid position)."""

    def __init__(self, dim: int, img_size: Sequence[int], grid_size: Sequence[int],
                 kernel: Sequence[int], stride, pad, dil, offset: Optional[Tensor], batch: int,
                 dtype, device):
        self.dim = dim
        self.img_size = tuple(img_size)
        self.grid_size = tuple(grid_size)
        K = math.prod(kernel)
        P = math.prod(grid_size)
        self.K, self.P = K, P
        # integer base coordinate per axis: grid*stride - pad + tap*dil
        taps = list(itertools.product(*[range(k) for k in kernel]))
        grids = torch.stack(torch.meshgrid(*[torch.arange(g, device=device) for g in grid_size],
                                           indexing="ij"), 0).reshape(dim, P)
        tap_t = torch.tensor(taps, device=device).reshape(K, dim).t()  # [dim, K]
        s = torch.tensor(stride, device=device).view(dim, 1, 1)
        p = torch.tensor(pad, device=device).view(dim, 1, 1)
        d = torch.tensor(dil, device=device).view(dim, 1, 1)
        base = grids.view(dim, 1, P) * s - p + tap_t.view(dim, K, 1) * d  # [dim, K, P]
        base = base.to(dtype).permute(1, 0, 2)  # [K, dim, P]
        if offset is not None:
            og = offset.shape[1] // (K * dim)
            off = offset.reshape(batch, og, K, dim, P)
            pos = base.view(1, 1, K, dim, P) + off
            self.deformable = True
        else:
            og = 1
            pos = base.view(1, 1, K, dim, P).expand(batch, 1, K, dim, P)
            self.deformable = False
        self.og = og
        fl = torch.floor(pos)
        self.fr = pos - fl  # [B, og, K, dim, P]
        self.fl = fl.to(torch.int64)
        strides = [math.prod(img_size[a + 1:]) for a in range(dim)]
        self.corners = []
        for bits in itertools.product((0, 1), repeat=dim):
            if not self.deformable and any(bits):
                continue  # integer sampling touches one point only
            flat = torch.zeros_like(self.fl[:, :, :, 0])
            valid = torch.ones_like(flat, dtype=torch.bool)
            w_axis = []
            for a in range(dim):
                ia = self.fl[:, :, :, a] + bits[a]
                valid &= (ia >= 0) & (ia < img_size[a])
                flat = flat + ia * strides[a]
                w_axis.append(self.fr[:, :, :, a] if bits[a] else 1 - self.fr[:, :, :, a])
            flat = torch.where(valid, flat, torch.zeros_like(flat))
            self.corners.append((bits, flat, valid.to(dtype), w_axis))

    def corner_weight(self, corner, deriv_axis: Optional[int] = None) -> Tensor:
        bits, _, valid, w_axis = corner
        w = valid.clone()
        for a in range(self.dim):
            if deriv_axis is not None and a == deriv_axis:
                w = w * (1.0 if bits[a] else -1.0)
            else:
                w = w * w_axis[a]
        return w  # [B, og, K, P]

    def gather(self, img: Tensor, deriv_axis: Optional[int] = None) -> Tensor:
        """img [B, C, *img_size] -> [B, C, K, P] sampled values (no mask)."""
        B, C = img.shape[:2]
        S = math.prod(self.img_size)
        cg = C // self.og
        im = img.reshape(B, self.og, cg, S)
        out = torch.zeros(B, self.og, cg, self.K * self.P, dtype=img.dtype, device=img.device)
        for corner in self.corners:
            w = self.corner_weight(corner, deriv_axis).reshape(B, self.og, 1, self.K * self.P)
            idx = corner[1].reshape(B, self.og, 1, self.K * self.P).expand(B, self.og, cg, -1)
            out = out + w * torch.gather(im, 3, idx)
        return out.reshape(B, C, self.K, self.P)

    def scatter(self, vals: Tensor, C: int) -> Tensor:
        """vals [B, C, K, P] -> image [B, C, *img_size] accumulated on the corners."""
        B = vals.shape[0]
        S = math.prod(self.img_size)
        cg = C // self.og
        v = vals.reshape(B, self.og, cg, self.K * self.P)
        img = torch.zeros(B, self.og, cg, S, dtype=vals.dtype, device=vals.device)
        for corner in self.corners:
            w = self.corner_weight(corner).reshape(B, self.og, 1, self.K * self.P)
            idx = corner[1].reshape(B, self.og, 1, self.K * self.P).expand(B, self.og, cg, -1)
            img.scatter_add_(3, idx, w * v)
        return img.reshape(B, C, *self.img_size)


def _expand_mask(mask: Optional[Tensor], B: int, C: int, K: int, P: int, like: Tensor) -> Tensor:
    if mask is None:
        return torch.ones(1, 1, 1, 1, dtype=like.dtype, device=like.device)
    mg = mask.shape[1] // K
    m = mask.reshape(B, mg, 1, K, P).expand(B, mg, C // mg, K, P)
    return m.reshape(B, C, K, P)


def _conv_out_size(in_size, kernel, stride, pad, dil):
    return tuple((i + 2 * p - (d * (k - 1) + 1)) // s + 1
                 for i, k, s, p, d in zip(in_size, kernel, stride, pad, dil))


def _tconv_out_size(in_size, kernel, stride, pad, dil, opad):
    return tuple((i - 1) * s - 2 * p + d * (k - 1) + 1 + op
                 for i, k, s, p, d, op in zip(in_size, kernel, stride, pad, dil, opad))


# --------------------------------------------------------------------------------------
# the three primitives
# --------------------------------------------------------------------------------------
def _sample_gemm(plan: _Plan, img: Tensor, weight: Tensor, mask: Optional[Tensor], groups: int) -> Tensor:
    """dense[b, d, p] = sum_{s', tap} W[d, s', tap] * mask * sample(img[b, s], pos)."""
    B, C = img.shape[:2]
    K, P = plan.K, plan.P
    col = plan.gather(img) * _expand_mask(mask, B, C, K, P, img)
    Dn = weight.shape[0]
    W = weight.reshape(groups, Dn // groups, C // groups, K)
    out = torch.einsum("gdsk,bgskp->bgdp", W, col.reshape(B, groups, C // groups, K, P))
    return out.reshape(B, Dn, *plan.grid_size), col


def _gemm_columns(plan: _Plan, dense: Tensor, weight: Tensor, groups: int, C: int) -> Tensor:
    """col[b, s, tap, p] = sum_{d in group(s)} W[d, s', tap] * dense[b, d, p]."""
    B, Dn = dense.shape[:2]
    W = weight.reshape(groups, Dn // groups, C // groups, plan.K)
    col = torch.einsum("gdsk,bgdp->bgskp", W, dense.reshape(B, groups, Dn // groups, plan.P))
    return col.reshape(B, C, plan.K, plan.P)


def _coord_grads(plan: _Plan, col: Tensor, img: Tensor, offset: Optional[Tensor], mask: Optional[Tensor]):
    B, C = img.shape[:2]
    K, P, dim = plan.K, plan.P, plan.dim
    m = _expand_mask(mask, B, C, K, P, img)
    g_off = None
    if offset is not None:
        parts = []
        for a in range(dim):
            dS = plan.gather(img, deriv_axis=a)
            parts.append((col * m * dS).reshape(B, plan.og, C // plan.og, K, P).sum(2))
        g_off = torch.stack(parts, 3).reshape(offset.shape)  # [B, og, K, dim, P]
    g_mask = None
    if mask is not None:
        mg = mask.shape[1] // K
        S_ = plan.gather(img)
        g_mask = (col * S_).reshape(B, mg, C // mg, K, P).sum(2).reshape(mask.shape)
    return g_off, g_mask


# --------------------------------------------------------------------------------------
# public restatements
# --------------------------------------------------------------------------------------
def deform_conv(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                mask: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                stride=1, padding=0, dilation=1, groups: int = 1) -> Tensor:
    dim = weight.dim() - 2
    stride, padding, dilation = (_ntuple(v, dim) for v in (stride, padding, dilation))
    kernel = tuple(weight.shape[2:])
    B = input.shape[0]
    grid = _conv_out_size(input.shape[2:], kernel, stride, padding, dilation)
    plan = _Plan(dim, input.shape[2:], grid, kernel, stride, padding, dilation, offset, B,
                 input.dtype, input.device)
    out, _ = _sample_gemm(plan, input, weight, mask, groups)
    if bias is not None:
        out = out + bias.view(1, -1, *([1] * dim))
    return out


def deform_conv_backward(grad: Tensor, input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                         mask: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                         stride=1, padding=0, dilation=1, groups: int = 1):
    dim = weight.dim() - 2
    stride, padding, dilation = (_ntuple(v, dim) for v in (stride, padding, dilation))
    kernel = tuple(weight.shape[2:])
    B, C = input.shape[:2]
    grid = tuple(grad.shape[2:])
    plan = _Plan(dim, input.shape[2:], grid, kernel, stride, padding, dilation, offset, B,
                 input.dtype, input.device)
    K, P = plan.K, plan.P
    m = _expand_mask(mask, B, C, K, P, input)
    col_g = _gemm_columns(plan, grad, weight, groups, C)
    g_input = plan.scatter(col_g * m, C)
    g_off, g_mask = _coord_grads(plan, col_g, input, offset, mask)
    col = plan.gather(input) * m
    Dn = weight.shape[0]
    g_w = torch.einsum("bgdp,bgskp->gdsk", grad.reshape(B, groups, Dn // groups, P),
                       col.reshape(B, groups, C // groups, K, P)).reshape(weight.shape)
    g_b = grad.sum(dim=[0] + list(range(2, 2 + dim))) if bias is not None else None
    return g_input, g_w, g_off, g_mask, g_b


def deform_conv_transpose(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                          mask: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                          stride=1, padding=0, output_padding=0, dilation=1, groups: int = 1) -> Tensor:
    dim = weight.dim() - 2
    stride, padding, output_padding, dilation = (
        _ntuple(v, dim) for v in (stride, padding, output_padding, dilation))
    kernel = tuple(weight.shape[2:])
    B = input.shape[0]
    C_out = weight.shape[1] * groups
    out_size = _tconv_out_size(input.shape[2:], kernel, stride, padding, dilation, output_padding)
    plan = _Plan(dim, out_size, input.shape[2:], kernel, stride, padding, dilation, offset, B,
                 input.dtype, input.device)
    col = _gemm_columns(plan, input, weight, groups, C_out)
    out = plan.scatter(col * _expand_mask(mask, B, C_out, plan.K, plan.P, input), C_out)
    if bias is not None:
        out = out + bias.view(1, -1, *([1] * dim))
    return out


def deform_conv_transpose_backward(grad: Tensor, input: Tensor, weight: Tensor,
                                   offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                                   bias: Optional[Tensor] = None, stride=1, padding=0,
                                   output_padding=0, dilation=1, groups: int = 1):
    dim = weight.dim() - 2
    stride, padding, output_padding, dilation = (
        _ntuple(v, dim) for v in (stride, padding, output_padding, dilation))
    kernel = tuple(weight.shape[2:])
    B, C_in = input.shape[:2]
    C_out = weight.shape[1] * groups
    plan = _Plan(dim, grad.shape[2:], input.shape[2:], kernel, stride, padding, dilation, offset, B,
                 input.dtype, input.device)
    K, P = plan.K, plan.P
    col = _gemm_columns(plan, input, weight, groups, C_out)
    g_off, g_mask = _coord_grads(plan, col, grad, offset, mask)
    g_input, T = _sample_gemm(plan, grad, weight, mask, groups)
    g_w = torch.einsum("bgdp,bgskp->gdsk", input.reshape(B, groups, C_in // groups, P),
                       T.reshape(B, groups, C_out // groups, K, P)).reshape(weight.shape)
    g_b = grad.sum(dim=[0] + list(range(2, 2 + dim))) if bias is not None else None
    return g_input, g_w, g_off, g_mask, g_b


def mask_softmax(mask: Tensor, kernel_size) -> Tensor:
    K = math.prod(kernel_size) if not isinstance(kernel_size, int) else kernel_size
    B = mask.shape[0]
    mg = mask.shape[1] // K
    if mg == 0:
        raise RuntimeError("mask has fewer channels than kernel taps")
    v = mask.reshape(B, mg, K, -1)
    return torch.softmax(v, dim=2).reshape(mask.shape)


def mask_softmax_backward(grad: Tensor, out: Tensor, kernel_size) -> Tensor:
    K = math.prod(kernel_size) if not isinstance(kernel_size, int) else kernel_size
    B = out.shape[0]
    mg = out.shape[1] // K
    g = grad.reshape(B, mg, K, -1)
    y = out.reshape(B, mg, K, -1)
    return (y * (g - (g * y).sum(2, keepdim=True))).reshape(out.shape)
