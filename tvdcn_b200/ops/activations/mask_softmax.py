"""Softmax over the kernel taps of each mask group.

Same signatures as tvdcn/ops/activations/mask_softmax.py:19-184.  CUDA tensors go through the
``tvdcn::mask_softmax{1,2,3}d`` operators (single-pass kernel, forward and backward); other tensors use
the reference's own definition, a ``torch.softmax`` over the tap axis of the 4-D view.
"""
import math
from typing import Optional, Tuple

import torch
from torch import Tensor, nn
from torch.nn.modules.utils import _single, _pair, _triple

from ...extension import _assert_has_ops

__all__ = [
    'mask_softmax1d', 'mask_softmax2d', 'mask_softmax3d',
    'MaskSoftmax1d', 'MaskSoftmax2d', 'MaskSoftmax3d',
]

_NTUPLE = {1: _single, 2: _pair, 3: _triple}


def _mask_softmax(mask: Tensor, kernel_size, dim: int) -> Tensor:
    ks = tuple(int(k) for k in _NTUPLE[dim](kernel_size))
    if mask.dim() != dim + 2:
        raise RuntimeError(f'mask_softmax{dim}d expects a {dim + 2}D mask, got size {tuple(mask.shape)}')
    taps = math.prod(ks)
    if mask.size(1) // taps == 0:
        raise RuntimeError(
            'The shape of the mask tensor at dimension 1 is not valid. It should be a multiple of '
            'prod(kernel_size).\nGot mask.size(1)={}, while prod(kernel_size)={}'.format(mask.size(1), taps))
    if mask.is_cuda:
        _assert_has_ops()
        return getattr(torch.ops.tvdcn, f'mask_softmax{dim}d')(mask, list(ks))
    groups = mask.size(1) // taps
    view = mask.view(mask.size(0), groups, taps, *mask.shape[2:])
    return torch.softmax(view, dim=2).view(mask.size(0), groups * taps, *mask.shape[2:])


def mask_softmax1d(mask: Tensor, kernel_size: Tuple[int]) -> Tensor:
    """mask: [batch, mask_groups * kernel_width, out_width]."""
    return _mask_softmax(mask, kernel_size, 1)


def mask_softmax2d(mask: Tensor, kernel_size: Tuple[int, int]) -> Tensor:
    """mask: [batch, mask_groups * kernel_height * kernel_width, out_height, out_width]."""
    return _mask_softmax(mask, kernel_size, 2)


def mask_softmax3d(mask: Tensor, kernel_size: Tuple[int, int, int]) -> Tensor:
    """mask: [batch, mask_groups * kd * kh * kw, out_depth, out_height, out_width]."""
    return _mask_softmax(mask, kernel_size, 3)


class _MaskSoftmaxNd(nn.Module):
    _dim = 0

    def __init__(self, kernel_size) -> None:
        super().__init__()
        self.kernel_size = tuple(_NTUPLE[self._dim](kernel_size))

    def forward(self, mask: Tensor, kernel_size: Optional[Tuple[int, ...]] = None) -> Tensor:
        return _mask_softmax(mask, kernel_size if kernel_size is not None else self.kernel_size, self._dim)

    def extra_repr(self) -> str:
        return f'kernel_size={self.kernel_size}'


class MaskSoftmax1d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax1d`."""
    _dim = 1


class MaskSoftmax2d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax2d`."""
    _dim = 2


class MaskSoftmax3d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax3d`."""
    _dim = 3
