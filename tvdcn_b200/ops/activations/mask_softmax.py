"""Softmax over the kernel taps of each mask group.

Same signatures as tvdcn/ops/activations/mask_softmax.py:19-184, and scriptable like them.  Every call goes
through the ``tvdcn::mask_softmax{1,2,3}d`` operators (single-pass CUDA kernel, forward and backward).  Like the
convolution operators they have CUDA kernels only: a CPU tensor is refused by the dispatcher, there is no
fallback to ``torch.softmax``.
"""
from typing import Optional, Tuple

import torch
from torch import Tensor, nn
from torch.nn.modules.utils import _single, _pair, _triple

from ...extension import _assert_has_ops

__all__ = [
    'mask_softmax1d', 'mask_softmax2d', 'mask_softmax3d',
    'MaskSoftmax1d', 'MaskSoftmax2d', 'MaskSoftmax3d',
]


def _check_mask(mask: Tensor, taps: int, dims: int) -> None:
    if mask.dim() != dims + 2:
        raise RuntimeError('mask_softmax{}d expects a {}D mask, got a {}D tensor'.format(dims, dims + 2, mask.dim()))
    if mask.size(1) // taps == 0:
        raise RuntimeError(
            'The shape of the mask tensor at dimension 1 is not valid. It should be a multiple of '
            'prod(kernel_size).\nGot mask.size(1)={}, while prod(kernel_size)={}'.format(mask.size(1), taps))


def mask_softmax1d(mask: Tensor, kernel_size: Tuple[int]) -> Tensor:
    """mask: [batch, mask_groups * kernel_width, out_width]."""
    if not torch.jit.is_scripting():
        kernel_size = _single(kernel_size)
    taps = kernel_size[0]
    _check_mask(mask, taps, 1)
    _assert_has_ops()
    return torch.ops.tvdcn.mask_softmax1d(mask, [kernel_size[0]])


def mask_softmax2d(mask: Tensor, kernel_size: Tuple[int, int]) -> Tensor:
    """mask: [batch, mask_groups * kernel_height * kernel_width, out_height, out_width]."""
    if not torch.jit.is_scripting():
        kernel_size = _pair(kernel_size)
    taps = kernel_size[0] * kernel_size[1]
    _check_mask(mask, taps, 2)
    _assert_has_ops()
    return torch.ops.tvdcn.mask_softmax2d(mask, [kernel_size[0], kernel_size[1]])


def mask_softmax3d(mask: Tensor, kernel_size: Tuple[int, int, int]) -> Tensor:
    """mask: [batch, mask_groups * kd * kh * kw, out_depth, out_height, out_width]."""
    if not torch.jit.is_scripting():
        kernel_size = _triple(kernel_size)
    taps = kernel_size[0] * kernel_size[1] * kernel_size[2]
    _check_mask(mask, taps, 3)
    _assert_has_ops()
    return torch.ops.tvdcn.mask_softmax3d(mask, [kernel_size[0], kernel_size[1], kernel_size[2]])


class _MaskSoftmaxNd(nn.Module):
    def extra_repr(self) -> str:
        return f'kernel_size={self.kernel_size}'


class MaskSoftmax1d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax1d`."""

    def __init__(self, kernel_size) -> None:
        super().__init__()
        self.kernel_size: Tuple[int] = _single(kernel_size)

    def forward(self, mask: Tensor, kernel_size: Optional[Tuple[int]] = None) -> Tensor:
        return mask_softmax1d(mask, kernel_size if kernel_size is not None else self.kernel_size)


class MaskSoftmax2d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax2d`."""

    def __init__(self, kernel_size) -> None:
        super().__init__()
        self.kernel_size: Tuple[int, int] = _pair(kernel_size)

    def forward(self, mask: Tensor, kernel_size: Optional[Tuple[int, int]] = None) -> Tensor:
        return mask_softmax2d(mask, kernel_size if kernel_size is not None else self.kernel_size)


class MaskSoftmax3d(_MaskSoftmaxNd):
    """Module form of :func:`mask_softmax3d`."""

    def __init__(self, kernel_size) -> None:
        super().__init__()
        self.kernel_size: Tuple[int, int, int] = _triple(kernel_size)

    def forward(self, mask: Tensor, kernel_size: Optional[Tuple[int, int, int]] = None) -> Tensor:
        return mask_softmax3d(mask, kernel_size if kernel_size is not None else self.kernel_size)
