"""Transposed deformable convolution: functional operators and ``nn.Module`` wrappers.

Public names, argument order and defaults are those of the reference
(tvdcn/ops/deform_conv_transpose.py:29-196 functions, :203-790 modules).

Layouts (taps = prod(kernel_size)):
  input   [batch, in_channels, *in_size]
  weight  [in_channels, out_channels // groups, *kernel_size]
  offset  [batch, offset_groups * taps * D, *in_size]   -- on the INPUT grid
  mask    [batch, mask_groups * taps, *in_size]
Offset and mask groups divide the OUTPUT channels (the image the columns are scattered into).
"""
from typing import Callable, List, Optional, Union

import torch
from torch import Tensor

from .deform_conv import _DeformConvNd, _PackedMixin, _NTUPLE, _ints
from ..extension import _assert_has_ops

__all__ = [
    'deform_conv_transpose1d', 'deform_conv_transpose2d', 'deform_conv_transpose3d',
    'DeformConvTranspose1d', 'DeformConvTranspose2d', 'DeformConvTranspose3d',
    'PackedDeformConvTranspose1d', 'PackedDeformConvTranspose2d', 'PackedDeformConvTranspose3d',
]


def _deform_conv_transpose(dim, input, weight, offset, mask, bias, stride, padding, output_padding, dilation,
                           groups):
    _assert_has_ops()
    op = getattr(torch.ops.tvdcn, f'deform_conv_transpose{dim}d')
    return op(input, weight, offset, mask, bias, _ints(stride, dim), _ints(padding, dim),
              _ints(output_padding, dim), _ints(dilation, dim), groups)


def deform_conv_transpose1d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride=1, padding=0,
                            output_padding=0, dilation=1, groups: int = 1) -> Tensor:
    """1D transposed deformable convolution."""
    return _deform_conv_transpose(1, input, weight, offset, mask, bias, stride, padding, output_padding,
                                  dilation, groups)


def deform_conv_transpose2d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride=1, padding=0,
                            output_padding=0, dilation=1, groups: int = 1) -> Tensor:
    """2D transposed deformable convolution."""
    return _deform_conv_transpose(2, input, weight, offset, mask, bias, stride, padding, output_padding,
                                  dilation, groups)


def deform_conv_transpose3d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride=1, padding=0,
                            output_padding=0, dilation=1, groups: int = 1) -> Tensor:
    """3D transposed deformable convolution."""
    return _deform_conv_transpose(3, input, weight, offset, mask, bias, stride, padding, output_padding,
                                  dilation, groups)


# noinspection PyMethodOverriding
class _DeformConvTransposeNd(_DeformConvNd):
    _transposed = True

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, bias: bool = True, padding_mode: str = 'zeros',
                 device=None, dtype=None) -> None:
        nt = _NTUPLE[self._dim]
        # _ConvNd stores the weight as [in, out // groups, *k] when transposed=True
        super(_DeformConvNd, self).__init__(
            in_channels, out_channels, nt(kernel_size), nt(stride), nt(padding), nt(dilation),
            True, nt(output_padding), groups, bias, padding_mode, device=device, dtype=dtype)

    def _output_padding(self, input: Tensor, output_size: Optional[List[int]]) -> List[int]:
        """output_padding that makes the result ``output_size`` (same rule as nn.ConvTransposeNd)."""
        if output_size is None:
            return list(self.output_padding)
        d = self._dim
        lead = 2 if input.dim() == d + 2 else 1
        output_size = list(output_size)
        if len(output_size) == lead + d:
            output_size = output_size[lead:]
        if len(output_size) != d:
            raise ValueError('ConvTranspose{}D: for {}D input, output_size must have {} or {} elements (got {})'
                             .format(d, input.dim(), d, lead + d, len(output_size)))
        res = []
        for a in range(d):
            lo = ((input.size(a + lead) - 1) * self.stride[a] - 2 * self.padding[a]
                  + self.dilation[a] * (self.kernel_size[a] - 1) + 1)
            hi = lo + self.stride[a] - 1
            if not lo <= output_size[a] <= hi:
                raise ValueError('requested an output size of {}, but valid sizes range from {} to {} '
                                 '(for an input of {})'.format(output_size, lo, hi, tuple(input.shape[lead:])))
            res.append(output_size[a] - lo)
        return res

    def _conv_transpose_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor],
                                mask: Optional[Tensor], bias: Optional[Tensor],
                                output_size: Optional[List[int]] = None) -> Tensor:
        if self.padding_mode != 'zeros':
            raise ValueError(f'Only `zeros` padding mode is supported for {type(self).__name__}.')
        return _deform_conv_transpose(self._dim, input, weight, offset, mask, bias, self.stride, self.padding,
                                      self._output_padding(input, output_size), self.dilation, self.groups)

    def forward(self, input: Tensor, offset: Optional[Tensor], mask: Optional[Tensor] = None,
                output_size: Optional[List[int]] = None) -> Tensor:
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)


class DeformConvTranspose1d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose1d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 1


class DeformConvTranspose2d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose2d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 2


class DeformConvTranspose3d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose3d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 3


# noinspection PyMethodOverriding
class _PackedDeformConvTransposeNd(_PackedMixin, _DeformConvTransposeNd):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, offset_groups: int = 1, mask_groups: int = 1,
                 bias: bool = True, generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, output_padding,
                         groups, bias, padding_mode, device, dtype)
        # offsets live on the input grid: pointwise generators (reference: deform_conv_transpose.py:617-637)
        self._init_packed(offset_groups, mask_groups, generator_bias, deformable, modulated,
                          offset_activation, mask_activation, dict(kernel_size=1), device, dtype)

    def forward(self, input: Tensor, output_size: Optional[List[int]] = None) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)


class PackedDeformConvTranspose1d(_PackedDeformConvTransposeNd):
    """:class:`DeformConvTranspose1d` that computes its own offset (and mask) from the input."""
    _dim = 1


class PackedDeformConvTranspose2d(_PackedDeformConvTransposeNd):
    """:class:`DeformConvTranspose2d` that computes its own offset (and mask) from the input."""
    _dim = 2


class PackedDeformConvTranspose3d(_PackedDeformConvTransposeNd):
    """:class:`DeformConvTranspose3d` that computes its own offset (and mask) from the input."""
    _dim = 3
