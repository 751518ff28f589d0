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
from torch.nn.common_types import _size_1_t, _size_2_t, _size_3_t
from torch.nn.modules.conv import _ConvTransposeNd

from .deform_conv import _PackedMixin, _NTUPLE, _list1, _list2, _list3
from ..extension import _assert_has_ops

__all__ = [
    'deform_conv_transpose1d', 'deform_conv_transpose2d', 'deform_conv_transpose3d',
    'DeformConvTranspose1d', 'DeformConvTranspose2d', 'DeformConvTranspose3d',
    'PackedDeformConvTranspose1d', 'PackedDeformConvTranspose2d', 'PackedDeformConvTranspose3d',
]


def deform_conv_transpose1d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride: _size_1_t = 1,
                            padding: _size_1_t = 0, output_padding: _size_1_t = 0, dilation: _size_1_t = 1,
                            groups: int = 1) -> Tensor:
    """1D transposed deformable convolution."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv_transpose1d(input, weight, offset, mask, bias, _list1(stride),
                                                   _list1(padding), _list1(output_padding), _list1(dilation),
                                                   groups)


def deform_conv_transpose2d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride: _size_2_t = 1,
                            padding: _size_2_t = 0, output_padding: _size_2_t = 0, dilation: _size_2_t = 1,
                            groups: int = 1) -> Tensor:
    """2D transposed deformable convolution."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv_transpose2d(input, weight, offset, mask, bias, _list2(stride),
                                                   _list2(padding), _list2(output_padding), _list2(dilation),
                                                   groups)


def deform_conv_transpose3d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None,
                            mask: Optional[Tensor] = None, bias: Optional[Tensor] = None, stride: _size_3_t = 1,
                            padding: _size_3_t = 0, output_padding: _size_3_t = 0, dilation: _size_3_t = 1,
                            groups: int = 1) -> Tensor:
    """3D transposed deformable convolution."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv_transpose3d(input, weight, offset, mask, bias, _list3(stride),
                                                   _list3(padding), _list3(output_padding), _list3(dilation),
                                                   groups)


################################################################################
# Modules (all of them compile under torch.jit.script, like the reference's)
################################################################################
# noinspection PyMethodOverriding
class _DeformConvTransposeNd(_ConvTransposeNd):
    """Shared constructor on top of torch's transposed-convolution base, which stores the weight as
    [in, out // groups, *k], rejects non-zero padding modes and turns ``output_size`` into output_padding."""
    _dim = 0

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, bias: bool = True, padding_mode: str = 'zeros',
                 device=None, dtype=None) -> None:
        nt = _NTUPLE[self._dim]
        super().__init__(in_channels, out_channels, nt(kernel_size), nt(stride), nt(padding), nt(dilation),
                         True, nt(output_padding), groups, bias, padding_mode, device=device, dtype=dtype)

    def _conv_transpose_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor],
                                mask: Optional[Tensor], bias: Optional[Tensor],
                                output_size: Optional[List[int]] = None) -> Tensor:
        raise NotImplementedError

    def forward(self, input: Tensor, offset: Optional[Tensor], mask: Optional[Tensor] = None,
                output_size: Optional[List[int]] = None) -> Tensor:
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)

    def extra_repr(self):
        s = super().extra_repr()
        if getattr(self, 'offset_groups', 1) != 1:
            s += ', offset_groups={offset_groups}'
        if getattr(self, 'mask_groups', 1) != 1:
            s += ', mask_groups={mask_groups}'
        if hasattr(self, 'deformable') and not self.deformable:
            s += ', deformable=False'
        if hasattr(self, 'modulated') and not self.modulated:
            s += ', modulated=False'
        return s.format(**self.__dict__)


class DeformConvTranspose1d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose1d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 1

    def _conv_transpose_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor],
                                mask: Optional[Tensor], bias: Optional[Tensor],
                                output_size: Optional[List[int]] = None) -> Tensor:
        _assert_has_ops()
        output_padding = self._output_padding(input, output_size, self.stride, self.padding, self.kernel_size, 1,
                                              self.dilation)
        return torch.ops.tvdcn.deform_conv_transpose1d(input, weight, offset, mask, bias, self.stride, self.padding,
                                                       output_padding, self.dilation, self.groups)


class DeformConvTranspose2d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose2d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 2

    def _conv_transpose_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor],
                                mask: Optional[Tensor], bias: Optional[Tensor],
                                output_size: Optional[List[int]] = None) -> Tensor:
        _assert_has_ops()
        output_padding = self._output_padding(input, output_size, self.stride, self.padding, self.kernel_size, 2,
                                              self.dilation)
        return torch.ops.tvdcn.deform_conv_transpose2d(input, weight, offset, mask, bias, self.stride, self.padding,
                                                       output_padding, self.dilation, self.groups)


class DeformConvTranspose3d(_DeformConvTransposeNd):
    """See :func:`deform_conv_transpose3d`.  ``forward(input, offset, mask=None, output_size=None)``."""
    _dim = 3

    def _conv_transpose_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor],
                                mask: Optional[Tensor], bias: Optional[Tensor],
                                output_size: Optional[List[int]] = None) -> Tensor:
        _assert_has_ops()
        output_padding = self._output_padding(input, output_size, self.stride, self.padding, self.kernel_size, 3,
                                              self.dilation)
        return torch.ops.tvdcn.deform_conv_transpose3d(input, weight, offset, mask, bias, self.stride, self.padding,
                                                       output_padding, self.dilation, self.groups)


def _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, output_padding, groups,
                 offset_groups, mask_groups, bias, generator_bias, deformable, modulated, offset_activation,
                 mask_activation, padding_mode, device, dtype):
    _DeformConvTransposeNd.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation,
                                    output_padding, groups, bias, padding_mode, device, dtype)
    # offsets live on the input grid: pointwise generators (reference: deform_conv_transpose.py:617-637)
    self._init_packed(offset_groups, mask_groups, generator_bias, deformable, modulated,
                      offset_activation, mask_activation, dict(kernel_size=1), device, dtype)


# noinspection PyMethodOverriding
class PackedDeformConvTranspose1d(_PackedMixin, DeformConvTranspose1d):
    """:class:`DeformConvTranspose1d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, offset_groups: int = 1, mask_groups: int = 1,
                 bias: bool = True, generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, output_padding, groups,
                     offset_groups, mask_groups, bias, generator_bias, deformable, modulated, offset_activation,
                     mask_activation, padding_mode, device, dtype)

    def forward(self, input: Tensor, output_size: Optional[List[int]] = None) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)


# noinspection PyMethodOverriding
class PackedDeformConvTranspose2d(_PackedMixin, DeformConvTranspose2d):
    """:class:`DeformConvTranspose2d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, offset_groups: int = 1, mask_groups: int = 1,
                 bias: bool = True, generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, output_padding, groups,
                     offset_groups, mask_groups, bias, generator_bias, deformable, modulated, offset_activation,
                     mask_activation, padding_mode, device, dtype)

    def forward(self, input: Tensor, output_size: Optional[List[int]] = None) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)


# noinspection PyMethodOverriding
class PackedDeformConvTranspose3d(_PackedMixin, DeformConvTranspose3d):
    """:class:`DeformConvTranspose3d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 output_padding=0, groups: int = 1, offset_groups: int = 1, mask_groups: int = 1,
                 bias: bool = True, generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, output_padding, groups,
                     offset_groups, mask_groups, bias, generator_bias, deformable, modulated, offset_activation,
                     mask_activation, padding_mode, device, dtype)

    def forward(self, input: Tensor, output_size: Optional[List[int]] = None) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_transpose_forward(input, self.weight, offset, mask, self.bias, output_size)
