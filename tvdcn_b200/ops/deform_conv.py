"""Deformable convolution: functional operators and ``nn.Module`` wrappers.

Public names, argument order, defaults and tensor layouts are those of the reference
(tvdcn/ops/deform_conv.py:30-199 for the functions, :206-751 for the modules); the arithmetic runs in
the ``torch.ops.tvdcn.deform_conv{1,2,3}d`` CUDA operators of this package.

Layouts (D = 1, 2, 3; taps = prod(kernel_size)):
  input   [batch, in_channels, *in_size]               (a missing batch axis is accepted)
  weight  [out_channels, in_channels // groups, *kernel_size]
  offset  [batch, offset_groups * taps * D, *out_size]  channel = (group * taps + tap) * D + axis
  mask    [batch, mask_groups * taps, *out_size]
  bias    [out_channels]
``offset=None`` samples the integer grid, ``mask=None`` multiplies by one; with both absent the operator
is an ordinary convolution.
"""
from typing import Callable, List, Optional, Tuple, Union

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from torch.nn import init
from torch.nn.common_types import _size_1_t, _size_2_t, _size_3_t
from torch.nn.modules.conv import _ConvNd
from torch.nn.modules.utils import _single, _pair, _triple

from .activations import MaskSigmoid, MaskSoftmax1d, MaskSoftmax2d, MaskSoftmax3d
from ..extension import _assert_has_ops

__all__ = [
    'deform_conv1d', 'deform_conv2d', 'deform_conv3d',
    'DeformConv1d', 'DeformConv2d', 'DeformConv3d',
    'PackedDeformConv1d', 'PackedDeformConv2d', 'PackedDeformConv3d',
]

_NTUPLE = {1: _single, 2: _pair, 3: _triple}
_MASK_SOFTMAX = {1: MaskSoftmax1d, 2: MaskSoftmax2d, 3: MaskSoftmax3d}
_CONV = {1: nn.Conv1d, 2: nn.Conv2d, 3: nn.Conv3d}


# The dispatcher wants a list for every SymInt[D] argument and does not broadcast a bare int; these do it, in
# eager mode and under TorchScript alike.
def _list1(v: _size_1_t) -> List[int]:
    if isinstance(v, int):
        return [v]
    return [v[0]]


def _list2(v: _size_2_t) -> List[int]:
    if isinstance(v, int):
        return [v, v]
    return [v[0], v[1]]


def _list3(v: _size_3_t) -> List[int]:
    if isinstance(v, int):
        return [v, v, v]
    return [v[0], v[1], v[2]]


def deform_conv1d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride: _size_1_t = 1, padding: _size_1_t = 0,
                  dilation: _size_1_t = 1, groups: int = 1) -> Tensor:
    """1D deformable convolution; returns [batch, out_channels, out_width]."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv1d(input, weight, offset, mask, bias, _list1(stride), _list1(padding),
                                         _list1(dilation), groups)


def deform_conv2d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride: _size_2_t = 1, padding: _size_2_t = 0,
                  dilation: _size_2_t = 1, groups: int = 1) -> Tensor:
    """2D deformable convolution (DCNv1 / DCNv2); returns [batch, out_channels, out_height, out_width]."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv2d(input, weight, offset, mask, bias, _list2(stride), _list2(padding),
                                         _list2(dilation), groups)


def deform_conv3d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride: _size_3_t = 1, padding: _size_3_t = 0,
                  dilation: _size_3_t = 1, groups: int = 1) -> Tensor:
    """3D deformable convolution; returns [batch, out_channels, out_depth, out_height, out_width]."""
    _assert_has_ops()
    return torch.ops.tvdcn.deform_conv3d(input, weight, offset, mask, bias, _list3(stride), _list3(padding),
                                         _list3(dilation), groups)


################################################################################
# Modules (all of them compile under torch.jit.script, like the reference's)
################################################################################
def _resolve_mask_activation(mask_activation, dim, kernel_size):
    if isinstance(mask_activation, str):
        if mask_activation == 'sigmoid':
            return MaskSigmoid(scale=2.)
        if mask_activation == 'softmax':
            return _MASK_SOFTMAX[dim](kernel_size)
        raise ValueError('only "sigmoid" and "softmax" activations are supported for mask')
    return mask_activation


# noinspection PyMethodOverriding
class _DeformConvNd(_ConvNd):
    """Shared constructor; subclasses fix ``_dim`` and the operator call."""
    _dim = 0

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        nt = _NTUPLE[self._dim]
        padding_ = padding if isinstance(padding, str) else nt(padding)
        super().__init__(in_channels, out_channels, nt(kernel_size), nt(stride), padding_, nt(dilation),
                         False, nt(0), groups, bias, padding_mode, device=device, dtype=dtype)

    def _conv_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor], mask: Optional[Tensor],
                      bias: Optional[Tensor]) -> Tensor:
        raise NotImplementedError

    def forward(self, input: Tensor, offset: Optional[Tensor], mask: Optional[Tensor] = None) -> Tensor:
        return self._conv_forward(input, self.weight, offset, mask, self.bias)

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


class DeformConv1d(_DeformConvNd):
    """See :func:`deform_conv1d`.  ``forward(input, offset, mask=None)``."""
    _dim = 1

    def _conv_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor], mask: Optional[Tensor],
                      bias: Optional[Tensor]) -> Tensor:
        if self.padding_mode != 'zeros':
            return deform_conv1d(F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode),
                                 weight, offset, mask, bias, self.stride, (0,), self.dilation, self.groups)
        return deform_conv1d(input, weight, offset, mask, bias, self.stride, self.padding, self.dilation,
                             self.groups)


class DeformConv2d(_DeformConvNd):
    """See :func:`deform_conv2d`.  ``forward(input, offset, mask=None)``."""
    _dim = 2

    def _conv_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor], mask: Optional[Tensor],
                      bias: Optional[Tensor]) -> Tensor:
        if self.padding_mode != 'zeros':
            return deform_conv2d(F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode),
                                 weight, offset, mask, bias, self.stride, (0, 0), self.dilation, self.groups)
        return deform_conv2d(input, weight, offset, mask, bias, self.stride, self.padding, self.dilation,
                             self.groups)


class DeformConv3d(_DeformConvNd):
    """See :func:`deform_conv3d`.  ``forward(input, offset, mask=None)``."""
    _dim = 3

    def _conv_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor], mask: Optional[Tensor],
                      bias: Optional[Tensor]) -> Tensor:
        if self.padding_mode != 'zeros':
            return deform_conv3d(F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode),
                                 weight, offset, mask, bias, self.stride, (0, 0, 0), self.dilation, self.groups)
        return deform_conv3d(input, weight, offset, mask, bias, self.stride, self.padding, self.dilation,
                             self.groups)


class _PackedMixin:
    """Owns the offset / mask generator convolutions of the packed modules.

    Generators are zero-initialised so a fresh module starts as an ordinary convolution
    (reference: tvdcn/ops/deform_conv.py:567-613).
    """

    def _init_packed(self, offset_groups, mask_groups, generator_bias, deformable, modulated,
                     offset_activation, mask_activation, generator_kwargs, device, dtype):
        for name, n in (('offset_groups', offset_groups), ('mask_groups', mask_groups)):
            if self.in_channels % n != 0:
                raise ValueError(f'in_channels must be divisible by {name}')
            if self.out_channels % n != 0:
                raise ValueError(f'out_channels must be divisible by {name}')
        if isinstance(offset_activation, str):
            raise ValueError('currently, no activation is supported for offset')
        mask_activation = _resolve_mask_activation(mask_activation, self._dim, self.kernel_size)

        self.offset_groups = offset_groups
        self.mask_groups = mask_groups
        self.deformable = deformable
        self.modulated = modulated
        taps = 1
        for k in self.kernel_size:
            taps *= k
        conv = _CONV[self._dim]
        if deformable:
            self.offset_generator = conv(self.in_channels, self._dim * taps * offset_groups, groups=offset_groups,
                                         bias=generator_bias, device=device, dtype=dtype, **generator_kwargs)
        else:
            self.register_module('offset_generator', None)
        if modulated:
            self.mask_generator = conv(self.in_channels, taps * mask_groups, groups=mask_groups,
                                       bias=generator_bias, device=device, dtype=dtype, **generator_kwargs)
        else:
            self.register_module('mask_generator', None)
        self.offset_activation = offset_activation
        self.mask_activation = mask_activation
        self.reset_parameters()

    def reset_parameters(self) -> None:
        if not hasattr(self, 'modulated'):
            return  # called by _ConvNd.__init__ before the generators exist
        super().reset_parameters()
        for gen in (self.offset_generator, self.mask_generator):
            if gen is not None:
                init.zeros_(gen.weight)
                if gen.bias is not None:
                    init.zeros_(gen.bias)

    def _offset_and_mask(self, input: Tensor) -> Tuple[Optional[Tensor], Optional[Tensor]]:
        offset: Optional[Tensor] = None
        mask: Optional[Tensor] = None
        if self.offset_generator is not None:
            offset = self.offset_generator(input)
            if self.offset_activation is not None:
                offset = self.offset_activation(offset)
        if self.mask_generator is not None:
            mask = self.mask_generator(input)
            if self.mask_activation is not None:
                mask = self.mask_activation(mask)
        return offset, mask


def _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, offset_groups,
                 mask_groups, bias, generator_bias, deformable, modulated, offset_activation, mask_activation,
                 padding_mode, device, dtype):
    _DeformConvNd.__init__(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                           padding_mode, device, dtype)
    # generators see the same window as the main kernel so offset / mask land on the output grid
    gen = dict(kernel_size=self.kernel_size, stride=self.stride, padding=self.padding, dilation=self.dilation)
    self._init_packed(offset_groups, mask_groups, generator_bias, deformable, modulated,
                      offset_activation, mask_activation, gen, device, dtype)


# noinspection PyMethodOverriding
class PackedDeformConv1d(_PackedMixin, DeformConv1d):
    """:class:`DeformConv1d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, offset_groups: int = 1, mask_groups: int = 1, bias: bool = True,
                 generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, offset_groups,
                     mask_groups, bias, generator_bias, deformable, modulated, offset_activation, mask_activation,
                     padding_mode, device, dtype)

    def forward(self, input: Tensor) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_forward(input, self.weight, offset, mask, self.bias)


# noinspection PyMethodOverriding
class PackedDeformConv2d(_PackedMixin, DeformConv2d):
    """:class:`DeformConv2d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, offset_groups: int = 1, mask_groups: int = 1, bias: bool = True,
                 generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, offset_groups,
                     mask_groups, bias, generator_bias, deformable, modulated, offset_activation, mask_activation,
                     padding_mode, device, dtype)

    def forward(self, input: Tensor) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_forward(input, self.weight, offset, mask, self.bias)


# noinspection PyMethodOverriding
class PackedDeformConv3d(_PackedMixin, DeformConv3d):
    """:class:`DeformConv3d` that computes its own offset (and mask) from the input."""

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, offset_groups: int = 1, mask_groups: int = 1, bias: bool = True,
                 generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        _packed_init(self, in_channels, out_channels, kernel_size, stride, padding, dilation, groups, offset_groups,
                     mask_groups, bias, generator_bias, deformable, modulated, offset_activation, mask_activation,
                     padding_mode, device, dtype)

    def forward(self, input: Tensor) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_forward(input, self.weight, offset, mask, self.bias)
