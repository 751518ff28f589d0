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
from typing import Callable, Optional, Union

import torch
import torch.nn.functional as F
from torch import Tensor, nn
from torch.nn import init
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


def _ints(v, dim: int):
    # the dispatcher wants lists for SymInt[D] arguments; ints are broadcast here
    return [int(e) for e in _NTUPLE[dim](v)]


def _deform_conv(dim, input, weight, offset, mask, bias, stride, padding, dilation, groups):
    _assert_has_ops()
    op = getattr(torch.ops.tvdcn, f'deform_conv{dim}d')
    return op(input, weight, offset, mask, bias,
              _ints(stride, dim), _ints(padding, dim), _ints(dilation, dim), groups)


def deform_conv1d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride=1, padding=0, dilation=1, groups: int = 1) -> Tensor:
    """1D deformable convolution; returns [batch, out_channels, out_width]."""
    return _deform_conv(1, input, weight, offset, mask, bias, stride, padding, dilation, groups)


def deform_conv2d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride=1, padding=0, dilation=1, groups: int = 1) -> Tensor:
    """2D deformable convolution (DCNv1 / DCNv2); returns [batch, out_channels, out_height, out_width]."""
    return _deform_conv(2, input, weight, offset, mask, bias, stride, padding, dilation, groups)


def deform_conv3d(input: Tensor, weight: Tensor, offset: Optional[Tensor] = None, mask: Optional[Tensor] = None,
                  bias: Optional[Tensor] = None, stride=1, padding=0, dilation=1, groups: int = 1) -> Tensor:
    """3D deformable convolution; returns [batch, out_channels, out_depth, out_height, out_width]."""
    return _deform_conv(3, input, weight, offset, mask, bias, stride, padding, dilation, groups)


################################################################################
# Modules
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
    """Shared implementation; subclasses fix ``_dim``."""
    _dim = 0
    _transposed = False

    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, bias: bool = True, padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        nt = _NTUPLE[self._dim]
        padding_ = padding if isinstance(padding, str) else nt(padding)
        super().__init__(in_channels, out_channels, nt(kernel_size), nt(stride), padding_, nt(dilation),
                         False, nt(0), groups, bias, padding_mode, device=device, dtype=dtype)

    def _conv_forward(self, input: Tensor, weight: Tensor, offset: Optional[Tensor], mask: Optional[Tensor],
                      bias: Optional[Tensor]) -> Tensor:
        if self.padding_mode != 'zeros':
            padded = F.pad(input, self._reversed_padding_repeated_twice, mode=self.padding_mode)
            return _deform_conv(self._dim, padded, weight, offset, mask, bias, self.stride,
                                (0,) * self._dim, self.dilation, self.groups)
        return _deform_conv(self._dim, input, weight, offset, mask, bias, self.stride, self.padding,
                            self.dilation, self.groups)

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


class DeformConv2d(_DeformConvNd):
    """See :func:`deform_conv2d`.  ``forward(input, offset, mask=None)``."""
    _dim = 2


class DeformConv3d(_DeformConvNd):
    """See :func:`deform_conv3d`.  ``forward(input, offset, mask=None)``."""
    _dim = 3


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

    def _offset_and_mask(self, input: Tensor):
        offset = mask = None
        if self.deformable and self.offset_generator is not None:
            offset = self.offset_generator(input)
            if self.offset_activation is not None:
                offset = self.offset_activation(offset)
        if self.modulated and self.mask_generator is not None:
            mask = self.mask_generator(input)
            if self.mask_activation is not None:
                mask = self.mask_activation(mask)
        return offset, mask


# noinspection PyMethodOverriding
class _PackedDeformConvNd(_PackedMixin, _DeformConvNd):
    def __init__(self, in_channels: int, out_channels: int, kernel_size, stride=1, padding=0, dilation=1,
                 groups: int = 1, offset_groups: int = 1, mask_groups: int = 1, bias: bool = True,
                 generator_bias: bool = False, deformable: bool = True, modulated: bool = False,
                 offset_activation: Optional[Union[str, Callable]] = None,
                 mask_activation: Optional[Union[str, Callable]] = 'sigmoid',
                 padding_mode: str = 'zeros', device=None, dtype=None) -> None:
        super().__init__(in_channels, out_channels, kernel_size, stride, padding, dilation, groups, bias,
                         padding_mode, device, dtype)
        # generators see the same window as the main kernel so offset / mask land on the output grid
        gen = dict(kernel_size=self.kernel_size, stride=self.stride, padding=self.padding, dilation=self.dilation)
        self._init_packed(offset_groups, mask_groups, generator_bias, deformable, modulated,
                          offset_activation, mask_activation, gen, device, dtype)

    def forward(self, input: Tensor) -> Tensor:
        offset, mask = self._offset_and_mask(input)
        return self._conv_forward(input, self.weight, offset, mask, self.bias)


class PackedDeformConv1d(_PackedDeformConvNd):
    """:class:`DeformConv1d` that computes its own offset (and mask) from the input."""
    _dim = 1


class PackedDeformConv2d(_PackedDeformConvNd):
    """:class:`DeformConv2d` that computes its own offset (and mask) from the input."""
    _dim = 2


class PackedDeformConv3d(_PackedDeformConvNd):
    """:class:`DeformConv3d` that computes its own offset (and mask) from the input."""
    _dim = 3
