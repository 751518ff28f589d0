"""Operators and module wrappers with the names of ``tvdcn.ops``: deformable convolution (1d/2d/3d, plain and
transposed, functional and ``nn.Module`` forms, packed variants with their own offset / mask generators) and the
mask activations."""
from . import activations, deform_conv, deform_conv_transpose
from .activations import *
from .deform_conv import *
from .deform_conv_transpose import *

__all__ = list(activations.__all__) + list(deform_conv.__all__) + list(deform_conv_transpose.__all__)
