"""Activations applied to the modulation mask before it reaches the deformable convolution."""
from . import mask_sigmoid as _sigmoid, mask_softmax as _softmax
from .mask_sigmoid import *
from .mask_softmax import *

__all__ = list(_sigmoid.__all__) + list(_softmax.__all__)
