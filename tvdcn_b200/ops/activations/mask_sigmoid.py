"""Scaled sigmoid for modulation masks.

Same call as the reference's (tvdcn/ops/activations/mask_sigmoid.py:11-39).  Elementwise and plain torch: there is
nothing here for a dedicated kernel to win.  The default scale of 2 makes a zero-initialised mask generator produce
a mask of ones, i.e. a packed module starts out as an ordinary (unmodulated) convolution.
"""
import torch
from torch import Tensor, nn

__all__ = ['mask_sigmoid', 'MaskSigmoid']


def mask_sigmoid(mask: Tensor, scale: float = 2.0) -> Tensor:
    """``scale * sigmoid(mask)``; ``scale`` must be positive."""
    if not scale > 0:
        raise ValueError('scale must be positive. Got scale={}'.format(scale))
    return torch.sigmoid(mask).mul(scale)


class MaskSigmoid(nn.Module):
    """Module form of :func:`mask_sigmoid` with a fixed scale."""

    def __init__(self, scale: float = 2.0) -> None:
        super().__init__()
        if not scale > 0:
            raise ValueError('scale must be positive. Got scale={}'.format(scale))
        self.scale = float(scale)

    def extra_repr(self) -> str:
        return 'scale={}'.format(self.scale)

    def forward(self, mask: Tensor) -> Tensor:
        return torch.sigmoid(mask).mul(self.scale)
