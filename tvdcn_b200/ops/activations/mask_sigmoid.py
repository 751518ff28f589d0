"""Scaled sigmoid for modulation masks (API of tvdcn/ops/activations/mask_sigmoid.py:11-39; plain torch)."""
import torch
from torch import Tensor, nn

__all__ = ['mask_sigmoid', 'MaskSigmoid']


def mask_sigmoid(mask: Tensor, scale: float = 2.0) -> Tensor:
    """``sigmoid(mask) * scale``; with ``scale=2`` a zero-initialised mask generator yields ones."""
    if scale <= 0:
        raise ValueError('scale must be positive. Got scale={}'.format(scale))
    return torch.sigmoid(mask) * scale


class MaskSigmoid(nn.Module):
    """Module form of :func:`mask_sigmoid`."""

    def __init__(self, scale: float = 2.0):
        super().__init__()
        self.scale = float(scale)

    def forward(self, mask: Tensor) -> Tensor:
        return mask_sigmoid(mask, self.scale)
