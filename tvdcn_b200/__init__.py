"""B200-native (sm_100a) deformable convolution with the tvdcn operator API.

Same public names as the reference package (tvdcn/__init__.py:1-4): ``tvdcn_b200.ops`` holds the
functional operators and the ``nn.Module`` wrappers; ``has_ops`` / ``with_cuda`` / ``cuda_version`` /
``cuda_arch_list`` report on the loaded extension.  ``import tvdcn_b200 as tvdcn`` is the intended
drop-in spelling.
"""
from . import ops
from ._version import __version__
from .extension import _HAS_OPS, has_ops, cuda_version, cuda_arch_list, with_cuda
from .ops import *
