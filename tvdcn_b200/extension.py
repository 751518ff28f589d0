"""Loads the native libraries and reports on them (mirrors tvdcn/extension.py:78-80, 159-188).

``_C.so`` registers the ``torch.ops.tvdcn.*`` operators; ``libtvdcn_b200.so`` is the C ABI it calls
(also reachable through :func:`c_abi` for callers that bind it directly).  There is no fallback:
when ``_C.so`` is missing every operator call raises.
"""
from __future__ import annotations

import ctypes
import os
from typing import List

import torch

__all__ = ['has_ops', 'with_cuda', 'cuda_version', 'cuda_arch_list', 'c_abi', 'load_error']

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
_EXT_PATH = os.path.join(_PKG_DIR, '_C.so')
_LIB_PATH = os.path.join(_PKG_DIR, 'libtvdcn_b200.so')

_HAS_OPS = False
_LOAD_ERROR = None


def _has_ops() -> bool:
    # replaced by a function that returns True once the extension is loaded; a plain function (not a
    # module-level flag) so that TorchScript can compile callers of _assert_has_ops()
    return False


def _load() -> None:
    global _HAS_OPS, _LOAD_ERROR
    if not os.path.exists(_EXT_PATH):
        _LOAD_ERROR = f'{_EXT_PATH} not found; build it with `python -m tvdcn_b200.build`'
        return
    try:
        torch.ops.load_library(_EXT_PATH)
        _HAS_OPS = True
    except (OSError, RuntimeError) as e:  # pragma: no cover - depends on the install
        _LOAD_ERROR = f'could not load {_EXT_PATH}: {e}'


_load()

if _HAS_OPS:
    def _has_ops() -> bool:  # noqa: F811
        return True


def _assert_has_ops() -> None:
    if not _has_ops():
        raise RuntimeError(
            'tvdcn_b200: the compiled extension is not available and there is no fallback path. '
            'Build it with `python -m tvdcn_b200.build`; tvdcn_b200.extension.load_error() has the detail.')


def load_error():
    """Why the compiled extension could not be loaded (None when it was)."""
    return _LOAD_ERROR


def has_ops() -> bool:
    """True when the compiled extension was found and loaded."""
    return _HAS_OPS


def cuda_version() -> int:
    """CUDA runtime version the extension was compiled with (-1 without the extension)."""
    if not _HAS_OPS:
        return -1
    return torch.ops.tvdcn._cuda_version()


def with_cuda() -> bool:
    """True when the extension carries CUDA kernels (always, once it is loaded)."""
    return cuda_version() != -1


def cuda_arch_list() -> List[str]:
    """Architectures the kernels were compiled for."""
    if not _HAS_OPS:
        return []
    return torch.ops.tvdcn._cuda_arch_flags().split()


_CABI = None


def c_abi() -> ctypes.CDLL:
    """The C ABI shared library (declarations: include/tvdcn_b200.h)."""
    global _CABI
    if _CABI is None:
        if not os.path.exists(_LIB_PATH):
            raise RuntimeError(f'{_LIB_PATH} not found; build it with `python -m tvdcn_b200.build`')
        _CABI = ctypes.CDLL(_LIB_PATH)
    return _CABI
