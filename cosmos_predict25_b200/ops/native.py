"""Loader for the in-tree sm_100a extension (``_C.so`` beside this file).

The library registers its operators under ``torch.ops.cosmos_b200``. It is built by
``cosmos_predict25_b200.ops.build.build_extension`` (also reachable as
``python -m cosmos_predict25_b200.ops.build``). On a machine with a GPU a missing library
is an error: nothing silently falls back to eager PyTorch for CUDA tensors.
"""

from __future__ import annotations

import contextlib
import os
import threading

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_C.so")
_lock = threading.Lock()
_loaded = False


def lib_path() -> str:
    return _LIB_PATH


def available() -> bool:
    """True when the compiled extension exists on disk."""
    return os.path.exists(_LIB_PATH)


def load():
    """Load the extension once and return the ``torch.ops.cosmos_b200`` namespace."""
    global _loaded
    if not _loaded:
        with _lock:
            if not _loaded:
                if not os.path.exists(_LIB_PATH):
                    raise RuntimeError(
                        f"native extension {_LIB_PATH} is missing; run `python -m cosmos_predict25_b200.ops.build` "
                        "(CUDA tensors are never served by a PyTorch fallback)"
                    )
                torch.ops.load_library(_LIB_PATH)
                _loaded = True
    return torch.ops.cosmos_b200


_forward_mode = False


def forward_mode() -> bool:
    """True inside ``forward_mode_ad()``: element-wise and GEMM operators then run as plain torch ops (which carry
    forward-mode tangents) and only attention uses its kernel, through a function with a JVP rule."""
    return _forward_mode


@contextlib.contextmanager
def forward_mode_ad():
    global _forward_mode
    prev, _forward_mode = _forward_mode, True
    try:
        yield
    finally:
        _forward_mode = prev


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors go to the extension; CPU tensors (and everything in forward-mode AD) go to the PyTorch oracle."""
    return t.is_cuda and not _forward_mode


_launch_count = 0


def count_launch(n: int = 1) -> None:
    """Host-side tally of kernels launched by this package (bench.py reports it)."""
    global _launch_count
    _launch_count += n


def launches() -> int:
    return _launch_count


def reset_launches() -> None:
    global _launch_count
    _launch_count = 0
