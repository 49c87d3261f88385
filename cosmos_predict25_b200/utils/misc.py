"""Small runtime helpers: architecture-invariant RNG, seeding, nested-batch utilities, timers.

Parity targets: ``arch_invariant_rand``, ``set_random_seed``, ``to``, ``get_data_batch_size``,
``TrainingTimer``, ``timer`` (cosmos_predict2/_src/imaginaire/utils/misc.py:157-391).
"""

from __future__ import annotations

import collections
import contextlib
import functools
import random
import time
from typing import Any, Callable, Dict, Optional, Tuple

import numpy as np
import torch


def arch_invariant_rand(shape, dtype: torch.dtype, device, seed: Optional[int] = None) -> torch.Tensor:
    """Standard-normal noise that is identical on every GPU architecture: drawn with NumPy's
    Mersenne Twister on the host, then moved to the device."""
    rng = np.random.RandomState(seed)
    return torch.from_numpy(rng.standard_normal(tuple(shape)).astype(np.float32)).to(dtype=dtype, device=device)


def set_random_seed(seed: int, by_rank: bool = False) -> int:
    if by_rank and torch.distributed.is_available() and torch.distributed.is_initialized():
        seed += torch.distributed.get_rank()
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    return seed


def to(data: Any, device=None, dtype=None, memory_format=torch.preserve_format) -> Any:
    """Recursively move tensors of a nested container; floating tensors also take ``dtype``."""
    if isinstance(data, torch.Tensor):
        if dtype is not None and data.is_floating_point():
            return data.to(device=device, dtype=dtype, non_blocking=True)
        return data.to(device=device, non_blocking=True)
    if isinstance(data, collections.abc.Mapping):
        return type(data)({k: to(v, device, dtype, memory_format) for k, v in data.items()})
    if isinstance(data, (list, tuple)) and not isinstance(data, str):
        return type(data)(to(v, device, dtype, memory_format) for v in data)
    return data


def get_data_batch_size(data: Any) -> int:
    """Batch size of the first tensor found in a nested batch."""
    if isinstance(data, torch.Tensor):
        return data.shape[0]
    if isinstance(data, collections.abc.Mapping):
        for v in data.values():
            try:
                return get_data_batch_size(v)
            except ValueError:
                continue
    if isinstance(data, (list, tuple)) and not isinstance(data, str):
        for v in data:
            try:
                return get_data_batch_size(v)
            except ValueError:
                continue
    raise ValueError("no tensor in batch")


class TrainingTimer:
    """Named wall-clock sections averaged over a logging window (dataloader / forward / backward / optimizer)."""

    def __init__(self):
        self.results: Dict[str, list] = collections.defaultdict(list)

    @contextlib.contextmanager
    def __call__(self, name: str):
        t0 = time.perf_counter()
        try:
            yield
        finally:
            self.results[name].append(time.perf_counter() - t0)

    def reset(self):
        self.results.clear()

    def compute_average_results(self) -> Dict[str, float]:
        return {k: sum(v) / max(len(v), 1) for k, v in self.results.items()}


class DeviceTimer:
    """CUDA-event section timer (device time, no host sync until ``elapsed_ms`` is read)."""

    def __init__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.stop = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.stop.record()

    def elapsed_ms(self) -> float:
        self.stop.synchronize()
        return self.start.elapsed_time(self.stop)


def timer(label: str) -> Callable:
    def deco(fn):
        @functools.wraps(fn)
        def wrapped(*a, **k):
            t0 = time.perf_counter()
            out = fn(*a, **k)
            from . import log
            log.debug(f"{label}: {time.perf_counter() - t0:.3f}s")
            return out
        return wrapped
    return deco


def count_params(model: torch.nn.Module) -> int:
    return sum(p.numel() for p in model.parameters())
