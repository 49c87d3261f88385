"""Composite loaders: image/video interleaving, cached replay with background prefetch, and an I/O watchdog.

Parity targets: ``IterativeJointDataLoader`` (cosmos_predict2/_src/predict2/datasets/joint_dataloader.py:25-89),
``CachedReplayDataLoader`` (cosmos_predict2/_src/predict2/datasets/cached_replay_dataloader.py:260-476),
``OperationWatchdog`` (cosmos_predict2/_src/predict2/datasets/watchdog.py:27).
"""

from __future__ import annotations

import queue
import random
import threading
import time
from typing import Callable, Dict, Iterable, Iterator, List, Optional

from ..utils import log


class IterativeJointDataLoader:
    """Round-robin over named loaders by integer ratios: with ratios {image: 1, video: 2} the global batch ids
    0,1,2,... map to image, video, video, image, ... Each batch is tagged with ``dataset_name``."""

    def __init__(self, dataloaders: Dict[str, Dict]):
        self.loaders = {k: v["dataloader"] for k, v in dataloaders.items()}
        self.ratios = {k: int(v.get("ratio", 1)) for k, v in dataloaders.items()}
        self.names = [k for k, r in self.ratios.items() if r > 0]
        self.ratio_sum = sum(self.ratios[k] for k in self.names)
        self.schedule: List[str] = []
        for k in self.names:
            self.schedule += [k] * self.ratios[k]
        self.global_id = 0

    def __len__(self):
        return sum(len(self.loaders[k]) for k in self.names)

    def __iter__(self) -> Iterator:
        iters = {k: iter(self.loaders[k]) for k in self.names}
        while True:
            name = self.schedule[self.global_id % self.ratio_sum]
            try:
                batch = next(iters[name])
            except StopIteration:
                iters[name] = iter(self.loaders[name])
                try:
                    batch = next(iters[name])
                except StopIteration:
                    return
            batch["dataset_name"] = name
            self.global_id += 1
            yield batch


class OperationWatchdog:
    """Context manager that logs a warning from a helper thread if the wrapped operation takes too long."""

    def __init__(self, name: str = "operation", warning_threshold: float = 60.0, interval: float = 30.0):
        self.name, self.threshold, self.interval = name, warning_threshold, interval
        self._stop = threading.Event()
        self.warnings = 0

    def _watch(self, t0):
        while not self._stop.wait(min(self.interval, self.threshold)):
            el = time.time() - t0
            if el >= self.threshold:
                self.warnings += 1
                log.warning(f"{self.name} is taking {el:.0f}s (threshold {self.threshold:.0f}s)", rank0_only=False)

    def __enter__(self):
        self._stop.clear()
        self._t = threading.Thread(target=self._watch, args=(time.time(),), daemon=True)
        self._t.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._t.join(timeout=1.0)


# ---- batch-level augmentations for the cached loader (cached_replay_dataloader.py:28-258 of the reference) -----------------------
def _grid_starts(full: int, out: int, n: int) -> List[int]:
    """Start offsets of ``n`` crops of length ``out`` spread over ``full``: centred for one crop, else on a regular grid with a
    random shift inside each cell."""
    if out > full:
        raise ValueError("Output dimensions cannot be larger than original dimensions")
    if n == 1:
        return [(full - out) // 2]
    step = max(1, (full - out) // (n - 1))
    return [min(full - out, i * step + random.randrange(max(1, step))) for i in range(n)]


def generate_multiple_image_batches(data_batch: Dict, nh: int, nw: int, output_height: int, output_width: int) -> List[Dict]:
    """``nh * nw`` copies of the batch whose ``images`` [B, C, H, W] are crops spread over the original."""
    import copy
    img = data_batch["images"]
    out = []
    for h0 in _grid_starts(img.shape[-2], output_height, nh):
        for w0 in _grid_starts(img.shape[-1], output_width, nw):
            b = copy.deepcopy(data_batch)
            b["images"] = img[..., h0:h0 + output_height, w0:w0 + output_width]
            out.append(b)
    return out


def generate_multiple_video_batches(data_batch: Dict, nt: int, nh: int, nw: int, output_length: int, output_height: int,
                                    output_width: int) -> List[Dict]:
    """``nt * nh * nw`` copies whose ``video`` [B, C, T, H, W] are space-time crops spread over the original."""
    import copy
    vid = data_batch["video"]
    out = []
    for t0 in _grid_starts(vid.shape[2], output_length, nt):
        for h0 in _grid_starts(vid.shape[3], output_height, nh):
            for w0 in _grid_starts(vid.shape[4], output_width, nw):
                b = copy.deepcopy(data_batch)
                b["video"] = vid[:, :, t0:t0 + output_length, h0:h0 + output_height, w0:w0 + output_width]
                out.append(b)
    return out


def duplicate_batches(data_batch: Dict, n: int) -> List[Dict]:
    import copy
    return [copy.deepcopy(data_batch) for _ in range(n)]


_DUP_RNG = random.Random(123)


def duplicate_batches_random(data_batch: Dict, n: float) -> List[Dict]:
    """``floor(n)`` or ``ceil(n)`` copies, so that the expected number of copies is ``n``."""
    import copy
    import math
    lo, hi = int(math.floor(n)), int(math.ceil(n))
    k = lo if _DUP_RNG.uniform(lo, hi) > n else hi
    return [copy.deepcopy(data_batch) for _ in range(k)]


def concatenate_batches(n: int, data_batches: List[Dict]) -> List[Dict]:
    """Merge ``n`` batches into one, for all ``len / n`` groups (group i takes batches i, i + m, i + 2m ...): tensors are
    concatenated along the batch axis, lists are joined, a string keeps the first value, anything else becomes a list."""
    import torch
    if n <= 0:
        raise ValueError("n must be a positive integer")
    if len(data_batches) % n != 0:
        raise ValueError(f"Length of data_batches ({len(data_batches)}) must be divisible by n ({n})")
    m = len(data_batches) // n
    out = []
    for i in range(m):
        group = [data_batches[j * m + i] for j in range(n)]
        merged: Dict = {}
        for key in {k for b in group for k in b}:
            vals = [b[key] for b in group if key in b]
            first = next((v for v in vals if v is not None), None)
            if first is None:
                merged[key] = None
            elif isinstance(first, torch.Tensor):
                merged[key] = torch.cat(vals, dim=0)
            elif isinstance(first, str):
                merged[key] = vals[0]
            elif isinstance(first, list):
                merged[key] = [x for v in vals for x in v]
            else:
                merged[key] = vals
        out.append(merged)
    return out


def get_cached_replay_dataloader(use_cache: bool = False, cache_size: int = 32, concat_size: int = 1,
                                 cache_augment_fn: Optional[Callable] = None, cache_replay_name: str = "cached_replay_dataloader",
                                 webdataset: bool = False, **kwargs):
    """A torch ``DataLoader(**kwargs)``, wrapped in the cached loader when ``use_cache``."""
    from torch.utils.data import DataLoader
    loader = DataLoader(**kwargs)
    if not use_cache:
        return loader
    return CachedReplayDataLoader(loader, cache_size=cache_size, cache_augmentation_fn=cache_augment_fn, concat_size=concat_size,
                                  name=cache_replay_name)


class CachedReplayDataLoader:
    """Prefetches batches from a base loader on a background thread into a bounded cache; each fetched batch is
    passed through ``cache_augmentation_fn`` (which may return several batches: crops, duplicates) and can be
    replayed ``cache_replay_n`` times, trading data diversity for loader throughput."""

    def __init__(self, dataloader: Iterable, cache_size: int = 8, cache_replay_n: int = 1,
                 cache_augmentation_fn: Optional[Callable] = None, shuffle_cache: bool = False, watchdog_threshold: float = 120.0,
                 concat_size: int = 1, name: str = "cached_replay_dataloader"):
        self.base = dataloader
        self.concat_size, self.name = max(1, concat_size), name
        self.cache_size = cache_size
        self.replay_n = max(1, cache_replay_n)
        self.aug = cache_augmentation_fn
        self.shuffle = shuffle_cache
        self.watchdog_threshold = watchdog_threshold
        self._q: "queue.Queue" = queue.Queue(maxsize=cache_size)
        self._thread: Optional[threading.Thread] = None
        self._stop = threading.Event()
        self._error: Optional[BaseException] = None

    def _producer(self):
        try:
            for batch in self.base:
                items = self.aug(batch) if self.aug is not None else [batch]
                if not isinstance(items, (list, tuple)):
                    items = [items]
                for it in items:
                    for _ in range(self.replay_n):
                        while not self._stop.is_set():
                            try:
                                self._q.put(it, timeout=0.2)
                                break
                            except queue.Full:
                                continue
                        if self._stop.is_set():
                            return
        except BaseException as e:
            self._error = e
        finally:
            self._q.put(StopIteration)

    def __iter__(self):
        if self.concat_size == 1:
            yield from self._iter_single()
            return
        group: List = []
        for item in self._iter_single():                # ``concat_size`` cached batches become one (batch axis)
            group.append(item)
            if len(group) == self.concat_size:
                yield concatenate_batches(self.concat_size, group)[0]
                group = []

    def _iter_single(self):
        self.close()
        self._stop.clear()
        self._q = queue.Queue(maxsize=self.cache_size)
        self._thread = threading.Thread(target=self._producer, daemon=True, name="cached-replay-prefetch")
        self._thread.start()
        pool: List = []
        while True:
            with OperationWatchdog("dataloader prefetch", self.watchdog_threshold):
                item = self._q.get()
            if item is StopIteration:
                if self._error is not None:
                    raise self._error
                while pool:
                    yield pool.pop(random.randrange(len(pool)))
                return
            if self.shuffle:
                pool.append(item)
                if len(pool) >= self.cache_size:
                    yield pool.pop(random.randrange(len(pool)))
            else:
                yield item

    def __len__(self):
        return len(self.base) * self.replay_n

    def close(self):
        if self._thread is not None and self._thread.is_alive():
            self._stop.set()
            try:
                while True:
                    self._q.get_nowait()
            except queue.Empty:
                pass
            self._thread.join(timeout=2.0)
        self._thread = None
