"""Profiler and memory-snapshot contexts for the training loop.

Parity target: ``maybe_enable_profiling`` / ``maybe_enable_memory_snapshot`` (cosmos_predict2/_src/imaginaire/utils/profiling.py:36-139):
a torch profiler with a (wait, warmup, active=1) schedule repeating every ``profile_freq`` steps that writes one gzip'd
chrome trace per target rank under ``<job dir>/torch_trace/iteration_<n>/``; a CUDA memory-history recorder that dumps a
snapshot every ``profile_freq`` steps and once more on an out-of-memory error (``iteration_<n>_exit``).
"""

from __future__ import annotations

import contextlib
import os
import pickle
import time
from dataclasses import dataclass, field
from typing import List

import torch

from . import distributed, log

TORCH_TRACE_WARMUP = 3
MEMORY_SNAPSHOT_MAX_ENTRIES = 100000


@dataclass
class ProfilingConfig:
    enable_profiling: bool = False
    enable_memory_snapshot: bool = False
    profile_freq: int = 10
    target_ranks: List[int] = field(default_factory=lambda: [0])
    record_shape: bool = False
    profile_memory: bool = False
    with_stack: bool = False
    with_modules: bool = False
    first_n_rank: int = 8


@contextlib.contextmanager
def maybe_enable_profiling(cfg: ProfilingConfig, job_dir: str, *, global_step: int = 0):
    if not cfg.enable_profiling:
        yield None
        return
    trace_dir = os.path.join(job_dir, "torch_trace")
    os.makedirs(trace_dir, exist_ok=True)
    rank = distributed.get_rank()

    def trace_handler(prof):
        d = os.path.join(trace_dir, f"iteration_{prof.step_num}")
        os.makedirs(d, exist_ok=True)
        t0 = time.monotonic()
        if rank in cfg.target_ranks:
            prof.export_chrome_trace(f"{d}/rank{rank}_trace.json.gz")
        log.info(f"trace of step {prof.step_num} written in {time.monotonic() - t0:.2f} s")

    warmup, active = TORCH_TRACE_WARMUP, 1
    wait = cfg.profile_freq - (active + warmup)
    assert wait >= 0, "profile_freq must be greater than or equal to warmup + active"
    acts = [torch.profiler.ProfilerActivity.CPU]
    if torch.cuda.is_available():
        acts.append(torch.profiler.ProfilerActivity.CUDA)
    with torch.profiler.profile(activities=acts, schedule=torch.profiler.schedule(wait=wait, warmup=warmup, active=active),
                                on_trace_ready=trace_handler, record_shapes=cfg.record_shape, profile_memory=cfg.profile_memory,
                                with_stack=cfg.with_stack, with_modules=cfg.with_modules) as prof:
        prof.step_num = global_step
        yield prof


class MemoryProfiler:
    def __init__(self, cfg: ProfilingConfig, snapshot_dir: str, step_num: int):
        self.cfg, self.dir, self.step_num = cfg, snapshot_dir, step_num
        self.rank = distributed.get_rank()
        if torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=MEMORY_SNAPSHOT_MAX_ENTRIES)

    def step(self, exit_ctx: bool = False):
        self.step_num += 1
        if not exit_ctx and self.step_num % self.cfg.profile_freq != 0:
            return
        cur = self.step_num if not exit_ctx else self.step_num - 1      # "iteration_0_exit" when iteration 1 ran out of memory
        d = os.path.join(self.dir, f"iteration_{cur}" + ("_exit" if exit_ctx else ""))
        os.makedirs(d, exist_ok=True)
        if self.rank in self.cfg.target_ranks:
            snap = torch.cuda.memory._snapshot() if torch.cuda.is_available() else {"segments": [], "device_traces": []}
            with open(f"{d}/rank{self.rank}_memory_snapshot.pickle", "wb") as f:
                pickle.dump(snap, f)
        log.info(f"memory snapshot of step {cur} written to {d}")


@contextlib.contextmanager
def maybe_enable_memory_snapshot(cfg: ProfilingConfig, job_dir: str, *, global_step: int = 0):
    if not cfg.enable_memory_snapshot:
        yield None
        return
    d = os.path.join(job_dir, "memory_snapshot")
    os.makedirs(d, exist_ok=True)
    prof = MemoryProfiler(cfg, d, global_step)
    try:
        yield prof
    except torch.cuda.OutOfMemoryError:
        prof.step(exit_ctx=True)
        raise
