"""Straggler detection: which rank is slow, and is this rank slower than it used to be.

Parity target: ``StragglerDetectorV2`` (cosmos_predict2/_src/imaginaire/utils/misc.py:539-667), which wraps an external
CUPTI-based package. This implementation has no external dependency: named sections are timed on the device with CUDA
events recorded on the current stream (host clock on CPU), so a section measures the GPU work enqueued inside it
regardless of where the host synchronises; every ``report_freq`` iterations the per-section medians are all-gathered and

* the relative score of rank r is  min over ranks of the total section time / total section time of r   (1.0 = fastest),
* the individual score of a rank is  its best total so far / its current total                           (1.0 = as fast as ever).

Ranks whose relative score is below ``1 / max_diff`` are stragglers; ``slowdown_count`` raises after the same condition
has been seen ``thres`` reports in a row (``raise_error``).
"""

from __future__ import annotations

import contextlib
import time
from collections import defaultdict
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class BufferCnt:
    """Counts consecutive positives; ``__call__(flag)`` returns True when the count exceeds ``thres``."""

    def __init__(self, thres: int = 10, reset_over_thres: bool = False):
        self.cnt, self.thres, self.reset_over_thres = 0, thres, reset_over_thres

    def __call__(self, expre: bool, thres: Optional[int] = None) -> bool:
        self.cnt = self.cnt + 1 if expre else 0
        thres = self.thres if thres is None else thres
        if self.cnt >= thres:
            if self.reset_over_thres:
                self.cnt = 0
            return True
        return False

    def reset(self):
        self.cnt = 0


@dataclass
class StragglerReport:
    sections: List[str]
    section_ms: torch.Tensor                      # [world, n_sections] median ms per section
    gpu_relative_perf_scores: Dict[int, float]
    gpu_individual_perf_scores: Dict[int, float]

    def identify_stragglers(self, gpu_rel_threshold: float = 0.7, gpu_indiv_threshold: float = 0.7) -> Dict[str, List[int]]:
        return {"straggler_gpus_relative": [r for r, s in self.gpu_relative_perf_scores.items() if s < gpu_rel_threshold],
                "straggler_gpus_individual": [r for r, s in self.gpu_individual_perf_scores.items() if s < gpu_indiv_threshold]}


class StragglerDetector:
    def __init__(self, enabled: bool = True, report_freq: int = 100, profile_freq: int = 1, max_diff: float = 2.0, raise_error: bool = True,
                 group=None, slowdown_thres: int = 10):
        self.enabled, self.report_freq, self.profile_freq = enabled, report_freq, max(1, profile_freq)
        self.max_diff, self.raise_error, self.group = max_diff, raise_error, group
        self.name = type(self).__name__
        self.slowdown_count = BufferCnt(thres=slowdown_thres, reset_over_thres=True)
        self._pending: Dict[str, List] = defaultdict(list)
        self._samples: Dict[str, List[float]] = defaultdict(list)
        self._best_total: Optional[float] = None
        self._calls = 0

    def initialize(self):
        self._pending.clear()
        self._samples.clear()

    @contextlib.contextmanager
    def profile_section(self, name: str, section_enabled: bool = True, profile_cuda: bool = True):
        self._calls += 1
        if not (self.enabled and section_enabled) or (self._calls % self.profile_freq):
            yield
            return
        if profile_cuda and torch.cuda.is_available():
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            try:
                yield
            finally:
                b.record()
                self._pending[name].append((a, b))
        else:
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._samples[name].append((time.perf_counter() - t0) * 1e3)

    def _drain(self):
        for name, evs in self._pending.items():
            for a, b in evs:
                b.synchronize()
                self._samples[name].append(a.elapsed_time(b))
        self._pending.clear()

    def generate_report(self, iteration: int) -> Optional[StragglerReport]:
        """Collective over the group on report iterations (every rank must call it). Returns the report on every rank."""
        if not self.enabled or iteration % self.report_freq != 0:
            return None
        self._drain()
        names = sorted(self._samples)
        if dist.is_available() and dist.is_initialized():      # all ranks must agree on the section list
            gathered: List = [None] * dist.get_world_size(self.group)
            dist.all_gather_object(gathered, names, group=self.group)
            names = sorted(set().union(*map(set, gathered)))
        local = torch.tensor([float(torch.tensor(self._samples[n]).median()) if self._samples.get(n) else 0.0 for n in names],
                             dtype=torch.float64)
        self._samples.clear()
        if dist.is_available() and dist.is_initialized():
            world = dist.get_world_size(self.group)
            dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(self.group) == "nccl" else torch.device("cpu")
            buf = [torch.zeros_like(local, device=dev) for _ in range(world)]
            dist.all_gather(buf, local.to(dev), group=self.group)
            table = torch.stack([b.cpu() for b in buf])
            rank = dist.get_rank(self.group)
        else:
            table, rank = local[None], 0
        totals = table.sum(dim=1).clamp_min(1e-9)
        rel = {r: float(totals.min() / totals[r]) for r in range(table.shape[0])}
        mine = float(totals[rank])
        self._best_total = mine if self._best_total is None else min(self._best_total, mine)
        indiv_local = torch.tensor([self._best_total / mine], dtype=torch.float64)
        if dist.is_available() and dist.is_initialized():
            ib = [torch.zeros_like(indiv_local, device=dev) for _ in range(table.shape[0])]
            dist.all_gather(ib, indiv_local.to(dev), group=self.group)
            indiv = {r: float(x) for r, x in enumerate(ib)}
        else:
            indiv = {0: float(indiv_local)}
        report = StragglerReport(names, table, rel, indiv)
        found = report.identify_stragglers(gpu_rel_threshold=1.0 / self.max_diff)["straggler_gpus_relative"]
        if self.slowdown_count(len(found) > 0) and self.raise_error:
            raise RuntimeError(f"stragglers detected repeatedly: ranks {found}, relative scores {rel}")
        return report

    def wandb_info(self, report: StragglerReport) -> Dict[str, float]:
        info = {f"{self.name}/relative_gpu_perf_{r}": s for r, s in report.gpu_relative_perf_scores.items()}
        for j, key in enumerate(report.sections):
            for r in range(report.section_ms.shape[0]):
                info[f"{self.name}/{key}_{r:03d}"] = float(report.section_ms[r, j]) / 1e3
            info[f"slowest_rank/slowest_{key}_rank"] = int(report.section_ms[:, j].argmax())
        scores = torch.tensor([report.gpu_relative_perf_scores[r] for r in sorted(report.gpu_relative_perf_scores)])
        info[f"slowest_rank/{self.name}_rank"] = int(scores.argmin())
        info[f"slowest_rank/{self.name}_relative_perf"] = float(scores.min())
        return info


StragglerDetectorV2 = StragglerDetector
