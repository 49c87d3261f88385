"""Optimizer and learning-rate schedule.

``ShardedAdamW`` is the optimizer-shaped facade over ``ShardedEngine.step``: AdamW with fp32 master
weights on the local shards, global-norm clipping, EMA and the bf16 write-back in one fused pass
per unit. It replaces the reference's FusedAdam-on-DTensor + separate clip/EMA/copy passes
(cosmos_predict2/_src/predict2/utils/fused_adam_dtensor.py:23-408,
cosmos_predict2/_src/predict2/utils/optim_instantiate.py:39-89). Unlike the reference, the fp32
masters ARE part of the optimizer state dict, so a resume is bit-exact.

``LambdaLinearScheduler`` / ``LambdaWarmUpCosineScheduler`` reproduce the warm-up + linear (or
cosine) multiplier of cosmos_predict2/_src/common/functional/lr_scheduler.py:157-178.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence

import numpy as np
import torch


@dataclass
class OptimizerConfig:
    lr: float = 2 ** -14.5
    betas: Sequence[float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 1e-3
    max_grad_norm: Optional[float] = 1.0


@dataclass
class SchedulerConfig:
    kind: str = "lambdalinear"        # lambdalinear | warmup_cosine | constant
    warm_up_steps: Sequence[int] = (2000,)
    cycle_lengths: Sequence[int] = (10_000_000,)
    f_start: Sequence[float] = (1.0e-6,)
    f_max: Sequence[float] = (1.0,)
    f_min: Sequence[float] = (1.0,)


class ShardedAdamW:
    """torch.optim-like facade (``param_groups``, ``step``, ``zero_grad``, ``state_dict``)."""

    def __init__(self, engine, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 max_grad_norm: Optional[float] = None):
        self.engine = engine
        self.defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay)
        self.param_groups: List[Dict[str, Any]] = [dict(self.defaults, params=[s.param for u in engine.units for s in u.slots],
                                                       initial_lr=lr)]
        self.max_grad_norm = max_grad_norm
        self.ema_beta: Optional[float] = None
        self.last_grad_norm: Optional[torch.Tensor] = None
        self.state: Dict = {}

    def step(self, closure=None):
        g = self.param_groups[0]
        self.last_grad_norm = self.engine.step(lr=g["lr"], betas=g["betas"], eps=g["eps"], weight_decay=g["weight_decay"],
                                               max_grad_norm=self.max_grad_norm, ema_beta=self.ema_beta)
        return None

    def zero_grad(self, set_to_none: bool = False):
        self.engine.zero_grad()

    def state_dict(self) -> Dict[str, Any]:
        """Flattened per-parameter state of the *local shard* (``state.<name>.<field>``) + hyper-parameters."""
        out: Dict[str, Any] = {}
        for which in ("exp_avg", "exp_avg_sq", "master"):
            for name, (local, shape, row0) in self.engine.sharded_state(which).items():
                out[f"state.{name}.{which}"] = local
        return self._hyper(out)

    def _hyper(self, out: Dict[str, Any]) -> Dict[str, Any]:
        out["state.step"] = torch.tensor(self.engine.step_count, dtype=torch.int64)
        g = self.param_groups[0]
        out["param_groups.lr"] = g["lr"]
        out["param_groups.betas"] = list(g["betas"])
        out["param_groups.eps"] = g["eps"]
        out["param_groups.weight_decay"] = g["weight_decay"]
        return out

    def consolidated_state_dict(self) -> Dict[str, Any]:
        """The same keys as ``state_dict`` but with every tensor gathered to its full (unsharded) shape. A collective
        over the shard group: every rank calls it and every rank gets the whole state, so a single-file checkpoint
        written by one rank restores all shards (the per-shard ``state_dict`` of one rank does not)."""
        out: Dict[str, Any] = {"consolidated": True}
        for which in ("exp_avg", "exp_avg_sq", "master"):
            for name, t in self.engine.full_state_dict(which).items():
                out[f"state.{name}.{which}"] = t
        return self._hyper(out)

    def load_consolidated_state_dict(self, sd: Dict[str, Any]):
        """Inverse of ``consolidated_state_dict``: every rank cuts its own rows out of the full tensors."""
        for which in ("exp_avg", "exp_avg_sq", "master"):
            part = {k[len("state."):-len(which) - 1]: v for k, v in sd.items()
                    if k.startswith("state.") and k.endswith("." + which)}
            if part:
                self.engine.load_full_state_dict(part, which=which, strict=False)
        self._load_hyper(sd)
        self.engine.restore_params()

    def load_state_dict(self, sd: Dict[str, Any]):
        if sd.get("consolidated", False):
            return self.load_consolidated_state_dict(sd)
        for which in ("exp_avg", "exp_avg_sq", "master"):
            for name, (local, shape, row0) in self.engine.sharded_state(which).items():
                key = f"state.{name}.{which}"
                if key in sd:
                    local.copy_(sd[key].to(local))
        self._load_hyper(sd)
        self.engine.restore_params()

    def _load_hyper(self, sd: Dict[str, Any]):
        if "state.step" in sd:
            self.engine.step_count = int(sd["state.step"])
        g = self.param_groups[0]
        for k in ("lr", "eps", "weight_decay"):
            if f"param_groups.{k}" in sd:
                g[k] = float(sd[f"param_groups.{k}"])
        if "param_groups.betas" in sd:
            g["betas"] = tuple(float(b) for b in sd["param_groups.betas"])


class LambdaLinearScheduler:
    """Piecewise multiplier over cycles: linear warm-up f_start->f_max, then linear f_max->f_min."""

    def __init__(self, warm_up_steps, f_min, f_max, f_start, cycle_lengths, verbosity_interval: int = 0):
        assert len(warm_up_steps) == len(f_min) == len(f_max) == len(f_start) == len(cycle_lengths)
        self.lr_warm_up_steps = list(warm_up_steps)
        self.f_start, self.f_min, self.f_max = list(f_start), list(f_min), list(f_max)
        self.cycle_lengths = list(cycle_lengths)
        self.cum_cycles = np.cumsum([0] + list(self.cycle_lengths))

    def find_in_interval(self, n: int) -> int:
        for i, cl in enumerate(self.cum_cycles[1:]):
            if n <= cl:
                return i
        return len(self.cycle_lengths) - 1

    def schedule(self, n: int) -> float:
        c = self.find_in_interval(n)
        n = n - self.cum_cycles[c]
        if n < self.lr_warm_up_steps[c]:
            return (self.f_max[c] - self.f_start[c]) / self.lr_warm_up_steps[c] * n + self.f_start[c]
        return self.f_min[c] + (self.f_max[c] - self.f_min[c]) * (self.cycle_lengths[c] - n) / (
            self.cycle_lengths[c] - self.lr_warm_up_steps[c])

    def __call__(self, n: int) -> float:
        return float(self.schedule(n))


class LambdaWarmUpCosineScheduler(LambdaLinearScheduler):
    def schedule(self, n: int) -> float:
        c = self.find_in_interval(n)
        n = n - self.cum_cycles[c]
        if n < self.lr_warm_up_steps[c]:
            return (self.f_max[c] - self.f_start[c]) / self.lr_warm_up_steps[c] * n + self.f_start[c]
        t = min((n - self.lr_warm_up_steps[c]) / (self.cycle_lengths[c] - self.lr_warm_up_steps[c]), 1.0)
        return self.f_min[c] + 0.5 * (self.f_max[c] - self.f_min[c]) * (1 + math.cos(t * math.pi))


class LambdaLR:
    """Multiplies each group's ``initial_lr`` by ``fn(last_epoch)`` (the torch LambdaLR contract)."""

    def __init__(self, optimizer, fn, last_epoch: int = -1):
        self.optimizer, self.fn = optimizer, fn
        self.last_epoch = last_epoch
        self.step()

    def step(self):
        self.last_epoch += 1
        for g in self.optimizer.param_groups:
            g["lr"] = g["initial_lr"] * self.fn(self.last_epoch)

    def get_last_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups]

    def state_dict(self):
        return {"last_epoch": self.last_epoch}

    def load_state_dict(self, sd):
        self.last_epoch = int(sd["last_epoch"])
        for g in self.optimizer.param_groups:
            g["lr"] = g["initial_lr"] * self.fn(self.last_epoch)


def build_optimizer(cfg: OptimizerConfig, engine) -> ShardedAdamW:
    cfg = cfg or OptimizerConfig()
    return ShardedAdamW(engine, lr=cfg.lr, betas=cfg.betas, eps=cfg.eps, weight_decay=cfg.weight_decay,
                        max_grad_norm=cfg.max_grad_norm)


def build_scheduler(cfg: SchedulerConfig, optimizer) -> LambdaLR:
    cfg = cfg or SchedulerConfig(kind="constant")
    if cfg.kind == "constant":
        return LambdaLR(optimizer, lambda n: 1.0)
    cls = {"lambdalinear": LambdaLinearScheduler, "warmup_cosine": LambdaWarmUpCosineScheduler}[cfg.kind]
    return LambdaLR(optimizer, cls(cfg.warm_up_steps, cfg.f_min, cfg.f_max, cfg.f_start, cfg.cycle_lengths))
