"""Callback bus and the stock callbacks.

Parity targets: ``Callback`` / ``CallBackGroup`` (cosmos_predict2/_src/imaginaire/utils/callback.py:47-308),
``EveryN`` (cosmos_predict2/_src/imaginaire/callbacks/every_n.py:27), ``IterSpeed``
(cosmos_predict2/_src/predict2/callbacks/iter_speed.py:30-106), ``HeartBeat`` (.../heart_beat.py:29-106),
``DeviceMonitor`` (.../device_monitor.py:80-196), ``GradClip`` (.../grad_clip.py:56-112),
``ManualGarbageCollection`` (cosmos_predict2/_src/imaginaire/callbacks/manual_gc.py:22-49),
``WandbCallback`` (cosmos_predict2/_src/predict2/callbacks/wandb_log.py:59-242, logging to JSONL when
wandb is unavailable/disabled), ``DetailedDataLoadingSpeedMonitor`` (.../dataloading_monitor.py:28-95),
``NVTXCallback`` and ``LowPrecisionCallback`` (callback.py:500-608).
"""

from __future__ import annotations

import gc
import json
import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist

from ..utils import log


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


class Callback:
    """Base class: every hook is a no-op. ``trainer`` and ``config`` are attached by the group."""

    trainer = None
    config = None

    def on_train_start(self, model, iteration: int = 0): ...
    def on_training_step_start(self, model, data, iteration: int = 0): ...
    def on_before_forward(self, iteration: int = 0): ...
    def on_after_forward(self, iteration: int = 0): ...
    def on_before_backward(self, model, loss, iteration: int = 0): ...
    def on_after_backward(self, model, iteration: int = 0): ...
    def on_before_dataloading(self, iteration: int = 0): ...
    def on_after_dataloading(self, iteration: int = 0): ...
    def on_optimizer_init_start(self): ...
    def on_optimizer_init_end(self): ...
    def on_before_optimizer_step(self, model, optimizer, scheduler, iteration: int = 0): ...
    def on_before_zero_grad(self, model, optimizer, scheduler, iteration: int = 0): ...
    def on_training_step_end(self, model, data, output, loss, iteration: int = 0): ...
    def on_validation_start(self, model, dataloader_val, iteration: int = 0): ...
    def on_validation_step_start(self, model, data, iteration: int = 0): ...
    def on_validation_step_end(self, model, data, output, loss, iteration: int = 0): ...
    def on_validation_end(self, model, iteration: int = 0): ...
    def on_load_checkpoint_start(self, model): ...
    def on_load_checkpoint_end(self, model, iteration: int = 0, checkpoint_path: Optional[str] = None): ...
    def on_load_checkpoint(self, model, state_dict): ...
    def on_save_checkpoint_start(self, model, iteration: int = 0): ...
    def on_save_checkpoint_end(self, model, iteration: int = 0): ...
    def on_save_checkpoint_success(self, iteration: int = 0, elapsed_time: float = 0): ...
    def on_save_checkpoint(self, model, state_dict): ...
    def on_train_end(self, model, iteration: int = 0): ...
    def on_app_end(self): ...


class CallBackGroup:
    """Fans every hook out to the registered callbacks in order."""

    def __init__(self, callbacks: List[Callback], trainer=None, config=None):
        self._callbacks = list(callbacks)
        for cb in self._callbacks:
            cb.trainer, cb.config = trainer, config

    def append(self, cb: Callback):
        self._callbacks.append(cb)

    def __getattr__(self, name: str):
        if not name.startswith("on_"):
            raise AttributeError(name)

        def fan_out(*args, **kwargs):
            for cb in self._callbacks:
                getattr(cb, name)(*args, **kwargs)

        return fan_out


class EveryN(Callback):
    """Runs ``every_n_impl`` each ``every_n`` iterations (and optionally at iteration 1), with a barrier after."""

    def __init__(self, every_n: Optional[int] = None, step_size: int = 1, barrier_after_run: bool = True,
                 run_at_start: bool = False):
        self.every_n = every_n
        self.step_size = step_size
        self.barrier_after_run = barrier_after_run
        self.run_at_start = run_at_start
        if every_n == 0:
            self.every_n = None

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        if self.every_n is None:
            return
        gstep = iteration // self.step_size
        should = (iteration == 1 and self.run_at_start) or (gstep % self.every_n == 0 and iteration % self.step_size == 0)
        if should:
            self.every_n_impl(self.trainer, model, data, output, loss, iteration)
            if self.barrier_after_run and _world() > 1:
                dist.barrier()

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        raise NotImplementedError


class IterSpeed(EveryN):
    """Seconds per iteration over the window; the first ``hit_thres`` iterations are reported one by one
    (with a device synchronise) in the exact format the reference's golden-loss test parses:
    ``Iteration k: Hit counter: k/5 | Loss: x.xxxx | Time: y.yys``."""

    def __init__(self, every_n: int = 20, hit_thres: int = 5, save_s3: bool = False):
        super().__init__(every_n, barrier_after_run=False)
        self.hit_thres = hit_thres
        self.hit_counter = 0
        self.time = None
        self.last_iter = 0
        self.history: List[Dict[str, float]] = []

    def on_train_start(self, model, iteration: int = 0):
        self.time = time.time()
        self.last_iter = iteration

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        if self.hit_counter < self.hit_thres:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            now = time.time()
            self.hit_counter += 1
            log.info(f"Iteration {iteration}: Hit counter: {self.hit_counter}/{self.hit_thres} | "
                     f"Loss: {float(loss):.4f} | Time: {now - (self.time or now):.2f}s")
            self.time, self.last_iter = now, iteration
            return
        super().on_training_step_end(model, data, output, loss, iteration)

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        now = time.time()
        n = max(iteration - self.last_iter, 1)
        spi = (now - self.time) / n
        self.history.append({"iteration": iteration, "sec_per_iter": spi})
        log.info(f"{iteration} : iter_speed {spi:.2f} seconds per iteration | Loss: {float(loss):.4f}")
        self.time, self.last_iter = now, iteration


class HeartBeat(EveryN):
    """Writes a timestamp file at most every ``update_interval_in_minutes`` so an external supervisor can
    detect a dead job."""

    def __init__(self, every_n: int = 10, update_interval_in_minutes: float = 20, save_path: Optional[str] = None):
        super().__init__(every_n, barrier_after_run=False)
        self.interval = update_interval_in_minutes * 60
        self.save_path = save_path
        self.last = 0.0

    def _write(self, tag: str, iteration: int):
        if _rank() != 0:
            return
        path = self.save_path or os.path.join(self.config.output_dir if self.config else ".", "heart_beat.json")
        os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
        with open(path, "w") as f:
            json.dump({"time": time.time(), "iteration": iteration, "event": tag}, f)
        self.last = time.time()

    def on_train_start(self, model, iteration: int = 0):
        self._write("train_start", iteration)

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        if time.time() - self.last >= self.interval:
            self._write("heartbeat", iteration)

    def on_train_end(self, model, iteration: int = 0):
        self._write("train_end", iteration)


class DeviceMonitor(EveryN):
    """Host RSS, peak device memory and (when NVML is importable) temperature / power / utilisation /
    SM clock, gathered from all ranks to rank 0. Reads settings only; never changes them."""

    def __init__(self, every_n: int = 200, log_memory_detail: bool = False):
        super().__init__(every_n, barrier_after_run=False)
        self.records: List[Dict[str, Any]] = []

    def sample(self) -> Dict[str, float]:
        import psutil
        rec = {"cpu_rss_gb": psutil.Process().memory_info().rss / 2 ** 30}
        if torch.cuda.is_available():
            rec["peak_gpu_mem_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
            rec["peak_gpu_mem_reserved_gb"] = torch.cuda.max_memory_reserved() / 2 ** 30
            try:
                import pynvml
                pynvml.nvmlInit()
                h = pynvml.nvmlDeviceGetHandleByIndex(torch.cuda.current_device())
                mem = pynvml.nvmlDeviceGetMemoryInfo(h)
                rec.update(nvml_used_gb=mem.used / 2 ** 30, nvml_free_gb=mem.free / 2 ** 30,
                           temperature=pynvml.nvmlDeviceGetTemperature(h, pynvml.NVML_TEMPERATURE_GPU),
                           power_w=pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0,
                           util=pynvml.nvmlDeviceGetUtilizationRates(h).gpu,
                           sm_clock_mhz=pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
            except Exception:
                pass
        return rec

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        rec = self.sample()
        if _world() > 1:
            gathered = [None] * _world()
            dist.all_gather_object(gathered, rec)
        else:
            gathered = [rec]
        if _rank() == 0:
            self.records.append({"iteration": iteration, "ranks": gathered})
            log.info(f"{iteration} : device monitor " + ", ".join(f"{k}={v:.2f}" for k, v in gathered[0].items()))


class GradClip(Callback):
    """Sets the clipping threshold the optimizer kernel applies and records the global gradient norm.
    NaN/Inf scrubbing and the clip itself run inside the fused reduce/optimizer kernels."""

    def __init__(self, clip_norm: float = 1.0, force_finite: bool = True):
        self.clip_norm = clip_norm
        self.force_finite = force_finite
        self.history: List[torch.Tensor] = []

    def on_before_optimizer_step(self, model, optimizer, scheduler, iteration: int = 0):
        optimizer.max_grad_norm = self.clip_norm

    def on_before_zero_grad(self, model, optimizer, scheduler, iteration: int = 0):
        if optimizer.last_grad_norm is not None:
            self.history.append(optimizer.last_grad_norm.detach())
            if len(self.history) > 1000:
                self.history = self.history[-1000:]


class ManualGarbageCollection(EveryN):
    """Disables Python's automatic GC and collects generation 1 every N steps so all ranks pause together."""

    def __init__(self, every_n: int = 5, warm_up: int = 5):
        super().__init__(every_n, barrier_after_run=False)
        self.warm_up = warm_up
        self.disabled = False

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        if iteration < self.warm_up:
            return
        if not self.disabled:
            gc.disable()
            self.disabled = True
        super().on_training_step_end(model, data, output, loss, iteration)

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        gc.collect(1)

    def on_train_end(self, model, iteration: int = 0):
        gc.enable()


class WandbCallback(Callback):
    """Window-averaged, all-reduced loss / lr / timers / unstable-loss counts. Writes to wandb when it is
    importable and ``mode == 'online'``; always appends to ``<output_dir>/metrics.jsonl``."""

    def __init__(self, logging_iter: int = 20, mode: str = "disabled", project: str = "cosmos_b200", name: str = "run"):
        self.logging_iter = logging_iter
        self.mode = mode
        self.project, self.name = project, name
        self.losses: List[torch.Tensor] = []
        self.unstable = 0
        self._wandb = None

    def on_train_start(self, model, iteration: int = 0):
        if self.mode == "online" and _rank() == 0:
            try:
                import wandb
                self._wandb = wandb.init(project=self.project, name=self.name, resume="allow", id=self._run_id())
            except Exception as e:  # no network: keep the JSONL sink
                log.warning(f"wandb unavailable ({e}); logging to metrics.jsonl only")

    def _run_id(self) -> str:
        """The run id lives next to the checkpoints, so a job restarted from its checkpoint continues the same run
        (cosmos_predict2/_src/imaginaire/utils/wandb_util.py:36-118)."""
        import uuid
        out_dir = self.config.output_dir if self.config else "."
        path = os.path.join(out_dir, "checkpoints", "wandb_id.txt")
        if os.path.exists(path):
            rid = open(path).read().strip()
            if rid:
                return rid
        rid = uuid.uuid4().hex[:8]
        os.makedirs(os.path.dirname(path), exist_ok=True)
        with open(path, "w") as f:
            f.write(rid + "\n")
        return rid

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        l = loss.detach().float()
        self.losses.append(l)
        if iteration % self.logging_iter != 0 or not self.losses:
            return
        stacked = torch.stack(self.losses)
        finite = torch.isfinite(stacked)
        n_bad = int((~finite).sum())
        mean = stacked[finite].mean() if finite.any() else torch.zeros((), device=stacked.device)
        if _world() > 1:
            buf = torch.stack([mean, torch.tensor(float(n_bad), device=mean.device)])
            dist.all_reduce(buf)
            mean, n_bad = buf[0] / _world(), int(buf[1])
        self.unstable += n_bad
        rec = {"iteration": iteration, "train/loss": float(mean), "train/unstable_count": self.unstable}
        if self.trainer is not None:
            rec["optim/lr"] = self.trainer.scheduler.get_last_lr()[0]
            for k, v in self.trainer.timer.compute_average_results().items():
                rec[f"timer/{k}"] = v
            self.trainer.timer.reset()
            if self.trainer.optimizer.last_grad_norm is not None:
                rec["clip_grad_norm"] = float(self.trainer.optimizer.last_grad_norm)
        self.losses = []
        if _rank() == 0:
            out_dir = self.config.output_dir if self.config else "."
            with open(os.path.join(out_dir, "metrics.jsonl"), "a") as f:
                f.write(json.dumps(rec) + "\n")
            if self._wandb is not None:
                self._wandb.log(rec, step=iteration)

    def on_train_end(self, model, iteration: int = 0):
        if self._wandb is not None:
            self._wandb.finish()


class DetailedDataLoadingSpeedMonitor(EveryN):
    """Time spent waiting for the dataloader vs. stepping, gathered over ranks."""

    def __init__(self, every_n: int = 100):
        super().__init__(every_n, barrier_after_run=False)
        self.t_step_end = None
        self.wait = 0.0
        self.step = 0.0
        self._t0 = None

    def on_training_step_start(self, model, data, iteration: int = 0):
        now = time.time()
        if self.t_step_end is not None:
            self.wait += now - self.t_step_end
        self._t0 = now

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        now = time.time()
        if self._t0 is not None:
            self.step += now - self._t0
        self.t_step_end = now
        super().on_training_step_end(model, data, output, loss, iteration)

    def every_n_impl(self, trainer, model, data, output, loss, iteration):
        t = torch.tensor([self.wait, self.step], dtype=torch.float64)
        if _world() > 1:
            dev = model.device_ if hasattr(model, "device_") else "cpu"
            parts = [torch.zeros(2, dtype=torch.float64, device=dev) for _ in range(_world())]
            dist.all_gather(parts, t.to(dev))
            t = torch.stack(parts).mean(0).cpu()
        log.info(f"{iteration} : dataloading wait {t[0]:.2f}s, step {t[1]:.2f}s over the window")
        self.wait = self.step = 0.0


class NVTXCallback(Callback):
    """NVTX ranges around the step phases (visible in Nsight Systems)."""

    def __init__(self, synchronize: bool = False):
        self.sync = synchronize

    def _push(self, name):
        if torch.cuda.is_available():
            if self.sync:
                torch.cuda.synchronize()
            torch.cuda.nvtx.range_push(name)

    def _pop(self):
        if torch.cuda.is_available():
            if self.sync:
                torch.cuda.synchronize()
            torch.cuda.nvtx.range_pop()

    def on_training_step_start(self, model, data, iteration: int = 0):
        self._push(f"step_{iteration}")

    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        self._pop()


class LowPrecisionCallback(Callback):
    """Casts floating inputs of a batch to the model precision (skipping keys that must stay fp32). The
    master->bf16 parameter copy of the reference's version happens inside the optimizer kernel here."""

    def __init__(self, update_iter: int = 1, skip_keys=("fps", "padding_mask", "latents")):
        self.skip = set(skip_keys)

    def on_training_step_start(self, model, data, iteration: int = 0):
        for k, v in list(data.items()):
            if isinstance(v, torch.Tensor) and v.is_floating_point() and k not in self.skip:
                data[k] = v.to(model.precision)
