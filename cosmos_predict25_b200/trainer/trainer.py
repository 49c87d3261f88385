"""Training loop.

Parity target: ``ImaginaireTrainer`` (cosmos_predict2/_src/imaginaire/trainer.py:46-354): distributed
init, seeding, callback bus, checkpointer, gradient accumulation, section timers, SIGALRM watchdog,
validation, profiler hooks. The loop body itself is ``train_step``: the public single-step API
(host batch in, loss out) that tools and benchmarks call directly.

Differences by design: no GradScaler (bf16 compute with fp32 masters needs none; the field is kept in
the trainer checkpoint for format parity), gradient clipping / EMA / master-weight write-back happen
inside the optimizer kernel, and the host->device copy of a batch is issued from pinned memory on the
compute stream so it overlaps the previous step's optimizer.
"""

from __future__ import annotations

import os
import signal
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

from ..utils import log, misc
from .callbacks import Callback, CallBackGroup
from .optim import OptimizerConfig, SchedulerConfig


@dataclass
class TrainerConfig:
    max_iter: int = 1000
    grad_accum_iter: int = 1
    logging_iter: int = 20
    validation_iter: int = 0
    max_val_iter: Optional[int] = None
    save_iter: int = 0
    seed: int = 0
    timeout_period: int = 0            # seconds; 0 disables the SIGALRM watchdog
    run_validation: bool = False
    distributed_parallelism: str = "fsdp"   # fsdp | ddp: read by cli/train.py, which turns it into the shard / replicate groups
    cudnn_deterministic: bool = False
    memory_format: str = "preserve"
    profile: bool = False
    profile_freq: int = 0
    output_dir: str = field(default_factory=lambda: os.path.join(
        os.environ.get("IMAGINAIRE_OUTPUT_ROOT", "/tmp/imaginaire4-output"), "cosmos_b200", "default", "run"))


class Trainer:
    def __init__(self, config: TrainerConfig, model, optimizer_config: Optional[OptimizerConfig] = None,
                 scheduler_config: Optional[SchedulerConfig] = None, callbacks: Optional[List[Callback]] = None,
                 checkpointer=None):
        self.config = config
        self.model = model
        misc.set_random_seed(config.seed, by_rank=True)
        if config.cudnn_deterministic:
            torch.backends.cudnn.deterministic = True
            torch.backends.cudnn.benchmark = False
        torch.backends.cuda.matmul.allow_tf32 = True
        torch.backends.cudnn.allow_tf32 = True
        os.makedirs(config.output_dir, exist_ok=True)
        self.callbacks = CallBackGroup(callbacks or [], trainer=self, config=config)
        self.checkpointer = checkpointer
        if checkpointer is not None and getattr(checkpointer, "callbacks", 0) is None:
            checkpointer.callbacks = self.callbacks   # on_save_checkpoint_* / on_load_checkpoint_* reach the callback bus
        self.timer = misc.TrainingTimer()
        model.on_train_start()
        self.optimizer, self.scheduler = model.init_optimizer_scheduler(optimizer_config or OptimizerConfig(),
                                                                        scheduler_config or SchedulerConfig(kind="constant"))
        self.iteration = 0
        self.grad_accum_count = 0
        if checkpointer is not None:
            self.iteration = checkpointer.load(model, self.optimizer, self.scheduler, trainer=self)
        if config.timeout_period > 0:
            signal.signal(signal.SIGALRM, _timeout_handler)
        self._pinned_cache: Dict[str, torch.Tensor] = {}

    # ---- host -> device ---------------------------------------------------------------------------------
    def to_device(self, batch: Dict[str, Any]) -> Dict[str, Any]:
        dev = self.model.device_
        out = {}
        for k, v in batch.items():
            if isinstance(v, torch.Tensor) and v.device != dev:
                out[k] = v.to(dev, non_blocking=True)
            else:
                out[k] = v
        return out

    # ---- one optimisation step --------------------------------------------------------------------------
    def train_step(self, batch: Dict[str, Any], return_loss_tensor: bool = False):
        """Forward, backward and (on the accumulation boundary) the optimizer step for one host or
        device batch. Returns the loss as a Python float (a device->host read of 4 bytes) unless
        ``return_loss_tensor``."""
        cfg = self.config
        model = self.model
        batch = self.to_device(batch)
        self.callbacks.on_training_step_start(model, batch, iteration=self.iteration)
        last_micro = (self.grad_accum_count + 1) == cfg.grad_accum_iter
        engine = getattr(model, "engine", None)        # the sharded engine of the video models; a plain module has none
        if engine is not None:
            engine.set_requires_gradient_sync(last_micro)
        with self.timer("forward"):
            out, loss = model.training_step(batch, self.iteration)
        with self.timer("backward"):
            (loss / cfg.grad_accum_iter).backward()
        self.grad_accum_count += 1
        if last_micro:
            with self.timer("optimizer_step"):
                self.callbacks.on_before_optimizer_step(model, self.optimizer, self.scheduler, iteration=self.iteration)
                if engine is not None:
                    self.optimizer.ema_beta = model.ema_beta(self.iteration + 1) if model.config.ema.enabled else None
                self.optimizer.step()
                self.scheduler.step()
                self.callbacks.on_before_zero_grad(model, self.optimizer, self.scheduler, iteration=self.iteration)
                model.on_before_zero_grad(self.optimizer, self.scheduler, iteration=self.iteration)
                if engine is None:
                    self.optimizer.zero_grad(set_to_none=True)   # the engine's optimizer kernel clears its gradients itself
            self.grad_accum_count = 0
            self.iteration += 1
        if last_micro and cfg.logging_iter and self.iteration % cfg.logging_iter == 0:
            self.check_health()   # the logging callbacks synchronise on this iteration anyway
        self.callbacks.on_training_step_end(model, batch, out, loss, iteration=self.iteration)
        return loss.detach() if return_loss_tensor else float(loss.detach().float().item())

    def check_health(self) -> None:
        """Raise if a kernel with a bounded wait (peer barrier, exchange) gave up: its successors ran on stale data, so the
        run must stop before anything is saved."""
        engine = getattr(self.model, "engine", None)
        if engine is not None and hasattr(engine, "check_health"):
            engine.check_health()

    def _save(self) -> None:
        self.check_health()
        self.checkpointer.save(self.model, self.optimizer, self.scheduler, self.iteration, trainer=self)

    # ---- full loop ---------------------------------------------------------------------------------------------
    def train(self, dataloader_train: Iterable, dataloader_val: Optional[Iterable] = None):
        cfg = self.config
        self.callbacks.on_train_start(self.model, iteration=self.iteration)
        log.info(f"training from iteration {self.iteration} to {cfg.max_iter}")
        done = self.iteration >= cfg.max_iter
        try:
            self._loop(dataloader_train, dataloader_val, done)
        finally:
            if cfg.timeout_period > 0:
                signal.alarm(0)   # a pending alarm must not outlive the loop, whichever way it ends
        if self.checkpointer is not None and cfg.save_iter:
            if self.iteration % cfg.save_iter != 0:  # otherwise the loop has just written this iteration
                self._save()
            getattr(self.checkpointer, "close", self.checkpointer.finalize)()   # waits for the save in flight, ends a writer process
        self.check_health()
        self.callbacks.on_train_end(self.model, iteration=self.iteration)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()

    def _loop(self, dataloader_train: Iterable, dataloader_val: Optional[Iterable], done: bool) -> None:
        cfg = self.config
        while not done:
            data_iter = iter(dataloader_train)
            while True:
                with self.timer("dataloader_train"):
                    try:
                        batch = next(data_iter)
                    except StopIteration:
                        break
                if cfg.timeout_period > 0:
                    signal.alarm(cfg.timeout_period)
                before = self.iteration
                self.train_step(batch, return_loss_tensor=True)
                if self.iteration != before:
                    if cfg.save_iter and self.checkpointer is not None and self.iteration % cfg.save_iter == 0:
                        self._save()
                    if cfg.run_validation and cfg.validation_iter and dataloader_val is not None \
                            and self.iteration % cfg.validation_iter == 0:
                        self.validate(dataloader_val)
                if self.iteration >= cfg.max_iter:
                    done = True
                    break

    @torch.no_grad()
    def validate(self, dataloader_val: Iterable) -> float:
        self.callbacks.on_validation_start(self.model, dataloader_val, iteration=self.iteration)
        self.model.eval()
        losses = []
        with self.model.ema_scope("validation"):
            for i, batch in enumerate(dataloader_val):
                if self.config.max_val_iter is not None and i >= self.config.max_val_iter:
                    break
                batch = self.to_device(batch)
                self.callbacks.on_validation_step_start(self.model, batch, iteration=self.iteration)
                out, loss = self.model.training_step(batch, self.iteration)
                losses.append(loss.detach().float())
                self.callbacks.on_validation_step_end(self.model, batch, out, loss, iteration=self.iteration)
        self.model.train()
        mean = torch.stack(losses).mean() if losses else torch.zeros(())
        if dist.is_available() and dist.is_initialized():
            mean = mean.to(self.model.device_)
            dist.all_reduce(mean, op=dist.ReduceOp.AVG if mean.is_cuda else dist.ReduceOp.SUM)
            if not mean.is_cuda:
                mean /= dist.get_world_size()
        self.callbacks.on_validation_end(self.model, iteration=self.iteration)
        return float(mean)


def _timeout_handler(signum, frame):
    """Watchdog: the alarm is re-armed after every successful iteration; firing means a hung step."""
    raise TimeoutError("training step exceeded trainer.timeout_period seconds")


class ImaginaireTrainer:
    """The reference's entry object: built from the WHOLE config, then ``train(model, dataloader_train, dataloader_val)``
    (cosmos_predict2/_src/imaginaire/trainer.py:58-150). Construction joins the process group (NCCL on GPUs, gloo without),
    seeds every generator per rank, creates the job's output directory, the callback bus from ``config.trainer.callbacks`` and the
    checkpointer from ``config.checkpoint.type`` (the legacy ``.pt`` checkpointer when none is named). ``train`` hands over to
    ``Trainer``, the loop of this package; a model that lacks the video models' device attribute gets it from its parameters."""

    def __init__(self, config):
        from ..utils import distributed
        from ..utils.lazy_config import _locate, instantiate
        self.config = config
        distributed.init()
        t = config["trainer"]
        misc.set_random_seed(t.get("seed", 0), by_rank=True)
        self.output_dir = config.job_path_local
        os.makedirs(self.output_dir, exist_ok=True)
        cbs = [instantiate(v) for v in (t.get("callbacks") or {}).values() if v is not None]
        self.callbacks = CallBackGroup(cbs, trainer=self, config=config)
        kind = config["checkpoint"].get("type")
        if kind:
            cls = _locate(kind) if isinstance(kind, str) else kind
            self.checkpointer = cls() if cls.__name__ == "DummyCheckpointer" else cls(config["checkpoint"], self.output_dir, self.callbacks)
        else:
            from ..checkpoint.ddp import Checkpointer
            self.checkpointer = Checkpointer(config["checkpoint"], self.output_dir, self.callbacks)
        self.training_timer = misc.TrainingTimer()

    def _trainer_config(self) -> TrainerConfig:
        t, c = self.config["trainer"], self.config["checkpoint"]
        timeout = t.get("timeout_period", 0)
        return TrainerConfig(max_iter=t["max_iter"], grad_accum_iter=t.get("grad_accum_iter", 1), logging_iter=t["logging_iter"],
                             validation_iter=t.get("validation_iter", 0), max_val_iter=t.get("max_val_iter"),
                             save_iter=c.get("save_iter", 0), seed=t.get("seed", 0), timeout_period=timeout if timeout < 10 ** 8 else 0,
                             run_validation=t.get("run_validation", False), distributed_parallelism=t.get("distributed_parallelism", "ddp"),
                             cudnn_deterministic=(t.get("cudnn") or {}).get("deterministic", False), output_dir=self.output_dir)

    def train(self, model, dataloader_train, dataloader_val=None) -> None:
        from ..utils.lazy_config import is_lazy, instantiate
        if not hasattr(model, "device_"):
            p = next(model.parameters(), None)
            model.device_ = p.device if p is not None else torch.device("cpu")
        opt, sch = self.config.get("optimizer"), self.config.get("scheduler")
        opt = opt if is_lazy(opt) else instantiate(opt)
        sch = sch if is_lazy(sch) else instantiate(sch)
        inner = Trainer(self._trainer_config(), model, opt, sch, list(self.callbacks._callbacks), self.checkpointer)
        self.inner = inner
        model.train()
        inner.train(dataloader_train, dataloader_val)
