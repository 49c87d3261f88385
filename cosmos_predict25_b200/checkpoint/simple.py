"""Non-distributed checkpointers: ``DummyCheckpointer`` (no I/O; tests, smoke runs) and ``PtCheckpointer``, the legacy
layout ``iter_%09d_{model,optim,scheduler}.pt`` + ``iter_%09d.pt`` (trainer state) + ``latest_checkpoint.txt`` written
by the first data-parallel rank from host copies on a background thread.

Parity targets: cosmos_predict2/_src/imaginaire/checkpointer/dummy.py:25, .../ddp.py:35-446 (layout, resume priority,
``strict_resume``, ``scheduler.last_epoch = iteration``, background thread save).
"""

from __future__ import annotations

import os
import threading
from typing import Optional

import torch
import torch.distributed as dist

from ..utils import log


def _rank():
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _optim_state(optimizer) -> dict:
    """Optimizer state that ONE file can restore on every rank. A sharded optimizer's ``state_dict`` holds only the
    calling rank's rows; writing rank 0's copy and loading it everywhere would put rank 0's rows into every shard.
    Such optimizers expose ``consolidated_state_dict`` (a collective that gathers full tensors), used here."""
    if optimizer is None:
        return {}
    if hasattr(optimizer, "consolidated_state_dict"):
        return optimizer.consolidated_state_dict()
    return optimizer.state_dict()


class DummyCheckpointer:
    def __init__(self, *a, **k):
        pass

    def save(self, model, optimizer, scheduler, iteration, grad_scaler=None, trainer=None):
        pass

    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, trainer=None) -> int:
        return 0

    def finalize(self):
        pass


class PtCheckpointer:
    def __init__(self, config_checkpoint, job_dir: str, callbacks=None):
        self.cfg = config_checkpoint
        self.dir = os.path.join(job_dir, "checkpoints")
        self.load_path = config_checkpoint.get("load_path") or None
        self.load_training_state = config_checkpoint.get("load_training_state", False)
        self.only_load_scheduler_state = config_checkpoint.get("only_load_scheduler_state", False)
        self.strict_resume = config_checkpoint.get("strict_resume", True)
        self.callbacks = callbacks
        self._thread: Optional[threading.Thread] = None

    def _latest(self):
        f = os.path.join(self.dir, "latest_checkpoint.txt")
        return open(f).read().strip() if os.path.exists(f) else None

    def save(self, model, optimizer, scheduler, iteration, grad_scaler=None, trainer=None):
        self.finalize()
        name = f"iter_{iteration:09d}"
        cpu = lambda sd: {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in sd.items()}
        parts = {"model": cpu(model.state_dict()), "optim": cpu(_optim_state(optimizer)),
                 "scheduler": scheduler.state_dict() if scheduler is not None else {}}
        trainer_state = {"iteration": iteration, "grad_scaler": grad_scaler.state_dict() if grad_scaler is not None else {}}

        def work():
            if _rank() == 0:
                os.makedirs(self.dir, exist_ok=True)
                for k, v in parts.items():
                    torch.save(v, os.path.join(self.dir, f"{name}_{k}.pt"))
                torch.save(trainer_state, os.path.join(self.dir, f"{name}.pt"))
                with open(os.path.join(self.dir, "latest_checkpoint.txt"), "w") as f:
                    f.write(name + "\n")
                log.info(f"saved checkpoint {name}")

        self._thread = threading.Thread(target=work, daemon=True)
        self._thread.start()

    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, trainer=None) -> int:
        latest = self._latest()
        if latest is not None:
            base, resume = os.path.join(self.dir, latest), {"model", "optim", "scheduler", "trainer"}
        elif self.load_path:
            base = self.load_path[:-3] if self.load_path.endswith(".pt") else self.load_path
            if base.endswith("_model"):
                base = base[:-6]
            resume = {"model", "optim", "scheduler", "trainer"} if self.load_training_state else \
                ({"model", "scheduler"} if self.only_load_scheduler_state else {"model"})
        else:
            return 0
        iteration = 0
        mp = base + "_model.pt" if os.path.exists(base + "_model.pt") else base + ".pt"
        if "model" in resume:
            sd = torch.load(mp, map_location="cpu", weights_only=False)
            model.load_state_dict(sd, strict=self.strict_resume)
        if "optim" in resume and optimizer is not None and os.path.exists(base + "_optim.pt"):
            optimizer.load_state_dict(torch.load(base + "_optim.pt", map_location="cpu", weights_only=False))
        if "trainer" in resume and os.path.exists(base + ".pt") and os.path.exists(base + "_model.pt"):
            trainer_state = torch.load(base + ".pt", map_location="cpu", weights_only=False)
            iteration = int(trainer_state["iteration"])
            if grad_scaler is not None and trainer_state.get("grad_scaler"):
                grad_scaler.load_state_dict(trainer_state["grad_scaler"])
        if "scheduler" in resume and scheduler is not None and os.path.exists(base + "_scheduler.pt"):
            scheduler.load_state_dict(torch.load(base + "_scheduler.pt", map_location="cpu", weights_only=False))
            if iteration:
                scheduler.last_epoch = iteration
        log.info(f"loaded checkpoint {base} at iteration {iteration}")
        return iteration

    def finalize(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None


class ModelParallelPtCheckpointer(PtCheckpointer):
    """``PtCheckpointer`` for models split over a model-parallel group: every model-parallel rank of the first data-parallel
    replica writes its own ``iter_%09d_{model,optim}_mp_{rank}.pt``; scheduler and trainer state are written once
    (cosmos_predict2/_src/imaginaire/checkpointer/tp.py:20-42). ``mp_rank`` / ``dp_rank`` are callables so that the class
    works with any group layout (and without a process group in tests)."""

    def __init__(self, config_checkpoint, job_dir: str, callbacks=None, mp_rank=lambda: 0, dp_rank=lambda: 0):
        super().__init__(config_checkpoint, job_dir, callbacks)
        self.mp_rank, self.dp_rank = mp_rank, dp_rank

    def _suffix(self, key: str) -> str:
        return f"_{key}_mp_{self.mp_rank()}.pt" if key in ("model", "optim") else f"_{key}.pt"

    def _extra_model_state(self, model) -> dict:
        return {}

    def _load_extra_model_state(self, model, sd: dict) -> dict:
        return sd

    def save(self, model, optimizer, scheduler, iteration, grad_scaler=None, trainer=None):
        self.finalize()
        name = f"iter_{iteration:09d}"
        cpu = lambda sd: {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in sd.items()}
        model_sd = cpu(model.state_dict())
        model_sd.update(self._extra_model_state(model))
        parts = {"model": model_sd, "optim": cpu(_optim_state(optimizer)),
                 "scheduler": scheduler.state_dict() if scheduler is not None else {}}
        first_replica, first_mp = self.dp_rank() == 0, self.mp_rank() == 0

        def work():
            if not first_replica:
                return
            os.makedirs(self.dir, exist_ok=True)
            for k in ("model", "optim"):
                torch.save(parts[k], os.path.join(self.dir, name + self._suffix(k)))
            if first_mp:
                torch.save(parts["scheduler"], os.path.join(self.dir, name + self._suffix("scheduler")))
                torch.save({"iteration": iteration, "grad_scaler": {}}, os.path.join(self.dir, f"{name}.pt"))
                with open(os.path.join(self.dir, "latest_checkpoint.txt"), "w") as f:
                    f.write(name + "\n")

        self._thread = threading.Thread(target=work, daemon=True)
        self._thread.start()

    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, trainer=None) -> int:
        latest = self._latest()
        if latest is None:
            return 0
        base = os.path.join(self.dir, latest)
        sd = torch.load(base + self._suffix("model"), map_location="cpu", weights_only=False)
        sd = self._load_extra_model_state(model, sd)
        model.load_state_dict(sd, strict=self.strict_resume)
        if optimizer is not None and os.path.exists(base + self._suffix("optim")):
            optimizer.load_state_dict(torch.load(base + self._suffix("optim"), map_location="cpu", weights_only=False))
        iteration = int(torch.load(base + ".pt", map_location="cpu", weights_only=False)["iteration"])
        if scheduler is not None and os.path.exists(base + self._suffix("scheduler")):
            scheduler.load_state_dict(torch.load(base + self._suffix("scheduler"), map_location="cpu", weights_only=False))
        return iteration


class ModelParallelEmaPtCheckpointer(ModelParallelPtCheckpointer):
    """Model-parallel checkpointer whose model file also carries the EMA weights under the key ``ema``
    (cosmos_predict2/_src/imaginaire/checkpointer/tp_ema.py:26-90). ``get_ema`` / ``set_ema`` read and write the EMA state
    dict of the model (by default ``model.ema_state_dict()`` / ``model.load_ema_state_dict(sd)`` when present)."""

    def __init__(self, *a, get_ema=None, set_ema=None, **k):
        super().__init__(*a, **k)
        self.get_ema, self.set_ema = get_ema, set_ema

    def _extra_model_state(self, model) -> dict:
        getter = self.get_ema or getattr(model, "ema_state_dict", None)
        if getter is None:
            return {}
        ema = getter() if self.get_ema is None else getter(model)
        return {"ema": {k: (v.detach().cpu() if isinstance(v, torch.Tensor) else v) for k, v in ema.items()}}

    def _load_extra_model_state(self, model, sd: dict) -> dict:
        sd = dict(sd)
        ema = sd.pop("ema", None)
        if ema is not None:
            if self.set_ema is not None:
                self.set_ema(model, ema)
            elif hasattr(model, "load_ema_state_dict"):
                model.load_ema_state_dict(ema)
        return sd


def broadcast_object(obj, src: int = 0, group=None):
    """Broadcast a picklable object; a no-op without a process group (checkpointer/safe_broadcast.py:27 of the reference
    guards the same call against un-initialised process groups)."""
    if not (dist.is_available() and dist.is_initialized()):
        return obj
    box = [obj]
    dist.broadcast_object_list(box, src=src, group=group)
    return box[0]
