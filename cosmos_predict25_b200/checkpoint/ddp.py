"""The legacy ``.pt`` checkpointer behind the reference's calling convention.

``Checkpointer(config_checkpoint, config_job, callbacks)`` with ``save(model, optimizer, scheduler, grad_scaler, iteration)`` and
``load(model, optimizer, scheduler, grad_scaler) -> iteration``, ``checkpoint_dir_local`` and ``finalize()``
(cosmos_predict2/_src/imaginaire/checkpointer/ddp.py:35-440, base.py:28-175). Files are those of ``PtCheckpointer``
(``checkpoints/iter_%09d_{model,optim,scheduler}.pt``, ``iter_%09d.pt`` with the iteration and the gradient scaler's state,
``latest_checkpoint.txt``), so either class resumes what the other wrote. A model wrapped for data parallelism (``.module``) is
saved and loaded without the wrapper's prefix. With ``save_to_object_store.enabled`` the finished files are also copied under
``s3://<bucket>/<project>/<group>/<name>/checkpoints`` through easy_io; ``load_from_object_store.enabled`` fetches them from there
first when the local directory has no ``latest_checkpoint.txt``.
"""

from __future__ import annotations

import os
from typing import Optional

import torch

from ..utils import log
from .simple import PtCheckpointer, _rank


def _unwrap(model):
    return model.module if isinstance(model, torch.nn.parallel.DistributedDataParallel) else model


class Checkpointer(PtCheckpointer):
    KEYS_TO_SAVE = ["model", "optim", "scheduler", "trainer"]

    def __init__(self, config_checkpoint, config_job, callbacks=None, disable_async: bool = False):
        job_dir = config_job if isinstance(config_job, str) else config_job.path_local
        super().__init__(config_checkpoint, job_dir, callbacks)
        self.config_checkpoint = config_checkpoint
        self.disable_async = disable_async
        self._object_store_dirname = None if isinstance(config_job, str) else os.path.join(config_job.path, "checkpoints")
        save_store, load_store = config_checkpoint.get("save_to_object_store"), config_checkpoint.get("load_from_object_store")
        self.save_to_object_store = bool(getattr(save_store, "enabled", False))
        self.load_from_object_store = bool(getattr(load_store, "enabled", False))
        self._save_store, self._load_store = save_store, load_store
        self._pending_upload: Optional[str] = None

    @property
    def checkpoint_dir_local(self) -> str:
        return self.dir

    # ---- object store -----------------------------------------------------------------------------------------------------
    def _remote(self, store, name: str) -> str:
        return f"s3://{store.bucket}/{self._object_store_dirname}/{name}"

    def _backend(self, store) -> dict:
        return {"backend_args": {"backend": "s3", "s3_credential_path": store.credentials}}

    def _upload(self, name: str) -> None:
        from ..utils.easy_io import easy_io
        for suffix in ("_model.pt", "_optim.pt", "_scheduler.pt", ".pt"):
            easy_io.copyfile_from_local(os.path.join(self.dir, name + suffix), self._remote(self._save_store, name + suffix),
                                        **self._backend(self._save_store))
        easy_io.put_text(name + "\n", self._remote(self._save_store, "latest_checkpoint.txt"), **self._backend(self._save_store))

    def _download_latest(self) -> None:
        from ..utils.easy_io import easy_io
        kw = self._backend(self._load_store)
        latest = self._remote(self._load_store, "latest_checkpoint.txt")
        if not easy_io.exists(latest, **kw):
            return
        name = easy_io.get_text(latest, **kw).strip()
        os.makedirs(self.dir, exist_ok=True)
        for suffix in ("_model.pt", "_optim.pt", "_scheduler.pt", ".pt"):
            easy_io.copyfile_to_local(self._remote(self._load_store, name + suffix), os.path.join(self.dir, name + suffix), **kw)
        with open(os.path.join(self.dir, "latest_checkpoint.txt"), "w") as f:
            f.write(name + "\n")

    # ---- the reference's call order ---------------------------------------------------------------------------------------
    def save(self, model, optimizer, scheduler, grad_scaler=None, iteration: int = 0, trainer=None) -> None:
        if isinstance(grad_scaler, int):             # this package's trainer passes (..., iteration, grad_scaler=None)
            grad_scaler, iteration = (iteration if not isinstance(iteration, int) else None), grad_scaler
        if self.callbacks is not None:
            self.callbacks.on_save_checkpoint_start(model, iteration)
        super().save(_unwrap(model), optimizer, scheduler, iteration, grad_scaler)
        if self.disable_async or self.save_to_object_store:
            super().finalize()
        if self.save_to_object_store and _rank() == 0:
            self._upload(f"iter_{iteration:09d}")
        if self.callbacks is not None:
            self.callbacks.on_save_checkpoint_end(model=None, iteration=iteration)

    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, trainer=None) -> int:
        if self.callbacks is not None:
            self.callbacks.on_load_checkpoint_start(model)
        if self.load_from_object_store and self._latest() is None and _rank() == 0:
            self._download_latest()
        if torch.distributed.is_available() and torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
            torch.distributed.barrier()              # every rank reads what rank 0 wrote / fetched
        iteration = super().load(_unwrap(model), optimizer, scheduler, grad_scaler)
        latest = self._latest()
        if self.callbacks is not None:
            self.callbacks.on_load_checkpoint_end(model, iteration=iteration, checkpoint_path=latest)
        log.info(f"checkpointer: resumed at iteration {iteration}")
        return iteration
