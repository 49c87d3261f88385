"""Distributed checkpointing in the reference's on-disk format.

Layout: ``<job>/checkpoints/iter_%09d/{model,optim,scheduler,trainer}/{.metadata,__<rank>_0.distcp}`` plus
``<job>/checkpoints/latest_checkpoint.txt`` holding ``iter_%09d``. Model keys are ``net.<param>`` (compute
dtype) and ``net_ema.<param>`` (fp32); every parameter is a dim-0 sharded DTensor when the job is
distributed, so torch DCP can reshard on load. Parity target: ``DistributedCheckpointer``
(cosmos_predict2/_src/predict2/checkpointer/dcp.py:16-732) incl. resume priority (``latest_checkpoint.txt``
beats ``load_path``), ``load_training_state`` / ``only_load_scheduler_state`` / ``keys_not_to_resume`` /
``strict_resume``, ``load_ema_to_reg``, skipping of ``_extra_state`` keys, size-mismatch-tolerant loading and the
asynchronous save path (staging to shared pinned host memory, write by a child process per rank whose group is separate from
the trainer's - ``async_writer.py`` -, success callback; ``dcp_async_writer: "thread"`` keeps the write in a thread of the
trainer's process instead).

Unlike the reference the optimizer state contains the fp32 master weights, so resuming is bit-exact.
"""

from __future__ import annotations

import os
import threading
import time
from typing import Any, Dict, List, Optional, Set

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import DefaultLoadPlanner, DefaultSavePlanner, FileSystemReader, FileSystemWriter

from ..utils import log

KEYS = ("model", "optim", "scheduler", "trainer")


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1


def _rank() -> int:
    return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0


def _as_dtensor(local: torch.Tensor, shape, mesh):
    """Wrap a rank's dim-0 chunk as a DTensor of global ``shape``: ``Shard(0)`` on a 1-D mesh, ``[Replicate(), Shard(0)]`` on the
    (replicate, shard) mesh of hybrid sharding."""
    from torch.distributed.tensor import DTensor, Replicate, Shard
    shape = torch.Size(shape)
    stride = torch.empty(shape, device="meta").stride() if len(shape) else ()
    placements = [Shard(0)] if mesh.ndim == 1 else [Replicate(), Shard(0)]
    return DTensor.from_local(local, mesh, placements, run_check=False, shape=shape, stride=stride)


class _Mesh:
    _cache: Dict[Any, Any] = {}

    @classmethod
    def get(cls, device_type: str, shard_size: Optional[int] = None):
        """1-D mesh over the world, or - when the state is sharded over ``shard_size`` < world ranks and replicated across the
        groups (hybrid sharding; rank = replica * shard_size + shard index, as ``parallel.mesh.build_groups`` lays them out) -
        the 2-D (replicate, shard) mesh."""
        W = dist.get_world_size()
        P = W if shard_size in (None, W) else int(shard_size)
        key = (device_type, W, P)
        if key not in cls._cache:
            from torch.distributed.device_mesh import init_device_mesh
            if P == W:
                cls._cache[key] = init_device_mesh(device_type, (W,), mesh_dim_names=("shard",))
            else:
                assert W % P == 0, (W, P)
                cls._cache[key] = init_device_mesh(device_type, (W // P, P), mesh_dim_names=("replicate", "shard"))
        return cls._cache[key]


class ModelWrapper:
    """Checkpoint view of a model that owns a ``ShardedEngine``: sharded ``net.*`` / ``net_ema.*`` entries."""

    def __init__(self, model, load_ema_to_reg: bool = False):
        self.model = model
        self.load_ema_to_reg = load_ema_to_reg

    def _entries(self):
        eng = self.model.engine
        out = []
        for which, prefix, dtype in (("master", "net.", self.model.precision), ("ema", "net_ema.", torch.float32)):
            if which == "ema" and not self.model.config.ema.enabled:
                continue
            for name, (local, shape, row0) in eng.sharded_state(which).items():
                out.append((prefix + name, which, name, local, shape, dtype))
        return out

    def state_dict(self) -> Dict[str, Any]:
        sd: Dict[str, Any] = {}
        sharded = _dist_on() and self.model.engine.P > 1
        mesh = _Mesh.get(self.model.device_.type, self.model.engine.P) if sharded else None
        for key, which, name, local, shape, dtype in self._entries():
            t = local.detach().to(dtype).clone()
            sd[key] = _as_dtensor(t, shape, mesh) if sharded and len(shape) > 0 else t
        pnames = {n for n, _ in self.model.net.named_parameters()}
        for k, v in self.model.net.state_dict().items():
            if k not in pnames:
                sd["net." + k] = v
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        eng = self.model.engine
        for key, which, name, local, shape, dtype in self._entries():
            src_key = key
            if self.load_ema_to_reg and which == "master" and ("net_ema." + name) in sd:
                src_key = "net_ema." + name
            if src_key not in sd:
                continue
            t = sd[src_key]
            t = t.to_local() if hasattr(t, "to_local") else t
            if t.numel() != local.numel():
                continue
            local.copy_(t.reshape(local.shape).to(local))
        pnames = {n for n, _ in self.model.net.named_parameters()}
        bufs = {k[len("net."):]: v for k, v in sd.items() if k.startswith("net.") and k[len("net."):] not in pnames}
        self.model.net.load_state_dict(bufs, strict=False)
        eng.restore_params()


class OptimizerWrapper:
    """Flattened optimizer state of the local shards under the names torch's flattened optimizer state dict gives them when the
    optimizer is looked at from the model object (``state.net.<param>.<exp_avg|exp_avg_sq>``: what the reference writes,
    checkpointer/dcp.py:283-307 there), plus this engine's fp32 masters (``state.net.<param>.master``) and its single step count.
    ``prefix=""`` reads checkpoints of this package written before the names carried the ``net.`` part."""

    def __init__(self, model, optimizer, prefix: str = "net."):
        self.model, self.optimizer, self.prefix = model, optimizer, prefix

    def _ckpt_key(self, k: str) -> str:
        return "state." + self.prefix + k[len("state."):] if k.startswith("state.") and k != "state.step" else k

    def state_dict(self, for_load: bool = False) -> Dict[str, Any]:
        sd = {}
        sharded = _dist_on() and self.model.engine.P > 1
        mesh = _Mesh.get(self.model.device_.type, self.model.engine.P) if sharded else None
        shapes = {n: shp for n, (_, shp, _) in self.model.engine.sharded_state("master").items()}
        if for_load and shapes:
            # torch's flattened optimizer state (what the reference writes) keeps the step count per parameter; this engine has
            # one count, stored as ``state.step``. When reading, ask for one parameter's count too, so either layout resumes.
            sd[f"state.{self.prefix}{next(iter(shapes))}.step"] = torch.tensor(-1.0)
        for k, v in self.optimizer.state_dict().items():
            if isinstance(v, torch.Tensor) and k.startswith("state.") and k != "state.step":
                name = k[len("state."):].rsplit(".", 1)[0]
                t = v.detach().clone()
                sd[self._ckpt_key(k)] = _as_dtensor(t, shapes[name], mesh) if sharded and len(shapes[name]) > 0 else t
            else:
                sd[k] = v
        return sd

    def load_state_dict(self, sd: Dict[str, Any]) -> None:
        flat = {k: (v.to_local() if hasattr(v, "to_local") else v) for k, v in sd.items()}
        per_param = [k for k in flat if k.startswith("state.") and k.endswith(".step") and k != "state.step"]
        steps = [float(flat.pop(k)) for k in per_param]
        if steps and max(steps) > float(flat.get("state.step", 0)):
            flat["state.step"] = torch.tensor(int(max(steps)), dtype=torch.int64)
        strip = len("state." + self.prefix)
        flat = {("state." + k[strip:] if k.startswith("state." + self.prefix) else k): v for k, v in flat.items()}
        self.optimizer.load_state_dict(flat)


class _TolerantLoadPlanner(DefaultLoadPlanner):
    """Skips keys missing from the checkpoint and (optionally) tensors whose stored size differs."""

    def __init__(self, allow_mismatched_size: bool = False):
        super().__init__(allow_partial_load=True)
        self.allow_mismatched_size = allow_mismatched_size

    def set_up_planner(self, state_dict, metadata=None, is_coordinator=False):
        if metadata is not None:
            drop = [k for k in state_dict if k.endswith("._extra_state")]
            if self.allow_mismatched_size:
                for k, v in state_dict.items():
                    md = metadata.state_dict_metadata.get(k)
                    if md is not None and hasattr(md, "size") and hasattr(v, "shape") and tuple(md.size) != tuple(v.shape):
                        log.warning(f"checkpoint size mismatch for {k}: {tuple(md.size)} vs {tuple(v.shape)}; skipped")
                        drop.append(k)
            for k in drop:
                state_dict.pop(k, None)
        super().set_up_planner(state_dict, metadata, is_coordinator)


class DistributedCheckpointer:
    def __init__(self, config_checkpoint: Dict[str, Any], job_dir: str, callbacks=None, disable_async: bool = False):
        c = config_checkpoint
        self.cfg = c
        self.job_dir = job_dir
        self.ckpt_dir = os.path.join(job_dir, "checkpoints")
        self.callbacks = callbacks
        self.load_path = c.get("load_path") or None
        self.load_training_state = c.get("load_training_state", False)
        self.only_load_scheduler_state = c.get("only_load_scheduler_state", False)
        self.strict_resume = c.get("strict_resume", True)
        self.keys_not_to_resume: List[str] = list(c.get("keys_not_to_resume", []))
        self.load_ema_to_reg = c.get("load_ema_to_reg", False)
        self.allow_mismatched = c.get("dcp_allow_mismatched_size", False)
        self.async_mode = bool(c.get("dcp_async_mode_enabled", False)) and not disable_async
        self.async_writer = str(c.get("dcp_async_writer", "process"))
        if self.async_writer not in ("process", "thread"):
            raise ValueError(f"dcp_async_writer must be 'process' or 'thread', got {self.async_writer!r}")
        self._writer = None                       # ProcessWriter, created on the first asynchronous save
        self._bg: Optional[threading.Thread] = None
        self._bg_error: Optional[BaseException] = None
        self._cpu_group = None

    # ---- paths ----------------------------------------------------------------------------------------------
    @staticmethod
    def iter_name(iteration: int) -> str:
        return f"iter_{iteration:09d}"

    def _latest_file(self) -> str:
        return os.path.join(self.ckpt_dir, "latest_checkpoint.txt")

    def _read_latest(self) -> Optional[str]:
        f = self._latest_file()
        if os.path.exists(f):
            name = open(f).read().strip()
            return name or None
        return None

    def _write_latest(self, name: str) -> None:
        if _rank() == 0:
            os.makedirs(self.ckpt_dir, exist_ok=True)
            tmp = self._latest_file() + ".tmp"
            with open(tmp, "w") as f:
                f.write(name + "\n")
            os.replace(tmp, self._latest_file())

    def keys_to_resume_during_load(self):
        """(keys to load, checkpoint dir). A checkpoint of this very job wins over ``load_path``."""
        latest = self._read_latest()
        if latest is not None:
            return set(KEYS), os.path.join(self.ckpt_dir, latest)
        if self.load_path:
            path = self.load_path
            if os.path.isdir(path) and os.path.exists(os.path.join(path, "latest_checkpoint.txt")):
                path = os.path.join(path, open(os.path.join(path, "latest_checkpoint.txt")).read().strip())
            if self.load_training_state:
                keys = set(KEYS)
            elif self.only_load_scheduler_state:
                keys = {"model", "scheduler"}
            else:
                keys = {"model"}
            return keys, path
        return set(), None

    # ---- load --------------------------------------------------------------------------------------------------
    def load(self, model, optimizer=None, scheduler=None, grad_scaler=None, trainer=None) -> int:
        if self.callbacks is not None:
            self.callbacks.on_load_checkpoint_start(model)
        keys, path = self.keys_to_resume_during_load()
        keys = {k for k in keys if k not in self.keys_not_to_resume}
        iteration = 0
        if path is None:
            log.info("no checkpoint to load; training from scratch")
            return 0
        if path.endswith(".pt"):
            sd = torch.load(path, map_location="cpu", weights_only=False)
            model.load_state_dict(sd, strict=False, load_ema_to_reg=self.load_ema_to_reg)
            log.info(f"loaded consolidated checkpoint {path}")
            return 0
        if _dist_on():
            dist.barrier()
        try:
            iteration = self._load_parts(model, optimizer, scheduler, keys, path)
        except BaseException as e:
            # torch's CheckpointException derives from BaseException; callers that guard with ``except Exception`` must see it
            if isinstance(e, (Exception, KeyboardInterrupt, SystemExit)):
                raise
            raise RuntimeError(f"checkpoint {path} is damaged or incomplete: {e}") from e
        log.info(f"loaded checkpoint {path} (keys {sorted(keys)}), iteration {iteration}")
        if self.callbacks is not None:
            self.callbacks.on_load_checkpoint_end(model, iteration=iteration, checkpoint_path=path)
        return iteration

    def _load_parts(self, model, optimizer, scheduler, keys, path: str) -> int:
        iteration = 0
        for key in KEYS:
            if key not in keys:
                continue
            sub = os.path.join(path, key)
            if not os.path.isdir(sub):
                if self.strict_resume and key in ("model",):
                    raise FileNotFoundError(sub)
                log.warning(f"checkpoint part {sub} missing; skipped")
                continue
            reader = FileSystemReader(sub)
            if key == "model":
                w = ModelWrapper(model, self.load_ema_to_reg)
                sd = w.state_dict()
                if self.load_ema_to_reg:
                    sd = {k: v for k, v in sd.items() if not (k.startswith("net.") and ("net_ema." + k[4:]) in sd)}
                dcp.load(sd, storage_reader=reader, planner=_TolerantLoadPlanner(self.allow_mismatched or not self.strict_resume))
                w.load_state_dict(sd)
            elif key == "optim" and optimizer is not None:
                stored = reader.read_metadata().state_dict_metadata
                legacy = not any(k.startswith("state.net.") for k in stored)
                w = OptimizerWrapper(model, optimizer, prefix="" if legacy else "net.")
                sd = w.state_dict(for_load=True)
                dcp.load(sd, storage_reader=reader, planner=_TolerantLoadPlanner(self.allow_mismatched))
                w.load_state_dict(sd)
            elif key == "scheduler" and scheduler is not None:
                sd = {"last_epoch": torch.tensor(scheduler.state_dict()["last_epoch"])}
                dcp.load(sd, storage_reader=reader, planner=_TolerantLoadPlanner())
                scheduler.load_state_dict({"last_epoch": int(sd["last_epoch"])})
            elif key == "trainer":
                sd = {"iteration": torch.tensor(0), "grad_scaler_scale": torch.tensor(1.0)}
                dcp.load(sd, storage_reader=reader, planner=_TolerantLoadPlanner())
                iteration = int(sd["iteration"])
        return iteration

    # ---- save --------------------------------------------------------------------------------------------------
    def _state_dicts(self, model, optimizer, scheduler, iteration: int) -> Dict[str, Dict[str, Any]]:
        return {
            "model": ModelWrapper(model).state_dict(),
            "optim": OptimizerWrapper(model, optimizer).state_dict() if optimizer is not None else {},
            "scheduler": {"last_epoch": torch.tensor(scheduler.state_dict()["last_epoch"])} if scheduler is not None else {},
            "trainer": {"iteration": torch.tensor(iteration), "grad_scaler_scale": torch.tensor(1.0)},
        }

    def _write(self, sds: Dict[str, Dict[str, Any]], name: str, group=None) -> None:
        t0 = time.time()
        for key, sd in sds.items():
            if not sd:
                continue
            path = os.path.join(self.ckpt_dir, name, key)
            if _rank() == 0:
                os.makedirs(path, exist_ok=True)
            dcp.save(sd, storage_writer=FileSystemWriter(path, thread_count=4),
                     planner=DefaultSavePlanner(dedup_save_to_lowest_rank=True), process_group=group)
        self._write_latest(name)
        if self.callbacks is not None:
            self.callbacks.on_save_checkpoint_success(iteration=int(name.split("_")[1]), elapsed_time=time.time() - t0)

    @staticmethod
    def _to_host(sd: Dict[str, Any]) -> Dict[str, Any]:
        """Stage a state dict to host memory (pinned when a GPU is present); DTensors keep their placement."""
        out = {}
        for k, v in sd.items():
            if hasattr(v, "to_local"):
                from torch.distributed.tensor import DTensor
                loc = v.to_local()
                if loc.is_cuda:
                    host = torch.empty(loc.shape, dtype=loc.dtype, pin_memory=True)
                    host.copy_(loc, non_blocking=True)
                    mesh = _Mesh.get("cpu", v.device_mesh.shape[-1])
                    out[k] = DTensor.from_local(host, mesh, v.placements, run_check=False, shape=v.shape, stride=v.stride())
                else:
                    out[k] = v
            elif isinstance(v, torch.Tensor) and v.is_cuda:
                host = torch.empty(v.shape, dtype=v.dtype, pin_memory=True)
                host.copy_(v, non_blocking=True)
                out[k] = host
            else:
                out[k] = v
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()
        return out

    def save(self, model, optimizer, scheduler, iteration: int, grad_scaler=None, trainer=None) -> None:
        if self.callbacks is not None:
            self.callbacks.on_save_checkpoint_start(model, iteration)
        name = self.iter_name(iteration)
        sds = self._state_dicts(model, optimizer, scheduler, iteration)
        if self.async_mode and self.async_writer == "process":
            self.finalize()  # one save in flight at a time
            if self._writer is None:
                from .async_writer import ProcessWriter
                self._writer = ProcessWriter()
            try:
                self._writer.submit(sds, self.ckpt_dir, name)
            except BaseException as e:  # a writer that cannot start must not end the training run
                self._bg_error = e
        elif self.async_mode:
            self.finalize()  # one save in flight at a time
            staged = {k: self._to_host(v) for k, v in sds.items()}
            if _dist_on() and self._cpu_group is None:
                self._cpu_group = dist.new_group(backend="gloo")

            def work():
                try:
                    self._write(staged, name, group=self._cpu_group)
                except BaseException as e:  # reported on the next save / finalize, never kills training
                    self._bg_error = e

            self._bg = threading.Thread(target=work, name="dcp-async-save", daemon=True)
            self._bg.start()
        else:
            self._write(sds, name)
        if self.callbacks is not None:
            self.callbacks.on_save_checkpoint_end(model, iteration)

    def finalize(self) -> None:
        """Wait for the save in flight; report (never raise) its failure. Collective when the job is distributed: a failure on
        one rank makes every rank restart its writer, so the writers' group stays in step."""
        if self._writer is not None:
            msg = self._writer.wait()
            failed = msg is not None and msg[1] is not None
            if _dist_on() and (msg is not None or self._bg_error is not None):
                flags = [None] * dist.get_world_size()
                dist.all_gather_object(flags, bool(failed or self._bg_error is not None))
                if any(flags) and not failed:
                    self._writer.close()
                    failed_elsewhere = True
                else:
                    failed_elsewhere = False
                if failed_elsewhere and self._bg_error is None:
                    self._bg_error = RuntimeError("checkpoint save failed on another rank")
            if failed:
                self._bg_error = RuntimeError(msg[1])
            elif msg is not None and self._bg_error is None and self.callbacks is not None:
                self.callbacks.on_save_checkpoint_success(iteration=int(msg[0].split("_")[1]), elapsed_time=msg[2])
        if self._bg is not None:
            self._bg.join()
            self._bg = None
        if self._bg_error is not None:
            e, self._bg_error = self._bg_error, None
            log.error(f"asynchronous checkpoint save failed: {e!r}")

    def close(self) -> None:
        """Finish the save in flight and end the writer process."""
        self.finalize()
        if self._writer is not None:
            self._writer.close()
            self._writer = None


def convert_distcp_to_pt(dcp_model_dir: str, out_dir: str) -> Dict[str, str]:
    """Consolidate ``<iter>/model`` into ``model.pt`` (all keys), ``model_ema_fp32.pt`` and
    ``model_ema_bf16.pt`` (EMA weights renamed ``net_ema.`` -> ``net.``), like the reference's release script
    (scripts/convert_distcp_to_pt.py:63-125)."""
    from torch.distributed.checkpoint.format_utils import dcp_to_torch_save
    os.makedirs(out_dir, exist_ok=True)
    full = os.path.join(out_dir, "model.pt")
    dcp_to_torch_save(dcp_model_dir, full)
    sd = torch.load(full, map_location="cpu", weights_only=False)
    ema = {k.replace("net_ema.", "net.", 1): v for k, v in sd.items() if k.startswith("net_ema.")}
    paths = {"model": full}
    if ema:
        p32, p16 = os.path.join(out_dir, "model_ema_fp32.pt"), os.path.join(out_dir, "model_ema_bf16.pt")
        torch.save(ema, p32)
        torch.save({k: (v.bfloat16() if v.is_floating_point() else v) for k, v in ema.items()}, p16)
        paths.update(ema_fp32=p32, ema_bf16=p16)
    return paths
