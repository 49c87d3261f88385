"""Checkpointer of the vision-language training stack (Reason1 / Qwen).

On-disk layout (torch DCP, like the world model's): ``<job>/checkpoints/iter_%09d/{model,optim,scheduler,trainer}`` plus the
``latest_checkpoint.txt`` pointer; additionally, at iteration 0, the model is exported part by part - ``llm``, ``vision_encoder``,
``mm_projector`` - under the parameter names of the released Hugging Face checkpoints, so that each part can seed another run.
Loading accepts either layout: a full ``model`` directory of this checkpointer or the per-part directories (names are mapped
back). Asynchronous saves go through the writer processes of ``async_writer.py``.

Parity target: cosmos_predict2/_src/reason1/parallelisms/dcp_checkpointer.py:103-491 (per-part export at iteration 0, background
process with its own group, pinned shared staging) and planner.py:25-57 (name mapping between the training modules and the
Hugging Face layout).
"""

from __future__ import annotations

import os
import time
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.distributed.checkpoint as dcp
from torch.distributed.checkpoint import DefaultLoadPlanner, FileSystemReader

from ..utils import log
from .async_writer import ProcessWriter, write_state_dicts

# training-module prefix -> (part directory, Hugging Face prefix)
PARTS = (
    ("visual.merger.", "mm_projector", "visual.merger."),
    ("visual.", "vision_encoder", "visual."),
    ("language_model.", "llm", "model."),
    ("model.", "llm", "model."),
    ("lm_head.", "llm", "lm_head."),
)


def to_hf_parts(state: Dict[str, torch.Tensor]) -> Dict[str, Dict[str, torch.Tensor]]:
    """Split a training state dict into the three exported parts, keys renamed to the Hugging Face layout."""
    out: Dict[str, Dict[str, torch.Tensor]] = {"llm": {}, "vision_encoder": {}, "mm_projector": {}}
    for k, v in state.items():
        for prefix, part, hf_prefix in PARTS:
            if k.startswith(prefix):
                out[part][hf_prefix + k[len(prefix):]] = v
                break
        else:
            raise KeyError(f"parameter {k!r} belongs to no exported part")
    return out


def from_hf_parts(parts: Dict[str, Dict[str, torch.Tensor]], wanted: List[str]) -> Dict[str, torch.Tensor]:
    """Inverse of ``to_hf_parts`` for the keys ``wanted`` (the training model's own names)."""
    flat: Dict[str, torch.Tensor] = {}
    for k in wanted:
        for prefix, part, hf_prefix in PARTS:
            if k.startswith(prefix):
                src = hf_prefix + k[len(prefix):]
                if src in parts.get(part, {}):
                    flat[k] = parts[part][src]
                break
    return flat


class VLMCheckpointer:
    def __init__(self, job_dir: str, async_mode: bool = False, export_parts_at_start: bool = True):
        self.ckpt_dir = os.path.join(job_dir, "checkpoints")
        self.async_mode = async_mode
        self.export_parts_at_start = export_parts_at_start
        self._writer: Optional[ProcessWriter] = None
        self.last_error: Optional[str] = None

    @staticmethod
    def _rank() -> int:
        return dist.get_rank() if dist.is_available() and dist.is_initialized() else 0

    def _state(self, model, optimizers, schedulers, iteration: int) -> Dict[str, Dict[str, Any]]:
        sds: Dict[str, Dict[str, Any]] = {"model": dict(model.state_dict())}
        optim: Dict[str, Any] = {}
        for name, opt in (optimizers or {}).items():
            sd = opt.state_dict()
            for pid, st in sd["state"].items():
                for kk, vv in st.items():
                    optim[f"{name}.state.{pid}.{kk}"] = vv
            optim[f"{name}.param_groups"] = sd["param_groups"]
        sds["optim"] = optim
        sds["scheduler"] = {f"{n}.last_epoch": torch.tensor(s.last_epoch) for n, s in (schedulers or {}).items()}
        sds["trainer"] = {"iteration": torch.tensor(iteration)}
        if iteration == 0 and self.export_parts_at_start:
            for part, sd in to_hf_parts(sds["model"]).items():
                if sd:
                    sds[part] = sd
        return sds

    def save(self, model, optimizers=None, schedulers=None, iteration: int = 0) -> None:
        name = f"iter_{iteration:09d}"
        sds = self._state(model, optimizers, schedulers, iteration)
        if self.async_mode:
            self.finalize()
            if self._writer is None:
                self._writer = ProcessWriter()
            try:
                self._writer.submit(sds, self.ckpt_dir, name)
            except BaseException as e:      # a writer that cannot start must not end the training run
                self.last_error = repr(e)
                log.error(f"asynchronous checkpoint save could not start: {e!r}")
        else:
            t0 = time.time()
            write_state_dicts(sds, self.ckpt_dir, name, self._rank())
            log.info(f"checkpoint {name} written in {time.time() - t0:.1f} s")

    def finalize(self) -> None:
        if self._writer is not None:
            msg = self._writer.wait()
            if msg is not None and msg[1] is not None:
                self.last_error = msg[1]
                log.error(f"asynchronous checkpoint save failed: {msg[1]}")

    def close(self) -> None:
        self.finalize()
        if self._writer is not None:
            self._writer.close()
            self._writer = None

    # ---- load -----------------------------------------------------------------------------------------------------------
    def latest(self) -> Optional[str]:
        f = os.path.join(self.ckpt_dir, "latest_checkpoint.txt")
        return open(f).read().strip() if os.path.exists(f) else None

    @staticmethod
    def _read(path: str, template: Dict[str, Any]) -> Dict[str, Any]:
        sd = {k: (torch.empty_like(v) if isinstance(v, torch.Tensor) else v) for k, v in template.items()}
        dcp.load(sd, storage_reader=FileSystemReader(path), planner=DefaultLoadPlanner(allow_partial_load=True))
        return sd

    def load(self, model, optimizers=None, schedulers=None, name: Optional[str] = None, parts_only: bool = False) -> int:
        """Restore ``model`` (and the training state) from checkpoint ``name`` (default: the latest). ``parts_only``: read the
        per-part export (``llm`` / ``vision_encoder`` / ``mm_projector``) instead of the full ``model`` directory. Returns the
        iteration."""
        name = name or self.latest()
        if name is None:
            return 0
        root = os.path.join(self.ckpt_dir, name)
        own = model.state_dict()
        if parts_only:
            tmpl = to_hf_parts(own)
            parts = {p: self._read(os.path.join(root, p), sd) for p, sd in tmpl.items() if sd and os.path.isdir(os.path.join(root, p))}
            model.load_state_dict(from_hf_parts(parts, list(own.keys())), strict=False)
            return int(name.split("_")[1])
        model.load_state_dict(self._read(os.path.join(root, "model"), own))
        if optimizers and os.path.isdir(os.path.join(root, "optim")):
            # a fresh optimizer has no state yet: the tensors to read are taken from the checkpoint's own metadata
            meta = FileSystemReader(os.path.join(root, "optim")).read_metadata().state_dict_metadata
            tmpl: Dict[str, Any] = {}
            for k, m in meta.items():
                if hasattr(m, "size") and ".state." in k:
                    tmpl[k] = torch.empty(tuple(m.size), dtype=m.properties.dtype)
            got = self._read(os.path.join(root, "optim"), tmpl) if tmpl else {}
            for oname, opt in optimizers.items():
                sd = opt.state_dict()
                state: Dict[int, Dict[str, Any]] = {}
                for k, v in got.items():
                    head, _, rest = k.partition(".state.")
                    if head != oname:
                        continue
                    pid, _, kk = rest.partition(".")
                    state.setdefault(int(pid), {})[kk] = v
                if state:
                    sd["state"] = state
                    opt.load_state_dict(sd)
        if schedulers and os.path.isdir(os.path.join(root, "scheduler")):
            got = self._read(os.path.join(root, "scheduler"), {f"{n}.last_epoch": torch.tensor(0) for n in schedulers})
            for n, s in schedulers.items():
                s.last_epoch = int(got[f"{n}.last_epoch"])
        return int(name.split("_")[1])
