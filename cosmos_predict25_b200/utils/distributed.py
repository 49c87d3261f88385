"""Process-group bootstrap and small rank helpers.

Parity target: cosmos_predict2/_src/imaginaire/utils/distributed.py:49-443: ``init`` (env:// rendezvous, NCCL on GPUs,
timeout from ``TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC``, CPU affinity from NVML topology - read-only NVML calls), rank
helpers, ``barrier``, ``all_gather_tensor``, ``dist_reduce_tensor``, ``sync_model_states``. gloo is selected
automatically when no GPU is present (CPU test worlds).
"""

from __future__ import annotations

import datetime
import os
from typing import List, Optional

import torch
import torch.distributed as dist

from . import log


def init(backend: Optional[str] = None) -> int:
    """Initialise torch.distributed from the torchrun environment (no-op when already initialised or single
    process). Returns the local rank."""
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if dist.is_available() and dist.is_initialized():
        return local_rank
    if "RANK" not in os.environ or int(os.environ.get("WORLD_SIZE", "1")) == 1 and "MASTER_ADDR" not in os.environ:
        if torch.cuda.is_available():
            torch.cuda.set_device(local_rank)
        return local_rank
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    use_cuda = torch.cuda.is_available()
    backend = backend or ("nccl" if use_cuda else "gloo")
    timeout = datetime.timedelta(seconds=int(os.environ.get("TORCH_NCCL_HEARTBEAT_TIMEOUT_SEC", "1800")))
    os.environ.setdefault("TORCH_NCCL_ASYNC_ERROR_HANDLING", "1")
    if use_cuda:
        torch.cuda.set_device(local_rank)
        _set_cpu_affinity(local_rank)
        dist.init_process_group(backend, init_method="env://", timeout=timeout, device_id=torch.device("cuda", local_rank))
    else:
        dist.init_process_group(backend, init_method="env://", timeout=timeout)
    return local_rank


def _set_cpu_affinity(local_rank: int) -> None:
    """Pin the process to the CPUs NVML reports as closest to its GPU (reads topology only)."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        n = os.cpu_count() or 1
        words = pynvml.nvmlDeviceGetCpuAffinity(h, (n + 63) // 64)
        cpus = [i * 64 + b for i, w in enumerate(words) for b in range(64) if (w >> b) & 1 and i * 64 + b < n]
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception as e:  # containers often hide the topology; affinity is an optimisation only
        log.debug(f"cpu affinity not set: {e}")


def get_rank(group=None) -> int:
    return dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0


def get_world_size(group=None) -> int:
    return dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1


def is_rank0() -> bool:
    return get_rank() == 0


def barrier() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.barrier()


def all_gather_tensor(t: torch.Tensor) -> List[torch.Tensor]:
    if get_world_size() == 1:
        return [t]
    out = [torch.empty_like(t) for _ in range(get_world_size())]
    dist.all_gather(out, t.contiguous())
    return out


def dist_reduce_tensor(t: torch.Tensor, rank: int = 0, reduce: str = "mean") -> torch.Tensor:
    """Reduce to ``rank`` with mean / sum / max / min."""
    if get_world_size() == 1:
        return t
    t = t.clone()
    op = {"mean": dist.ReduceOp.SUM, "sum": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX, "min": dist.ReduceOp.MIN}[reduce]
    dist.reduce(t, dst=rank, op=op)
    if reduce == "mean" and get_rank() == rank:
        t /= get_world_size()
    return t


@torch.no_grad()
def sync_model_states(model: torch.nn.Module, group=None, src: int = 0, params: bool = True, buffers: bool = True) -> None:
    """Broadcast parameters / buffers from ``src`` so that all ranks start identical."""
    if get_world_size(group) == 1:
        return
    tensors = (list(model.parameters()) if params else []) + (list(model.buffers()) if buffers else [])
    for t in tensors:
        dist.broadcast(t.data, src=src, group=group)


def destroy() -> None:
    if dist.is_available() and dist.is_initialized():
        dist.destroy_process_group()


class DistributedDataParallel(torch.nn.parallel.DistributedDataParallel):
    """Data-parallel wrapper whose ``training_step`` runs the wrapped model's ``training_step`` THROUGH the wrapper's forward, so
    that the gradient hooks see it (imaginaire/utils/distributed.py:205-232 of the reference): ``forward`` is swapped for the
    step for the duration of one call and restored inside it."""

    def training_step(self, *args, **kwargs):
        original_forward = self.module.forward

        def step(*a, **k):
            self.module.forward = original_forward
            return self.module.training_step(*a, **k)

        self.module.forward = step
        return self(*args, **kwargs)


def parallel_model_wrapper(config_ddp, model: torch.nn.Module) -> torch.nn.Module:
    """Wrap for data parallelism when a process group exists; the model itself otherwise."""
    if dist.is_available() and dist.is_initialized():
        kw = dict(find_unused_parameters=getattr(config_ddp, "find_unused_parameters", False),
                  static_graph=getattr(config_ddp, "static_graph", False), broadcast_buffers=getattr(config_ddp, "broadcast_buffers", True))
        if torch.cuda.is_available():
            kw.update(device_ids=[torch.cuda.current_device()], output_device=torch.cuda.current_device())
        return DistributedDataParallel(model, **kw)
    return model
