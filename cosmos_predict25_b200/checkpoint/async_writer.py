"""Checkpoint writer in a child process per rank.

The trainer stages a state dict into host memory that both processes can see and hands it to a long-lived child; the children of
all ranks form their own gloo group and run the collective ``torch.distributed.checkpoint.save`` among themselves, so neither
the planning collectives nor the file writes share the trainer's process, its GIL or its NCCL communicators. The trainer only
waits for the previous save when the next one starts (or in ``finalize``). Parity target: the asynchronous path of the
reference's checkpointer (cosmos_predict2/_src/predict2/checkpointer/dcp.py:327-406: a checkpoint process with its own process
group fed through queues; pinned shared staging buffers :579-636).

A failure in the child (a full disk, an unwritable directory, a killed process) is reported to the trainer as a message or is
seen as a dead process; it never raises into the training loop, the ``latest_checkpoint.txt`` pointer keeps naming the last
complete checkpoint, and the next save starts a fresh child.
"""

from __future__ import annotations

import os
import queue
import socket
import time
import traceback
from typing import Any, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def pack_state_dict(sd: Dict[str, Any], staging: Optional[Dict[str, torch.Tensor]] = None) -> List[Tuple]:
    """Turn a state dict into picklable entries whose tensors live in shared host memory.

    Entry: ``(key, "dtensor", local, global_shape, placements, mesh_shape)`` for a DTensor (placements as ``("S", dim)`` /
    ``("R",)`` per mesh dimension), ``(key, "tensor", t)`` for a plain
    tensor, ``(key, "object", obj)`` for anything else. ``staging`` keeps the shared buffers between saves (same key and
    shape: reused, so a save allocates nothing after the first one)."""
    out: List[Tuple] = []
    copies = []
    for k, v in sd.items():
        if hasattr(v, "to_local"):
            loc = v.to_local()
            spec = tuple(("S", int(p.dim)) if getattr(p, "dim", None) is not None else ("R",) for p in v.placements)
            host = _stage(k, loc, staging)
            copies.append((host, loc))
            out.append((k, "dtensor", host, tuple(v.shape), spec, tuple(v.device_mesh.shape)))
        elif isinstance(v, torch.Tensor):
            host = _stage(k, v, staging)
            copies.append((host, v))
            out.append((k, "tensor", host))
        else:
            out.append((k, "object", v))
    for host, src in copies:
        host.copy_(src.detach(), non_blocking=src.is_cuda)
    if torch.cuda.is_available() and any(src.is_cuda for _, src in copies):
        torch.cuda.current_stream().synchronize()
    return out


def _stage(key: str, src: torch.Tensor, staging: Optional[Dict[str, torch.Tensor]]) -> torch.Tensor:
    buf = None if staging is None else staging.get(key)
    if buf is None or buf.shape != src.shape or buf.dtype != src.dtype:
        buf = torch.empty(src.shape, dtype=src.dtype).share_memory_()
        if src.is_cuda and buf.numel() > 0:
            # page-lock the shared pages so the device-to-host copy runs at full speed and asynchronously
            try:
                torch.cuda.cudart().cudaHostRegister(buf.data_ptr(), buf.numel() * buf.element_size(), 0)
            except Exception:
                pass
        if staging is not None:
            staging[key] = buf
    return buf


_meshes: Dict[Tuple, Any] = {}


def _cpu_mesh(shape: Tuple[int, ...]):
    if shape not in _meshes:
        from torch.distributed.device_mesh import init_device_mesh
        names = ("shard",) if len(shape) == 1 else ("replicate", "shard")
        _meshes[shape] = init_device_mesh("cpu", shape, mesh_dim_names=names)
    return _meshes[shape]


def unpack_state_dict(entries: List[Tuple], distributed: bool) -> Dict[str, Any]:
    sd: Dict[str, Any] = {}
    for e in entries:
        k, kind = e[0], e[1]
        if kind == "dtensor" and distributed:
            from torch.distributed.tensor import DTensor, Replicate, Shard
            _, _, local, shape, spec, mesh_shape = e
            shape = torch.Size(shape)
            stride = torch.empty(shape, device="meta").stride() if len(shape) else ()
            placements = [Shard(p[1]) if p[0] == "S" else Replicate() for p in spec]
            sd[k] = DTensor.from_local(local, _cpu_mesh(tuple(mesh_shape)), placements, run_check=False, shape=shape, stride=stride)
        else:
            sd[k] = e[2]
    return sd


def write_state_dicts(sds: Dict[str, Dict[str, Any]], ckpt_dir: str, name: str, rank: int, group=None) -> None:
    """``<ckpt_dir>/<name>/<key>/`` for every non-empty part, then the ``latest_checkpoint.txt`` pointer (rank 0, atomically)."""
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import DefaultSavePlanner, FileSystemWriter
    for key, sd in sds.items():
        if not sd:
            continue
        path = os.path.join(ckpt_dir, name, key)
        if rank == 0:
            os.makedirs(path, exist_ok=True)
        dcp.save(sd, storage_writer=FileSystemWriter(path, thread_count=4),
                 planner=DefaultSavePlanner(dedup_save_to_lowest_rank=True), process_group=group)
    if rank == 0:
        os.makedirs(ckpt_dir, exist_ok=True)
        latest = os.path.join(ckpt_dir, "latest_checkpoint.txt")
        with open(latest + ".tmp", "w") as f:
            f.write(name + "\n")
        os.replace(latest + ".tmp", latest)


def _writer_main(rank: int, world: int, addr: str, port: int, jobs, done) -> None:
    """Body of the child: join the writers' gloo group, then serve save jobs until ``None`` arrives."""
    try:
        torch.set_num_threads(2)
        if world > 1:
            dist.init_process_group("gloo", init_method=f"tcp://{addr}:{port}", rank=rank, world_size=world)
        done.put(("ready", None, 0.0))
    except BaseException:
        done.put(("ready", traceback.format_exc(), 0.0))
        return
    while True:
        job = jobs.get()
        if job is None:
            break
        name, ckpt_dir, payload = job
        t0 = time.time()
        try:
            sds = {key: unpack_state_dict(entries, world > 1) for key, entries in payload.items()}
            write_state_dicts(sds, ckpt_dir, name, rank, group=None)
            done.put((name, None, time.time() - t0))
        except BaseException:
            done.put((name, traceback.format_exc(), time.time() - t0))
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()


class ProcessWriter:
    """Owner of the child process of this rank. ``submit`` hands over a packed state dict, ``wait`` returns ``(name, error or
    None, seconds)`` of the save in flight, ``close`` ends the child."""

    def __init__(self, start_timeout_s: float = 120.0):
        self._proc = None
        self._jobs = None
        self._done = None
        self._pending: Optional[str] = None
        self._staging: Dict[str, Dict[str, torch.Tensor]] = {}
        self._start_timeout_s = start_timeout_s

    def _start(self) -> None:
        on = dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1
        rank, world = (dist.get_rank(), dist.get_world_size()) if on else (0, 1)
        addr, port = os.environ.get("MASTER_ADDR", "127.0.0.1"), 0
        if on:
            box = [_free_port() if rank == 0 else 0]
            dist.broadcast_object_list(box, src=0)
            port = int(box[0])
        ctx = mp.get_context("spawn")
        self._jobs, self._done = ctx.Queue(), ctx.Queue()
        self._proc = ctx.Process(target=_writer_main, args=(rank, world, addr, port, self._jobs, self._done),
                                 name="cosmos-b200-checkpoint-writer", daemon=True)
        self._proc.start()
        tag, err, _ = self._get(self._start_timeout_s)
        if tag != "ready" or err is not None:
            self._kill()
            raise RuntimeError(f"checkpoint writer process did not start: {err or tag}")

    def _get(self, timeout_s: Optional[float]):
        """Next message of the child; a child that died without one is reported as a failure."""
        t0 = time.time()
        while True:
            try:
                return self._done.get(timeout=0.2)
            except queue.Empty:
                if self._proc is None or not self._proc.is_alive():
                    try:
                        return self._done.get(timeout=0.2)
                    except queue.Empty:
                        code = None if self._proc is None else self._proc.exitcode
                        return (self._pending or "?", f"checkpoint writer process exited with code {code}", 0.0)
                if timeout_s is not None and time.time() - t0 > timeout_s:
                    return (self._pending or "?", f"no answer from the checkpoint writer within {timeout_s:.0f} s", 0.0)

    def _kill(self) -> None:
        if self._proc is not None:
            if self._proc.is_alive():
                self._proc.terminate()
            self._proc.join(timeout=5)
        self._proc = self._jobs = self._done = None
        self._pending = None

    def alive(self) -> bool:
        return self._proc is not None and self._proc.is_alive()

    def submit(self, sds: Dict[str, Dict[str, Any]], ckpt_dir: str, name: str) -> None:
        assert self._pending is None, "wait() for the save in flight first"
        if not self.alive():
            self._kill()
            self._start()
        payload = {key: pack_state_dict(sd, self._staging.setdefault(key, {})) for key, sd in sds.items()}
        self._jobs.put((name, ckpt_dir, payload))
        self._pending = name

    def wait(self, timeout_s: Optional[float] = None) -> Optional[Tuple[str, Optional[str], float]]:
        if self._pending is None:
            return None
        msg = self._get(timeout_s)
        self._pending = None
        if msg[1] is not None:
            self._kill()          # its group may be out of step with the other ranks' writers: start over next time
        return msg

    def close(self) -> None:
        if self._proc is not None and self._proc.is_alive() and self._pending is None:
            self._jobs.put(None)
            self._proc.join(timeout=10)
        self._kill()
