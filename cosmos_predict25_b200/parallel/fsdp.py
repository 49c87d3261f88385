"""Sharded-parameter engine: the FSDP/ZeRO equivalent of this framework.

What the reference does with torch FSDP2 (``fully_shard`` per DiT block + final layer + timestep
embedder + root; cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:1688-1699,
cosmos_predict2/_src/predict2/models/text2world_model_rectified_flow.py:177-249) is restated here
for a 180 GB-per-GPU machine:

  * Parameters are grouped into the same *units*. Every parameter is sharded on dim 0 into
    ``ceil(rows/P)``-row chunks (the FSDP2 / DTensor ``Shard(0)`` layout, so checkpoints interoperate).
  * Each rank owns, per unit, one contiguous shard holding its chunk of every parameter:
    fp32 master weights, Adam moments, an optional fp32 EMA, and the fp32 reduced gradient.
  * The full bf16 parameters of all units stay resident in HBM (4 GB for 2B, 29 GB for 14B). The
    all-gather moves out of the forward pass: the optimizer kernel writes each updated bf16 chunk
    straight into every peer's full buffer.
  * HSDP / DDP: with a ``replicate_group`` the reduced gradient shard is summed once more over the
    ranks that hold the same shard in other replicas (cosmos_predict2/_src/common/utils/fsdp_helper.py:97-159).
    A shard group of one rank plus a replicate group over the world is plain data parallelism
    (cosmos_predict2/_src/imaginaire/utils/distributed.py:173-264): every rank keeps the whole state.
  * Gradients are accumulated by autograd directly into a flat bf16 buffer with the full-parameter
    layout (``param.grad`` are views). When a unit's backward is complete, its reduce-scatter runs
    on a side stream: either NCCL/gloo ``reduce_scatter`` (the baseline twin) or the peer-memory
    kernel that reads the chunk from every peer over NVLink, sums in fp32, scrubs NaN/Inf and
    accumulates the squared-norm partial used for global-norm clipping.
  * ``step`` clips by the global norm, runs the fused AdamW (+EMA, + bf16 write-back) on shards.

The same code runs on CPU tensors with the gloo backend (tests) using the PyTorch oracle ops.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import native, ref


def _group_size_rank(group) -> Tuple[int, int]:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


@dataclass
class ParamSlot:
    name: str
    param: nn.Parameter
    shape: torch.Size
    rows: int
    cols: int
    chunk_rows: int          # ceil(rows / P)
    full_offset: int         # element offset of the (row-padded) parameter in the full buffer
    shard_offset: int        # element offset of this rank's chunk in the shard buffer

    @property
    def chunk_numel(self) -> int:
        return self.chunk_rows * self.cols

    @property
    def padded_numel(self) -> int:
        return self.chunk_numel  # per rank; times P for the full buffer


class FlatUnit:
    """One gather/reduce group: a set of parameters with flat full and shard buffers."""

    def __init__(self, name: str, named_params: Sequence[Tuple[str, nn.Parameter]], group, compute_dtype: torch.dtype,
                 use_ema: bool, device: torch.device, alloc=None):
        self.name = name
        self.group = group
        self.P, self.rank = _group_size_rank(group)
        self.compute_dtype = compute_dtype
        self.device = device
        P = self.P
        self.slots: List[ParamSlot] = []
        full_off = shard_off = 0
        for n, p in named_params:
            rows = p.shape[0] if p.ndim > 0 else 1
            cols = p.numel() // max(rows, 1)
            chunk_rows = (rows + P - 1) // P
            cn = chunk_rows * cols
            self.slots.append(ParamSlot(n, p, p.shape, rows, cols, chunk_rows, full_off, shard_off))
            # each parameter (and each shard segment) starts 16-byte aligned in bf16; chunks of one
            # parameter are back to back so the parameter view stays contiguous
            full_off += cn * P + ((-cn * P) % 8)
            shard_off += cn + ((-cn) % 8)
        self.full_numel = full_off
        self.shard_numel = shard_off
        alloc = alloc or (lambda numel, dtype: torch.zeros(numel, dtype=dtype, device=device))
        self._alloc = alloc
        # full-layout buffers (peer-visible when alloc hands out symmetric memory)
        self.full = alloc(self.full_numel, compute_dtype)
        self.grad_full = alloc(self.full_numel, compute_dtype)
        # shard-layout state
        self.master = torch.zeros(self.shard_numel, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros_like(self.master)
        self.exp_avg_sq = torch.zeros_like(self.master)
        self.grad_shard = torch.zeros_like(self.master)
        self.ema = torch.zeros_like(self.master) if use_ema else None
        self.sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self._init_from_params()
        self._pending = 0
        self._n_trainable = len(self.slots)
        self.reduced = False

    # ---- layout helpers ------------------------------------------------------------------
    def _stride(self, s: ParamSlot) -> int:
        """Elements between consecutive ranks' chunks of one parameter in the full buffer."""
        return s.chunk_numel

    def full_view(self, s: ParamSlot, buf: torch.Tensor) -> torch.Tensor:
        """The parameter-shaped view of slot ``s`` inside a full-layout buffer."""
        return buf[s.full_offset: s.full_offset + s.rows * s.cols].view(s.shape)

    def chunk_in_full(self, s: ParamSlot, buf: torch.Tensor, r: int) -> torch.Tensor:
        stride = self._stride(s)
        return buf[s.full_offset + r * stride: s.full_offset + r * stride + s.chunk_numel]

    def chunk_in_shard(self, s: ParamSlot, buf: torch.Tensor) -> torch.Tensor:
        return buf[s.shard_offset: s.shard_offset + s.chunk_numel]

    def local_rows(self, s: ParamSlot) -> Tuple[int, int]:
        lo = min(self.rank * s.chunk_rows, s.rows)
        hi = min(lo + s.chunk_rows, s.rows)
        return lo, hi

    def segment_table(self) -> torch.Tensor:
        """int64 [n_slots, 4]: (full_offset, rank_stride, shard_offset, chunk_numel) for the kernels."""
        rows = [[s.full_offset, self._stride(s), s.shard_offset, s.chunk_numel] for s in self.slots]
        return torch.tensor(rows, dtype=torch.int64)

    # ---- initialisation ---------------------------------------------------------------------
    @torch.no_grad()
    def _init_from_params(self):
        for s in self.slots:
            src = s.param.detach().to(device=self.device, dtype=torch.float32).reshape(s.rows, s.cols)
            lo, hi = self.local_rows(s)
            n = (hi - lo) * s.cols
            self.chunk_in_shard(s, self.master)[:n].copy_(src[lo:hi].reshape(-1))
            for r in range(self.P):
                rlo = min(r * s.chunk_rows, s.rows)
                rhi = min(rlo + s.chunk_rows, s.rows)
                m = (rhi - rlo) * s.cols
                self.chunk_in_full(s, self.full, r)[:m].copy_(src[rlo:rhi].reshape(-1).to(self.compute_dtype))
        if self.ema is not None:
            self.ema.copy_(self.master)
        self.bind_params()

    def bind_params(self):
        """Point every parameter (and its .grad) at its view in the flat buffers."""
        for s in self.slots:
            s.param.data = self.full_view(s, self.full)
            s.param.grad = self.full_view(s, self.grad_full)

    # ---- collectives ---------------------------------------------------------------------------
    @torch.no_grad()
    def reduce_scatter_grads(self, transport: str, scale: float):
        """grad_shard <- scale * sum over ranks of this rank's chunk; sumsq <- ||grad_shard||^2."""
        if self.P == 1:
            self._local_grad_to_shard(scale)
        elif transport == "nccl":
            tmp = torch.zeros(self.P, self.shard_numel, dtype=self.compute_dtype, device=self.device)
            for s in self.slots:
                stride = self._stride(s)
                src = self.grad_full[s.full_offset: s.full_offset + stride * self.P].view(self.P, stride)
                tmp[:, s.shard_offset: s.shard_offset + stride].copy_(src)
            # (alignment gaps of tmp stay uninitialised; they are never read back)
            out = torch.empty(self.shard_numel, dtype=self.compute_dtype, device=self.device)
            if self.device.type == "cpu":
                flat = tmp.float()
                dist.all_reduce(flat, group=self.group)
                red = flat[self.rank]
            else:
                dist.reduce_scatter_tensor(out, tmp, group=self.group)
                red = out.float()
            red = torch.nan_to_num(red * scale, nan=0.0, posinf=0.0, neginf=0.0)
            self.grad_shard.copy_(red)
            self.sumsq.copy_(red.pow(2).sum().view(1))
        else:
            raise ValueError(f"transport {transport!r} is handled by PeerFlatUnit")
        self.reduced = True

    @torch.no_grad()
    def all_reduce_replicas(self, group):
        """HSDP / DDP: sum the reduced shard over the replicas (the 1/replicas factor is part of ``scale``)."""
        dist.all_reduce(self.grad_shard, group=group)
        self.sumsq.copy_(self.grad_shard.pow(2).sum().view(1))

    def _local_grad_to_shard(self, scale: float):
        if self.device.type == "cuda":
            ops = native.load()
            ops.grad_cast_norm(self.grad_full, self.grad_shard, self.sumsq, float(scale))
            native.count_launch()
        else:
            g = torch.nan_to_num(self.grad_full.float() * scale, nan=0.0, posinf=0.0, neginf=0.0)
            self.grad_shard.copy_(g)
            self.sumsq.copy_(g.pow(2).sum().view(1))

    @torch.no_grad()
    def all_gather_params(self, transport: str, src: Optional[torch.Tensor] = None):
        """Rebuild the full bf16 buffer from every rank's master shard (or ``src`` shard)."""
        shard = (self.master if src is None else src).to(self.compute_dtype)
        if self.P == 1:
            self.full.copy_(shard)
            return
        tmp = torch.empty(self.P, self.shard_numel, dtype=self.compute_dtype, device=self.device)
        dist.all_gather_into_tensor(tmp.view(-1), shard.contiguous(), group=self.group)
        for s in self.slots:
            stride = self._stride(s)
            dst = self.full[s.full_offset: s.full_offset + stride * self.P].view(self.P, stride)
            dst.copy_(tmp[:, s.shard_offset: s.shard_offset + stride])

    # ---- optimizer math on the shard ----------------------------------------------------------
    @torch.no_grad()
    def adamw(self, *, lr, beta1, beta2, eps, weight_decay, step, clip_coef: torch.Tensor, ema_beta: Optional[float]):
        if self.device.type == "cuda":
            ops = native.load()
            ops.adamw_ema_shard(self.master, self.grad_shard, self.exp_avg, self.exp_avg_sq,
                                self.ema if self.ema is not None else None,
                                self.full if self.P == 1 else None, clip_coef,
                                float(lr), float(beta1), float(beta2), float(eps), float(weight_decay), int(step),
                                float(ema_beta if ema_beta is not None else -1.0))
            native.count_launch()
        else:
            g = self.grad_shard * clip_coef.to(self.grad_shard)
            ref.adamw_step(self.master, g, self.exp_avg, self.exp_avg_sq, lr=lr, beta1=beta1, beta2=beta2, eps=eps,
                           weight_decay=weight_decay, step=step)
            if self.ema is not None and ema_beta is not None:
                self.ema.mul_(ema_beta).add_(self.master, alpha=1.0 - ema_beta)
            if self.P == 1:
                self.full.copy_(self.master.to(self.compute_dtype))

    @torch.no_grad()
    def zero_grad(self):
        self.grad_full.zero_()
        self.reduced = False
        self._pending = 0


class ShardedEngine:
    """Owns the flat units of one network and drives reduce-scatter, clipping, AdamW, EMA and the
    parameter all-gather."""

    def __init__(self, net: nn.Module, group=None, compute_dtype: torch.dtype = torch.bfloat16, use_ema: bool = True,
                 transport: str = "nccl", units: Optional[List[nn.Module]] = None, device: Optional[torch.device] = None,
                 grad_divide: Optional[float] = None, replicate_group=None):
        self.net = net
        self.group = group
        self.P, self.rank = _group_size_rank(group)
        self.replicate_group = replicate_group
        self.R = _group_size_rank(replicate_group)[0]
        if self.R == 1:
            self.replicate_group = None
        self.transport = transport
        self.compute_dtype = compute_dtype
        first = next(net.parameters())
        self.device = device or first.device
        self.grad_scale = 1.0 / (grad_divide if grad_divide is not None else self.P * self.R)
        unit_modules = units if units is not None else (net.fsdp_units() if hasattr(net, "fsdp_units") else [])
        claimed = set()
        self.units: List[FlatUnit] = []
        name_of = {id(p): n for n, p in net.named_parameters()}
        alloc = self._make_alloc()
        for i, m in enumerate(unit_modules):
            named = [(name_of[id(p)], p) for p in m.parameters() if p.requires_grad and id(p) not in claimed]
            claimed.update(id(p) for _, p in named)
            if named:
                self.units.append(self._make_unit(f"unit{i}", named, use_ema, alloc))
        rest = [(n, p) for n, p in net.named_parameters() if p.requires_grad and id(p) not in claimed]
        if rest:
            self.units.append(self._make_unit("root", rest, use_ema, alloc))
        # non-parameter floating buffers follow the compute dtype only if they already did
        self._sync_grads = True
        self._comm_stream = torch.cuda.Stream(device=self.device) if self.device.type == "cuda" else None
        self._install_hooks()
        self.step_count = 0

    # transports that need special memory override these two
    def _make_alloc(self):
        return None

    def _make_unit(self, name, named, use_ema, alloc) -> FlatUnit:
        return FlatUnit(name, named, self.group, self.compute_dtype, use_ema, self.device, alloc)

    # ---- backward hooks -----------------------------------------------------------------------------
    def _install_hooks(self):
        for u in self.units:
            for s in u.slots:
                s.param.register_post_accumulate_grad_hook(self._make_hook(u))

    def _make_hook(self, unit: FlatUnit):
        def hook(_param):
            unit._pending += 1
            if unit._pending == unit._n_trainable and self._sync_grads:
                self._reduce_unit(unit)
        return hook

    def set_requires_gradient_sync(self, flag: bool):
        """False while accumulating micro-batches: gradients stay local until the last one."""
        self._sync_grads = flag

    def _reduce_unit(self, unit: FlatUnit):
        def run():
            unit.reduce_scatter_grads(self.transport, self.grad_scale)
            if self.replicate_group is not None:
                unit.all_reduce_replicas(self.replicate_group)
        if self._comm_stream is not None:
            self._comm_stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self._comm_stream):
                run()
        else:
            run()

    def check_health(self) -> None:
        """Raise if a kernel recorded an error in the device's error word (a bounded wait that ran out: the kernel returned
        early and its output is not valid). Synchronises the device; the trainer calls it where it synchronises anyway."""
        if self.device.type == "cuda" and native.available():
            code = int(native.load().kernel_error(self.device.index, True))
            if code != 0:
                raise RuntimeError(f"a kernel gave up a bounded wait (error code {code}); the step's results are not valid")

    def finish_backward(self):
        """Reduce any unit whose hook did not fire (unused parameters) and join the comm stream."""
        for u in self.units:
            if not u.reduced:
                self._reduce_unit(u)
        if self._comm_stream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._comm_stream)

    # ---- optimizer step -----------------------------------------------------------------------------------
    @torch.no_grad()
    def grad_norm(self) -> torch.Tensor:
        total = torch.stack([u.sumsq for u in self.units]).sum().view(1)
        if self.P > 1:
            dist.all_reduce(total, group=self.group)
        return total.sqrt()

    @torch.no_grad()
    def step(self, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
             max_grad_norm: Optional[float] = None, ema_beta: Optional[float] = None) -> torch.Tensor:
        """Global-norm clip, AdamW on shards, EMA, refresh of the full bf16 parameters, zero grads.
        Returns the pre-clip gradient norm (a 1-element device tensor; no host sync)."""
        self.finish_backward()
        self.step_count += 1
        norm = self.grad_norm()
        if max_grad_norm is not None and max_grad_norm > 0:
            clip = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0)
        else:
            clip = torch.ones_like(norm)
        for u in self.units:
            u.adamw(lr=lr, beta1=betas[0], beta2=betas[1], eps=eps, weight_decay=weight_decay, step=self.step_count,
                    clip_coef=clip, ema_beta=ema_beta)
            if self.P > 1:
                u.all_gather_params(self.transport)
            u.zero_grad()
        return norm

    def zero_grad(self):
        for u in self.units:
            u.zero_grad()

    # ---- EMA swap ---------------------------------------------------------------------------------------------
    @torch.no_grad()
    def load_ema_into_params(self):
        for u in self.units:
            assert u.ema is not None, "EMA is disabled"
            u.all_gather_params(self.transport, src=u.ema)

    @torch.no_grad()
    def restore_params(self):
        for u in self.units:
            u.all_gather_params(self.transport)

    # ---- state for checkpoints --------------------------------------------------------------------------------
    def _slot_local(self, u: FlatUnit, s: ParamSlot, buf: torch.Tensor) -> torch.Tensor:
        lo, hi = u.local_rows(s)
        local = u.chunk_in_shard(s, buf)[: (hi - lo) * s.cols]
        return local.view(hi - lo, *s.shape[1:]) if len(s.shape) > 0 else local.view(())

    def sharded_state(self, which: str = "master") -> Dict[str, Tuple[torch.Tensor, torch.Size, int]]:
        """{param name: (local chunk view, global shape, row offset)} for which in
        {master, ema, exp_avg, exp_avg_sq}."""
        out = {}
        for u in self.units:
            buf = getattr(u, which)
            if buf is None:
                continue
            for s in u.slots:
                lo, _ = u.local_rows(s)
                out[s.name] = (self._slot_local(u, s, buf), s.shape, lo)
        return out

    @torch.no_grad()
    def full_state_dict(self, which: str = "master", dtype: Optional[torch.dtype] = None) -> Dict[str, torch.Tensor]:
        """Consolidated (unsharded) tensors on every rank."""
        out = {}
        for u in self.units:
            buf = getattr(u, which)
            if buf is None:
                continue
            if u.P > 1:
                tmp = torch.empty(u.P, u.shard_numel, dtype=buf.dtype, device=u.device)
                dist.all_gather_into_tensor(tmp.view(-1), buf.contiguous(), group=u.group)
            else:
                tmp = buf.view(1, -1)
            for s in u.slots:
                t = tmp[:, s.shard_offset: s.shard_offset + s.chunk_numel].reshape(u.P * s.chunk_rows, s.cols)[: s.rows]
                t = t.reshape(s.shape).clone()
                out[s.name] = t.to(dtype) if dtype is not None else t
        return out

    @torch.no_grad()
    def load_full_state_dict(self, sd: Dict[str, torch.Tensor], which: str = "master", strict: bool = True):
        """Load consolidated tensors into this rank's shards (and refresh params for master)."""
        missing = []
        for u in self.units:
            buf = getattr(u, which)
            if buf is None:
                continue
            for s in u.slots:
                if s.name not in sd:
                    missing.append(s.name)
                    continue
                src = sd[s.name].to(device=u.device, dtype=buf.dtype).reshape(s.rows, s.cols)
                lo, hi = u.local_rows(s)
                u.chunk_in_shard(s, buf)[: (hi - lo) * s.cols].copy_(src[lo:hi].reshape(-1))
        if strict and missing:
            raise KeyError(f"missing keys: {missing[:8]}{'...' if len(missing) > 8 else ''}")
        if which == "master":
            self.restore_params()
        return missing

    def num_parameters(self) -> int:
        return sum(s.param.numel() for u in self.units for s in u.slots)
