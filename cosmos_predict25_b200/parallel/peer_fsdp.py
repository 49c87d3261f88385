"""Sharded engine whose collectives are fused into kernels over NVLink peer memory.

Same state layout and semantics as ``fsdp.ShardedEngine`` (its NCCL twin), but:

  * the flat full-parameter and full-gradient buffers of all units live in one symmetric arena, so
    every rank can address every peer's copy;
  * reduce-scatter = ``rs_cast_norm_peer``: a rank READS its chunk of each peer's gradient buffer, sums in
    fp32, applies 1/world, scrubs NaN/Inf, stores the fp32 shard and the squared-norm partial - one
    kernel instead of NCCL reduce-scatter + cast + nan_to_num + norm;
  * optimizer + all-gather = ``adamw_push_peer``: AdamW/EMA on the fp32 shard; the global gradient norm is
    formed from every rank's published squared sum (read over NVLink) and the clip coefficient applied
    in-kernel; the updated bf16 chunk is STORED into every peer's full parameter buffer, so the forward
    pass of the next step needs no all-gather at all.

Ordering between ranks uses ``PeerContext.barrier`` (bounded device-side waits): one before a unit's
gradients are read (all peers have produced them), one before the optimizer (all squared sums are final
and all gradient reads are done, so gradients may be zeroed), one after it (all parameter stores have
landed). Requires every parameter's per-rank chunk to be a multiple of 8 elements (true for the DiT
presets at 2/4/8 ranks); otherwise use the NCCL twin.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import native
from .fsdp import FlatUnit, ShardedEngine, _group_size_rank
from .symm import PeerContext, SymmetricArena


def check_segment_table(segs: torch.Tensor, world: int, full_numel: int, shard_numel: int) -> None:
    """Bound every (full_offset, rank_stride, shard_offset, chunk_numel) row of a unit's segment table against the buffers
    the kernels will index with it. Runs once on the host copy when a unit is built: the kernels themselves take the table
    on trust, and a row that runs past a buffer would be an out-of-bounds access to a peer's memory."""
    for i, (full_off, stride, shard_off, n) in enumerate(segs.tolist()):
        if min(full_off, stride, shard_off, n) < 0 or stride < n:
            raise ValueError(f"segment {i}: negative field or rank stride {stride} below the chunk size {n}")
        if n % 8 != 0 or full_off % 8 != 0 or shard_off % 4 != 0:
            raise ValueError(f"segment {i}: offsets and sizes must keep 16-byte alignment")
        if full_off + (world - 1) * stride + n > full_numel:
            raise ValueError(f"segment {i} runs past the full buffer ({full_off} + {world - 1} * {stride} + {n} > {full_numel})")
        if shard_off + n > shard_numel:
            raise ValueError(f"segment {i} runs past the shard ({shard_off} + {n} > {shard_numel})")


class PeerFlatUnit(FlatUnit):
    def __init__(self, *args, peer_alloc=None, **kwargs):
        self._peer_alloc = peer_alloc
        self._ptrs = {}
        super().__init__(*args, alloc=self._alloc_symmetric, **kwargs)
        for s in self.slots:
            if s.chunk_numel % 8 != 0:
                raise ValueError(f"parameter {s.name}: per-rank chunk of {s.chunk_numel} elements is not a multiple of 8; "
                                 "use sharding_transport='nccl'")
        table = self.segment_table()
        check_segment_table(table, self.P, self.full_numel, self.shard_numel)
        self.segs = table.to(self.device)
        self.full_ptrs = self._ptrs[id(self.full)]
        self.grad_ptrs = self._ptrs[id(self.grad_full)]

    def _alloc_symmetric(self, numel, dtype):
        st = self._peer_alloc(numel, dtype)
        self._ptrs[id(st.tensor)] = st.ptrs
        return st.tensor


class PeerShardedEngine(ShardedEngine):
    def __init__(self, net, group=None, compute_dtype: torch.dtype = torch.bfloat16, use_ema: bool = True,
                 transport: str = "peer", units=None, device: Optional[torch.device] = None, grad_divide=None,
                 replicate_group=None):
        P, _ = _group_size_rank(group)
        dev = device or next(net.parameters()).device
        assert dev.type == "cuda" and P > 1, "the peer engine needs CUDA devices and more than one rank"
        esize = torch.empty((), dtype=compute_dtype).element_size()
        total = sum(p.numel() for p in net.parameters() if p.requires_grad)
        # 2 full-layout buffers (params, grads) + per-parameter padding + flags / slots
        nbytes = 2 * (total * esize + 64 * 1024 * max(1, len(list(net.parameters())))) + (1 << 20)
        self.arena = SymmetricArena(nbytes, group if group is not None else dist.group.WORLD, dev)
        self.ctx = PeerContext(group, dev, arena=self.arena)
        self.sumsq_slot = self.arena.alloc(64, torch.float32)
        self.norm_out = torch.zeros(1, dtype=torch.float32, device=dev)
        super().__init__(net, group=group, compute_dtype=compute_dtype, use_ema=use_ema, transport="peer", units=units,
                         device=dev, grad_divide=grad_divide, replicate_group=replicate_group)
        torch.cuda.synchronize(dev)
        dist.barrier(self.ctx.group)  # every rank's buffers are initialised before any peer touches them

    def _make_unit(self, name, named, use_ema, alloc):
        return PeerFlatUnit(name, named, self.group, self.compute_dtype, use_ema, self.device,
                            peer_alloc=lambda n, dt: self.arena.alloc(n, dt))

    # ---- reduce-scatter fused with cast / scale / scrub / norm partial -----------------------------------
    def _reduce_unit(self, unit):
        ops = self.ctx.ops
        self._comm_stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._comm_stream):
            self.ctx.barrier()  # every peer has finished this unit's backward
            ops.rs_cast_norm_peer(unit.grad_ptrs, unit.segs, unit.grad_shard, unit.sumsq, self.sumsq_slot.tensor[:1],
                                  self.rank, float(self.grad_scale))
            native.count_launch(2)
            if self.replicate_group is not None:
                # HSDP: the kernel has added this unit's squared sum to the published slot; swap it for the replica-summed one
                self.sumsq_slot.tensor[:1].sub_(unit.sumsq)
                unit.all_reduce_replicas(self.replicate_group)
                self.sumsq_slot.tensor[:1].add_(unit.sumsq)
        unit.reduced = True

    def check_health(self) -> None:
        """A device barrier that ran out of time only records an error word and returns, and the kernels after it would
        then work on stale peer data. The trainer calls this wherever it synchronises anyway (logging, before a
        checkpoint is written, end of training) so that such a run stops instead of saving a damaged state."""
        self.ctx.check()

    @torch.no_grad()
    def grad_norm(self) -> torch.Tensor:
        total = self.sumsq_slot.tensor[:1].clone()
        dist.all_reduce(total, group=self.group)
        return total.sqrt()

    # ---- AdamW + EMA + all-gather by peer stores ------------------------------------------------------------
    @torch.no_grad()
    def step(self, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
             max_grad_norm: Optional[float] = None, ema_beta: Optional[float] = None) -> torch.Tensor:
        ops = self.ctx.ops
        self.finish_backward()
        self.step_count += 1
        self.ctx.barrier()  # all squared sums final, all peer reads of gradients done
        for u in self.units:
            ops.adamw_push_peer(u.full_ptrs, self.sumsq_slot.ptrs, u.segs, u.master, u.grad_shard, u.exp_avg, u.exp_avg_sq,
                                u.ema, self.rank, float(max_grad_norm or 0.0), float(lr), float(betas[0]), float(betas[1]),
                                float(eps), float(weight_decay), self.step_count,
                                float(ema_beta if ema_beta is not None else -1.0), self.norm_out)
            native.count_launch()
            u.zero_grad()
        norm = self.norm_out.clone()
        self.ctx.barrier()  # every rank's parameter stores have landed; squared sums no longer needed
        self.sumsq_slot.tensor.zero_()
        return norm

    # EMA swap and restore go through the NCCL path of the base class (cold paths)
