"""Sharded engine that does NOT keep the full bf16 parameters of the transformer blocks resident: the FSDP all-gather is fused
into the GEMM that consumes each weight.

What FSDP2 does per block - all-gather the parameters before the block's forward, free them after it, gather again in backward
(cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:1688-1699,
cosmos_predict2/_src/predict2/models/text2world_model_rectified_flow.py:177-249) - is restated for peer memory:

  * every rank keeps, per resharded unit, only its own ``Shard(0)`` chunk of every parameter as bf16 (``shard16``, in the
    symmetric arena so that peers can read it) beside the fp32 master / moment / EMA shards of the base engine;
  * all resharded units share ONE full-size workspace; their parameters' ``.data`` are views into it. A large matrix is
    brought into the workspace by the GEMM that multiplies with it: ``gemm_bf16_gather`` pulls the row shards from their owners
    with plain peer loads in 256-row groups while its tensor-core tiles already run on the groups that have landed
    (``ops/csrc/gemm_tcgen05.cu``, template flag GATHER), in the forward and again in the input-gradient GEMM;
  * the small parameters of a unit (norm weights, AdaLN matrices, biases) are gathered by one peer-read kernel when the unit's
    module is entered (forward, the recompute pass of activation checkpointing, and a backward that runs without recompute);
  * the optimizer writes the updated bf16 chunk into the local ``shard16`` only - the parameter push into every peer's resident
    copy of the base engine disappears.

Units that are not resharded (final layer, timestep embedder, root) behave as in ``PeerShardedEngine``. Resident bf16 parameter
memory per rank drops from the model size to model size / P + one unit (2B, 8 ranks: 3.9 GB -> 0.63 GB; 14B: 27 GB -> 4.2 GB).
Weights of a resharded unit are valid only while that unit runs, so code that reads several units' parameters at once
(building the cross-attention K/V cache of all blocks for sampling) needs the resident engine.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import native
from .fsdp import _group_size_rank
from .peer_fsdp import PeerFlatUnit, PeerShardedEngine

BIG_NUMEL = 1 << 20          # matrices at least this large are gathered inside their GEMM


@dataclass
class GatherInfo:
    """What ``ops.functional.linear`` needs to run a weight through the gather GEMM."""

    shard_ptrs: List[int]     # address of this parameter's chunk on every rank
    chunk_rows: int
    counters: torch.Tensor    # int32 scratch, one per 256 rows


class ReshardFlatUnit(PeerFlatUnit):
    """A unit whose full-layout parameter buffer is the engine's shared workspace."""

    def __init__(self, *args, workspace_alloc=None, gather_ids=None, **kwargs):
        """``gather_ids``: ids of the parameters whose consumer is ``ops.functional.linear`` (the only caller that can bring a
        weight in through the gather GEMM); every other parameter is gathered when the unit is entered."""
        self._workspace_alloc = workspace_alloc
        self._alloc_calls = 0
        super().__init__(*args, **kwargs)
        P = self.P
        dev = self.device
        st = self._peer_alloc(self.shard_numel, self.compute_dtype)
        self.shard16, self.shard16_ptrs = st.tensor, st.ptrs
        self.shard16.copy_(self.master.to(self.compute_dtype))
        esize = self.shard16.element_size()
        small_rows = []
        self.big_slots = []
        for s in self.slots:
            big = (len(s.shape) == 2 and s.param.numel() >= BIG_NUMEL and s.rows % (8 * P) == 0 and s.cols % 64 == 0
                   and (gather_ids is None or id(s.param) in gather_ids))
            if big:
                self.big_slots.append(s)
                n_groups = (s.rows + 255) // 256
                s.param._cb200_gather = GatherInfo([p + s.shard_offset * esize for p in self.shard16_ptrs], s.chunk_rows,
                                                   torch.zeros(n_groups, dtype=torch.int32, device=dev))
            else:
                small_rows.append([s.full_offset, self._stride(s), s.shard_offset, s.chunk_numel])
        self.small_segs = torch.tensor(small_rows, dtype=torch.int64, device=dev) if small_rows else None

    def _alloc_symmetric(self, numel, dtype):
        # FlatUnit asks for the full parameter buffer first, then for the full gradient buffer
        self._alloc_calls += 1
        if self._alloc_calls == 1:
            ws = self._workspace_alloc(numel, dtype)
            self._ptrs[id(ws)] = None            # never addressed by peers
            return ws
        return super()._alloc_symmetric(numel, dtype)

    @torch.no_grad()
    def gather_small(self):
        """Bring every small parameter of this unit into the workspace (the large ones arrive inside their GEMMs)."""
        if self.small_segs is not None:
            native.load().gather_slots_peer(self.shard16_ptrs, self.small_segs, self.full)
            native.count_launch()

    @torch.no_grad()
    def refresh_shard16(self, src: Optional[torch.Tensor] = None):
        self.shard16.copy_((self.master if src is None else src).to(self.compute_dtype))


class ReshardEngine(PeerShardedEngine):
    """``PeerShardedEngine`` with the block units resharded (see the module docstring). ``reshard`` selects the units by index;
    default: the units that are entries of ``net.blocks``."""

    def __init__(self, net, group=None, compute_dtype: torch.dtype = torch.bfloat16, use_ema: bool = True, transport: str = "peer",
                 units=None, device=None, grad_divide=None, replicate_group=None, reshard: Optional[List[int]] = None):
        unit_modules = units if units is not None else (net.fsdp_units() if hasattr(net, "fsdp_units") else [])
        blocks = set(id(b) for b in getattr(net, "blocks", []))
        self._reshard_ids = set(reshard) if reshard is not None else {i for i, m in enumerate(unit_modules) if id(m) in blocks}
        self._unit_modules = list(unit_modules)
        self._workspace: Optional[torch.Tensor] = None
        self._make_count = 0
        super().__init__(net, group=group, compute_dtype=compute_dtype, use_ema=use_ema, transport=transport, units=unit_modules,
                         device=device, grad_divide=grad_divide, replicate_group=replicate_group)
        self._current: Optional[ReshardFlatUnit] = None
        net._params_sharded = True            # code that reads several blocks' parameters in one kernel must not run
        for u in self.units:
            if isinstance(u, ReshardFlatUnit):
                mod = u.module
                mod.register_forward_pre_hook(self._enter(u))
                mod.register_full_backward_pre_hook(self._enter_backward(u))
        torch.cuda.synchronize(self.device)
        dist.barrier(self.ctx.group)          # every rank's shard16 is initialised before a peer reads it

    # ---- construction -------------------------------------------------------------------------------------
    def _workspace_alloc(self, numel, dtype):
        if self._workspace is None:
            self._workspace = torch.zeros(numel, dtype=dtype, device=self.device)
        assert numel <= self._workspace.numel(), "resharded units must not exceed the first one in size"
        return self._workspace[:numel]

    def _make_unit(self, name, named, use_ema, alloc):
        idx = int(name[4:]) if name.startswith("unit") else -1
        if idx in self._reshard_ids:
            from ..models.dit import FusedLinear
            mod = self._unit_modules[idx]
            gather_ids = {id(m.weight) for m in mod.modules() if isinstance(m, FusedLinear)}
            u = ReshardFlatUnit(name, named, self.group, self.compute_dtype, use_ema, self.device,
                                peer_alloc=lambda n, dt: self.arena.alloc(n, dt), workspace_alloc=self._workspace_alloc,
                                gather_ids=gather_ids)
            u.module = mod
            return u
        return super()._make_unit(name, named, use_ema, alloc)

    def _enter(self, unit: ReshardFlatUnit):
        def hook(_module, _args):
            unit.gather_small()
            self._current = unit
        return hook

    def _enter_backward(self, unit: ReshardFlatUnit):
        def hook(_module, _grad_output):
            if self._current is not unit:        # no recompute pass has just refilled the workspace for this unit
                unit.gather_small()
                self._current = unit
        return hook

    # ---- optimizer ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def step(self, *, lr: float, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
             max_grad_norm: Optional[float] = None, ema_beta: Optional[float] = None) -> torch.Tensor:
        ops = self.ctx.ops
        self.finish_backward()
        self.step_count += 1
        self.ctx.barrier()                        # all squared sums final, all peer reads of gradients done
        norm = self.grad_norm()
        clip = torch.clamp(max_grad_norm / (norm + 1e-6), max=1.0) if max_grad_norm else torch.ones_like(norm)
        for u in self.units:
            if isinstance(u, ReshardFlatUnit):
                ops.adamw_ema_shard(u.master, u.grad_shard, u.exp_avg, u.exp_avg_sq, u.ema, u.shard16, clip, float(lr), float(betas[0]),
                                    float(betas[1]), float(eps), float(weight_decay), self.step_count,
                                    float(ema_beta if ema_beta is not None else -1.0))
            else:
                ops.adamw_push_peer(u.full_ptrs, self.sumsq_slot.ptrs, u.segs, u.master, u.grad_shard, u.exp_avg, u.exp_avg_sq,
                                    u.ema, self.rank, float(max_grad_norm or 0.0), float(lr), float(betas[0]), float(betas[1]),
                                    float(eps), float(weight_decay), self.step_count,
                                    float(ema_beta if ema_beta is not None else -1.0), self.norm_out)
            native.count_launch()
            u.zero_grad()
        self._current = None
        self.ctx.barrier()                        # parameter stores (resident units) and shard16 updates are visible to every rank
        self.sumsq_slot.tensor.zero_()
        return norm

    # ---- EMA swap / restore ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def load_ema_into_params(self):
        for u in self.units:
            assert u.ema is not None, "EMA is disabled"
            if isinstance(u, ReshardFlatUnit):
                u.refresh_shard16(u.ema)
            else:
                u.all_gather_params(self.transport, src=u.ema)
        self._sync_shards()

    @torch.no_grad()
    def restore_params(self):
        for u in self.units:
            if isinstance(u, ReshardFlatUnit):
                u.refresh_shard16()
            else:
                u.all_gather_params(self.transport)
        self._sync_shards()

    def _sync_shards(self):
        self._current = None
        if getattr(self, "ctx", None) is not None:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.ctx.group)

    # ---- accounting -------------------------------------------------------------------------------------------------
    def resident_parameter_bytes(self) -> int:
        """bf16 parameter bytes this rank keeps between steps: shards of the resharded units, the shared workspace and the full
        buffers of the resident units."""
        n = self._workspace.numel() if self._workspace is not None else 0
        for u in self.units:
            n += u.shard_numel if isinstance(u, ReshardFlatUnit) else u.full_numel
        return n * torch.empty((), dtype=self.compute_dtype).element_size()
