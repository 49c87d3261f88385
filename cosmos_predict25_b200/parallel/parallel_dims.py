"""Five-way parallel layout (pipeline, replicated data, sharded data, context, tensor) and its device mesh.

Parity target: ``ParallelDims`` (cosmos_predict2/_src/reason1/parallelisms/parallel_dims.py:25-160): degrees must multiply to
the world size (``dp_shard = -1`` is inferred; a mismatching ``dp_replicate`` is recomputed with a warning); the mesh keeps
only the dimensions larger than one, ordered ``pp, dp_replicate, dp_shard, cp, tp`` (tp innermost = adjacent GPUs), and
flattened views ``dp`` (data loading), ``dp_shard_cp`` (parameter sharding) and ``dp_cp`` (loss all-reduce) are created.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Tuple

from ..utils import log

ORDER = ("pp", "dp_replicate", "dp_shard", "cp", "tp")


@dataclass
class ParallelDims:
    dp_replicate: int = 1
    dp_shard: int = -1
    cp: int = 1
    tp: int = 1
    pp: int = 1
    world_size: int = 1
    enable_loss_parallel: bool = False

    def __post_init__(self):
        self._validate()

    def _validate(self):
        for d in (self.dp_replicate, self.cp, self.tp, self.pp):
            assert d >= 1, "Parallelism degree should be >= 1, except for dp_shard"
        assert self.dp_shard == -1 or self.dp_shard >= 1, "dp_shard must be -1 or >= 1"
        rest = self.dp_replicate * self.cp * self.tp * self.pp
        if self.dp_shard < 0:
            self.dp_shard = self.world_size // rest
        assert self.dp_shard >= 1
        if self.dp_replicate * self.dp_shard * self.cp * self.tp * self.pp != self.world_size:
            log.warning(f"invalid parallel dims: dp_replicate({self.dp_replicate}) * dp_shard({self.dp_shard}) * cp({self.cp}) * "
                        f"tp({self.tp}) * pp({self.pp}) != WORLD_SIZE({self.world_size}); recomputing dp_replicate")
            self.dp_replicate = self.world_size // (self.dp_shard * self.cp * self.tp * self.pp)
            assert self.dp_replicate * self.dp_shard * self.cp * self.tp * self.pp == self.world_size, "degrees do not divide the world size"

    def mesh_shape(self) -> Tuple[List[int], List[str]]:
        dims, names = [], []
        for name in ORDER:
            d = getattr(self, name)
            if d > 1:
                dims.append(d)
                names.append(name)
        return dims, names

    def flattened_views(self) -> Dict[str, List[str]]:
        dp, dp_shard_cp, dp_cp = [], [], []
        if self.dp_replicate_enabled:
            dp.append("dp_replicate")
            dp_cp.append("dp_replicate")
        if self.dp_shard_enabled:
            dp.append("dp_shard")
            dp_shard_cp.append("dp_shard")
            dp_cp.append("dp_shard")
        if self.cp_enabled:
            dp_shard_cp.append("cp")
            dp_cp.append("cp")
        return {k: v for k, v in (("dp", dp), ("dp_shard_cp", dp_shard_cp), ("dp_cp", dp_cp)) if v}

    def build_mesh(self, device_type: str):
        from torch.distributed.device_mesh import init_device_mesh
        dims, names = self.mesh_shape()
        if not dims:
            dims, names = [1], ["dp_shard"]
        mesh = init_device_mesh(device_type, tuple(dims), mesh_dim_names=tuple(names))
        for flat, parts in self.flattened_views().items():
            parts = [p for p in parts if p in names]
            if parts:
                mesh[tuple(parts)]._flatten(mesh_dim_name=flat)
        return mesh

    def coordinates(self, rank: int) -> Dict[str, int]:
        """Position of ``rank`` along every dimension (tp fastest)."""
        out, r = {}, rank
        for name in reversed(ORDER):
            d = getattr(self, name)
            out[name] = r % d
            r //= d
        return out

    dp_enabled = property(lambda s: s.dp_replicate > 1 or s.dp_shard > 1)
    dp_replicate_enabled = property(lambda s: s.dp_replicate > 1)
    dp_shard_enabled = property(lambda s: s.dp_shard > 1)
    cp_enabled = property(lambda s: s.cp > 1)
    tp_enabled = property(lambda s: s.tp > 1)
    pp_enabled = property(lambda s: s.pp > 1)
    loss_parallel_enabled = property(lambda s: s.tp > 1 and s.enable_loss_parallel)
    non_data_parallel_size = property(lambda s: s.cp * s.tp * s.pp)
