"""Process-group layout: data-parallel sharding (FSDP / HSDP) x context parallel.

Parity targets: ``hsdp_device_mesh`` (cosmos_predict2/_src/common/utils/fsdp_helper.py:97-159) and the
Megatron ``parallel_state`` groups the reference trainer creates (cosmos_predict2/_src/imaginaire/trainer.py:86-97):
context-parallel group, data-parallel group, data-parallel-with-CP group. Ranks are laid out with the
context-parallel dimension fastest, so a CP group is a set of adjacent GPUs of one NVSwitch domain.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, List, Optional

import torch.distributed as dist


@dataclass
class ParallelGroups:
    world_size: int = 1
    rank: int = 0
    cp_size: int = 1
    dp_size: int = 1
    shard_size: int = 1
    replicate_size: int = 1
    cp: Any = None          # ranks that share one sample, sequence-sharded
    dp: Any = None          # ranks holding different samples (same cp index)
    fsdp: Any = None        # ranks over which parameters are sharded (dp x cp within one replica)
    replicate: Any = None   # HSDP: ranks holding the same shard in different replicas

    @property
    def cp_rank(self) -> int:
        return self.rank % self.cp_size

    @property
    def dp_rank(self) -> int:
        return self.rank // self.cp_size


def build_groups(world_size: Optional[int] = None, cp_size: int = 1, shard_size: Optional[int] = None) -> ParallelGroups:
    """Create the groups (every rank must call this with the same arguments)."""
    if not (dist.is_available() and dist.is_initialized()) or (world_size or dist.get_world_size()) == 1:
        return ParallelGroups()
    W, r = dist.get_world_size(), dist.get_rank()
    assert W % cp_size == 0, f"world {W} not divisible by cp {cp_size}"
    dp_size = W // cp_size
    shard_size = W if shard_size in (None, -1, 0) else shard_size
    assert W % shard_size == 0 and shard_size % cp_size == 0, "shard group must contain whole CP groups"
    g = ParallelGroups(world_size=W, rank=r, cp_size=cp_size, dp_size=dp_size, shard_size=shard_size,
                       replicate_size=W // shard_size)
    if cp_size > 1:
        for i in range(dp_size):
            ranks = list(range(i * cp_size, (i + 1) * cp_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                g.cp = grp
    if dp_size > 1 and cp_size > 1:
        for j in range(cp_size):
            ranks = list(range(j, W, cp_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                g.dp = grp
    elif dp_size > 1:
        g.dp = dist.group.WORLD
    if shard_size == W:
        g.fsdp = dist.group.WORLD
    elif shard_size == 1:
        g.fsdp, g.replicate = None, dist.group.WORLD   # plain data parallelism: nothing is sharded
    else:
        for i in range(W // shard_size):
            ranks = list(range(i * shard_size, (i + 1) * shard_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                g.fsdp = grp
        for j in range(shard_size):
            ranks = list(range(j, W, shard_size))
            grp = dist.new_group(ranks)
            if r in ranks:
                g.replicate = grp
    return g


def hsdp_device_mesh(replica_group_size: Optional[int] = None, sharding_group_size: Optional[int] = None):
    """(replicate, shard) sizes with the reference's defaulting rules: shard defaults to the local world."""
    W = dist.get_world_size() if dist.is_initialized() else 1
    if sharding_group_size is None:
        sharding_group_size = W
    if replica_group_size is None:
        replica_group_size = W // sharding_group_size
    assert replica_group_size * sharding_group_size == W, "replicate x shard must equal the world size"
    return replica_group_size, sharding_group_size
