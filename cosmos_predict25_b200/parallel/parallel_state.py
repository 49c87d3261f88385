"""Process-wide registry of the model-parallel groups, with the accessor names of Megatron's ``parallel_state``.

The reference keeps its groups in ``megatron.core.parallel_state`` (created in cosmos_predict2/_src/imaginaire/trainer.py:86-97
and read all over its models, checkpointers and inference scripts). This package passes ``ParallelGroups`` objects explicitly;
this module is the same information behind the global accessors, for code written against the reference:
``initialize_model_parallel(context_parallel_size=...)`` builds the groups once (context-parallel ranks adjacent), the getters
return groups / ranks / sizes, ``destroy_model_parallel()`` forgets them. Tensor, pipeline and expert parallelism of the
video models do not exist here (size 1, rank 0); the data-parallel group "with context parallel" is the world.
"""

from __future__ import annotations

from typing import Optional

import torch.distributed as dist

from .mesh import ParallelGroups, build_groups

_GROUPS: Optional[ParallelGroups] = None
_SELF_GROUP = None


def initialize_model_parallel(tensor_model_parallel_size: int = 1, pipeline_model_parallel_size: int = 1,
                              context_parallel_size: int = 1, expert_model_parallel_size: int = 1, **unused) -> ParallelGroups:
    global _GROUPS
    if tensor_model_parallel_size != 1 or pipeline_model_parallel_size != 1 or expert_model_parallel_size != 1:
        raise NotImplementedError("the video models are parallelised over data (sharded) and context only")
    assert _GROUPS is None, "model parallel is already initialized"
    _GROUPS = build_groups(cp_size=context_parallel_size)
    return _GROUPS


def set_groups(groups: ParallelGroups) -> None:
    """Publish groups that were built elsewhere (the training entry point builds them itself)."""
    global _GROUPS
    _GROUPS = groups


def is_initialized() -> bool:
    return _GROUPS is not None


model_parallel_is_initialized = is_initialized


def destroy_model_parallel() -> None:
    global _GROUPS, _SELF_GROUP
    _GROUPS = _SELF_GROUP = None


def _groups() -> ParallelGroups:
    assert _GROUPS is not None, "model parallel is not initialized"
    return _GROUPS


def _self_group():
    """A group of this rank alone: what a size-1 model-parallel dimension looks like to callers that ask for a group object."""
    global _SELF_GROUP
    if _SELF_GROUP is None and dist.is_available() and dist.is_initialized():
        for r in range(dist.get_world_size()):
            g = dist.new_group([r])
            if r == dist.get_rank():
                _SELF_GROUP = g
    return _SELF_GROUP


# ---- context parallel ------------------------------------------------------------------------------------------------------
def get_context_parallel_group(check_initialized: bool = True):
    return _groups().cp if (check_initialized or _GROUPS is not None) else None


def get_context_parallel_world_size() -> int:
    return _groups().cp_size


def get_context_parallel_rank() -> int:
    return _groups().cp_rank


# ---- data parallel ---------------------------------------------------------------------------------------------------------
def get_data_parallel_group(with_context_parallel: bool = False):
    g = _groups()
    if with_context_parallel:
        return dist.group.WORLD if dist.is_available() and dist.is_initialized() else None
    return g.dp


def get_data_parallel_world_size(with_context_parallel: bool = False) -> int:
    g = _groups()
    return g.world_size if with_context_parallel else g.dp_size


def get_data_parallel_rank(with_context_parallel: bool = False) -> int:
    g = _groups()
    return g.rank if with_context_parallel else g.dp_rank


# ---- dimensions of size one ------------------------------------------------------------------------------------------------
def get_model_parallel_group():
    _groups()
    return _self_group()


get_tensor_model_parallel_group = get_model_parallel_group


def get_tensor_model_parallel_world_size() -> int:
    return 1


def get_tensor_model_parallel_rank() -> int:
    return 0


def get_pipeline_model_parallel_world_size() -> int:
    return 1


def get_pipeline_model_parallel_rank() -> int:
    return 0


def get_expert_model_parallel_world_size() -> int:
    return 1


def get_expert_model_parallel_rank() -> int:
    return 0
