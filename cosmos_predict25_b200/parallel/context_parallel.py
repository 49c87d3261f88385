"""Tensor utilities for context (sequence) parallelism.

Split a tensor along the sequence dim by rank, concatenate shards back (with or without gradient),
broadcast tensors whose shape the receivers do not know, and the composed broadcast-then-split used
for inputs created on the lowest rank of a context-parallel group. Behaviour follows
cosmos_predict2/_src/predict2/utils/context_parallel.py:26-191. These are cold paths (once per
step or per sample) and deliberately stay on torch.distributed (NCCL on GPUs, gloo on CPU).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist


def _size_rank(group):
    if group is None or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def split_inputs_cp(x: torch.Tensor, seq_dim: int, cp_group) -> torch.Tensor:
    """Return this rank's contiguous chunk of ``x`` along ``seq_dim``."""
    P, r = _size_rank(cp_group)
    if P == 1:
        return x
    assert x.shape[seq_dim] % P == 0, f"dim {seq_dim} of size {x.shape[seq_dim]} not divisible by cp size {P}"
    n = x.shape[seq_dim] // P
    return x.narrow(seq_dim, r * n, n).contiguous()


def cat_outputs_cp(x: torch.Tensor, seq_dim: int, cp_group) -> torch.Tensor:
    """All-gather shards and concatenate along ``seq_dim`` (no gradient)."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return x
    outs = [torch.empty_like(x) for _ in range(P)]
    dist.all_gather(outs, x.contiguous(), group=cp_group)
    return torch.cat(outs, dim=seq_dim)


class _GatherCat(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim, group):
        ctx.seq_dim, ctx.group = seq_dim, group
        return cat_outputs_cp(x, seq_dim, group)

    @staticmethod
    def backward(ctx, g):
        P, r = _size_rank(ctx.group)
        n = g.shape[ctx.seq_dim] // P
        return g.narrow(ctx.seq_dim, r * n, n).contiguous(), None, None


def cat_outputs_cp_with_grad(x: torch.Tensor, seq_dim: int, cp_group) -> torch.Tensor:
    """Like ``cat_outputs_cp`` but differentiable: the gradient of the concatenation is this
    rank's slice of the incoming gradient."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return x
    return _GatherCat.apply(x, seq_dim, cp_group)


_DTYPES = [torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.int16,
           torch.int8, torch.uint8, torch.bool]


def robust_broadcast(x: Optional[torch.Tensor], src: int, group, device=None) -> torch.Tensor:
    """Broadcast a tensor whose shape/dtype only the source knows: header (ndim, dtype id, dims)
    first, then the payload. ``src`` is a global rank."""
    rank = dist.get_rank()
    dev = device if device is not None else (x.device if x is not None else torch.device("cpu"))
    header = torch.zeros(10, dtype=torch.int64, device=dev)
    if rank == src:
        assert x is not None and x.ndim <= 8
        header[0] = x.ndim
        header[1] = _DTYPES.index(x.dtype)
        header[2:2 + x.ndim] = torch.tensor(list(x.shape), dtype=torch.int64)
    dist.broadcast(header, src, group=group)
    h = header.tolist()
    shape, dtype = h[2:2 + h[0]], _DTYPES[h[1]]
    if rank != src:
        x = torch.empty(shape, dtype=dtype, device=dev)
    else:
        x = x.to(dev).contiguous()
    dist.broadcast(x, src, group=group)
    return x


def broadcast(item, cp_group):
    """Broadcast a tensor (or any picklable object) from the lowest rank of ``cp_group``."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return item
    src = dist.get_global_rank(cp_group, 0) if cp_group is not dist.group.WORLD and cp_group is not None else 0
    if isinstance(item, torch.Tensor):
        return robust_broadcast(item, src, cp_group)
    box = [item]
    dist.broadcast_object_list(box, src, group=cp_group)
    return box[0]


def broadcast_split_tensor(x: torch.Tensor, seq_dim: int, cp_group) -> torch.Tensor:
    """Make every rank see rank-0's tensor, then keep the local chunk along ``seq_dim``."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return x
    x = broadcast(x, cp_group)
    return split_inputs_cp(x, seq_dim, cp_group)
