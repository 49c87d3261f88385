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


def robust_broadcast(x: Optional[torch.Tensor], src: int, group, device=None):
    """Broadcast from global rank ``src`` something whose kind, shape and dtype only the source knows.
    A 10-word header goes first: (kind, ndim, dtype id, dims...), kind 0 = tensor, 1 = picklable object;
    then the payload. Receivers may pass anything (it is ignored)."""
    rank = dist.get_rank()
    is_src = rank == src
    if device is None:
        device = x.device if isinstance(x, torch.Tensor) else torch.device("cpu")
        if dist.get_backend(group) == "nccl" and device.type != "cuda":
            device = torch.device("cuda", torch.cuda.current_device())
    header = torch.zeros(10, dtype=torch.int64, device=device)
    if is_src:
        if isinstance(x, torch.Tensor):
            assert x.ndim <= 7
            header[0] = 0
            header[1] = x.ndim
            header[2] = _DTYPES.index(x.dtype)
            if x.ndim:
                header[3:3 + x.ndim] = torch.tensor(list(x.shape), dtype=torch.int64)
        else:
            header[0] = 1
    dist.broadcast(header, src, group=group)
    h = header.tolist()
    if h[0] == 1:
        box = [x if is_src else None]
        dist.broadcast_object_list(box, src, group=group)
        return box[0]
    shape, dtype = h[3:3 + h[1]], _DTYPES[h[2]]
    buf = x.to(device).contiguous() if is_src else torch.empty(shape, dtype=dtype, device=device)
    dist.broadcast(buf, src, group=group)
    return buf


def broadcast(item, cp_group):
    """Broadcast a tensor (or any picklable object) from the lowest rank of ``cp_group``."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return item
    src = dist.get_global_rank(cp_group, 0) if cp_group is not None else 0
    return robust_broadcast(item, src, cp_group)


def broadcast_split_tensor(x: torch.Tensor, seq_dim: int, cp_group) -> torch.Tensor:
    """Make every rank see rank-0's tensor, then keep the local chunk along ``seq_dim``."""
    P, _ = _size_rank(cp_group)
    if P == 1:
        return x
    x = broadcast(x, cp_group)
    return split_inputs_cp(x, seq_dim, cp_group)
