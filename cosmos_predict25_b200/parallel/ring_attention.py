"""Ring (point-to-point) context-parallel self-attention.

The reference exposes this as the ``cp_comm_type="p2p"`` alternative to the Ulysses all-to-all: TransformerEngine's
``DotProductAttention.set_context_parallel_group(..., cp_comm_type="p2p")`` (cosmos_predict2/_src/predict2/networks/
minimal_v4_dit.py:361-371,446-448; Wan2.1 configs select it, cosmos_predict2/_src/predict2/networks/wan2pt1.py:378-384).
Unlike Ulysses it does not need the head count to divide by the group size and never holds the whole sequence of a head
on one GPU: every rank keeps its query shard and the key / value shards travel round the ring.

Forward, P ranks, step i = 0 .. P-1: attend the local queries to the key / value shard that originated on rank
(r - i) mod P, which gives a partial output and its log-sum-exp; partial results merge exactly:
``lse = logaddexp(lse_a, lse_b)``, ``o = o_a * exp(lse_a - lse) + o_b * exp(lse_b - lse)``. While a shard is being
attended to, the next one is already in flight (send to r+1, receive from r-1).

Backward: with the merged ``o`` and ``lse`` the contribution of one key / value shard to dq, dk, dv is what the ordinary
attention backward computes when it is handed those global statistics (P_block = exp(S_block * scale - lse),
delta = rowsum(do * o)), so the backward walks the ring once more: dq accumulates locally, dk / dv travel with their
shard and arrive home after P steps. The per-shard products run on this package's attention kernels on the GPU and on
the closed-form PyTorch expressions on the CPU (gloo tests).
"""

from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import functional as ops
from ..ops import native, ref


def _rotate(tensors, group, rank: int, size: int):
    """Start sending ``tensors`` to rank+1 and receiving the same shapes from rank-1; returns (received buffers, requests)."""
    nxt, prv = (rank + 1) % size, (rank - 1) % size
    if group is not None and group is not dist.group.WORLD:
        nxt, prv = dist.get_global_rank(group, nxt), dist.get_global_rank(group, prv)
    recv = [torch.empty_like(t) for t in tensors]
    p2p = []
    for t, r in zip(tensors, recv):
        p2p.append(dist.P2POp(dist.isend, t.contiguous(), nxt, group))
        p2p.append(dist.P2POp(dist.irecv, r, prv, group))
    return recv, dist.batch_isend_irecv(p2p)


def _block_fwd(q, k, v, scale) -> Tuple[torch.Tensor, torch.Tensor]:
    """(o fp32 [B,S,H,D], lse fp32 [B,H,S]) of the local queries against one key / value shard."""
    if ops.native_attention_supported(q, k) and native.use_native(q):
        o, lse = native.load().fa_fwd(q.contiguous(), k.contiguous(), v.contiguous(), scale)
        native.count_launch()
        return o.float(), lse
    o, lse = ref.attention(q.float(), k.float(), v.float(), scale)
    return o, lse


def _block_bwd(do, q, k, v, o, lse, scale):
    """dq, dk, dv of one shard given the *global* output and log-sum-exp of the query rows."""
    if ops.native_attention_supported(q, k) and native.use_native(q) and hasattr(native.load(), "fa_bwd"):
        dq, dk, dv = native.load().fa_bwd(do.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), o.contiguous(), lse.contiguous(),
                                          scale)
        native.count_launch(3)
        return dq.float(), dk.float(), dv.float()
    qf, kf, vf, dof, of = (t.float().transpose(1, 2) for t in (q, k, v, do, o))     # [B,H,S,D]
    p = torch.exp(torch.matmul(qf, kf.transpose(-1, -2)) * scale - lse.unsqueeze(-1))
    dv = torch.matmul(p.transpose(-1, -2), dof)
    dp = torch.matmul(dof, vf.transpose(-1, -2))
    delta = (dof * of).sum(-1, keepdim=True)
    ds = p * (dp - delta) * scale
    dq = torch.matmul(ds, kf)
    dk = torch.matmul(ds.transpose(-1, -2), qf)
    return dq.transpose(1, 2), dk.transpose(1, 2), dv.transpose(1, 2)


def _merge(o, lse, o_i, lse_i):
    """Exact merge of two partial softmax results; o [B,S,H,D] fp32, lse [B,H,S] fp32."""
    new = torch.logaddexp(lse, lse_i)
    wa = torch.exp(lse - new).transpose(1, 2).unsqueeze(-1)
    wb = torch.exp(lse_i - new).transpose(1, 2).unsqueeze(-1)
    return o * wa + o_i * wb, new


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, group):
        size, rank = dist.get_world_size(group), dist.get_rank(group)
        kv = [k.contiguous(), v.contiguous()]
        o = lse = None
        for step in range(size):
            if step + 1 < size:
                nxt, reqs = _rotate(kv, group, rank, size)
            o_i, lse_i = _block_fwd(q, kv[0], kv[1], scale)
            o, lse = (o_i, lse_i) if o is None else _merge(o, lse, o_i, lse_i)
            if step + 1 < size:
                for r in reqs:
                    r.wait()
                kv = nxt
        out = o.to(q.dtype)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.scale, ctx.group = scale, group
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse = ctx.saved_tensors
        group, scale = ctx.group, ctx.scale
        size, rank = dist.get_world_size(group), dist.get_rank(group)
        do = do.contiguous()
        kv = [k.contiguous(), v.contiguous()]
        dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
        dkv = [torch.zeros(k.shape, dtype=torch.float32, device=k.device), torch.zeros(v.shape, dtype=torch.float32, device=v.device)]
        for step in range(size):
            if step + 1 < size:
                nxt, reqs = _rotate(kv, group, rank, size)
            dq_i, dk_i, dv_i = _block_bwd(do, q, kv[0], kv[1], o, lse, scale)
            dq += dq_i
            dkv[0] += dk_i
            dkv[1] += dv_i
            if step + 1 < size:
                for r in reqs:
                    r.wait()
                kv = nxt
            # the gradient accumulators follow their shard round the ring; after the last step one more hop brings
            # every shard's gradient back to the rank that owns the shard
            moved, reqs_g = _rotate(dkv, group, rank, size)
            for r in reqs_g:
                r.wait()
            dkv = moved
        return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype), None, None


def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scale: Optional[float] = None) -> torch.Tensor:
    """Non-causal self-attention over a sequence sharded on dim 1 across ``group``; q, k, v: [B, S_loc, H, D]."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ops.attention(q, k, v, scale)
    return _RingAttention.apply(q, k, v, scale, group)
