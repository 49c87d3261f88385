"""Ulysses (all-to-all) context parallelism for self-attention.

Activations stay sharded along the sequence (whole latent frames per rank) everywhere except
inside self-attention, where q, k, v are exchanged so that each rank holds the *full* sequence
for ``H / cp`` heads, and the attention output is exchanged back. The backward of each exchange
is the reverse exchange. Semantics follow the reference
(cosmos_predict2/_src/predict2/networks/a2a_cp.py:45-226).

Two transports implement the exchange:
  * ``torch.distributed.all_to_all_single`` (NCCL on GPUs, gloo on CPU test worlds): the twin
    kept as baseline and as oracle;
  * the peer-memory transport in ``symm.py``: a kernel of this package writes each head slice
    straight into the destination rank's buffer over NVLink (selected when the group has a
    symmetric workspace attached through ``attach_peer_transport``).
"""

from __future__ import annotations

from typing import Optional, Tuple

import math

import torch
import torch.distributed as dist

from ..ops import functional as ops

_peer_transports = {}


def group_size_rank(group) -> Tuple[int, int]:
    if group is None or not dist.is_available() or not dist.is_initialized():
        return 1, 0
    return dist.get_world_size(group), dist.get_rank(group)


def attach_peer_transport(group, transport) -> None:
    """Route the exchanges of ``group`` through a peer-memory transport (see symm.PeerAllToAll)."""
    _peer_transports[id(group)] = transport


def detach_peer_transport(group) -> None:
    _peer_transports.pop(id(group), None)


def _a2a(inp: torch.Tensor, group) -> torch.Tensor:
    out = torch.empty_like(inp)
    try:
        dist.all_to_all_single(out, inp, group=group)
    except RuntimeError:
        # gloo builds without alltoall: emulate with P point-to-point rounds (CPU test worlds only)
        P, r = group_size_rank(group)
        chunks_in = list(inp.chunk(P, dim=0))
        chunks_out = list(out.chunk(P, dim=0))
        chunks_out[r].copy_(chunks_in[r])
        reqs = []
        for p in range(P):
            if p != r:
                reqs.append(dist.isend(chunks_in[p].contiguous(), dist.get_global_rank(group, p), group=group))
                reqs.append(dist.irecv(chunks_out[p], dist.get_global_rank(group, p), group=group))
        for q in reqs:
            q.wait()
    return out


def seq_to_head(x: torch.Tensor, group) -> torch.Tensor:
    """[B, S_loc, H, D] (all heads, local tokens) -> [B, S_loc*P, H/P, D] (all tokens, local heads)."""
    P, _ = group_size_rank(group)
    B, S, H, D = x.shape
    assert H % P == 0, f"heads {H} not divisible by context-parallel size {P}"
    t = _peer_transports.get(id(group))
    if t is not None and x.is_cuda:
        return t.seq_to_head(x)
    send = x.view(B, S, P, H // P, D).permute(2, 0, 1, 3, 4).contiguous()  # [P, B, S, H/P, D]
    recv = _a2a(send, group)  # slot p = tokens of rank p for my heads
    return recv.permute(1, 0, 2, 3, 4).reshape(B, P * S, H // P, D)


def head_to_seq(x: torch.Tensor, group) -> torch.Tensor:
    """[B, S_loc*P, H/P, D] -> [B, S_loc, H, D]; the inverse of ``seq_to_head``."""
    P, _ = group_size_rank(group)
    B, SP, Hl, D = x.shape
    S = SP // P
    t = _peer_transports.get(id(group))
    if t is not None and x.is_cuda:
        return t.head_to_seq(x)
    send = x.view(B, P, S, Hl, D).permute(1, 0, 2, 3, 4).contiguous()  # [P, B, S, Hl, D]
    recv = _a2a(send, group)  # slot p = my tokens for heads of rank p
    return recv.permute(1, 2, 0, 3, 4).reshape(B, S, P * Hl, D)


class _SeqToHead(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return seq_to_head(x, group)

    @staticmethod
    def backward(ctx, g):
        return head_to_seq(g.contiguous(), ctx.group), None


class _HeadToSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return head_to_seq(x, group)

    @staticmethod
    def backward(ctx, g):
        return seq_to_head(g.contiguous(), ctx.group), None


class _ScatterHeadsFused(torch.autograd.Function):
    """q, k: per-head RMSNorm (+RoPE) fused with the seq->head exchange; v: plain exchange; one barrier for
    the three. Backward: head->seq exchange of the gradients, then the RMSNorm/RoPE backward kernel."""

    @staticmethod
    def forward(ctx, q, k, v, wq, wk, rope, eps, transport):
        (qh, kh, vh), (rq, rk, _) = transport.scatter_heads([q, k, v], [wq, wk, None], rope, eps)
        ctx.save_for_backward(q, k, wq, wk, rq, rk)
        ctx.rope, ctx.transport = rope, transport
        return qh, kh, vh

    @staticmethod
    def backward(ctx, dqh, dkh, dvh):
        from ..ops import native
        ops_n = native.load()
        q, k, wq, wk, rq, rk = ctx.saved_tensors
        t = ctx.transport
        dqn, dkn, dv = t.head_to_seq_many([g.contiguous() for g in (dqh, dkh, dvh)])
        cos, sin = ctx.rope.cos_sin() if ctx.rope is not None else (None, None)
        dq, dwq = ops_n.rmsnorm_rope_bwd(dqn, q, wq, rq, cos, sin)
        dk, dwk = ops_n.rmsnorm_rope_bwd(dkn, k, wk, rk, cos, sin)
        native.count_launch(4)
        return dq, dk, dv, dwq.to(wq.dtype), dwk.to(wk.dtype), None, None, None


class _ProjectScatterHeads(torch.autograd.Function):
    """Training form of the GEMM-epilogue exchange: ``x @ Wq^T``, ``x @ Wk^T``, ``x @ Wv^T`` leave their GEMMs normalised,
    rotated and already in the owners' staging buffers (no projected tensor in sequence layout is read back, no stand-alone
    exchange kernel); the same epilogue keeps the raw q / k projections and their reciprocal RMS locally for the backward.
    Backward: head->seq exchange of the three gradients, RMSNorm / RoPE backward kernel, then the input- and weight-gradient
    GEMMs (a2a_cp.py:120-158 of the reference is the differentiable exchange this replaces)."""

    @staticmethod
    def forward(ctx, x, wq, wk, wv, nq, nk, rope, eps, transport):
        B, S, D = x.shape
        x2d = x.reshape(B * S, D)
        x2d = x2d if x2d.is_contiguous() else x2d.contiguous()
        (qh, kh, vh), (q_raw, k_raw, _), (rq, rk, _) = transport.project_scatter_heads(
            x2d, [wq, wk, wv], [nq, nk, None], rope, B, S, eps, keep_for_backward=True)
        ctx.save_for_backward(x2d, wq, wk, wv, nq, nk, q_raw, k_raw, rq, rk)
        ctx.rope, ctx.transport, ctx.x_shape = rope, transport, x.shape
        return qh, kh, vh

    @staticmethod
    def backward(ctx, dqh, dkh, dvh):
        from ..ops import native
        from ..ops.functional import gemm_nt
        ops_n = native.load()
        x2d, wq, wk, wv, nq, nk, q_raw, k_raw, rq, rk = ctx.saved_tensors
        t = ctx.transport
        dqn, dkn, dv = t.head_to_seq_many([g.contiguous() for g in (dqh, dkh, dvh)])
        cos, sin = ctx.rope.cos_sin() if ctx.rope is not None else (None, None)
        dq, dnq = ops_n.rmsnorm_rope_bwd(dqn, q_raw, nq, rq, cos, sin)
        dk, dnk = ops_n.rmsnorm_rope_bwd(dkn, k_raw, nk, rk, cos, sin)
        native.count_launch(4)
        M = x2d.shape[0]
        g2 = [g.reshape(M, -1) for g in (dq, dk, dv)]
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm_nt(g2[0], wq, None, "none", False, True)
            dx += gemm_nt(g2[1], wk, None, "none", False, True)
            dx += gemm_nt(g2[2], wv, None, "none", False, True)
            dx = dx.view(ctx.x_shape)
        dws = [gemm_nt(g, x2d, None, "none", True, True) if need else None
               for g, need in zip(g2, ctx.needs_input_grad[1:4])]
        return (dx, dws[0], dws[1], dws[2], dnq.to(nq.dtype), dnk.to(nk.dtype), None, None, None)


def ulysses_projected_attention_train(x, wq, wk, wv, q_norm_weight, k_norm_weight, rope, group, eps: float = 1e-6,
                                      scale: Optional[float] = None):
    """Differentiable self-attention on a sequence shard ``x [B, S_loc, D]`` with the sequence->head exchange in the epilogue of
    the q / k / v GEMMs; the attention output returns through the head->sequence exchange. Returns [B, S_loc, H, 128]."""
    t = _peer_transports[id(group)]
    qh, kh, vh = _ProjectScatterHeads.apply(x, wq, wk, wv, q_norm_weight, k_norm_weight, rope, eps, t)
    oh = ops.attention(qh, kh, vh, scale)
    return _HeadToSeq.apply(oh, group)


def projected_attention_train_available(x: torch.Tensor, group, head_dim: int) -> bool:
    """True when the training form of the GEMM-epilogue exchange can run (peer transport attached, bf16 CUDA activations,
    128-wide heads, native kernels selected, not in forward-mode AD)."""
    from ..ops import native
    from ..ops.functional import settings
    import os
    return (id(group) in _peer_transports and x.is_cuda and x.dtype == torch.bfloat16 and head_dim == 128
            and torch.is_grad_enabled() and native.use_native(x) and settings.attention == "native" and settings.gemm == "native"
            and x.shape[-1] % 64 == 0 and (x.numel() // x.shape[-1]) % 8 == 0
            and os.environ.get("COSMOS_B200_TRAIN_EXCHANGE", "gemm") == "gemm")


def ulysses_attention_fused(q_raw, k_raw, v, q_norm_weight, k_norm_weight, rope, group, eps: float = 1e-6,
                            scale: Optional[float] = None):
    """Self-attention on un-normalised q/k projections with the q/k epilogue chain (RMSNorm, RoPE) fused into
    the peer-memory all-to-all. Falls back to the unfused composition when no peer transport is attached."""
    from ..ops import native
    t = _peer_transports.get(id(group))
    if t is None or not q_raw.is_cuda or native.forward_mode():
        q = ops.rmsnorm_rope(q_raw, q_norm_weight, rope, eps)
        k = ops.rmsnorm_rope(k_raw, k_norm_weight, rope, eps)
        return ulysses_attention(q, k, v, group, scale)
    if not (torch.is_grad_enabled() and any(x.requires_grad for x in (q_raw, k_raw, v, q_norm_weight, k_norm_weight))):
        # inference: consume the staged tensors in place, nothing is kept for a backward pass
        (qh, kh, vh), _ = t.scatter_heads([q_raw.contiguous(), k_raw.contiguous(), v.contiguous()],
                                          [q_norm_weight, k_norm_weight, None], rope, eps, copy_out=False)
        return t.head_to_seq(ops.attention(qh, kh, vh, scale))
    qh, kh, vh = _ScatterHeadsFused.apply(q_raw.contiguous(), k_raw.contiguous(), v.contiguous(), q_norm_weight, k_norm_weight,
                                          rope, eps, t)
    oh = ops.attention(qh, kh, vh, scale)
    return _HeadToSeq.apply(oh, group)


def projected_attention_available(x: torch.Tensor, group, head_dim: int) -> bool:
    """True when ``ulysses_projected_attention`` can run: a peer transport is attached to ``group``, nothing needs a
    backward pass, and the activations are bf16 on the GPU with 128-wide heads."""
    from ..ops import native
    from ..ops.functional import settings
    return (id(group) in _peer_transports and x.is_cuda and x.dtype == torch.bfloat16 and head_dim == 128
            and not torch.is_grad_enabled() and native.use_native(x) and settings.attention == "native"
            and settings.gemm == "native")


def _attention_exchange_mode() -> str:
    """How the attention output returns to sequence layout in the inference path: "store" = the attention kernel writes every
    finished row into its owner's shard (one barrier, no extra kernel); "gather" = attention, then the stand-alone gather kernel
    (two barriers). Both are exact; COSMOS_B200_ATTN_EXCHANGE selects, the default is the one that measured faster end to end."""
    import os
    return os.environ.get("COSMOS_B200_ATTN_EXCHANGE", "store")


def ulysses_projected_attention(x, wq, wk, wv, q_norm_weight, k_norm_weight, rope, group, eps: float = 1e-6,
                                scale: Optional[float] = None):
    """Inference self-attention on a sequence shard ``x [B, S_loc, D]``: the three projection GEMMs write their
    heads, normalised and rotated, directly into the peers' staging buffers (exchange in the GEMM epilogue),
    attention runs on the staged tensors and stores its output rows directly into the sequence shards of their
    owners (exchange in the attention epilogue). No stand-alone exchange kernel runs; two device barriers per call.
    Returns [B, S_loc, H, 128], aliasing a staging buffer: consume it before the next four calls."""
    t = _peer_transports[id(group)]
    B, S, D = x.shape
    x2d = x.reshape(B * S, D)
    if not x2d.is_contiguous():
        x2d = x2d.contiguous()
    qh, kh, vh = t.project_scatter_heads(x2d, [wq, wk, wv], [q_norm_weight, k_norm_weight, None], rope, B, S, eps)
    scale = scale if scale is not None else 1.0 / math.sqrt(qh.shape[-1])
    if _attention_exchange_mode() == "store":
        return t.attention_scatter_seq(qh, kh, vh, scale)
    return t.head_to_seq(ops.attention(qh, kh, vh, scale))


def _exchange_dual(fn, x: torch.Tensor) -> torch.Tensor:
    """Apply the linear map ``fn`` to a (possibly dual) tensor: value and tangent are mapped one after the other."""
    import torch.autograd.forward_ad as fwAD
    primal, tangent = fwAD.unpack_dual(x)
    y = fn(primal.contiguous())
    if tangent is None:
        return y
    return fwAD.make_dual(y, fn(tangent.contiguous()))


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group, scale: Optional[float] = None):
    """Self-attention over a sequence sharded on dim 1 across ``group``."""
    P, _ = group_size_rank(group)
    if P == 1:
        return ops.attention(q, k, v, scale)
    from ..ops import native
    if native.forward_mode():
        # forward-mode AD (consistency distillation): the exchanges are linear, so primal and tangent travel separately
        qh, kh, vh = (_exchange_dual(lambda x: seq_to_head(x, group), x) for x in (q, k, v))
        return _exchange_dual(lambda x: head_to_seq(x, group), ops.attention(qh, kh, vh, scale))
    qh = _SeqToHead.apply(q, group)
    kh = _SeqToHead.apply(k, group)
    vh = _SeqToHead.apply(v, group)
    oh = ops.attention(qh, kh, vh, scale)
    return _HeadToSeq.apply(oh, group)
