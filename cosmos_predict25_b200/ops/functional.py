"""Differentiable front-ends of the fused ops.

CUDA tensors run the sm_100a kernels of the in-tree extension (forward and backward are
both hand-written kernels wrapped in ``torch.autograd.Function``); CPU tensors run the
PyTorch oracle in ``ref.py`` under ordinary autograd. The two contraction families that
also exist as vendor library calls (GEMM, attention) have a switch in ``settings`` so the
library twin can be timed against the hand-written kernel on the same box.
"""

from __future__ import annotations

import math
import os
from dataclasses import dataclass
from typing import Optional, Sequence, Tuple

import torch
import torch.autograd.forward_ad as fwAD
import torch.nn.functional as F

from . import native, ref


@dataclass
class OpSettings:
    """Which implementation serves the two contraction families on CUDA tensors.

    attention: "native" (tcgen05 flash attention of this package) or "cudnn"
               (torch SDPA pinned to the cuDNN backend: what the reference selects on sm_100,
               cosmos_predict2/_src/predict2/networks/attention.py:132-138).
    gemm:      "native" (tcgen05/TMA GEMM with fused epilogues) or "cublas" (torch.matmul).
    conv:      "native" (channels-last implicit-GEMM convolution kernel: the VAE decoder) or "cudnn" (torch convolutions).
    """

    attention: str = os.environ.get("COSMOS_B200_ATTENTION", "native")
    gemm: str = os.environ.get("COSMOS_B200_GEMM", "native")
    attention_bwd: str = os.environ.get("COSMOS_B200_ATTENTION_BWD", "native")
    conv: str = os.environ.get("COSMOS_B200_CONV", "native")


settings = OpSettings()


# --------------------------------------------------------------------------------------
# Forward-mode (tangent) paths. Inside ``native.forward_mode_ad()`` the network runs without autograd on dual tensors; each
# front-end unpacks (primal, tangent), runs a kernel that produces value and directional derivative together, and packs the
# result again, so the network JVP of the distillation step stays on this package's kernels.
# --------------------------------------------------------------------------------------
def _fm_native(x: torch.Tensor) -> bool:
    return native.forward_mode() and x.is_cuda and native.available() and settings.gemm == "native"


def _unpack(x):
    """(primal, tangent or None)."""
    if x is None:
        return None, None
    d = fwAD.unpack_dual(x)
    return d.primal, d.tangent


def _pack(p: torch.Tensor, t: Optional[torch.Tensor]) -> torch.Tensor:
    return p if t is None else fwAD.make_dual(p, t)


def _stacked_rows(p2d: torch.Tensor, t2d: torch.Tensor) -> Optional[torch.Tensor]:
    """[2M, K] view over primal and tangent when the tangent's rows follow the primal's in one allocation (the tangent kernels
    and the stacked GEMM below lay their results out that way), else None."""
    if not (p2d.is_contiguous() and t2d.is_contiguous() and p2d.dtype == t2d.dtype):
        return None
    if t2d.data_ptr() != p2d.data_ptr() + p2d.numel() * p2d.element_size():
        return None
    if p2d.untyped_storage().data_ptr() != t2d.untyped_storage().data_ptr():
        return None
    M, K = p2d.shape
    return torch.as_strided(p2d, (2 * M, K), (K, 1))


def _ln_modulate_fm(x, shift, scale, eps):
    px, tx = _unpack(x)
    ps, ts = _unpack(shift)
    pc, tc = _unpack(scale)
    B, T, L, D = px.shape
    f32 = lambda v: None if v is None else v.float().expand(B, T, D).contiguous().view(B * T, D)
    if tx is None:
        tx = torch.zeros_like(px)
    if (ts is None) != (tc is None):
        ts = torch.zeros_like(ps) if ts is None else ts
        tc = torch.zeros_like(pc) if tc is None else tc
    y, ty = native.load().ln_modulate_jvp(px.contiguous().view(-1, D), tx.contiguous().view(-1, D), f32(ps), f32(pc), f32(ts), f32(tc),
                                          L, eps)
    native.count_launch()
    return _pack(y.view(B, T, L, D), ty.view(B, T, L, D))


def _gate_residual_fm(x, gate, y):
    ops = native.load()
    px, tx = _unpack(x)
    pg, tg = _unpack(gate)
    py, ty = _unpack(y)
    B, T, L, D = px.shape
    g2 = lambda v: v.float().expand(B, T, D).contiguous().view(B * T, D)
    r2 = lambda v: v.contiguous().view(-1, D)
    out = ops.gate_residual_fwd(r2(px), g2(pg), r2(py), L)
    native.count_launch()
    t = tx
    if ty is not None:       # t = tx + gate * ty
        t = ops.gate_residual_fwd(r2(tx if tx is not None else torch.zeros_like(px)), g2(pg), r2(ty), L)
        native.count_launch()
    if tg is not None:       # t += tgate * y
        t = ops.gate_residual_fwd(r2(t if t is not None else torch.zeros_like(px)), g2(tg), r2(py), L)
        native.count_launch()
    return _pack(out.view(B, T, L, D), None if t is None else t.view(B, T, L, D))


def _rmsnorm_rope_fm(x, weight, rope, eps):
    px, tx = _unpack(x)
    cos, sin = rope.cos_sin() if rope is not None else (None, None)
    if tx is None:
        y, _ = native.load().rmsnorm_rope_fwd(px.contiguous(), weight, cos, sin, eps)
        native.count_launch()
        return y
    y, ty = native.load().rmsnorm_rope_jvp(px.contiguous(), tx.contiguous(), weight, cos, sin, eps)
    native.count_launch()
    return _pack(y, ty)


def _linear_fm(x, w, bias, act):
    """Primal and tangent rows through the tcgen05 GEMM: one call on the stacked [2M, K] rows when they are adjacent in memory
    (the weight is read once), two calls otherwise. The bias belongs to the primal only; GELU: y = gelu(pre), ty = gelu'(pre) tpre."""
    ops = native.load()
    px, tx = _unpack(x)
    lead, N = px.shape[:-1], w.shape[0]
    p2 = px.reshape(-1, px.shape[-1])
    p2 = p2 if p2.is_contiguous() else p2.contiguous()
    M = p2.shape[0]
    if tx is None:
        y = ops.gemm_bf16(p2, w, bias, _ACT_CODE[act], False, False)
        native.count_launch()
        return y.view(*lead, N)
    t2 = tx.reshape(-1, tx.shape[-1])
    t2 = t2 if t2.is_contiguous() else t2.contiguous()
    both = _stacked_rows(p2, t2)
    if both is not None:
        out = ops.gemm_bf16(both, w, None, 0, False, False)
        native.count_launch()
        pre, tpre = out[:M], out[M:]
    else:
        pre = ops.gemm_bf16(p2, w, None, 0, False, False)
        tpre = ops.gemm_bf16(t2, w, None, 0, False, False)
        native.count_launch(2)
    if bias is not None:
        pre += bias
    if act == "gelu":
        y, ty = ops.gelu_fwd(pre), ops.gelu_bwd(tpre, pre)
        native.count_launch(2)
    else:
        y, ty = pre, tpre
    return _pack(y.view(*lead, N), ty.view(*lead, N))


# --------------------------------------------------------------------------------------
# AdaLN: LayerNorm + modulate
# --------------------------------------------------------------------------------------
class _LnModulate(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale, eps):
        ops = native.load()
        B, T, L, D = x.shape
        xc = x.contiguous()
        shift_c = shift.float().contiguous()
        scale_c = scale.float().contiguous()
        y, mean, rstd = ops.ln_modulate_fwd(xc.view(B * T * L, D), shift_c.view(B * T, D), scale_c.view(B * T, D), L, eps)
        native.count_launch()
        ctx.save_for_backward(xc, scale_c, mean, rstd)
        ctx.dims = (B, T, L, D)
        ctx.in_dtypes = (shift.dtype, scale.dtype)
        return y.view(B, T, L, D)

    @staticmethod
    def backward(ctx, dy):
        ops = native.load()
        x, scale, mean, rstd = ctx.saved_tensors
        B, T, L, D = ctx.dims
        dx, dshift, dscale = ops.ln_modulate_bwd(
            dy.contiguous().view(B * T * L, D), x.view(B * T * L, D), mean, rstd, scale.view(B * T, D), L
        )
        native.count_launch(2)
        return (dx.view(B, T, L, D), dshift.view(B, T, D).to(ctx.in_dtypes[0]),
                dscale.view(B, T, D).to(ctx.in_dtypes[1]), None)


def ln_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """LayerNorm(x) * (1 + scale) + shift; x [B,T,L,D], shift/scale [B,T,D]."""
    if _fm_native(x) and x.dtype == torch.bfloat16:
        return _ln_modulate_fm(x, shift, scale, eps)
    if native.use_native(x):
        return _LnModulate.apply(x, shift, scale, eps)
    return ref.ln_modulate(x, shift, scale, eps)


# --------------------------------------------------------------------------------------
# gated residual
# --------------------------------------------------------------------------------------
class _GateResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, y):
        ops = native.load()
        B, T, L, D = x.shape
        gate_c = gate.float().contiguous()
        yc = y.contiguous()
        out = ops.gate_residual_fwd(x.contiguous().view(-1, D), gate_c.view(B * T, D), yc.view(-1, D), L)
        native.count_launch()
        ctx.save_for_backward(gate_c, yc)
        ctx.dims = (B, T, L, D)
        ctx.gate_dtype = gate.dtype
        return out.view(B, T, L, D)

    @staticmethod
    def backward(ctx, dout):
        ops = native.load()
        gate, y = ctx.saved_tensors
        B, T, L, D = ctx.dims
        dout = dout.contiguous()
        dy, dgate = ops.gate_residual_bwd(dout.view(-1, D), gate.view(B * T, D), y.view(-1, D), L)
        native.count_launch(2)
        return dout, dgate.view(B, T, D).to(ctx.gate_dtype), dy.view(B, T, L, D)


def gate_residual(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
    """x + gate * y; x,y [B,T,L,D], gate [B,T,D]."""
    if _fm_native(x) and x.dtype == torch.bfloat16:
        return _gate_residual_fm(x, gate, y.view_as(x))
    if native.use_native(x):
        return _GateResidual.apply(x, gate, y.view_as(x))
    return ref.gate_residual(x, gate, y.view_as(x))


# --------------------------------------------------------------------------------------
# per-head RMSNorm (+ RoPE)
# --------------------------------------------------------------------------------------
class RopeTable:
    """Rotary angles [S, D] (fp32, second half duplicates the first) with lazily cached cos/sin [S, D/2]."""

    def __init__(self, angles: torch.Tensor):
        self.angles = angles
        self._cs = None

    def cos_sin(self) -> Tuple[torch.Tensor, torch.Tensor]:
        if self._cs is None:
            half = self.angles[:, : self.angles.shape[1] // 2].float()
            self._cs = (half.cos().contiguous(), half.sin().contiguous())
        return self._cs


class _RmsNormRope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, rope, eps):
        ops = native.load()
        xc = x.contiguous()
        cos, sin = rope.cos_sin() if rope is not None else (None, None)
        y, rstd = ops.rmsnorm_rope_fwd(xc, weight, cos, sin, eps)
        native.count_launch()
        ctx.save_for_backward(xc, weight, rstd)
        ctx.rope = rope
        return y

    @staticmethod
    def backward(ctx, dy):
        ops = native.load()
        x, weight, rstd = ctx.saved_tensors
        cos, sin = ctx.rope.cos_sin() if ctx.rope is not None else (None, None)
        dx, dw = ops.rmsnorm_rope_bwd(dy.contiguous(), x, weight, rstd, cos, sin)
        native.count_launch(2)
        return dx, dw.to(weight.dtype), None, None


def rmsnorm_rope(x: torch.Tensor, weight: torch.Tensor, rope: Optional[RopeTable], eps: float = 1e-6) -> torch.Tensor:
    """Per-head RMSNorm then rotate-half RoPE (if a table is given); x [B,S,H,D]."""
    if _fm_native(x) and x.dtype == torch.bfloat16 and x.shape[-1] in (64, 128) and _unpack(weight)[1] is None:
        return _rmsnorm_rope_fm(x, weight, rope, eps)
    if native.use_native(x):
        return _RmsNormRope.apply(x, weight, rope, eps)
    return ref.rmsnorm_rope(x, weight, rope.angles if rope is not None else None, eps)


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale):
        ops = native.load()
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = ops.fa_fwd(q, k, v, scale)
        native.count_launch()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale = scale
        return o

    @staticmethod
    def backward(ctx, do):
        ops = native.load()
        q, k, v, o, lse = ctx.saved_tensors
        if hasattr(ops, "fa_bwd") and settings.attention_bwd == "native":
            dq, dk, dv = ops.fa_bwd(do.contiguous(), q, k, v, o, lse, ctx.scale)
            native.count_launch(3)
            return dq, dk, dv, None
        # library twin: recompute through cuDNN SDPA and let it differentiate
        with torch.enable_grad():
            qd, kd, vd = (t.detach().requires_grad_(True) for t in (q, k, v))
            out = _sdpa(qd, kd, vd, ctx.scale)
            dq, dk, dv = torch.autograd.grad(out, (qd, kd, vd), do)
        return dq, dk, dv, None


class _FlashAttentionJVP(torch.autograd.Function):
    """Attention with a forward-mode rule: ``jvp`` runs the tangent pass of the JVP kernel on the saved forward
    statistics; ``backward`` differentiates the primal only (the tangent is used under stop-gradient by consistency
    training), like the reference's Triton function (flash_attention_jvp_triton.py:436-520)."""

    @staticmethod
    def forward(q, k, v, scale):
        ops = native.load()
        o, lse = ops.fa_fwd(q.contiguous(), k.contiguous(), v.contiguous(), scale)
        native.count_launch()
        return o, lse

    @staticmethod
    def setup_context(ctx, inputs, output):
        q, k, v, scale = inputs
        o, lse = output
        ctx.scale = scale
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.save_for_forward(q, k, v, o, lse)
        ctx.mark_non_differentiable(lse)

    @staticmethod
    def jvp(ctx, tq, tk, tv, _tscale):
        ops = native.load()
        q, k, v, o, lse = ctx.saved_tensors
        z = lambda t, like: torch.zeros_like(like) if t is None else t.to(like.dtype).contiguous()
        to = ops.fa_jvp_tangent(q.contiguous(), k.contiguous(), v.contiguous(), z(tq, q), z(tk, k), z(tv, v), o, lse, ctx.scale)
        native.count_launch()
        return to, None      # lse is marked non-differentiable

    @staticmethod
    def backward(ctx, do, _dlse):
        ops = native.load()
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ops.fa_bwd(do.contiguous(), q.contiguous(), k.contiguous(), v.contiguous(), o, lse, ctx.scale)
        native.count_launch(3)
        return dq, dk, dv, None


def _sdpa(q, k, v, scale):
    """torch SDPA pinned to the cuDNN backend (flash / efficient as fall-backs), [B,S,H,D] layout."""
    from torch.nn.attention import SDPBackend, sdpa_kernel

    backends = [SDPBackend.CUDNN_ATTENTION, SDPBackend.FLASH_ATTENTION, SDPBackend.EFFICIENT_ATTENTION]
    if q.dtype == torch.float32:
        backends = [SDPBackend.EFFICIENT_ATTENTION, SDPBackend.MATH]
    with sdpa_kernel(backends):
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), scale=scale)
    return o.transpose(1, 2)


def native_attention_supported(q: torch.Tensor, k: torch.Tensor) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and native.available() and \
        hasattr(native.load(), "fa_fwd")


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """Non-causal softmax attention, layout [B, S, H, D] in and out."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return ref.attention(q, k, v, scale)[0]
    if native.forward_mode():
        if native_attention_supported(q, k):
            return _FlashAttentionJVP.apply(q, k, v, scale)[0]
        return ref.attention(q, k, v, scale)[0]      # explicit softmax: carries forward-mode tangents
    if settings.attention == "native" and native_attention_supported(q, k):
        return _FlashAttention.apply(q, k, v, scale)
    return _sdpa(q, k, v, scale)


def attention_jvp(q, k, v, tq, tk, tv, scale: Optional[float] = None):
    """Primal and tangent output of attention in one pass: returns (o, to)."""
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if q.is_cuda and native.available() and hasattr(native.load(), "fa_jvp") and q.dtype == torch.bfloat16 \
            and q.shape[-1] == 128:
        o, to, _ = native.load().fa_jvp(q.contiguous(), k.contiguous(), v.contiguous(), tq.contiguous(),
                                        tk.contiguous(), tv.contiguous(), scale)
        native.count_launch()
        return o, to
    o, to, _ = ref.attention_jvp(q, k, v, tq, tk, tv, scale)
    return o, to


# --------------------------------------------------------------------------------------
# GEMM with fused epilogue
# --------------------------------------------------------------------------------------
_ACT_CODE = {"none": 0, "gelu": 1}


def _native_gemm_ok(x2d: torch.Tensor, w: torch.Tensor) -> bool:
    if native.forward_mode():
        return False
    if settings.gemm != "native" or not x2d.is_cuda or x2d.dtype != torch.bfloat16 or w.dtype != torch.bfloat16:
        return False
    if not native.available() or not hasattr(native.load(), "gemm_bf16"):
        return False
    M, K = x2d.shape
    N = w.shape[0]
    return K % 64 == 0 and N % 8 == 0 and M >= 1


def gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none",
            trans_a: bool = False, trans_b: bool = False) -> torch.Tensor:
    """C[M,N] = op(A) @ op(B)^T-style contraction on the tcgen05 GEMM.

    With both flags False: A is [M,K] and B is [N,K] (both K-major, the nn.Linear form).
    trans_a: A is stored [K,M]; trans_b: B is stored [K,N].
    """
    ops = native.load()
    out = ops.gemm_bf16(a, b, bias, _ACT_CODE[act], trans_a, trans_b)
    native.count_launch()
    return out


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias, act):
        x2d = x.reshape(-1, x.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        if act == "gelu":
            y, pre = native.load().gemm_bf16_gelu_pre(x2d, w, bias)
            native.count_launch()
            ctx.save_for_backward(x2d, w, pre)
        else:
            y = gemm_nt(x2d, w, bias, "none")
            ctx.save_for_backward(x2d, w)
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        dy2d = dy.reshape(-1, dy.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        if ctx.act == "gelu":
            x2d, w, pre = ctx.saved_tensors
            ops = native.load()
            dy2d = ops.gelu_bwd(dy2d, pre)
            native.count_launch()
        else:
            x2d, w = ctx.saved_tensors
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # dX[M,K] = dY[M,N] @ W[N,K]: B operand stored [contract, out] -> trans_b
            dx = gemm_nt(dy2d, w, None, "none", False, True).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            # dW[N,K] = dY^T[N,M] @ X[M,K]: both operands stored [contract, out]
            dw = gemm_nt(dy2d, x2d, None, "none", True, True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2d.float().sum(0).to(dy.dtype)
        return dx, dw, db, None


class _LinearGather(torch.autograd.Function):
    """``_Linear`` for a weight whose rows are sharded over the ranks of the sharding group (``parallel/reshard_fsdp.py``): the
    all-gather runs inside the forward GEMM and again inside the input-gradient GEMM (``gemm_bf16_gather``); ``w`` is the
    parameter's view into the engine's workspace, which the kernel fills."""

    @staticmethod
    def forward(ctx, x, w, bias, act, info):
        ops = native.load()
        x2d = x.reshape(-1, x.shape[-1])
        if not x2d.is_contiguous():
            x2d = x2d.contiguous()
        pre = torch.empty(x2d.shape[0], w.shape[0], dtype=x2d.dtype, device=x2d.device) if act == "gelu" else None
        y = ops.gemm_bf16_gather(x2d, w, info.shard_ptrs, info.chunk_rows, info.counters, bias, _ACT_CODE[act], False, pre)
        native.count_launch()
        if act == "gelu":
            ctx.save_for_backward(x2d, w, pre)
        else:
            ctx.save_for_backward(x2d, w)
        ctx.act, ctx.has_bias, ctx.x_shape, ctx.info = act, bias is not None, x.shape, info
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        ops = native.load()
        dy2d = dy.reshape(-1, dy.shape[-1])
        if not dy2d.is_contiguous():
            dy2d = dy2d.contiguous()
        if ctx.act == "gelu":
            x2d, w, pre = ctx.saved_tensors
            dy2d = ops.gelu_bwd(dy2d, pre)
            native.count_launch()
        else:
            x2d, w = ctx.saved_tensors
        info = ctx.info
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            # the workspace may hold another unit's weights by now: the input-gradient GEMM gathers the rows again
            dx = ops.gemm_bf16_gather(dy2d, w, info.shard_ptrs, info.chunk_rows, info.counters, None, 0, True, None).view(ctx.x_shape)
            native.count_launch()
        if ctx.needs_input_grad[1]:
            dw = gemm_nt(dy2d, x2d, None, "none", True, True)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = dy2d.float().sum(0).to(dy.dtype)
        return dx, dw, db, None, None


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, act: str = "none") -> torch.Tensor:
    """act(x @ w.T + bias); act in {none, gelu(erf)}."""
    x2d_shape_ok = x.shape[-1] == w.shape[1]
    assert x2d_shape_ok, (x.shape, w.shape)
    info = getattr(w, "_cb200_gather", None)
    if info is not None:
        if not (x.is_cuda and x.dtype == torch.bfloat16 and not native.forward_mode()):
            raise RuntimeError("a resharded weight can only be used by the bf16 CUDA GEMM (its values live on other ranks)")
        return _LinearGather.apply(x, w, bias, act, info)
    if _fm_native(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[-1] % 64 == 0 and w.shape[0] % 8 == 0 \
            and x.numel() // x.shape[-1] % 8 == 0 and _unpack(w)[1] is None and (bias is None or _unpack(bias)[1] is None):
        return _linear_fm(x, w, bias, act)
    if x.is_cuda and _native_gemm_ok(x.reshape(-1, x.shape[-1]), w) and x.shape[-1] % 64 == 0 \
            and x.numel() // x.shape[-1] % 8 == 0:
        return _Linear.apply(x, w, bias, act)
    y = F.linear(x, w, bias)
    if act == "gelu":
        y = F.gelu(y)
    return y


class _LinearGateResidual(torch.autograd.Function):
    """``resid + gate * (h @ w^T)`` as ONE GEMM whose epilogue also stores the product (the gate gradient needs it): replaces the
    GEMM + gated-residual kernel pair of the training path. Backward: gate / product gradients by the gated-residual backward
    kernel, then the input- and weight-gradient GEMMs."""

    @staticmethod
    def forward(ctx, h, w, resid, gate):
        B, T, L, D = resid.shape
        h2d = h.reshape(-1, h.shape[-1])
        h2d = h2d if h2d.is_contiguous() else h2d.contiguous()
        gate_c = gate.float().contiguous().view(B * T, D)
        out, y = native.load().gemm_bf16_gate_residual_pre(h2d, w, resid.contiguous().view(-1, D), gate_c, L)
        native.count_launch()
        ctx.save_for_backward(h2d, w, gate_c, y)
        ctx.dims, ctx.h_shape, ctx.gate_dtype = (B, T, L, D), h.shape, gate.dtype
        return out.view(B, T, L, D)

    @staticmethod
    def backward(ctx, dout):
        ops = native.load()
        h2d, w, gate_c, y = ctx.saved_tensors
        B, T, L, D = ctx.dims
        dout = dout.contiguous()
        dy, dgate = ops.gate_residual_bwd(dout.view(-1, D), gate_c, y, L)
        native.count_launch(2)
        dh = dw = None
        if ctx.needs_input_grad[0]:
            dh = gemm_nt(dy, w, None, "none", False, True).view(ctx.h_shape)
        if ctx.needs_input_grad[1]:
            dw = gemm_nt(dy, h2d, None, "none", True, True)
        return dh, dw, dout, dgate.view(B, T, D).to(ctx.gate_dtype)


def linear_gate_residual(h: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """resid + gate * (h @ w.T); resid [B,T,L,D], gate [B,T,D], h [B,T*L,K]. Without autograd the gated
    residual is the GEMM epilogue (the product never goes to memory); with autograd the product is kept
    because the gate gradient needs it."""
    B, T, L, D = resid.shape
    needs_grad = torch.is_grad_enabled() and (h.requires_grad or w.requires_grad or resid.requires_grad or gate.requires_grad)
    h2d = h.reshape(-1, h.shape[-1])
    if resid.is_cuda and not needs_grad and _native_gemm_ok(h2d, w) and h2d.shape[0] % 8 == 0 \
            and getattr(w, "_cb200_gather", None) is None:
        out = native.load().gemm_bf16_gate_residual(h2d.contiguous(), w, resid.contiguous().view(-1, D),
                                                    gate.float().contiguous().view(B * T, D), L)
        native.count_launch()
        return out.view(B, T, L, D)
    if (resid.is_cuda and needs_grad and _native_gemm_ok(h2d, w) and h2d.shape[0] % 8 == 0 and w.shape[0] % 256 == 0
            and resid.dtype == torch.bfloat16 and getattr(w, "_cb200_gather", None) is None
            and hasattr(native.load(), "gemm_bf16_gate_residual_pre")):
        return _LinearGateResidual.apply(h, w, resid, gate)
    return gate_residual(resid, gate, linear(h, w).view(B, T, L, D))


# --------------------------------------------------------------------------------------
# small fused elementwise ops used by sampling
# --------------------------------------------------------------------------------------
# --------------------------------------------------------------------------------------
# Few-row fp32 linears, many weights per launch (AdaLN-LoRA modulation MLPs, timestep embedder)
# --------------------------------------------------------------------------------------
_ptr_tables: dict = {}


def _ptr_table(weights: Sequence[torch.Tensor]) -> torch.Tensor:
    """Device tensor with the base address of every weight; cached per address tuple (parameter storages do not move)."""
    key = tuple(w.data_ptr() for w in weights)
    t = _ptr_tables.get(key)
    if t is None:
        if len(_ptr_tables) > 4096:
            _ptr_tables.clear()
        t = torch.tensor(key, dtype=torch.int64, device=weights[0].device)
        _ptr_tables[key] = t
    return t


def _skinny_ok(a: torch.Tensor, weights: Sequence[torch.Tensor], ignore_forward_mode: bool = False) -> bool:
    if (native.forward_mode() and not ignore_forward_mode) or settings.gemm != "native" or not a.is_cuda or not native.available():
        return False
    w0 = weights[0]
    return (w0.dtype in (torch.bfloat16, torch.float32) and all(w.shape == w0.shape and w.dtype == w0.dtype and w.is_contiguous()
                                                                   for w in weights) and hasattr(native.load(), "skinny_bgemm"))


def _skinny_split(Z: int, R: int, N: int, K: int) -> int:
    """Ranges of the reduction per problem: enough CTAs to fill the GPU when the output is a few tiles and K is long."""
    tiles = Z * ((R + 63) // 64) * ((N + 63) // 64)
    return max(1, min((K + 255) // 256, 296 // max(tiles, 1), 65535 // Z))


def _skinny_call(ops, Z, R, N, K, *args):
    """args = the operator's arguments up to ``out_bf16``; splits long reductions and adds the partial sums."""
    out_bf16 = args[-1]
    S = 1 if out_bf16 else _skinny_split(Z, R, N, K)
    out = ops.skinny_bgemm(*args, S)
    native.count_launch()
    return out if S == 1 else out.view(Z, S, R, N).sum(1)


class _SkinnyLinears(torch.autograd.Function):
    """``out[z] = f(a[z]) @ W[z]^T (+ add)`` for Z weights of one shape in one launch; ``a`` is [R, K] (shared by every z) or
    [Z, R, K]; f is identity or SiLU. fp32 accumulate, fp32 result. Backward: two more launches of the same kernel."""

    @staticmethod
    def forward(ctx, a, add, silu, *weights):
        ops = native.load()
        Z = len(weights)
        N, K = weights[0].shape
        shared = a.dim() == 2
        R = a.shape[-2]
        a32 = a.float().contiguous()
        add32 = None if add is None else add.float().contiguous()
        bf16 = weights[0].dtype == torch.bfloat16
        out = _skinny_call(ops, Z, R, N, K, a32, 0 if shared else R * K, K, 1, _ptr_table(weights), None, 0, K, 1, bf16, add32,
                           0 if add32 is None else add32.shape[1], Z, R, N, K, bool(silu), False, False)
        ctx.save_for_backward(a32, *weights)
        ctx.meta = (Z, R, N, K, shared, bool(silu), bf16, None if add is None else (add.shape, add.dtype), a.dtype)
        return out

    @staticmethod
    def backward(ctx, dout):
        ops = native.load()
        a32, *weights = ctx.saved_tensors
        Z, R, N, K, shared, silu, bf16, add_meta, a_dtype = ctx.meta
        dout = dout.float().contiguous()
        da = dadd = None
        if ctx.needs_input_grad[0]:
            # da[z][r, k] = sum_n dout[z][r, n] W[z][n, k]: the weight is read along its rows (k contiguous in the output)
            da = _skinny_call(ops, Z, R, K, N, dout, R * N, N, 1, _ptr_table(weights), None, 0, 1, K, bf16, None, 0, Z, R, K, N, False,
                              False, False)
            if silu:
                sg = torch.sigmoid(a32)
                da = da * (sg * (1 + a32 * (1 - sg)))
            if shared:
                da = da.sum(0)
            da = da.to(a_dtype)
        if add_meta is not None and ctx.needs_input_grad[1]:
            dadd = dout.sum(0)
            if add_meta[0][1] < N:
                dadd = dadd[:, : add_meta[0][1]]
            dadd = dadd.to(add_meta[1])
        dws: Tuple = (None,) * Z
        if any(ctx.needs_input_grad[3:]):
            # dW[z][n, k] = sum_r dout[z][r, n] f(a[z][r, k]): the reduction runs over the few rows
            dw = _skinny_call(ops, Z, N, K, R, dout, R * N, 1, N, None, a32, 0 if shared else R * K, 1, K, False, None, 0, Z, N, K, R, False,
                              silu, bf16)
            dws = tuple(dw[z] for z in range(Z))
        return (da, dadd, None) + dws


def skinny_linears(a: torch.Tensor, weights: Sequence[torch.Tensor], silu: bool = False,
                   add: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``stack_z( f(a[z]) @ weights[z]^T ) + add`` in fp32 -> [Z, R, N]. ``a``: [R, K] shared by all weights or [Z, R, K];
    ``add``: [R, <= N] added to the leading columns of every z (the shared AdaLN-LoRA term)."""
    if _skinny_ok(a, weights):
        return _SkinnyLinears.apply(a, add, silu, *weights)
    if _fm_native(a) and not torch.is_grad_enabled() and _skinny_ok(a, weights, ignore_forward_mode=True) \
            and all(_unpack(w)[1] is None for w in weights):
        # value and tangent as stacked rows of one launch; the SiLU runs outside (its derivative scales the tangent)
        h = F.silu(a.float()) if silu else a.float()
        ph, th = _unpack(h)
        padd, tadd = _unpack(add)
        if th is None and tadd is None:
            return _SkinnyLinears.apply(ph, padd, False, *weights)
        R = ph.shape[-2]
        th = torch.zeros_like(ph) if th is None else th
        add2 = None
        if padd is not None:
            add2 = torch.cat([padd.float(), torch.zeros_like(padd, dtype=torch.float32) if tadd is None else tadd.float()], dim=0)
        out = _SkinnyLinears.apply(torch.cat([ph, th], dim=-2), add2, False, *weights)
        return _pack(out[:, :R], out[:, R:])
    h = a.float()
    if silu:
        h = torch.nn.functional.silu(h)
    outs = []
    for z, w in enumerate(weights):
        o = torch.nn.functional.linear(h if h.dim() == 2 else h[z], w.float())
        if add is not None:
            o = torch.cat([o[:, : add.shape[1]] + add.float(), o[:, add.shape[1]:]], dim=1) if add.shape[1] < o.shape[1] else o + add.float()
        outs.append(o)
    return torch.stack(outs)


def cfg_combine(cond: torch.Tensor, uncond: torch.Tensor, guidance: float) -> torch.Tensor:
    if cond.is_cuda and native.available() and hasattr(native.load(), "cfg_combine"):
        native.count_launch()
        return native.load().cfg_combine(cond.contiguous(), uncond.contiguous(), float(guidance))
    return ref.cfg_combine(cond, uncond, guidance)


def _sampler_native(*ts) -> bool:
    # contiguous already (a .contiguous() copy would cost the pass the kernel saves) and aligned for 16-byte accesses
    return (all(t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.data_ptr() % 16 == 0 for t in ts)
            and native.available() and not any(t.requires_grad for t in ts if torch.is_grad_enabled()))


def lincomb(xs, coeffs) -> torch.Tensor:
    """``sum_k coeffs[k] * xs[k]``: one pass over memory for a state update of the multistep sampler (fp32 on a GPU; anything
    else goes through torch)."""
    xs = list(xs)
    coeffs = [float(c) for c in coeffs]
    if 1 <= len(xs) <= 6 and _sampler_native(*xs) and all(x.shape == xs[0].shape for x in xs) and xs[0].numel() > 0:
        native.count_launch()
        return native.load().lincomb([x.contiguous() for x in xs], coeffs)
    return ref.lincomb(xs, coeffs)


def frame_blend(x, gt, noise, mask, flag=None, out_dtype=None) -> torch.Tensor:
    """Put conditioning frames back: ``keep * mask + x * (1 - mask)`` with ``keep = gt * flag`` or ``noise - gt`` (see
    ``ref.frame_blend``); on a GPU one kernel that can also write the network's bf16 input directly."""
    ts = [t for t in (x, gt, noise) if t is not None]
    B, C = x.shape[0], x.shape[1]
    S = x.numel() // max(B * C, 1)
    if (x.dim() >= 3 and _sampler_native(*ts) and all(t.shape == x.shape for t in ts) and mask.is_cuda and mask.numel() == B * S
            and mask.is_contiguous() and mask.data_ptr() % 16 == 0
            and S % 4 == 0 and out_dtype in (None, torch.float32, torch.bfloat16) and x.numel() > 0):
        native.count_launch()
        f = None if flag is None else flag.reshape(-1).float().contiguous()
        return native.load().frame_blend(x.contiguous(), gt.contiguous(), None if noise is None else noise.contiguous(),
                                         mask.float().contiguous(), f, out_dtype == torch.bfloat16)
    return ref.frame_blend(x, gt, noise, mask, flag, out_dtype)

