"""Flow-matching video DiT (AdaLN-LoRA blocks, 3-D RoPE, patch (1,2,2)).

Behavioural parity target: ``MiniTrainDIT`` and its ``MinimalV1LVGDiT`` wrapper in the reference
(cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:1245-1809,
cosmos_predict2/_src/predict2/networks/minimal_v1_lvg_dit.py:24-62). Parameter and buffer names
match the reference state dict (``x_embedder.proj.1.weight``, ``blocks.N.self_attn.q_proj.weight``,
``blocks.N.adaln_modulation_mlp.2.weight``, ``final_layer.linear.weight`` ...), so consolidated
``net.*`` / ``net_ema.*`` checkpoints load without a key map.

The layout differs from the reference on purpose: every block is five fused kernels
(LN+modulate, per-head RMSNorm+RoPE, attention, gated residual, GEMMs with epilogues) from
``cosmos_predict25_b200.ops``; context-dependent tensors that do not change across sampling steps
(projected text context, cross-attention K/V) can be cached by the caller.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Sequence, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..parallel import ulysses


@dataclass
class DiTConfig:
    """Hyper-parameters; defaults are the 2B network of the reference
    (cosmos_predict2/_src/predict2/configs/video2world/defaults/net.py:58-94)."""

    max_img_h: int = 240
    max_img_w: int = 240
    max_frames: int = 128
    in_channels: int = 16
    out_channels: int = 16
    patch_spatial: int = 2
    patch_temporal: int = 1
    concat_padding_mask: bool = True
    model_channels: int = 2048
    num_blocks: int = 28
    num_heads: int = 16
    mlp_ratio: float = 4.0
    crossattn_emb_channels: int = 1024
    use_crossattn_projection: bool = True
    crossattn_proj_in_channels: int = 100352
    pos_emb_cls: str = "rope3d"
    rope_h_extrapolation_ratio: float = 3.0
    rope_w_extrapolation_ratio: float = 3.0
    rope_t_extrapolation_ratio: float = 1.0
    rope_enable_fps_modulation: bool = False
    extra_per_block_abs_pos_emb: bool = False
    use_adaln_lora: bool = True
    adaln_lora_dim: int = 256
    use_wan_fp32_strategy: bool = True
    # LVG wrapper: one extra input channel carrying the condition mask, timestep scaling
    add_condition_mask_channel: bool = True
    timestep_scale: float = 0.001
    extra_image_context_dim: Optional[int] = None
    checkpoint_mode: str = "none"  # none | block_wise | save_attention
    # sparse self-attention (minimal_v4_dit.py:1279-1290, 1435-1436 of the reference): -1 = every block dense; otherwise see
    # ``replace_selfattn_op_with_sparse_attn_op``. ``natten_parameters``: one dict, or a list with one entry (or None) per block.
    n_dense_blocks: int = -1
    natten_parameters: Any = None

    @property
    def head_dim(self) -> int:
        return self.model_channels // self.num_heads


def _trunc_normal_(w: torch.Tensor, std: float) -> None:
    nn.init.trunc_normal_(w, std=std, a=-3 * std, b=3 * std)


class FusedLinear(nn.Linear):
    """nn.Linear whose forward goes through the tcgen05 GEMM front-end (optional fused GELU)."""

    def __init__(self, in_features, out_features, bias=False, act: str = "none"):
        super().__init__(in_features, out_features, bias=bias)
        self.act = act

    def forward(self, x):
        return ops.linear(x, self.weight, self.bias, self.act)


def _proj_gate_residual(proj: nn.Module, a: torch.Tensor, x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    """``x + gate * proj(a)``. A plain projection runs as one GEMM with the gated residual in its epilogue; a
    projection wrapped by a LoRA adapter adds the low-rank term to the GEMM input of the residual instead."""
    if isinstance(proj, FusedLinear) and proj.bias is None:
        return ops.linear_gate_residual(a, proj.weight, x, gate)
    B, T, L, D = x.shape
    return ops.gate_residual(x, gate, proj(a).view(B, T, L, D))


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def reset_parameters(self):
        nn.init.ones_(self.weight)

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class Patchify(nn.Module):
    """``b c (t r) (h m) (w n) -> b t h w (c r m n)``."""

    def __init__(self, spatial: int, temporal: int):
        super().__init__()
        self.m, self.r = spatial, temporal

    def forward(self, x):
        B, C, T, H, W = x.shape
        r, m = self.r, self.m
        x = x.view(B, C, T // r, r, H // m, m, W // m, m)
        x = x.permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, T // r, H // m, W // m, C * r * m * m)


class PatchEmbed(nn.Module):
    def __init__(self, spatial: int, temporal: int, in_channels: int, out_channels: int):
        super().__init__()
        self.dim = in_channels * spatial * spatial * temporal
        self.proj = nn.Sequential(Patchify(spatial, temporal), nn.Linear(self.dim, out_channels, bias=False))

    def init_weights(self):
        _trunc_normal_(self.proj[1].weight, 1.0 / math.sqrt(self.dim))

    def forward(self, x):
        return self.proj(x)


class Timesteps(nn.Module):
    """Sinusoidal embedding, cosine half first; always computed in fp32."""

    def __init__(self, num_channels: int):
        super().__init__()
        self.num_channels = num_channels

    def forward(self, t_B_T: torch.Tensor) -> torch.Tensor:
        half = self.num_channels // 2
        freq = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=t_B_T.device) / half)
        ang = t_B_T.float().unsqueeze(-1) * freq
        return torch.cat([ang.cos(), ang.sin()], dim=-1)


class FourierFeatures(nn.Module):
    """[B] -> [B, D] random Fourier features cos(2 pi (bandwidth f x + p)) with f ~ N(0, 1), p ~ U(0, 1) drawn once from a fixed seed
    (so every rank and every restart holds the same table); ``normalize`` scales by sqrt(2) for unit variance. An alternative
    noise-level embedding of the EDM-era networks (minimal_v4_dit.py:786-838 of the reference)."""

    def __init__(self, num_channels: int, bandwidth: float = 1.0, normalize: bool = False):
        super().__init__()
        g = torch.Generator().manual_seed(0)
        self.register_buffer("freqs", 2 * math.pi * bandwidth * torch.randn(num_channels, generator=g), persistent=True)
        self.register_buffer("phases", 2 * math.pi * torch.rand(num_channels, generator=g), persistent=True)
        self.gain = math.sqrt(2.0) if normalize else 1.0

    def forward(self, x: torch.Tensor, gain: float = 1.0) -> torch.Tensor:
        y = torch.outer(x.float(), self.freqs.float()) + self.phases.float()
        return (y.cos() * (self.gain * gain)).to(x.dtype)


class TimestepEmbedding(nn.Module):
    """Linear -> SiLU -> Linear(3D). With AdaLN-LoRA the *raw sinusoid* is the embedding that is
    passed on and the MLP output is the shared LoRA term (minimal_v4_dit.py:776-783)."""

    def __init__(self, in_features: int, out_features: int, use_adaln_lora: bool):
        super().__init__()
        self.in_dim, self.out_dim = in_features, out_features
        self.use_adaln_lora = use_adaln_lora
        self.linear_1 = nn.Linear(in_features, out_features, bias=not use_adaln_lora)
        self.activation = nn.SiLU()
        self.linear_2 = nn.Linear(out_features, 3 * out_features if use_adaln_lora else out_features, bias=False)

    def init_weights(self):
        _trunc_normal_(self.linear_1.weight, 1.0 / math.sqrt(self.in_dim))
        _trunc_normal_(self.linear_2.weight, 1.0 / math.sqrt(self.out_dim))

    def forward(self, sample):
        w1, w2 = self.linear_1.weight, self.linear_2.weight
        if self.linear_1.bias is None and sample.is_cuda and type(self.linear_1) is nn.Linear and type(self.linear_2) is nn.Linear:
            # two launches of the few-row fp32 GEMM kernel; the SiLU is applied while the second one loads its input
            lead = sample.shape[:-1]
            h = ops.skinny_linears(sample.reshape(-1, sample.shape[-1]), [w1])
            emb = ops.skinny_linears(h, [w2], silu=True)[0].view(*lead, -1).to(sample.dtype)
        else:
            h = F.linear(sample, w1.to(sample.dtype), None if self.linear_1.bias is None else self.linear_1.bias.to(sample.dtype))
            emb = F.linear(self.activation(h), w2.to(sample.dtype))
        if self.use_adaln_lora:
            return sample, emb
        return emb, None


class VideoRopePosition3DEmb(nn.Module):
    """3-D rotary angle table: head_dim split (t, h, w) = (D-2*(D//6*2), D//6*2, D//6*2), NTK scaling
    per axis, output [T*H*W, D] fp32 = cat([t,h,w] * 2) (minimal_v4_dit.py:534-662)."""

    def __init__(self, head_dim: int, len_h: int, len_w: int, len_t: int, base_fps: int = 24,
                 h_extrapolation_ratio: float = 1.0, w_extrapolation_ratio: float = 1.0,
                 t_extrapolation_ratio: float = 1.0, enable_fps_modulation: bool = True):
        super().__init__()
        self.max_h, self.max_w, self.max_t = len_h, len_w, len_t
        self.base_fps = base_fps
        self.enable_fps_modulation = enable_fps_modulation
        dim_h = head_dim // 6 * 2
        dim_t = head_dim - 2 * dim_h
        self._dim_h, self._dim_t = dim_h, dim_t
        self.register_buffer("seq", torch.arange(max(len_h, len_w, len_t), dtype=torch.float))
        self.register_buffer("dim_spatial_range", torch.arange(0, dim_h, 2)[: dim_h // 2].float() / dim_h)
        self.register_buffer("dim_temporal_range", torch.arange(0, dim_t, 2)[: dim_t // 2].float() / dim_t)
        self.h_ntk_factor = h_extrapolation_ratio ** (dim_h / (dim_h - 2))
        self.w_ntk_factor = w_extrapolation_ratio ** (dim_h / (dim_h - 2))
        self.t_ntk_factor = t_extrapolation_ratio ** (dim_t / (dim_t - 2))

    def reset_parameters(self):
        dev = self.dim_spatial_range.device
        self.seq = torch.arange(max(self.max_h, self.max_w, self.max_t)).float().to(dev)
        self.dim_spatial_range = torch.arange(0, self._dim_h, 2)[: self._dim_h // 2].float().to(dev) / self._dim_h
        self.dim_temporal_range = torch.arange(0, self._dim_t, 2)[: self._dim_t // 2].float().to(dev) / self._dim_t

    def generate(self, T: int, H: int, W: int, fps: Optional[torch.Tensor] = None,
                 t_offset: int = 0, t_total: Optional[int] = None) -> torch.Tensor:
        """Angles for frames [t_offset, t_offset+T) of a clip with t_total frames; [T*H*W, D]."""
        assert H <= self.max_h and W <= self.max_w, (H, W, self.max_h, self.max_w)
        h_freq = 1.0 / ((10000.0 * self.h_ntk_factor) ** self.dim_spatial_range.float())
        w_freq = 1.0 / ((10000.0 * self.w_ntk_factor) ** self.dim_spatial_range.float())
        t_freq = 1.0 / ((10000.0 * self.t_ntk_factor) ** self.dim_temporal_range.float())
        seq = self.seq.float()
        t_pos = seq[t_offset:t_offset + T]
        if self.enable_fps_modulation and fps is not None:
            t_pos = t_pos / fps[:1].float() * self.base_fps
        e_t = torch.outer(t_pos, t_freq)[:, None, None, :].expand(T, H, W, -1)
        e_h = torch.outer(seq[:H], h_freq)[None, :, None, :].expand(T, H, W, -1)
        e_w = torch.outer(seq[:W], w_freq)[None, None, :, :].expand(T, H, W, -1)
        emb = torch.cat([e_t, e_h, e_w] * 2, dim=-1)
        return emb.reshape(T * H * W, -1).float().contiguous()


class LearnablePosEmbAxis(nn.Module):
    """Additive per-axis learnable position embedding, L2-normalised (7B network only;
    minimal_v4_dit.py:665-719)."""

    def __init__(self, model_channels: int, len_h: int, len_w: int, len_t: int):
        super().__init__()
        self.pos_emb_h = nn.Parameter(torch.zeros(len_h, model_channels))
        self.pos_emb_w = nn.Parameter(torch.zeros(len_w, model_channels))
        self.pos_emb_t = nn.Parameter(torch.zeros(len_t, model_channels))

    def reset_parameters(self):
        std = 1.0 / math.sqrt(self.pos_emb_h.shape[1])
        for p in (self.pos_emb_h, self.pos_emb_w, self.pos_emb_t):
            _trunc_normal_(p.data, std)

    def generate(self, T, H, W, t_offset: int = 0):
        emb = (self.pos_emb_t[t_offset:t_offset + T, None, None, :] + self.pos_emb_h[None, :H, None, :]
               + self.pos_emb_w[None, None, :W, :])
        norm = torch.linalg.vector_norm(emb.float(), dim=-1, keepdim=True)
        norm = torch.add(1e-6, norm, alpha=math.sqrt(norm.numel() / emb.numel()))
        return (emb / norm.to(emb.dtype)).unsqueeze(0)


class Attention(nn.Module):
    """Self- or cross-attention with per-head RMSNorm on q,k and RoPE on self-attention q,k
    (minimal_v4_dit.py:286-449)."""

    def __init__(self, query_dim: int, context_dim: Optional[int], n_heads: int, head_dim: int):
        super().__init__()
        self.is_selfattn = context_dim is None
        context_dim = query_dim if context_dim is None else context_dim
        inner = n_heads * head_dim
        self.n_heads, self.head_dim = n_heads, head_dim
        self.query_dim, self.context_dim = query_dim, context_dim
        self.q_proj = FusedLinear(query_dim, inner)
        self.q_norm = RMSNorm(head_dim)
        self.k_proj = FusedLinear(context_dim, inner)
        self.k_norm = RMSNorm(head_dim)
        self.v_proj = FusedLinear(context_dim, inner)
        self.output_proj = FusedLinear(inner, query_dim)
        self.cp_group = None
        self.cp_comm_type = "a2a"  # "a2a": Ulysses exchange; "p2p": ring attention
        self.sparse_op = None      # NeighborhoodAttention in blocks switched to sparse self-attention
        self.video_size = None     # (T, H, W) of the whole token grid, set by the network before the blocks run

    def init_weights(self):
        _trunc_normal_(self.q_proj.weight, 1.0 / math.sqrt(self.query_dim))
        _trunc_normal_(self.k_proj.weight, 1.0 / math.sqrt(self.context_dim))
        _trunc_normal_(self.v_proj.weight, 1.0 / math.sqrt(self.context_dim))
        _trunc_normal_(self.output_proj.weight, 1.0 / math.sqrt(self.n_heads * self.head_dim))
        self.q_norm.reset_parameters()
        self.k_norm.reset_parameters()

    def _sparse_forward(self, x, rope, return_pre_proj):
        """Self-attention through the neighbourhood operator. Under context parallelism q/k/v are exchanged to
        (whole sequence, local heads) first, like the reference's a2a wrapper around NATTEN
        (minimal_v4_dit.py:1176-1192), and the output is exchanged back."""
        B, S, _ = x.shape
        q = ops.rmsnorm_rope(self.q_proj(x).view(B, S, self.n_heads, self.head_dim), self.q_norm.weight, rope, self.q_norm.eps)
        k = ops.rmsnorm_rope(self.k_proj(x).view(B, S, self.n_heads, self.head_dim), self.k_norm.weight, rope, self.k_norm.eps)
        v = self.v_proj(x).view(B, S, self.n_heads, self.head_dim)
        if self.cp_group is not None and ulysses.group_size_rank(self.cp_group)[0] > 1:
            q, k, v = (ulysses._SeqToHead.apply(t, self.cp_group) for t in (q, k, v))
            o = ulysses._HeadToSeq.apply(self.sparse_op(q, k, v, self.video_size), self.cp_group)
        else:
            o = self.sparse_op(q, k, v, self.video_size)
        o = o.reshape(B, S, self.n_heads * self.head_dim)
        return o if return_pre_proj else self.output_proj(o)

    def _plain_projections(self) -> bool:
        return all(type(p) is FusedLinear and p.bias is None and p.weight.dtype == torch.bfloat16
                   for p in (self.q_proj, self.k_proj, self.v_proj))

    def project_kv(self, context: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """K (normalised) and V of a context; constant across sampling steps for cross-attention."""
        B, S, _ = context.shape
        k = self.k_proj(context).view(B, S, self.n_heads, self.head_dim)
        v = self.v_proj(context).view(B, S, self.n_heads, self.head_dim)
        k = ops.rmsnorm_rope(k, self.k_norm.weight, None, self.k_norm.eps)
        return k, v

    def forward(self, x: torch.Tensor, context: Optional[torch.Tensor] = None, rope=None,
                kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, return_pre_proj: bool = False):
        B, S, _ = x.shape
        if self.is_selfattn and self.sparse_op is not None and self.video_size is not None:
            return self._sparse_forward(x, rope, return_pre_proj)
        if (self.is_selfattn and self.cp_group is not None and self.cp_comm_type == "a2a" and self._plain_projections()
                and ulysses.projected_attention_available(x, self.cp_group, self.head_dim)):
            # inference under context parallelism: the sequence->head exchange is the epilogue of the q/k/v GEMMs
            o = ulysses.ulysses_projected_attention(x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight,
                                                    self.q_norm.weight, self.k_norm.weight, rope, self.cp_group, self.q_norm.eps)
            o = o.reshape(B, S, self.n_heads * self.head_dim)
            return o if return_pre_proj else self.output_proj(o)
        if (self.is_selfattn and self.cp_group is not None and self.cp_comm_type == "a2a" and self._plain_projections()
                and all(getattr(p.weight, "_cb200_gather", None) is None for p in (self.q_proj, self.k_proj, self.v_proj))
                and ulysses.projected_attention_train_available(x, self.cp_group, self.head_dim)):
            # training under context parallelism: same GEMM-epilogue exchange, with the raw projections kept for the backward
            o = ulysses.ulysses_projected_attention_train(x, self.q_proj.weight, self.k_proj.weight, self.v_proj.weight,
                                                          self.q_norm.weight, self.k_norm.weight, rope, self.cp_group, self.q_norm.eps)
            o = o.reshape(B, S, self.n_heads * self.head_dim)
            return o if return_pre_proj else self.output_proj(o)
        q = self.q_proj(x).view(B, S, self.n_heads, self.head_dim)
        if self.is_selfattn:
            k = self.k_proj(x).view(B, S, self.n_heads, self.head_dim)
            v = self.v_proj(x).view(B, S, self.n_heads, self.head_dim)
            if self.cp_group is not None and self.cp_comm_type == "p2p":
                from ..parallel.ring_attention import ring_attention
                q = ops.rmsnorm_rope(q, self.q_norm.weight, rope, self.q_norm.eps)
                k = ops.rmsnorm_rope(k, self.k_norm.weight, rope, self.k_norm.eps)
                o = ring_attention(q, k, v, self.cp_group)
            elif self.cp_group is not None:
                o = ulysses.ulysses_attention_fused(q, k, v, self.q_norm.weight, self.k_norm.weight, rope, self.cp_group,
                                                    self.q_norm.eps)
            else:
                q = ops.rmsnorm_rope(q, self.q_norm.weight, rope, self.q_norm.eps)
                k = ops.rmsnorm_rope(k, self.k_norm.weight, rope, self.k_norm.eps)
                o = ops.attention(q, k, v)
        else:
            q = ops.rmsnorm_rope(q, self.q_norm.weight, None, self.q_norm.eps)
            k, v = kv if kv is not None else self.project_kv(context)
            o = ops.attention(q, k, v)
        o = o.reshape(B, S, self.n_heads * self.head_dim)
        return o if return_pre_proj else self.output_proj(o)


class I2VCrossAttention(Attention):
    """Cross-attention over a text context AND an image context: ``context = (text, image)``; the two attention results are added
    before the output projection; the image keys have their own projection and per-head norm (minimal_v4_dit.py:451-492)."""

    def __init__(self, query_dim: int, context_dim: int, n_heads: int, head_dim: int, img_latent_dim: int):
        super().__init__(query_dim, context_dim, n_heads, head_dim)
        inner = n_heads * head_dim
        self.k_img = FusedLinear(img_latent_dim, inner)
        self.v_img = FusedLinear(img_latent_dim, inner)
        self.k_img_norm = RMSNorm(head_dim)

    def init_weights(self):
        super().init_weights()
        inner = self.n_heads * self.head_dim
        nn.init.trunc_normal_(self.k_img.weight, std=1.0 / math.sqrt(inner))
        nn.init.trunc_normal_(self.v_img.weight, std=1.0 / math.sqrt(inner))
        self.k_img_norm.reset_parameters()

    def forward(self, x, context=None, rope=None, kv=None, return_pre_proj: bool = False):
        text, img = context
        B, S, _ = x.shape
        Si = img.shape[1]
        q = ops.rmsnorm_rope(self.q_proj(x).view(B, S, self.n_heads, self.head_dim), self.q_norm.weight, None, self.q_norm.eps)
        k, v = kv if kv is not None else self.project_kv(text)
        k_img = ops.rmsnorm_rope(self.k_img(img).view(B, Si, self.n_heads, self.head_dim), self.k_img_norm.weight, None, self.k_img_norm.eps)
        v_img = self.v_img(img).view(B, Si, self.n_heads, self.head_dim)
        o = (ops.attention(q, k, v) + ops.attention(q, k_img, v_img)).reshape(B, S, self.n_heads * self.head_dim)
        return o if return_pre_proj else self.output_proj(o)


class GPT2FeedForward(nn.Module):
    def __init__(self, d_model: int, d_ff: int):
        super().__init__()
        self.layer1 = FusedLinear(d_model, d_ff, act="gelu")
        self.layer2 = FusedLinear(d_ff, d_model)
        self.d_model, self.d_ff = d_model, d_ff

    def init_weights(self):
        _trunc_normal_(self.layer1.weight, 1.0 / math.sqrt(self.d_model))
        _trunc_normal_(self.layer2.weight, 1.0 / math.sqrt(self.d_ff))

    def forward(self, x):
        return self.layer2(self.layer1(x))


def _adaln_mlp(x_dim: int, lora_dim: int, n_chunks: int, use_lora: bool) -> nn.Sequential:
    if use_lora:
        return nn.Sequential(nn.SiLU(), nn.Linear(x_dim, lora_dim, bias=False), nn.Linear(lora_dim, n_chunks * x_dim, bias=False))
    return nn.Sequential(nn.SiLU(), nn.Linear(x_dim, n_chunks * x_dim, bias=False))


def _run_adaln(mlp: nn.Sequential, emb: torch.Tensor, lora: Optional[torch.Tensor], fp32: bool) -> torch.Tensor:
    """Modulation MLP; in fp32 when the fp32-island strategy is on (minimal_v4_dit.py:1131)."""
    h = emb.float() if fp32 else emb
    for m in mlp:
        if isinstance(m, nn.Linear):
            h = F.linear(h, m.weight.to(h.dtype))
        else:
            h = m(h)
    if lora is not None:
        h = h + lora.to(h.dtype)
    return h


def _plain_adaln(mlp: nn.Sequential) -> bool:
    return all(type(m) in (nn.Linear, nn.SiLU) for m in mlp)


def run_adaln_many(mlps: Sequence[nn.Sequential], emb: torch.Tensor, lora: Optional[torch.Tensor], fp32: bool) -> torch.Tensor:
    """The modulation MLPs ``mlps`` (same shapes) on one embedding in two launches of the few-row fp32 GEMM kernel:
    SiLU(emb) @ W1[z]^T for every z, then @ W2[z]^T + the shared LoRA term. Returns [Z, *emb.shape[:-1], n * D]
    (minimal_v4_dit.py:1131-1162)."""
    lead = emb.shape[:-1]
    e2 = emb.reshape(-1, emb.shape[-1])
    l2 = None if lora is None else lora.reshape(-1, lora.shape[-1])
    lins = [[m for m in mlp if isinstance(m, nn.Linear)] for mlp in mlps]
    if len(lins[0]) == 2:
        h = ops.skinny_linears(e2, [l[0].weight for l in lins], silu=True)
        out = ops.skinny_linears(h, [l[1].weight for l in lins], add=l2)
    else:
        out = ops.skinny_linears(e2, [l[0].weight for l in lins], silu=True, add=l2)
    out = out.view(len(mlps), *lead, out.shape[-1])
    return out if fp32 else out.to(emb.dtype)


class Block(nn.Module):
    """x += g1*SA(LNmod(x)); x += g2*CA(LNmod(x), ctx); x += g3*MLP(LNmod(x)) (minimal_v4_dit.py:993-1242)."""

    def __init__(self, cfg: DiTConfig):
        super().__init__()
        D = cfg.model_channels
        self.cfg = cfg
        self.self_attn = Attention(D, None, cfg.num_heads, cfg.head_dim)
        if cfg.extra_image_context_dim is None:
            self.cross_attn = Attention(D, cfg.crossattn_emb_channels, cfg.num_heads, cfg.head_dim)
        else:       # the image context arrives already projected to the model width
            self.cross_attn = I2VCrossAttention(D, cfg.crossattn_emb_channels, cfg.num_heads, cfg.head_dim, img_latent_dim=D)
        self.mlp = GPT2FeedForward(D, int(D * cfg.mlp_ratio))
        self.adaln_modulation_self_attn = _adaln_mlp(D, cfg.adaln_lora_dim, 3, cfg.use_adaln_lora)
        self.adaln_modulation_cross_attn = _adaln_mlp(D, cfg.adaln_lora_dim, 3, cfg.use_adaln_lora)
        self.adaln_modulation_mlp = _adaln_mlp(D, cfg.adaln_lora_dim, 3, cfg.use_adaln_lora)

    def adaln_mlps(self) -> Tuple[nn.Sequential, nn.Sequential, nn.Sequential]:
        return self.adaln_modulation_self_attn, self.adaln_modulation_cross_attn, self.adaln_modulation_mlp

    def init_weights(self):
        self.self_attn.init_weights()
        self.cross_attn.init_weights()
        self.mlp.init_weights()
        for mlp in self.adaln_mlps():
            lins = [m for m in mlp if isinstance(m, nn.Linear)]
            for lin in lins[:-1]:
                _trunc_normal_(lin.weight, 1.0 / math.sqrt(lin.in_features))
            nn.init.zeros_(lins[-1].weight)

    def forward(self, x: torch.Tensor, emb: torch.Tensor, context: torch.Tensor, rope: Optional[torch.Tensor],
                lora: Optional[torch.Tensor], extra_pos: Optional[torch.Tensor] = None,
                cross_kv: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, mods: Optional[torch.Tensor] = None) -> torch.Tensor:
        """x: [B,T,L,D] (L = H*W tokens of one latent frame); emb [B,T,D]; lora [B,T,3D]; ``mods`` [3,B,T,3D]: the block's three
        modulation outputs when the caller has computed those of all blocks in one launch."""
        if extra_pos is not None:
            x = x + extra_pos
        fp32 = self.cfg.use_wan_fp32_strategy
        B, T, L, D = x.shape
        if mods is None and emb.is_cuda and all(_plain_adaln(m) for m in self.adaln_mlps()):
            mods = run_adaln_many(self.adaln_mlps(), emb, lora, fp32)
        if mods is not None:
            (sh1, sc1, g1), (sh2, sc2, g2), (sh3, sc3, g3) = (mods[i].chunk(3, dim=-1) for i in range(3))
        else:
            sh1, sc1, g1 = _run_adaln(self.adaln_modulation_self_attn, emb, lora, fp32).chunk(3, dim=-1)
            sh2, sc2, g2 = _run_adaln(self.adaln_modulation_cross_attn, emb, lora, fp32).chunk(3, dim=-1)
            sh3, sc3, g3 = _run_adaln(self.adaln_modulation_mlp, emb, lora, fp32).chunk(3, dim=-1)

        h = ops.ln_modulate(x, sh1, sc1)
        o = self.self_attn(h.view(B, T * L, D), None, rope, return_pre_proj=True)
        x = _proj_gate_residual(self.self_attn.output_proj, o, x, g1)

        h = ops.ln_modulate(x, sh2, sc2)
        o = self.cross_attn(h.view(B, T * L, D), context, None, cross_kv, return_pre_proj=True)
        x = _proj_gate_residual(self.cross_attn.output_proj, o, x, g2)

        h = ops.ln_modulate(x, sh3, sc3)
        a = self.mlp.layer1(h.view(B, T * L, D))
        x = _proj_gate_residual(self.mlp.layer2, a, x, g3)
        return x


class FinalLayer(nn.Module):
    def __init__(self, cfg: DiTConfig):
        super().__init__()
        D = cfg.model_channels
        self.cfg = cfg
        out = cfg.patch_spatial * cfg.patch_spatial * cfg.patch_temporal * cfg.out_channels
        self.linear = nn.Linear(D, out, bias=False)
        self.adaln_modulation = _adaln_mlp(D, cfg.adaln_lora_dim, 2, cfg.use_adaln_lora)

    def init_weights(self):
        _trunc_normal_(self.linear.weight, 1.0 / math.sqrt(self.cfg.model_channels))
        lins = [m for m in self.adaln_modulation if isinstance(m, nn.Linear)]
        for lin in lins[:-1]:
            _trunc_normal_(lin.weight, 1.0 / math.sqrt(lin.in_features))
        nn.init.zeros_(lins[-1].weight)

    def forward(self, x, emb, lora):
        D = self.cfg.model_channels
        lora2 = lora[..., : 2 * D] if lora is not None else None
        if emb.is_cuda and _plain_adaln(self.adaln_modulation):
            shift, scale = run_adaln_many([self.adaln_modulation], emb, lora2, self.cfg.use_wan_fp32_strategy)[0].chunk(2, dim=-1)
        else:
            shift, scale = _run_adaln(self.adaln_modulation, emb, lora2, self.cfg.use_wan_fp32_strategy).chunk(2, dim=-1)
        h = ops.ln_modulate(x, shift, scale)
        return ops.linear(h, self.linear.weight)


@dataclass
class ContextCache:
    """Per-prompt tensors that are identical in every denoising call: the projected text context
    and each block's cross-attention K/V. The reference recomputes them 70 times per video."""

    context: torch.Tensor
    cross_kv: List[Tuple[torch.Tensor, torch.Tensor]] = field(default_factory=list)


def register_training_stats(module: nn.Module) -> None:
    """Scalar buffers that travel with the weights of every released network: samples seen, iterations, training hours
    (model_weights_stats.py:41-51 of the reference)."""
    for name in ("accum_video_sample_counter", "accum_image_sample_counter", "accum_iteration"):
        module.register_buffer(name, torch.tensor(0, dtype=torch.int64), persistent=True)
    module.register_buffer("accum_train_in_hours", torch.tensor(0.0, dtype=torch.float32), persistent=True)


class CosmosDiT(nn.Module):
    """The Predict2.5 network: text2world / image2world / video2world share it; the conditioning
    mask enters as an extra input channel and timesteps arrive in scheduler units (0..1000)."""

    def __init__(self, cfg: DiTConfig):
        super().__init__()
        self.cfg = cfg
        D = cfg.model_channels
        in_ch = cfg.in_channels + (1 if cfg.add_condition_mask_channel else 0) + (1 if cfg.concat_padding_mask else 0)
        self.x_embedder = PatchEmbed(cfg.patch_spatial, cfg.patch_temporal, in_ch, D)
        self.pos_embedder = VideoRopePosition3DEmb(
            head_dim=cfg.head_dim, len_h=cfg.max_img_h // cfg.patch_spatial, len_w=cfg.max_img_w // cfg.patch_spatial,
            len_t=cfg.max_frames // cfg.patch_temporal, h_extrapolation_ratio=cfg.rope_h_extrapolation_ratio,
            w_extrapolation_ratio=cfg.rope_w_extrapolation_ratio, t_extrapolation_ratio=cfg.rope_t_extrapolation_ratio,
            enable_fps_modulation=cfg.rope_enable_fps_modulation)
        if cfg.extra_per_block_abs_pos_emb:
            self.extra_pos_embedder = LearnablePosEmbAxis(D, cfg.max_img_h // cfg.patch_spatial,
                                                          cfg.max_img_w // cfg.patch_spatial,
                                                          cfg.max_frames // cfg.patch_temporal)
        self.t_embedder = nn.Sequential(Timesteps(D), TimestepEmbedding(D, D, cfg.use_adaln_lora))
        self.t_embedding_norm = RMSNorm(D, eps=1e-6)
        if cfg.use_crossattn_projection:
            self.crossattn_proj = nn.Sequential(
                nn.Linear(cfg.crossattn_proj_in_channels, cfg.crossattn_emb_channels, bias=True), nn.GELU())
        if cfg.extra_image_context_dim is not None:
            self.img_context_proj = nn.Sequential(nn.Linear(cfg.extra_image_context_dim, D, bias=True), nn.GELU())
        self.blocks = nn.ModuleList([Block(cfg) for _ in range(cfg.num_blocks)])
        self.final_layer = FinalLayer(cfg)
        # training statistics buffers kept for checkpoint parity (model_weights_stats.py:41-51)
        register_training_stats(self)
        self.cp_group = None
        self._fsdp = None
        if cfg.n_dense_blocks != -1:
            replace_selfattn_op_with_sparse_attn_op(self, cfg.n_dense_blocks, cfg.natten_parameters)

    # ---- initialisation ---------------------------------------------------------------
    def init_weights(self):
        self.x_embedder.init_weights()
        self.pos_embedder.reset_parameters()
        if self.cfg.extra_per_block_abs_pos_emb:
            self.extra_pos_embedder.reset_parameters()
        self.t_embedder[1].init_weights()
        for b in self.blocks:
            b.init_weights()
        self.final_layer.init_weights()
        self.t_embedding_norm.reset_parameters()
        if self.cfg.use_crossattn_projection:
            self.crossattn_proj[0].reset_parameters()
        if self.cfg.extra_image_context_dim is not None:
            self.img_context_proj[0].reset_parameters()

    # ---- context parallel ----------------------------------------------------------------
    def enable_context_parallel(self, group, comm_type: str = "a2a"):
        """Shard the sequence by latent frames over ``group``; only self-attention communicates. ``comm_type``: "a2a"
        (Ulysses all-to-all, the default) or "p2p" (ring attention: key / value shards travel round the group, no
        constraint on the head count)."""
        assert comm_type in ("a2a", "p2p"), comm_type
        self.cp_group = group
        for b in self.blocks:
            b.self_attn.cp_group = group
            b.self_attn.cp_comm_type = comm_type

    def disable_context_parallel(self):
        self.cp_group = None
        for b in self.blocks:
            b.self_attn.cp_group = None

    @property
    def is_context_parallel_enabled(self) -> bool:
        return self.cp_group is not None

    # ---- pieces of forward ---------------------------------------------------------------
    def project_context(self, crossattn_emb: torch.Tensor) -> torch.Tensor:
        if self.cfg.use_crossattn_projection:
            lin = self.crossattn_proj[0]
            return ops.linear(crossattn_emb.to(lin.weight.dtype), lin.weight, lin.bias, "gelu")
        return crossattn_emb

    def build_context_cache(self, crossattn_emb: torch.Tensor) -> ContextCache:
        ctx = self.project_context(crossattn_emb)
        return ContextCache(ctx, [b.cross_attn.project_kv(ctx) for b in self.blocks])

    def _embed(self, x_B_C_T_H_W, condition_mask, padding_mask):
        B, C, T, H, W = x_B_C_T_H_W.shape
        parts = [x_B_C_T_H_W]
        if self.cfg.add_condition_mask_channel:
            if condition_mask is None:
                condition_mask = x_B_C_T_H_W.new_zeros(B, 1, T, H, W)
            parts.append(condition_mask.to(x_B_C_T_H_W.dtype))
        if self.cfg.concat_padding_mask:
            if padding_mask is None:
                pm = x_B_C_T_H_W.new_zeros(B, 1, 1, H, W)
            else:
                pm = padding_mask.to(x_B_C_T_H_W.dtype)
                if pm.shape[-2:] != (H, W):
                    pm = F.interpolate(pm, size=(H, W), mode="nearest")
                pm = pm.view(B, 1, 1, H, W)
            parts.append(pm.expand(B, 1, T, H, W))
        x = torch.cat(parts, dim=1)
        lin = self.x_embedder.proj[1]
        tokens = self.x_embedder.proj[0](x).to(lin.weight.dtype)
        K = tokens.shape[-1]
        if tokens.is_cuda and tokens.dtype == torch.bfloat16 and K % 64 != 0:
            # the patch vector (72 values for 18 channels x 2 x 2) is zero-padded to the GEMM's 64-element k-block so that the
            # embedding runs on the tcgen05 GEMM like every other projection (minimal_v4_dit.py:867-877)
            pad = (-K) % 64
            return ops.linear(F.pad(tokens, (0, pad)), F.pad(lin.weight, (0, pad)))
        return ops.linear(tokens, lin.weight)

    def forward(self, x_B_C_T_H_W: torch.Tensor, timesteps_B_T: torch.Tensor, crossattn_emb: Optional[torch.Tensor],
                condition_video_input_mask_B_C_T_H_W: Optional[torch.Tensor] = None,
                fps: Optional[torch.Tensor] = None, padding_mask: Optional[torch.Tensor] = None,
                context_cache: Optional[ContextCache] = None, img_context_emb: Optional[torch.Tensor] = None,
                **_unused) -> torch.Tensor:
        """Velocity prediction. Under context parallelism every input is the local T-slice. ``img_context_emb`` [B, N, extra_image_
        context_dim]: tokens of a reference image for networks built with ``extra_image_context_dim``."""
        cfg = self.cfg
        x = self._embed(x_B_C_T_H_W, condition_video_input_mask_B_C_T_H_W, padding_mask)  # [B,T,H,W,D]
        B, T, H, W, D = x.shape
        cp_size, cp_rank = ulysses.group_size_rank(self.cp_group)
        rope = ops.RopeTable(self.pos_embedder.generate(T, H, W, fps, t_offset=cp_rank * T)) \
            if "rope" in cfg.pos_emb_cls else None
        extra = None
        if cfg.extra_per_block_abs_pos_emb:
            extra = self.extra_pos_embedder.generate(T, H, W, t_offset=cp_rank * T).to(x.dtype).reshape(1, T, H * W, D)

        if context_cache is not None:
            context, cross_kv = context_cache.context, context_cache.cross_kv
        else:
            context, cross_kv = self.project_context(crossattn_emb), None
        if cfg.extra_image_context_dim is not None:
            assert img_context_emb is not None, "this network was built with extra_image_context_dim: pass img_context_emb"
            lin = self.img_context_proj[0]
            context = (context, ops.linear(img_context_emb.to(lin.weight.dtype), lin.weight, lin.bias, "gelu"))

        if timesteps_B_T.ndim == 1:
            timesteps_B_T = timesteps_B_T.unsqueeze(1)
        t_in = timesteps_B_T.float() * cfg.timestep_scale
        sinus = self.t_embedder[0](t_in)
        if not cfg.use_wan_fp32_strategy:
            sinus = sinus.to(x.dtype)
        emb, lora = self.t_embedder[1](sinus)
        emb = self.t_embedding_norm(emb)
        if emb.shape[1] == 1 and T > 1:
            emb = emb.expand(B, T, -1)
            lora = lora.expand(B, T, -1) if lora is not None else None

        x = x.view(B, T, H * W, D)
        from .checkpointing import run_block
        for block in self.blocks:
            block.self_attn.video_size = (T * cp_size, H, W)

        all_mods = None
        if (not torch.is_grad_enabled() and emb.is_cuda and not getattr(self, "_params_sharded", False)
                and all(_plain_adaln(m) for b in self.blocks for m in b.adaln_mlps())):
            # the modulation vectors depend only on the timestep embedding: all 3 x L MLPs in two launches, once per forward
            all_mods = run_adaln_many([m for b in self.blocks for m in b.adaln_mlps()], emb, lora, cfg.use_wan_fp32_strategy)
        for i, block in enumerate(self.blocks):
            kv = cross_kv[i] if cross_kv else None
            mods = None if all_mods is None else all_mods[3 * i: 3 * i + 3]
            x = run_block(block, cfg.checkpoint_mode if self.training else "none", x, emb, context, rope, lora, extra, kv, mods)
        out = self.final_layer(x, emb, lora).view(B, T, H, W, -1)
        return self.unpatchify(out)

    def use_sparse_attention(self, n_dense_blocks: int = 0, natten_parameters=None) -> "CosmosDiT":
        return replace_selfattn_op_with_sparse_attn_op(self, n_dense_blocks, natten_parameters)

    def unpatchify(self, x_B_T_H_W_M):
        """``B T H W (p1 p2 t C) -> B C (T t) (H p1) (W p2)``."""
        B, T, H, W, _ = x_B_T_H_W_M.shape
        p, t = self.cfg.patch_spatial, self.cfg.patch_temporal
        x = x_B_T_H_W_M.view(B, T, H, W, p, p, t, -1)
        x = x.permute(0, 7, 1, 6, 2, 4, 3, 5)
        return x.reshape(B, -1, T * t, H * p, W * p)

    # ---- sharding ------------------------------------------------------------------------
    def fsdp_units(self) -> List[nn.Module]:
        """The parameter groups that are gathered / reduced together: one per block, then the
        final layer and the timestep embedder, then everything else at the root
        (grouping of minimal_v4_dit.py:1688-1699)."""
        return list(self.blocks) + [self.final_layer, self.t_embedder]


# ---- size presets (cosmos_predict2/_src/predict2/configs/video2world/defaults/net.py:26-110) ----
def dit_2b(**kw) -> DiTConfig:
    return DiTConfig(model_channels=2048, num_heads=16, num_blocks=28, **kw)


def dit_14b(**kw) -> DiTConfig:
    return DiTConfig(model_channels=5120, num_heads=40, num_blocks=36, **kw)


def dit_7b(**kw) -> DiTConfig:
    return DiTConfig(model_channels=4096, num_heads=32, num_blocks=28, extra_per_block_abs_pos_emb=True, **kw)


def dit_mini(**kw) -> DiTConfig:
    base = dict(model_channels=1024, num_heads=8, num_blocks=2)
    base.update(kw)
    return DiTConfig(**base)


def dit_tiny(**kw) -> DiTConfig:
    """The CPU test network: 2 blocks, hidden 256, 4 heads, context width 256 without projection."""
    base = dict(model_channels=256, num_heads=4, num_blocks=2, crossattn_emb_channels=256,
                use_crossattn_projection=False, max_img_h=64, max_img_w=64, max_frames=32, adaln_lora_dim=64)
    base.update(kw)
    return DiTConfig(**base)


NET_PRESETS = {"2B": dit_2b, "14B": dit_14b, "7B": dit_7b, "mini": dit_mini, "tiny": dit_tiny}


def replace_selfattn_op_with_sparse_attn_op(model, n_dense_blocks: int = 0, natten_parameters=None):
    """Switch the self-attention of DiT blocks to neighbourhood attention
    (minimal_v4_dit.py:1739-1812 of the reference). ``natten_parameters`` is one dict for all sparse blocks or a list
    with one entry per block (None keeps a block dense). ``n_dense_blocks``: -1 leaves the model alone; 0 makes every
    block sparse; 1 keeps the middle block dense; n > 1 keeps n blocks dense, spread evenly from first to last."""
    from ..modules.neighborhood_attn import NeighborhoodAttention
    if n_dense_blocks == -1:
        return model
    if natten_parameters is None:
        raise ValueError("natten_parameters is required when n_dense_blocks > -1")
    n = len(model.blocks)
    if isinstance(natten_parameters, (list, tuple)):
        if len(natten_parameters) != n:
            raise ValueError(f"got {len(natten_parameters)} parameter sets for {n} blocks")
        if n_dense_blocks > 0:
            raise ValueError("a per-block list already says which blocks stay dense: n_dense_blocks must be 0")
        per_block = list(natten_parameters)
    else:
        if n_dense_blocks >= n:
            raise ValueError(f"n_dense_blocks ({n_dense_blocks}) must be less than the number of blocks ({n})")
        dense = set()
        if n_dense_blocks == 1:
            dense.add(n // 2)
        elif n_dense_blocks > 1:
            dense.update(int(i) for i in torch.linspace(0, n - 1, n_dense_blocks).long().tolist())
        per_block = [None if i in dense else natten_parameters for i in range(n)]
    for i, (block, params) in enumerate(zip(model.blocks, per_block)):
        if params is not None:
            layer = dict(params)
            layer["layer_id"] = i
            block.self_attn.sparse_op = NeighborhoodAttention(layer, base_attn_op=ops.attention)
    return model
