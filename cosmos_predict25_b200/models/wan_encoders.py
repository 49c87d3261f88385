"""Encoders that condition the Wan2.1 models: CLIP ViT-H/14 vision tower, XLM-RoBERTa text tower, umT5 text encoder.

Parity targets: ``VisionTransformer`` / ``XLMRobertaCLIP`` / ``CLIPModel`` / ``Wan2pt1CLIPEmb``
(cosmos_predict2/_src/predict2/networks/clip.py:195-592), ``XLMRoberta`` (cosmos_predict2/_src/predict2/networks/xlm_roberta.py:24-180)
and the umT5 encoder used to pre-compute prompt embeddings (cosmos_predict2/_src/predict2/inference/get_umt5_emb.py:40-634).
Module / parameter names follow the released Wan2.1 checkpoints so their state dicts load unchanged.

All towers are inference-only feature extractors here (frozen, no dropout).
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from .conditioner import AbstractEmbModel, GeneralConditioner, ReMapkey, Text2WorldCondition, TextAttr


# ---- CLIP vision tower ---------------------------------------------------------------------------------------------------
class QuickGELU(nn.Module):
    def forward(self, x):
        return x * torch.sigmoid(1.702 * x)


class _LN(nn.LayerNorm):
    def forward(self, x):
        return super().forward(x.float()).type_as(x)


class ClipSelfAttention(nn.Module):
    def __init__(self, dim: int, num_heads: int, causal: bool = False):
        super().__init__()
        self.num_heads, self.head_dim, self.causal = num_heads, dim // num_heads, causal
        self.to_qkv = nn.Linear(dim, dim * 3)
        self.proj = nn.Linear(dim, dim)

    def forward(self, x):
        B, S, C = x.shape
        q, k, v = self.to_qkv(x).view(B, S, 3, self.num_heads, self.head_dim).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=self.causal)
        return self.proj(o.transpose(1, 2).reshape(B, S, C))


class ClipSwiGLU(nn.Module):
    def __init__(self, dim, mid):
        super().__init__()
        self.fc1, self.fc2, self.fc3 = nn.Linear(dim, mid), nn.Linear(dim, mid), nn.Linear(mid, dim)

    def forward(self, x):
        return self.fc3(F.silu(self.fc1(x)) * self.fc2(x))


class ClipAttentionBlock(nn.Module):
    def __init__(self, dim, mlp_ratio, num_heads, post_norm=False, causal=False, activation="quick_gelu", norm_eps=1e-5):
        super().__init__()
        self.post_norm = post_norm
        self.norm1 = _LN(dim, eps=norm_eps)
        self.attn = ClipSelfAttention(dim, num_heads, causal)
        self.norm2 = _LN(dim, eps=norm_eps)
        if activation == "swi_glu":
            self.mlp = ClipSwiGLU(dim, int(dim * mlp_ratio))
        else:
            act = QuickGELU() if activation == "quick_gelu" else nn.GELU()
            self.mlp = nn.Sequential(nn.Linear(dim, int(dim * mlp_ratio)), act, nn.Linear(int(dim * mlp_ratio), dim), nn.Dropout(0.0))

    def forward(self, x):
        if self.post_norm:
            x = x + self.norm1(self.attn(x))
            return x + self.norm2(self.mlp(x))
        x = x + self.attn(self.norm1(x))
        return x + self.mlp(self.norm2(x))


def pos_interpolate(pos: torch.Tensor, seq_len: int) -> torch.Tensor:
    if pos.size(1) == seq_len:
        return pos
    src, tar = int(math.sqrt(pos.size(1))), int(math.sqrt(seq_len))
    n = pos.size(1) - src * src
    grid = pos[:, n:].float().reshape(1, src, src, -1).permute(0, 3, 1, 2)
    grid = F.interpolate(grid, size=(tar, tar), mode="bicubic", align_corners=False).flatten(2).transpose(1, 2)
    return torch.cat([pos[:, :n], grid.to(pos.dtype)], dim=1)


class VisionTransformer(nn.Module):
    def __init__(self, image_size=224, patch_size=14, dim=1280, mlp_ratio=4, out_dim=1024, num_heads=16, num_layers=32,
                 pool_type="token", pre_norm=True, post_norm=False, activation="gelu", norm_eps=1e-5):
        super().__init__()
        assert pool_type in ("token", "token_fc")
        self.image_size, self.patch_size, self.dim, self.pool_type = image_size, patch_size, dim, pool_type
        self.num_patches = (image_size // patch_size) ** 2
        gain = 1.0 / math.sqrt(dim)
        self.patch_embedding = nn.Conv2d(3, dim, kernel_size=patch_size, stride=patch_size, bias=not pre_norm)
        self.cls_embedding = nn.Parameter(gain * torch.randn(1, 1, dim))
        self.pos_embedding = nn.Parameter(gain * torch.randn(1, self.num_patches + 1, dim))
        self.pre_norm = _LN(dim, eps=norm_eps) if pre_norm else None
        self.transformer = nn.Sequential(*[ClipAttentionBlock(dim, mlp_ratio, num_heads, post_norm, False, activation, norm_eps)
                                           for _ in range(num_layers)])
        self.post_norm = _LN(dim, eps=norm_eps)
        self.head = nn.Parameter(gain * torch.randn(dim, out_dim)) if pool_type == "token" else nn.Linear(dim, out_dim)

    def forward(self, x, interpolation: bool = False, use_31_block: bool = False):
        b = x.size(0)
        x = self.patch_embedding(x).flatten(2).permute(0, 2, 1)
        x = torch.cat([self.cls_embedding.expand(b, -1, -1).to(x.dtype), x], dim=1)
        e = pos_interpolate(self.pos_embedding, x.size(1)) if interpolation else self.pos_embedding
        x = x + e.to(x.dtype)
        if self.pre_norm is not None:
            x = self.pre_norm(x)
        if use_31_block:      # penultimate-layer tokens are what conditions the video model
            return self.transformer[:-1](x)
        return self.transformer(x)

    def pooled(self, x):
        x = self.post_norm(self.forward(x))[:, 0]
        return x @ self.head if isinstance(self.head, nn.Parameter) else self.head(x)


# ---- XLM-RoBERTa text tower -------------------------------------------------------------------------------------------------
class XLMRobertaLayer(nn.Module):
    def __init__(self, dim, num_heads, post_norm=True, eps=1e-5):
        super().__init__()
        self.post_norm = post_norm
        self.attn = nn.ModuleDict(dict(q=nn.Linear(dim, dim), k=nn.Linear(dim, dim), v=nn.Linear(dim, dim), o=nn.Linear(dim, dim)))
        self.num_heads = num_heads
        self.norm1 = nn.LayerNorm(dim, eps=eps)
        self.ffn = nn.Sequential(nn.Linear(dim, dim * 4), nn.GELU(), nn.Linear(dim * 4, dim), nn.Dropout(0.0))
        self.norm2 = nn.LayerNorm(dim, eps=eps)

    def _attn(self, x, mask):
        B, S, C = x.shape
        n = self.num_heads
        q, k, v = (self.attn[t](x).view(B, S, n, C // n).transpose(1, 2) for t in ("q", "k", "v"))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask)
        return self.attn["o"](o.transpose(1, 2).reshape(B, S, C))

    def forward(self, x, mask):
        if self.post_norm:
            x = self.norm1(x + self._attn(x, mask))
            return self.norm2(x + self.ffn(x))
        x = x + self._attn(self.norm1(x), mask)
        return x + self.ffn(self.norm2(x))


class XLMRoberta(nn.Module):
    def __init__(self, vocab_size=250002, max_seq_len=514, type_size=1, pad_id=1, dim=1024, num_heads=16, num_layers=24,
                 post_norm=True, eps=1e-5):
        super().__init__()
        self.pad_id, self.post_norm = pad_id, post_norm
        self.token_embedding = nn.Embedding(vocab_size, dim, padding_idx=pad_id)
        self.type_embedding = nn.Embedding(type_size, dim)
        self.pos_embedding = nn.Embedding(max_seq_len, dim, padding_idx=pad_id)
        self.blocks = nn.ModuleList([XLMRobertaLayer(dim, num_heads, post_norm, eps) for _ in range(num_layers)])
        self.norm = nn.LayerNorm(dim, eps=eps)

    def forward(self, ids):
        mask = ids.ne(self.pad_id).long()
        x = self.token_embedding(ids) + self.type_embedding(torch.zeros_like(ids)) + \
            self.pos_embedding(self.pad_id + torch.cumsum(mask, dim=1) * mask)
        if self.post_norm:
            x = self.norm(x)
        attn_mask = mask.view(ids.shape[0], 1, 1, -1).bool()
        for blk in self.blocks:
            x = blk(x, attn_mask)
        return x if self.post_norm else self.norm(x)


class XLMRobertaWithHead(XLMRoberta):
    def __init__(self, out_dim=1024, **kw):
        super().__init__(**kw)
        dim = self.token_embedding.embedding_dim
        mid = (dim + out_dim) // 2
        self.head = nn.Sequential(nn.Linear(dim, mid, bias=False), nn.GELU(), nn.Linear(mid, out_dim, bias=False))

    def forward(self, ids):
        x = super().forward(ids)
        m = ids.ne(self.pad_id).unsqueeze(-1).to(x)
        return self.head((x * m).sum(1) / m.sum(1))


class XLMRobertaCLIP(nn.Module):
    """open-clip xlm-roberta-large + ViT-H/14 (the Wan2.1 image-conditioning CLIP)."""

    def __init__(self, embed_dim=1024, image_size=224, patch_size=14, vision_dim=1280, vision_heads=16, vision_layers=32,
                 text_dim=1024, text_heads=16, text_layers=24, vocab_size=250002, max_text_len=514):
        super().__init__()
        self.image_size, self.max_text_len = image_size, max_text_len
        self.visual = VisionTransformer(image_size, patch_size, vision_dim, 4, embed_dim, vision_heads, vision_layers, "token",
                                        True, False, "gelu", 1e-5)
        self.textual = XLMRobertaWithHead(out_dim=embed_dim, vocab_size=vocab_size, max_seq_len=max_text_len, dim=text_dim,
                                          num_heads=text_heads, num_layers=text_layers)
        self.log_scale = nn.Parameter(math.log(1 / 0.07) * torch.ones([]))

    def forward(self, imgs, txt_ids):
        return self.visual.pooled(imgs), self.textual(txt_ids)


CLIP_MEAN, CLIP_STD = (0.48145466, 0.4578275, 0.40821073), (0.26862954, 0.26130258, 0.27577711)


class CLIPModel:
    """Frozen CLIP wrapper: ``visual(frames in [-1,1])`` -> penultimate-layer tokens [B, 257, 1280]."""

    def __init__(self, dtype=torch.float16, device="cpu", checkpoint_path: Optional[str] = None, model: Optional[XLMRobertaCLIP] = None):
        self.dtype, self.device = dtype, torch.device(device)
        self.model = (model or XLMRobertaCLIP()).to(self.device, dtype).eval().requires_grad_(False)
        if checkpoint_path:
            from ..utils.checkpoint_db import get_checkpoint_path
            self.model.load_state_dict(torch.load(get_checkpoint_path(checkpoint_path), map_location="cpu"), strict=True)

    @torch.no_grad()
    def visual(self, videos_B_C_H_W: torch.Tensor) -> torch.Tensor:
        size = (self.model.image_size,) * 2
        x = F.interpolate(videos_B_C_H_W.float(), size=size, mode="bicubic", align_corners=False) * 0.5 + 0.5
        mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1)
        std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1)
        return self.model.visual(((x - mean) / std).to(self.device, self.dtype), use_31_block=True)


# ---- Wan I2V conditioning -----------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class WanI2VCondition(Text2WorldCondition):
    frame_cond_crossattn_emb_B_L_D: Optional[torch.Tensor] = None
    y_B_C_T_H_W: Optional[torch.Tensor] = None


class Wan2pt1CLIPEmb(AbstractEmbModel):
    """(images | video, conditioning latents) -> CLIP tokens of the first frame and ``y`` = [4-channel first-frame mask, latents]."""

    def __init__(self, input_key: Sequence[str] = ("images", "video", "i2v_WAN2PT1_cond_latents"), dropout_rate: float = 0.0,
                 num_token: int = 257, dtype: str = "bfloat16", clip_model: Optional[CLIPModel] = None):
        super().__init__(list(input_key), None, dropout_rate)
        self.num_token, self.model_dim = num_token, 1280
        self.clip_model = clip_model
        self.dtype = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}[dtype]

    def random_dropout_input(self, x=None, dropout_rate=None, key=None):
        return None if x is None else super().random_dropout_input(x, dropout_rate, key)

    def forward(self, image_tensor=None, video_tensor=None, media_latents=None) -> Dict[str, torch.Tensor]:
        b, _, f, h, w = media_latents.shape
        mask = torch.zeros(b, 4, f, h, w, device=media_latents.device, dtype=self.dtype)
        if image_tensor is not None or video_tensor is None:
            ctx = torch.zeros(b, self.num_token, self.model_dim, device=media_latents.device, dtype=self.dtype)
        else:
            if self.clip_model is None:
                self.clip_model = CLIPModel(device=media_latents.device)
            ctx = self.clip_model.visual(video_tensor[:, :, 0]).to(media_latents.device, self.dtype)
            mask[:, :, :1] = 1.0
        return {"frame_cond_crossattn_emb_B_L_D": ctx, "y_B_C_T_H_W": torch.cat([mask, media_latents.to(self.dtype)], dim=1)}

    def details(self) -> str:
        return f"Input key: {self.input_key}\n\tOutput key: ['frame_cond_crossattn_emb_B_L_D', 'y_B_C_T_H_W']"


class WanI2VConditioner(GeneralConditioner):
    condition_cls = WanI2VCondition


def default_wan_i2v_conditioner(text_dropout: float = 0.2, clip_model: Optional[CLIPModel] = None) -> WanI2VConditioner:
    return WanI2VConditioner(fps=ReMapkey("fps", "fps"), padding_mask=ReMapkey("padding_mask", "padding_mask"),
                             text=TextAttr("t5_text_embeddings", text_dropout), frame_cond=Wan2pt1CLIPEmb(clip_model=clip_model))


# ---- umT5 encoder ---------------------------------------------------------------------------------------------------------------
class T5LayerNorm(nn.Module):
    def __init__(self, dim, eps=1e-6):
        super().__init__()
        self.eps, self.weight = eps, nn.Parameter(torch.ones(dim))

    def forward(self, x):
        x = x * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + self.eps).type_as(x)
        return self.weight.to(x.dtype) * x


class T5RelativeEmbedding(nn.Module):
    def __init__(self, num_buckets, num_heads, bidirectional=True, max_dist=128):
        super().__init__()
        self.num_buckets, self.bidirectional, self.max_dist = num_buckets, bidirectional, max_dist
        self.embedding = nn.Embedding(num_buckets, num_heads)

    def _bucket(self, rel):
        nb = self.num_buckets // 2 if self.bidirectional else self.num_buckets
        out = (rel > 0).long() * nb if self.bidirectional else torch.zeros_like(rel)
        rel = rel.abs() if self.bidirectional else -torch.min(rel, torch.zeros_like(rel))
        exact = nb // 2
        large = exact + (torch.log(rel.float().clamp_min(1) / exact) / math.log(self.max_dist / exact) * (nb - exact)).long()
        return out + torch.where(rel < exact, rel, large.clamp_max(nb - 1))

    def forward(self, lq, lk):
        dev = self.embedding.weight.device
        rel = torch.arange(lk, device=dev)[None, :] - torch.arange(lq, device=dev)[:, None]
        return self.embedding(self._bucket(rel)).permute(2, 0, 1).unsqueeze(0)      # [1, heads, lq, lk]


class T5SelfAttentionBlock(nn.Module):
    def __init__(self, dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos=False):
        super().__init__()
        self.num_heads = num_heads
        self.norm1 = T5LayerNorm(dim)
        self.attn = nn.ModuleDict(dict(q=nn.Linear(dim, dim_attn, bias=False), k=nn.Linear(dim, dim_attn, bias=False),
                                       v=nn.Linear(dim, dim_attn, bias=False), o=nn.Linear(dim_attn, dim, bias=False)))
        self.norm2 = T5LayerNorm(dim)
        self.ffn = nn.ModuleDict(dict(gate=nn.Sequential(nn.Linear(dim, dim_ffn, bias=False), nn.GELU(approximate="tanh")),
                                      fc1=nn.Linear(dim, dim_ffn, bias=False), fc2=nn.Linear(dim_ffn, dim, bias=False)))
        self.pos_embedding = None if shared_pos else T5RelativeEmbedding(num_buckets, num_heads, True)

    def forward(self, x, mask=None, pos_bias=None):
        B, S, _ = x.shape
        n = self.num_heads
        e = pos_bias if self.pos_embedding is None else self.pos_embedding(S, S)
        h = self.norm1(x)
        q, k, v = (self.attn[t](h).view(B, S, n, -1).transpose(1, 2) for t in ("q", "k", "v"))
        bias = e.to(q.dtype)
        if mask is not None:
            bias = bias.masked_fill(~mask.view(B, 1, 1, S).bool(), torch.finfo(q.dtype).min)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias, scale=1.0)       # T5 does not scale the scores
        x = x + self.attn["o"](o.transpose(1, 2).reshape(B, S, -1))
        h = self.norm2(x)
        return x + self.ffn["fc2"](self.ffn["fc1"](h) * self.ffn["gate"](h))


class UMT5Encoder(nn.Module):
    """umT5-XXL encoder (per-layer relative position bias, gated tanh-GELU FFN)."""

    def __init__(self, vocab=256384, dim=4096, dim_attn=4096, dim_ffn=10240, num_heads=64, num_layers=24, num_buckets=32, shared_pos=False):
        super().__init__()
        self.token_embedding = nn.Embedding(vocab, dim)
        self.pos_embedding = T5RelativeEmbedding(num_buckets, num_heads, True) if shared_pos else None
        self.blocks = nn.ModuleList([T5SelfAttentionBlock(dim, dim_attn, dim_ffn, num_heads, num_buckets, shared_pos)
                                     for _ in range(num_layers)])
        self.norm = T5LayerNorm(dim)

    def forward(self, ids, mask=None):
        x = self.token_embedding(ids)
        e = self.pos_embedding(x.size(1), x.size(1)) if self.pos_embedding is not None else None
        for blk in self.blocks:
            x = blk(x, mask, e)
        return self.norm(x)


class UMT5EncoderModel:
    """Tokenise + encode prompts to ``[B, text_len, 4096]`` zero-padded embeddings (the ``t5_text_embeddings`` of Wan batches)."""

    def __init__(self, text_len=512, dtype=torch.bfloat16, device="cpu", checkpoint_path: Optional[str] = None,
                 tokenizer=None, model: Optional[UMT5Encoder] = None):
        self.text_len, self.dtype, self.device = text_len, dtype, torch.device(device)
        self.model = (model or UMT5Encoder()).to(self.device, dtype).eval().requires_grad_(False)
        if checkpoint_path:
            from ..utils.checkpoint_db import get_checkpoint_path
            self.model.load_state_dict(torch.load(get_checkpoint_path(checkpoint_path), map_location="cpu"))
        self.tokenizer = tokenizer

    @torch.no_grad()
    def __call__(self, texts: List[str]) -> torch.Tensor:
        if self.tokenizer is None:
            raise RuntimeError("a tokenizer (e.g. transformers AutoTokenizer 'google/umt5-xxl') must be supplied")
        tok = self.tokenizer(texts, return_tensors="pt", padding="max_length", truncation=True, max_length=self.text_len,
                             add_special_tokens=True)
        ids, mask = tok["input_ids"].to(self.device), tok["attention_mask"].to(self.device)
        out = self.model(ids, mask)
        return out * mask.unsqueeze(-1).to(out.dtype)
