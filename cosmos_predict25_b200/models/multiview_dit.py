"""N-camera DiT: the views of one sample are stacked along the latent time axis.

Parity target: ``MultiViewDiT`` and its parts (cosmos_predict2/_src/predict2_multiview/networks/multiview_dit.py:40-578):
* self-attention runs over all views jointly (sequence = V * T * H * W tokens);
* cross-attention runs per view: view v's tokens attend only to view v's caption tokens (``MultiViewCrossAttention`` :40);
* every view gets the same 3-D rotary table, i.e. positions restart at 0 for each camera
  (``MultiCameraVideoRopePosition3DEmb`` :103);
* an optional learned per-camera embedding is concatenated to the input channels (``prepare_embedded_sequence`` :444);
* context parallelism splits the frames of every view, so a rank holds frames [r*T/P, (r+1)*T/P) of all V views.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as ops
from ..parallel import ulysses
from .dit import Attention, Block, ContextCache, CosmosDiT, DiTConfig, PatchEmbed


@dataclass
class MultiViewDiTConfig(DiTConfig):
    state_t: int = 8                    # latent frames per view
    n_cameras_emb: int = 7              # rows of the camera embedding table
    view_condition_dim: int = 7
    concat_view_embedding: bool = True
    context_tokens_per_view: int = 512
    timestep_scale: float = 0.001


class MultiViewCrossAttention(Attention):
    """Cross-attention restricted to each view's own caption: folds views into the batch axis."""

    def __init__(self, *args, tokens_per_view: int = 512, **kw):
        super().__init__(*args, **kw)
        self.tokens_per_view = tokens_per_view

    def _views(self, n_ctx: int) -> int:
        assert n_ctx % self.tokens_per_view == 0, (n_ctx, self.tokens_per_view)
        return n_ctx // self.tokens_per_view

    def project_kv(self, context: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        B, M, D = context.shape
        V = self._views(M)
        ctx = context.view(B, V, M // V, D).transpose(0, 1).reshape(V * B, M // V, D)   # (V B) M D
        return super().project_kv(ctx)

    def forward(self, x, context=None, rope=None, kv=None, return_pre_proj: bool = False):
        B, L, D = x.shape
        if kv is None:
            kv = self.project_kv(context)
        V = kv[0].shape[0] // B
        assert L % V == 0
        xv = x.view(B, V, L // V, D).transpose(0, 1).reshape(V * B, L // V, D)
        o = super().forward(xv, None, None, kv, return_pre_proj=return_pre_proj)
        return o.view(V, B, L // V, -1).transpose(0, 1).reshape(B, L, -1)


class MultiViewBlock(Block):
    def __init__(self, cfg: MultiViewDiTConfig):
        super().__init__(cfg)
        self.cross_attn = MultiViewCrossAttention(cfg.model_channels, cfg.crossattn_emb_channels, cfg.num_heads,
                                                  cfg.head_dim, tokens_per_view=cfg.context_tokens_per_view)


class MultiViewDiT(CosmosDiT):
    def __init__(self, cfg: MultiViewDiTConfig):
        super().__init__(cfg)
        D = cfg.model_channels
        if cfg.concat_view_embedding:
            in_ch = (cfg.in_channels + cfg.view_condition_dim + (1 if cfg.add_condition_mask_channel else 0)
                     + (1 if cfg.concat_padding_mask else 0))
            self.x_embedder = PatchEmbed(cfg.patch_spatial, cfg.patch_temporal, in_ch, D)
            self.view_embeddings = nn.Embedding(cfg.n_cameras_emb, cfg.view_condition_dim)
        self.blocks = nn.ModuleList([MultiViewBlock(cfg) for _ in range(cfg.num_blocks)])
        # the released multi-camera checkpoints hold one rotary-position module per camera count (``pos_embedder_options.
        # n_cameras_K.*``, multiview_dit.py:397-403 of the reference); their tables are identical - a view's positions do not
        # depend on the number of views - so the first one serves every count and the rest only keep the state dict's names
        import copy
        one = self._modules.pop("pos_embedder")
        self.pos_embedder_options = nn.ModuleDict({f"n_cameras_{k}": (one if k == 1 else copy.deepcopy(one))
                                                   for k in range(1, cfg.n_cameras_emb + 1)})

    def __getattr__(self, name):
        if name == "pos_embedder":
            return self._modules["pos_embedder_options"]["n_cameras_1"]
        return super().__getattr__(name)

    # ---- embedding ---------------------------------------------------------------------------------------------
    def n_views_of(self, local_T: int) -> int:
        cp_size, _ = ulysses.group_size_rank(self.cp_group)
        assert (local_T * cp_size) % self.cfg.state_t == 0, (local_T, cp_size, self.cfg.state_t)
        return (local_T * cp_size) // self.cfg.state_t

    def _view_channels(self, B: int, V: int, Tv: int, H: int, W: int, view_indices_B_T, like: torch.Tensor):
        cfg = self.cfg
        if view_indices_B_T is None:
            idx = torch.arange(V, device=like.device).clamp(max=cfg.n_cameras_emb - 1)
            e = self.view_embeddings(idx).t().reshape(1, -1, V, 1, 1, 1)                    # 1 D V 1 1 1
        else:
            idx = view_indices_B_T.to(like.device).long().clamp(max=cfg.n_cameras_emb - 1)
            e = self.view_embeddings(idx)                                                    # B (V T) D
            e = e.view(B, V, Tv, -1).permute(0, 3, 1, 2)[..., None, None]                    # B D V T 1 1
        return e.expand(B, e.shape[1], V, Tv, H, W).reshape(B, -1, V * Tv, H, W).to(like.dtype)

    def _embed_mv(self, x, condition_mask, padding_mask, view_indices_B_T):
        cfg = self.cfg
        B, C, T, H, W = x.shape
        parts = [x]
        if cfg.add_condition_mask_channel:
            parts.append((x.new_zeros(B, 1, T, H, W) if condition_mask is None else condition_mask.to(x.dtype)))
        if cfg.concat_padding_mask:
            if padding_mask is None:
                pm = x.new_zeros(B, 1, 1, H, W)
            else:
                pm = padding_mask.to(x.dtype)
                if pm.shape[-2:] != (H, W):
                    pm = F.interpolate(pm, size=(H, W), mode="nearest")
                pm = pm.view(B, 1, 1, H, W)
            parts.append(pm.expand(B, 1, T, H, W))
        if cfg.concat_view_embedding:
            V = self.n_views_of(T)
            parts.append(self._view_channels(B, V, T // V, H, W, view_indices_B_T, x))
        xin = torch.cat(parts, dim=1)
        lin = self.x_embedder.proj[1]
        return F.linear(self.x_embedder.proj[0](xin).to(lin.weight.dtype), lin.weight)

    def _rope(self, T: int, H: int, W: int, fps) -> torch.Tensor:
        V = self.n_views_of(T)
        _, cp_rank = ulysses.group_size_rank(self.cp_group)
        Tv = T // V
        one = self.pos_embedder.generate(Tv, H, W, fps, t_offset=cp_rank * Tv)              # [Tv*H*W, hd]
        return one.repeat(V, 1)

    # ---- forward ------------------------------------------------------------------------------------------------
    def forward(self, x_B_C_T_H_W, timesteps_B_T, crossattn_emb, condition_video_input_mask_B_C_T_H_W=None, fps=None,
                padding_mask=None, context_cache: Optional[ContextCache] = None, view_indices_B_T=None, **_unused):
        cfg = self.cfg
        x = self._embed_mv(x_B_C_T_H_W, condition_video_input_mask_B_C_T_H_W, padding_mask, view_indices_B_T)
        B, T, H, W, D = x.shape
        rope = ops.RopeTable(self._rope(T, H, W, fps))
        if context_cache is not None:
            context, cross_kv = context_cache.context, context_cache.cross_kv
        else:
            context, cross_kv = self.project_context(crossattn_emb), None
        if timesteps_B_T.ndim == 1:
            timesteps_B_T = timesteps_B_T.unsqueeze(1)
        sinus = self.t_embedder[0](timesteps_B_T.float() * cfg.timestep_scale)
        if not cfg.use_wan_fp32_strategy:
            sinus = sinus.to(x.dtype)
        emb, lora = self.t_embedder[1](sinus)
        emb = self.t_embedding_norm(emb)
        if emb.shape[1] == 1 and T > 1:
            emb = emb.expand(B, T, -1)
            lora = lora.expand(B, T, -1) if lora is not None else None
        x = x.view(B, T, H * W, D)
        from .checkpointing import run_block
        for i, block in enumerate(self.blocks):
            kv = cross_kv[i] if cross_kv else None
            x = run_block(block, cfg.checkpoint_mode if self.training else "none", x, emb, context, rope, lora, None, kv)
        out = self.final_layer(x, emb, lora).view(B, T, H, W, -1)
        return self.unpatchify(out)


def multiview_dit_2b(**kw) -> MultiViewDiTConfig:
    """2B multiview network (buttercup2p5_rectified_flow.py: 7 cameras, state_t 8, crossattn width 1024)."""
    base = dict(model_channels=2048, num_heads=16, num_blocks=28, state_t=8, n_cameras_emb=7, view_condition_dim=7,
                concat_view_embedding=True, rope_enable_fps_modulation=False, rope_h_extrapolation_ratio=3.0,
                rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=8.0 / 24.0)
    base.update(kw)
    return MultiViewDiTConfig(**base)


def multiview_dit_14b(**kw) -> MultiViewDiTConfig:
    return multiview_dit_2b(model_channels=5120, num_heads=40, num_blocks=36, **kw)


def multiview_dit_tiny(**kw) -> MultiViewDiTConfig:
    base = dict(model_channels=256, num_heads=4, num_blocks=2, crossattn_emb_channels=256, use_crossattn_projection=False,
                max_img_h=64, max_img_w=64, max_frames=32, adaln_lora_dim=64, state_t=2, n_cameras_emb=4,
                view_condition_dim=4, context_tokens_per_view=8)
    base.update(kw)
    return MultiViewDiTConfig(**base)
