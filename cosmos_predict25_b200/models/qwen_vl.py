"""Vision-language model of Reason1 (Qwen2.5-VL): vision tower + language tower, image / video features scattered into the
token embeddings, 3-D multimodal rotary positions (M-RoPE).

Parity target: ``Qwen2_5_VLModel`` inside cosmos_predict2/_src/reason1/networks/qwen2_5_vl.py (position rule ``get_rope_index``,
embedding scatter, rotary sections). The video model's text conditioning uses the language tower alone (``models/text_encoder.py``);
this wrapper serves prompts that contain images or video.

Positions: text tokens advance all three components (t, h, w) together; the tokens of an image or video take
(t index x seconds per temporal grid step x tokens per second, row, column) of their merged patch, offset by the position where the
vision block starts; the text after a vision block continues at the largest position used so far + 1. The rotary angle of
frequency i uses the t component for i in the first section, h for the second, w for the third (sections in rotary pairs).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from .qwen_vision import QwenVisionConfig, QwenVisionTower
from .text_encoder import QwenConfig, QwenLanguageModel


@dataclass
class QwenVLConfig:
    text: QwenConfig = field(default_factory=QwenConfig)
    vision: QwenVisionConfig = field(default_factory=QwenVisionConfig)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    mrope_section: Tuple[int, int, int] = (16, 24, 24)      # rotary pairs per position component; sums to head_dim / 2
    tokens_per_second: float = 2.0


def multimodal_positions(input_ids: torch.Tensor, image_grid_thw: Optional[torch.Tensor], video_grid_thw: Optional[torch.Tensor],
                         second_per_grid_ts: Optional[Sequence[float]], attention_mask: Optional[torch.Tensor], cfg: QwenVLConfig,
                         ) -> torch.Tensor:
    """[3, B, S] position components (t, h, w) of every token; padded positions get 1."""
    B, S = input_ids.shape
    merge = cfg.vision.spatial_merge_size
    if attention_mask is None:
        attention_mask = torch.ones_like(input_ids)
    if image_grid_thw is None and video_grid_thw is None:
        pos = (attention_mask.long().cumsum(-1) - 1).masked_fill(attention_mask == 0, 1)
        return pos[None].expand(3, B, S).clone()
    out = torch.ones(3, B, S, dtype=torch.long, device=input_ids.device)
    img_i = vid_i = 0
    for b in range(B):
        keep = attention_mask[b] == 1
        toks = input_ids[b][keep].tolist()
        parts: List[torch.Tensor] = []
        st = 0
        nxt = 0                                               # next free position
        while True:
            # next vision block: the first image / video placeholder at or after st
            ed_img = toks.index(cfg.image_token_id, st) if cfg.image_token_id in toks[st:] else len(toks) + 1
            ed_vid = toks.index(cfg.video_token_id, st) if cfg.video_token_id in toks[st:] else len(toks) + 1
            if min(ed_img, ed_vid) > len(toks):
                break
            if ed_img < ed_vid:
                t, h, w = (int(v) for v in image_grid_thw[img_i])
                img_i += 1
                step, ed = 0.0, ed_img
            else:
                t, h, w = (int(v) for v in video_grid_thw[vid_i])
                step = float(second_per_grid_ts[vid_i]) if second_per_grid_ts is not None else 1.0
                vid_i += 1
                ed = ed_vid
            gh, gw = h // merge, w // merge
            n_text = ed - st
            parts.append(torch.arange(n_text)[None].expand(3, -1) + nxt)
            base = nxt + n_text
            ti = (torch.arange(t)[:, None].expand(t, gh * gw) * step * cfg.tokens_per_second).long().reshape(-1)
            hi = torch.arange(gh)[None, :, None].expand(t, gh, gw).reshape(-1)
            wi = torch.arange(gw)[None, None, :].expand(t, gh, gw).reshape(-1)
            parts.append(torch.stack([ti, hi, wi]) + base)
            nxt = int(parts[-1].max()) + 1
            st = ed + t * gh * gw
        if st < len(toks):
            parts.append(torch.arange(len(toks) - st)[None].expand(3, -1) + nxt)
        out[:, b, keep] = torch.cat(parts, 1).to(out.device)
    return out


class QwenVLModel(nn.Module):
    def __init__(self, config: QwenVLConfig):
        super().__init__()
        self.config = config
        self.visual = QwenVisionTower(config.vision)
        self.language_model = QwenLanguageModel(config.text)

    def mrope(self, position_ids: torch.Tensor, dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        """cos, sin [B, 1, S, head_dim] from [3, B, S] positions: frequency i takes the component of its section."""
        c = self.config.text
        hd = c.hidden_size // c.num_attention_heads
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, hd, 2, dtype=torch.float32, device=position_ids.device) / hd))
        ang = position_ids[..., None].float() * inv                                # [3, B, S, hd / 2]
        sec = self.config.mrope_section
        assert sum(sec) == hd // 2, (sec, hd)
        which = torch.repeat_interleave(torch.arange(3, device=ang.device), torch.tensor(sec, device=ang.device))   # [hd / 2]
        ang = ang.gather(0, which[None, None, None, :].expand(1, *ang.shape[1:]))[0]                                # [B, S, hd / 2]
        emb = torch.cat([ang, ang], -1)
        return emb.cos()[:, None].to(dtype), emb.sin()[:, None].to(dtype)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                pixel_values: Optional[torch.Tensor] = None, image_grid_thw: Optional[torch.Tensor] = None,
                pixel_values_videos: Optional[torch.Tensor] = None, video_grid_thw: Optional[torch.Tensor] = None,
                second_per_grid_ts: Optional[Sequence[float]] = None) -> List[torch.Tensor]:
        """Every hidden state of the language tower [B, S, hidden] for prompts with image / video placeholders."""
        cfg = self.config
        lm = self.language_model
        emb = lm.embed_tokens(input_ids)
        for values, grid, token in ((pixel_values, image_grid_thw, cfg.image_token_id),
                                    (pixel_values_videos, video_grid_thw, cfg.video_token_id)):
            if values is None:
                continue
            feats = self.visual(values, grid).to(emb.dtype)
            where = input_ids == token
            assert int(where.sum()) == feats.shape[0], f"{int(where.sum())} placeholder tokens for {feats.shape[0]} vision features"
            emb = emb.masked_scatter(where[..., None].expand_as(emb), feats)
        pos = multimodal_positions(input_ids, image_grid_thw, video_grid_thw, second_per_grid_ts, attention_mask, cfg)
        return lm(None, attention_mask=attention_mask, inputs_embeds=emb, rope=self.mrope(pos, emb.dtype))

    def load_hf_state_dict(self, sd) -> None:
        """Hugging Face Qwen2.5-VL names: ``model.visual.*`` / ``visual.*`` and ``model.language_model.*`` / ``model.*``."""
        vis = {}
        for k, v in sd.items():
            for prefix in ("model.visual.", "visual."):
                if k.startswith(prefix):
                    vis[k[len(prefix):]] = v
        self.visual.load_state_dict(vis, strict=True)
        self.language_model.load_hf_state_dict({k: v for k, v in sd.items() if "visual." not in k and not k.startswith("lm_head")})
