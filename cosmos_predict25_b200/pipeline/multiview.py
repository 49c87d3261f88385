"""Multiview video-to-video inference.

Parity target: ``Vid2VidInference`` (cosmos_predict2/_src/predict2_multiview/scripts/inference.py:70-180): load the
experiment's model, optionally enable context parallelism, then for a dataloader batch compute (or take) the text
embeddings, sample with classifier-free guidance, decode every view with the tokenizer and stack the views either on
the time axis or on the height axis.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..models.multiview import NUM_CONDITIONAL_FRAMES_KEY
from ..models.text_encoder import HashTextEncoder, NUM_EMBEDDING_PADDING_TOKENS
from ..parallel.mesh import build_groups
from ..utils import log
from ..utils.model_loader import load_model_from_checkpoint


def to_model_input(batch: Dict, model) -> Dict:
    out = {}
    for k, v in batch.items():
        if isinstance(v, torch.Tensor):
            v = v.to(model.device_)
            if torch.is_floating_point(v):
                v = v.to(model.precision)
        out[k] = v
    return out


class Vid2VidInference:
    def __init__(self, experiment_name: str, ckpt_path: Optional[str], s3_credential_path: str = "", context_parallel_size: int = 1,
                 config_file: str = "cosmos_predict25_b200.configs.multiview", experiment_opts=None, text_encoder=None,
                 device=None, model=None, config=None):
        self.experiment_name, self.ckpt_path = experiment_name, ckpt_path
        self.context_parallel_size = context_parallel_size
        self.groups = build_groups(cp_size=context_parallel_size) if context_parallel_size > 1 else None
        self.process_group = self.groups.cp if self.groups is not None else None
        if model is None:
            model, config = load_model_from_checkpoint(experiment_name, ckpt_path, config_file=config_file, load_ema_to_reg=True,
                                                       experiment_opts=experiment_opts, device=device, cp_group=self.process_group)
        self.model, self.config = model, config
        self.model.cp_group = self.process_group
        if self.process_group is not None:
            self.model.net.enable_context_parallel(self.process_group)
        net_cfg = self.model.config.net
        self.text_dim = net_cfg.crossattn_proj_in_channels if net_cfg.use_crossattn_projection else net_cfg.crossattn_emb_channels
        self.text_encoder = text_encoder or self.model.text_encoder
        if self.text_encoder is None:
            log.warning("no text-encoder weights configured: prompts are mapped to deterministic pseudo-embeddings")
            self.text_encoder = HashTextEncoder(self.text_dim, self.model.config.tokens_per_view, device=self.model.device_,
                                                dtype=self.model.precision)
        self.batch_size = 1

    def compute_text_embeddings(self, batch: Dict) -> None:
        """One caption per view (joined by `` -- ``) -> ``[B, V*tokens_per_view, D]``; a single caption is repeated."""
        if "t5_text_embeddings" in batch:
            return
        V = int(batch["sample_n_views"].view(-1)[0]) if "sample_n_views" in batch else 1
        embs = []
        for cap in batch["ai_caption"]:
            parts = cap.split(" -- ")
            if len(parts) == 1:
                parts = parts * V
            assert len(parts) >= V, f"expected {V} view captions, got {len(parts)}"
            e = self.text_encoder.encode_prompts(parts[:V])                       # [V, L, D]
            embs.append(e.reshape(1, -1, e.shape[-1]))
        batch["t5_text_embeddings"] = torch.cat(embs, 0).to(self.model.device_, self.model.precision)

    @torch.no_grad()
    def generate_from_batch(self, data_batch: Dict, guidance: float = 7, seed: int = 1, num_steps: int = 35,
                            stack_mode: str = "time", decode: bool = True) -> torch.Tensor:
        batch = to_model_input(data_batch, self.model)
        self.compute_text_embeddings(batch)
        _, x0, _ = self.model.get_data_and_condition(dict(batch))
        sample = self.model.generate_samples_from_batch(batch, guidance=guidance, state_shape=tuple(x0.shape[1:]), n_sample=x0.shape[0],
                                                        seed=seed, num_steps=num_steps, is_negative_prompt=False)
        video = self.model.decode(sample) if (decode and self.model.tokenizer is not None) else sample
        if stack_mode == "height":
            V = sample.shape[2] // self.model.state_t
            B, C, VT, H, W = video.shape
            video = video.view(B, C, V, VT // V, H, W).permute(0, 1, 3, 2, 4, 5).reshape(B, C, VT // V, V * H, W)
        elif stack_mode != "time":
            raise ValueError(f"Invalid stack mode '{stack_mode}'. Must be one of: 'height', 'time'")
        return video

    def cleanup(self):
        if dist.is_initialized() and self.context_parallel_size > 1:
            dist.barrier()
