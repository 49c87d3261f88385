"""Text2World / Image2World / Video2World generation pipeline.

Parity target: ``Video2WorldInference`` (cosmos_predict2/_src/predict2/inference/video2world.py:282-519): build the model
from an experiment + checkpoint (EMA weights as regular ones), optional context parallelism over all ranks, read and
pre-process the conditioning image / video into a uint8 clip, compute prompt and negative-prompt embeddings,
sample 35 UniPC steps with classifier-free guidance, decode to pixels in [-1, 1].

Differences by design: cond / uncond run as one batch-2 forward with the text context and cross-attention K/V
cached across the 35 steps; the VAE decode is split into horizontal bands over the context-parallel group
(exact: boundary rows are exchanged) instead of being repeated on every rank.
"""

from __future__ import annotations

import os
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..models.text_encoder import HashTextEncoder, NUM_EMBEDDING_PADDING_TOKENS
from ..parallel.mesh import build_groups
from ..utils import log
from ..utils.model_loader import load_model_from_checkpoint
from ..utils.video_io import IMAGE_EXT, VIDEO_EXT, read_and_process_image, read_and_process_video

_RESOLUTIONS = {  # (H, W) per resolution key and aspect ratio
    "720": {"16,9": (704, 1280), "9,16": (1280, 704), "1,1": (960, 960), "4,3": (832, 1120), "3,4": (1120, 832)},
    "480": {"16,9": (432, 768), "9,16": (768, 432), "1,1": (640, 640), "4,3": (544, 736), "3,4": (736, 544)},
    "256": {"16,9": (192, 320), "9,16": (320, 192), "1,1": (256, 256), "4,3": (192, 256), "3,4": (256, 192)},
}


class Video2WorldInference:
    def __init__(self, experiment_name: str, ckpt_path: Optional[str], s3_credential_path: str = "", context_parallel_size: int = 1,
                 config_file: str = "cosmos_predict25_b200.configs.video2world", experiment_opts=None, text_encoder=None,
                 device=None, model=None, config=None):
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.context_parallel_size = context_parallel_size
        self.groups = build_groups(cp_size=context_parallel_size) if context_parallel_size > 1 else None
        cp_group = self.groups.cp if self.groups is not None else None
        if model is None:
            model, config = load_model_from_checkpoint(experiment_name, ckpt_path, config_file=config_file, load_ema_to_reg=True,
                                                       experiment_opts=experiment_opts, device=device, cp_group=cp_group)
        self.model, self.config = model, config
        self.model.cp_group = cp_group
        if cp_group is not None:
            self.model.shard_vae_encode = True     # every rank reads the same conditioning clip: encode it in row bands
            self.model.net.enable_context_parallel(cp_group)
            self._attach_peer_exchange(cp_group)
        self.device = self.model.device_
        net_cfg = self.model.config.net
        self.text_dim = net_cfg.crossattn_proj_in_channels if net_cfg.use_crossattn_projection else net_cfg.crossattn_emb_channels
        self.text_encoder = text_encoder or self.model.text_encoder
        if self.text_encoder is None:
            log.warning("no text-encoder weights configured: prompts are mapped to deterministic pseudo-embeddings")
            self.text_encoder = HashTextEncoder(self.text_dim, NUM_EMBEDDING_PADDING_TOKENS, device=self.device, dtype=self.model.precision)

    def _attach_peer_exchange(self, cp_group):
        if self.device_type() != "cuda":
            return
        try:
            from ..parallel import ulysses
            from ..parallel.symm import PeerAllToAll, PeerContext
            c = self.model.config
            tok = self.model.tokenizer
            per_rank = 2 * (c.state_t // self.context_parallel_size + 1) * 64 * 96 * c.net.model_channels
            ctx = PeerContext(cp_group, self.model.device_, arena_bytes=8 * (per_rank * 2 + 4096) + (1 << 20))
            ulysses.attach_peer_transport(cp_group, PeerAllToAll(ctx, max_elems=per_rank))
        except Exception as e:
            log.warning(f"peer-memory exchange unavailable ({e}); context parallelism uses NCCL all-to-all")

    def device_type(self) -> str:
        return self.model.device_.type

    # ---- inputs ------------------------------------------------------------------------------------------------
    def resolve_resolution(self, resolution: str = "none", aspect_ratio: str = "16,9"):
        if resolution and resolution != "none":
            h, w = (int(x) for x in resolution.split(","))
            return h, w
        return _RESOLUTIONS[str(self.model.config.resolution)][aspect_ratio]

    def _get_data_batch_input(self, video: torch.Tensor, prompt: str, num_latent_conditional_frames: int = 1,
                              negative_prompt: Optional[str] = None, use_neg_prompt: bool = True) -> Dict:
        B, C, T, H, W = video.shape
        batch = {"dataset_name": "video_data", "video": video.to(self.device),
                 "fps": torch.full((B,), 16.0, device=self.device), "padding_mask": torch.zeros(B, 1, H, W, device=self.device),
                 "num_conditional_frames": num_latent_conditional_frames, "ai_caption": [prompt] * B}
        batch["t5_text_embeddings"] = self.text_encoder.encode_prompts([prompt] * B).to(self.device, self.model.precision)
        if use_neg_prompt:
            if negative_prompt is None:          # the library call without a negative prompt uses the default one, like the CLI
                from ..config import DEFAULT_NEGATIVE_PROMPT as negative_prompt
            neg = negative_prompt
            batch["neg_t5_text_embeddings"] = self.text_encoder.encode_prompts([neg] * B).to(self.device, self.model.precision)
        return batch

    # ---- generation -------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate_vid2world(self, prompt: str, input_path: Optional[str], guidance: float = 7.0, num_video_frames: int = 77,
                           num_latent_conditional_frames: int = 1, resolution: str = "none", seed: int = 1,
                           negative_prompt: Optional[str] = None, num_steps: int = 35, aspect_ratio: str = "16,9",
                           input_video: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Returns the generated clip [B, 3, T, H, W] in [-1, 1]."""
        assert num_latent_conditional_frames in (0, 1, 2), "0 (text), 1 (image) or 2 (video) conditioning latent frames"
        tok = self.model.tokenizer
        n_frames = tok.get_pixel_num_frames(self.model.config.state_t) if tok is not None else num_video_frames
        H, W = self.resolve_resolution(resolution, aspect_ratio)
        if input_video is not None:
            vid = input_video
        elif num_latent_conditional_frames == 0 or not input_path:
            vid = torch.zeros(1, 3, n_frames, H, W, dtype=torch.uint8)
            num_latent_conditional_frames = 0
        else:
            ext = os.path.splitext(input_path)[1].lower()
            if ext in IMAGE_EXT:
                vid = read_and_process_image(input_path, (H, W), n_frames)
                num_latent_conditional_frames = min(num_latent_conditional_frames, 1)
            elif ext in VIDEO_EXT:
                vid = read_and_process_video(input_path, (H, W), n_frames, max(num_latent_conditional_frames, 1))
            else:
                raise ValueError(f"unsupported input {input_path}")
        batch = self._get_data_batch_input(vid, prompt, num_latent_conditional_frames, negative_prompt, use_neg_prompt=True)
        latents = self.model.generate_samples_from_batch(batch, guidance=guidance, seed=seed, is_negative_prompt=True,
                                                         num_steps=num_steps, shift=self.model.config.shift)
        if tok is None:
            return latents
        return self.model.decode(latents).float().clamp(-1, 1)

    def cleanup(self):
        if dist.is_initialized() and self.context_parallel_size > 1:
            dist.barrier()
