"""Image tokenizers kept for the legacy text-to-image paths.

Parity targets: ``BaseVAE`` / ``BasePretrainedImageVAE`` / ``JITVAE`` / ``StateDictVAE`` / ``SDVAE``
(cosmos_predict2/_src/predict2/tokenizers/base_vae.py:29-462). A pretrained image VAE is an (encoder, decoder) pair loaded
from TorchScript archives or from state dicts into a user-supplied module, wrapped with per-channel latent
normalisation ``(z - mean) / std`` and dtype handling. ``SDVAE`` wraps a Stable-Diffusion ``AutoencoderKL`` with its
fixed per-channel scale / bias and an optional 2x bilinear down/up-sampling around it.
"""

from __future__ import annotations

import os
from abc import ABC, abstractmethod
from typing import Optional

import torch
import torch.nn.functional as F


class BaseVAE(torch.nn.Module, ABC):
    def __init__(self, channel: int = 3, name: str = "vae"):
        super().__init__()
        self.channel, self.name = channel, name

    @property
    def latent_ch(self) -> int:
        return self.channel

    @abstractmethod
    def encode(self, state: torch.Tensor) -> torch.Tensor: ...

    @abstractmethod
    def decode(self, latent: torch.Tensor) -> torch.Tensor: ...

    @property
    def spatial_compression_factor(self) -> int:
        return 8


class BasePretrainedImageVAE(BaseVAE):
    def __init__(self, name: str, mean_std_fp: Optional[str] = None, latent_ch: int = 16, is_image: bool = True, is_bf16: bool = True,
                 load_mean_std: bool = True):
        super().__init__(latent_ch, name)
        self.dtype = torch.bfloat16 if is_bf16 else torch.float32
        self.is_image, self.load_mean_std = is_image, load_mean_std and bool(mean_std_fp)
        self.register_mean_std(mean_std_fp)
        self.encoder: Optional[torch.nn.Module] = None
        self.decoder: Optional[torch.nn.Module] = None

    def register_mean_std(self, mean_std_fp: Optional[str]) -> None:
        shape = [1, self.latent_ch, 1, 1] if self.is_image else [1, self.latent_ch, 1, 1, 1]
        if self.load_mean_std:
            from ..utils.easy_io import easy_io
            mean, std = easy_io.load(mean_std_fp)
            mean, std = torch.as_tensor(mean), torch.as_tensor(std)
        else:
            mean, std = torch.zeros(self.latent_ch), torch.ones(self.latent_ch)
        self.register_buffer("latent_mean", mean.to(self.dtype).reshape(*shape), persistent=False)
        self.register_buffer("latent_std", std.to(self.dtype).reshape(*shape), persistent=False)

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        in_dtype = state.dtype
        z = self.encoder(state.to(self.dtype))
        if isinstance(z, tuple):
            z = z[0]
        if not isinstance(z, torch.Tensor):
            raise ValueError("Invalid type of encoded state")
        return (z.to(in_dtype) - self.latent_mean.to(in_dtype)) / self.latent_std.to(in_dtype)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        in_dtype = latent.dtype
        latent = latent * self.latent_std.to(in_dtype) + self.latent_mean.to(in_dtype)
        return self.decoder(latent.to(self.dtype)).to(in_dtype)

    def reset_dtype(self, *args, **kwargs):
        self.decoder.to(self.dtype)
        self.encoder.to(self.dtype)


class JITVAE(BasePretrainedImageVAE):
    """Encoder / decoder stored as TorchScript archives."""

    def __init__(self, enc_fp: str, dec_fp: str, name: str, mean_std_fp: Optional[str] = None, latent_ch: int = 16, is_image: bool = True,
                 is_bf16: bool = True, load_mean_std: bool = True):
        super().__init__(name, mean_std_fp, latent_ch, is_image, is_bf16, load_mean_std)
        self.encoder = self._load(enc_fp)
        self.decoder = self._load(dec_fp)

    def _load(self, fp: str):
        m = torch.jit.load(fp, map_location="cpu")
        m.eval()
        for p in m.parameters():
            p.requires_grad = False
        return m.to(self.dtype)


class StateDictVAE(BasePretrainedImageVAE):
    """Encoder / decoder weights stored as state dicts for the ``encoder`` / ``decoder`` children of ``vae``."""

    def __init__(self, enc_fp: str, dec_fp: str, vae: torch.nn.Module, name: str, mean_std_fp: Optional[str] = None, latent_ch: int = 16,
                 is_image: bool = True, is_bf16: bool = True, load_mean_std: bool = True):
        super().__init__(name, mean_std_fp, latent_ch, is_image, is_bf16, load_mean_std)
        enc_sd = torch.load(enc_fp, map_location="cpu", weights_only=False)
        dec_sd = torch.load(dec_fp, map_location="cpu", weights_only=False)
        vae.encoder.load_state_dict(enc_sd)
        vae.decoder.load_state_dict(dec_sd)
        vae.eval().requires_grad_(False)
        self.vae = vae.to(self.dtype)
        self.encoder, self.decoder = self.vae.encoder, self.vae.decoder

    def reset_dtype(self, *args, **kwargs):
        self.vae.to(self.dtype)


class SDVAE(BaseVAE):
    SCALE = (4.17, 4.62, 3.71, 3.28)
    SHIFT = (5.81, 3.25, 0.12, -2.15)

    def __init__(self, batch_size: int = 16, count_std: bool = False, is_downsample: bool = True, vae: Optional[torch.nn.Module] = None,
                 dtype=torch.bfloat16):
        super().__init__(channel=4, name="sd_vae")
        self.dtype = dtype
        scale = torch.tensor(self.SCALE, dtype=dtype).reciprocal().reshape(1, -1, 1, 1)
        self.register_buffer("scale", scale, persistent=False)
        self.register_buffer("bias", -1.0 * torch.tensor(self.SHIFT, dtype=dtype).reshape(1, -1, 1, 1) * scale, persistent=False)
        self.batch_size, self.count_std, self.is_downsample = batch_size, count_std, is_downsample
        self.vae = (vae if vae is not None else self.load_vae()).eval().requires_grad_(False)
        self.reset_dtype()

    def reset_dtype(self, *args, **kwargs):
        self.vae.to(self.dtype)

    @staticmethod
    def load_vae():
        os.environ["HF_HUB_DISABLE_SYMLINKS_WARNING"] = "1"
        try:
            import diffusers
        except ImportError as e:
            raise ImportError("SDVAE needs the `diffusers` package (or pass `vae=` explicitly)") from e
        return diffusers.models.AutoencoderKL.from_pretrained("stabilityai/sd-vae-ft-mse", local_files_only=True)

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        if self.is_downsample:
            h, w = state.shape[-2:]
            state = F.interpolate(state, size=(h // 2, w // 2), mode="bilinear", align_corners=False)
        in_dtype = state.dtype
        dist = self.vae.encode(((state.to(self.dtype) + 1.0) / 2.0))["latent_dist"]
        z = dist.mean + torch.randn_like(dist.mean) * dist.std if self.count_std else dist.mean
        return (z * self.scale + self.bias).to(in_dtype)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        in_dtype = latent.dtype
        z = (latent.to(self.dtype) - self.bias) / self.scale
        x = torch.cat([self.vae.decode(b)["sample"] for b in z.split(self.batch_size)])
        if self.is_downsample:
            h, w = x.shape[-2:]
            x = F.interpolate(x, size=(h * 2, w * 2), mode="bilinear", align_corners=False)
        return x.to(in_dtype) * 2 - 1.0
