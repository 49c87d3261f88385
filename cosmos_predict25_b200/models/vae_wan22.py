"""Wan2.2 VAE: 48 latent channels, 16x16 spatial / 4x temporal compression.

Parity targets: ``patchify`` / ``AvgDown3D`` / ``DupUp3D`` / ``Down_ResidualBlock`` / ``Up_ResidualBlock`` / ``Encoder3d`` /
``Decoder3d`` / ``WanVAE_`` / ``WanVAE`` / ``Wan2pt2VAEInterface`` (cosmos_predict2/_src/predict2/tokenizers/wan2pt2.py:255-1133).
Differences from the 2.1 VAE: a 2x2 pixel (un)patchify in front of the network (3 -> 12 channels), residual groups with
parameter-free shortcuts (grouped average on the way down, channel duplication on the way up), separate encoder /
decoder widths (160 / 256) and a decoder whose groups do not halve their input width.

Streaming rules are the 2.1 ones (first pixel frame alone, then windows of 4; one latent frame per decoder step; the first
decoder step skips temporal up-sampling, so its duplicated shortcut drops the leading ``factor_t - 1`` frames). The carry-over
lives in the explicit ``StreamState`` of the 2.1 implementation.
"""

from __future__ import annotations

from typing import List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from .vae_wan import (AttentionBlock, CausalConv3d, ResidualBlock, Resample, RMS_norm, StreamState, VideoTokenizerInterface)

WAN22_LATENT_MEAN = [-0.2289, -0.0052, -0.1323, -0.2339, -0.2799, 0.0174, 0.1838, 0.1557, -0.1382, 0.0542, 0.2813, 0.0891,
                     0.1570, -0.0098, 0.0375, -0.1825, -0.2246, -0.1207, -0.0698, 0.5109, 0.2665, -0.2108, -0.2158, 0.2502,
                     -0.2055, -0.0322, 0.1109, 0.1567, -0.0729, 0.0899, -0.2799, -0.1230, -0.0313, -0.1649, 0.0117, 0.0723,
                     -0.2839, -0.2083, -0.0520, 0.3748, 0.0152, 0.1957, 0.1433, -0.2944, 0.3573, -0.0548, -0.1681, -0.0667]
WAN22_LATENT_STD = [0.4765, 1.0364, 0.4514, 1.1677, 0.5313, 0.4990, 0.4818, 0.5013, 0.8158, 1.0344, 0.5894, 1.0901,
                    0.6885, 0.6165, 0.8454, 0.4978, 0.5759, 0.3523, 0.7135, 0.6804, 0.5833, 1.4146, 0.8986, 0.5659,
                    0.7069, 0.5338, 0.4889, 0.4917, 0.4069, 0.4999, 0.6866, 0.4093, 0.5709, 0.6065, 0.6415, 0.4944,
                    0.5726, 1.2042, 0.5458, 1.6887, 0.3971, 1.0600, 0.3943, 0.5537, 0.5444, 0.4089, 0.7468, 0.7744]


def patchify(x: torch.Tensor, p: int) -> torch.Tensor:
    """``b c f (h q) (w r) -> b (c r q) f h w`` (4-D input: without f)."""
    if p == 1:
        return x
    if x.dim() == 4:
        b, c, H, W = x.shape
        return x.view(b, c, H // p, p, W // p, p).permute(0, 1, 5, 3, 2, 4).reshape(b, c * p * p, H // p, W // p)
    b, c, f, H, W = x.shape
    return x.view(b, c, f, H // p, p, W // p, p).permute(0, 1, 6, 4, 2, 3, 5).reshape(b, c * p * p, f, H // p, W // p)


def unpatchify(x: torch.Tensor, p: int) -> torch.Tensor:
    if p == 1:
        return x
    if x.dim() == 4:
        b, C, h, w = x.shape
        c = C // (p * p)
        return x.view(b, c, p, p, h, w).permute(0, 1, 4, 3, 5, 2).reshape(b, c, h * p, w * p)
    b, C, f, h, w = x.shape
    c = C // (p * p)
    return x.view(b, c, p, p, f, h, w).permute(0, 1, 4, 5, 3, 6, 2).reshape(b, c, f, h * p, w * p)


class AvgDown3D(nn.Module):
    """Space/time-to-channel followed by a mean over channel groups: a parameter-free down-sampling shortcut."""

    def __init__(self, in_channels, out_channels, factor_t, factor_s=1):
        super().__init__()
        self.in_channels, self.out_channels, self.factor_t, self.factor_s = in_channels, out_channels, factor_t, factor_s
        self.factor = factor_t * factor_s * factor_s
        assert in_channels * self.factor % out_channels == 0
        self.group_size = in_channels * self.factor // out_channels

    def forward(self, x):
        ft, fs = self.factor_t, self.factor_s
        pad_t = (ft - x.shape[2] % ft) % ft
        x = F.pad(x, (0, 0, 0, 0, pad_t, 0))
        B, C, T, H, W = x.shape
        x = x.view(B, C, T // ft, ft, H // fs, fs, W // fs, fs).permute(0, 1, 3, 5, 7, 2, 4, 6)
        x = x.reshape(B, self.out_channels, self.group_size, T // ft, H // fs, W // fs)
        return x.mean(dim=2)


class DupUp3D(nn.Module):
    """Channel duplication followed by channel-to-space/time: the matching up-sampling shortcut."""

    def __init__(self, in_channels, out_channels, factor_t, factor_s=1):
        super().__init__()
        self.in_channels, self.out_channels, self.factor_t, self.factor_s = in_channels, out_channels, factor_t, factor_s
        self.factor = factor_t * factor_s * factor_s
        assert out_channels * self.factor % in_channels == 0
        self.repeats = out_channels * self.factor // in_channels

    def forward(self, x, first_chunk: bool = False):
        ft, fs = self.factor_t, self.factor_s
        x = x.repeat_interleave(self.repeats, dim=1)
        B, _, T, H, W = x.shape
        x = x.view(B, self.out_channels, ft, fs, fs, T, H, W).permute(0, 1, 5, 2, 6, 3, 7, 4)
        x = x.reshape(B, self.out_channels, T * ft, H * fs, W * fs)
        return x[:, :, ft - 1:] if first_chunk else x


class Down_ResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout, mult, temperal_downsample=False, down_flag=False):
        super().__init__()
        self.avg_shortcut = AvgDown3D(in_dim, out_dim, 2 if temperal_downsample else 1, 2 if down_flag else 1)
        mods: List[nn.Module] = []
        for _ in range(mult):
            mods.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if down_flag:
            mods.append(Resample(out_dim, mode="downsample3d" if temperal_downsample else "downsample2d"))
        self.downsamples = nn.Sequential(*mods)

    def forward(self, x, state: Optional[StreamState] = None):
        h = x
        for m in self.downsamples:
            h = m(h, state)
        return h + self.avg_shortcut(x)


class Up_ResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout, mult, temperal_upsample=False, up_flag=False):
        super().__init__()
        self.avg_shortcut = DupUp3D(in_dim, out_dim, 2 if temperal_upsample else 1, 2) if up_flag else None
        self.temporal = temperal_upsample and up_flag
        mods: List[nn.Module] = []
        for _ in range(mult):
            mods.append(ResidualBlock(in_dim, out_dim, dropout))
            in_dim = out_dim
        if up_flag:
            mods.append(Resample(out_dim, mode="upsample3d" if temperal_upsample else "upsample2d"))
        self.upsamples = nn.Sequential(*mods)

    def forward(self, x, state: Optional[StreamState] = None):
        first = state is not None and self.temporal and state.get(self) is None
        if state is not None and self.temporal:
            state.set(self, True)
        h = x
        for m in self.upsamples:
            h = m(h, state)
        if self.avg_shortcut is None:
            return h
        return h + self.avg_shortcut(x, first_chunk=first)


class Encoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(), temperal_downsample=(False, True, True),
                 dropout=0.0):
        super().__init__()
        dims = [dim * u for u in [1] + list(dim_mult)]
        self.conv1 = CausalConv3d(12, dims[0], 3, padding=1)
        groups = []
        out_dim = dims[0]
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            t_down = temperal_downsample[i] if i < len(temperal_downsample) else False
            groups.append(Down_ResidualBlock(in_dim, out_dim, dropout, num_res_blocks, t_down, i != len(dim_mult) - 1))
        self.downsamples = nn.Sequential(*groups)
        self.middle = nn.Sequential(ResidualBlock(out_dim, out_dim, dropout), AttentionBlock(out_dim), ResidualBlock(out_dim, out_dim, dropout))
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, z_dim, 3, padding=1))

    def forward(self, x, state: Optional[StreamState] = None):
        x = self.conv1.stream(x, state)
        for g in self.downsamples:
            x = g(x, state)
        for m in self.middle:
            x = m(x, state)
        for m in self.head:
            x = m.stream(x, state) if isinstance(m, CausalConv3d) else m(x)
        return x


class Decoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(), temperal_upsample=(True, True, False),
                 dropout=0.0):
        super().__init__()
        dim_mult = list(dim_mult)
        dims = [dim * u for u in [dim_mult[-1]] + dim_mult[::-1]]
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]), ResidualBlock(dims[0], dims[0], dropout))
        groups = []
        out_dim = dims[0]
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            t_up = temperal_upsample[i] if i < len(temperal_upsample) else False
            groups.append(Up_ResidualBlock(in_dim, out_dim, dropout, num_res_blocks + 1, t_up, i != len(dim_mult) - 1))
        self.upsamples = nn.Sequential(*groups)
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, 12, 3, padding=1))

    def forward(self, x, state: Optional[StreamState] = None):
        x = self.conv1.stream(x, state)
        for m in self.middle:
            x = m(x, state)
        for g in self.upsamples:
            x = g(x, state)
        for m in self.head:
            x = m.stream(x, state) if isinstance(m, CausalConv3d) else m(x)
        return x


class _Resample22(Resample):
    """The 2.2 up-samplers keep their channel count (the 2.1 ones halve it)."""

    def __init__(self, dim, mode):
        super().__init__(dim, mode)
        if mode in ("upsample2d", "upsample3d"):
            self.resample[1] = nn.Conv2d(dim, dim, 3, padding=1)


def _use_22_resamplers(module: nn.Module):
    for name, child in list(module.named_children()):
        if type(child) is Resample and child.mode in ("upsample2d", "upsample3d"):
            setattr(module, name, _Resample22(child.dim, child.mode))
        else:
            _use_22_resamplers(child)


class Wan22VAE_(nn.Module):
    def __init__(self, dim=160, dec_dim=256, z_dim=48, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout=0.0, temporal_window=4):
        super().__init__()
        self.z_dim, self.temporal_window = z_dim, temporal_window
        td = list(temperal_downsample)
        self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, attn_scales, td, dropout)
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder3d(dec_dim, z_dim, dim_mult, num_res_blocks, attn_scales, td[::-1], dropout)
        _use_22_resamplers(self.decoder)

    def _scale(self, t, like):
        return t.view(1, self.z_dim, 1, 1, 1).to(like) if isinstance(t, torch.Tensor) else t

    def encode(self, x, scale):
        st = StreamState()
        x = patchify(x, 2)
        t, tw = x.shape[2], self.temporal_window
        outs = [self.encoder(x[:, :, :1], st)]
        n_full = (t - 1) // tw
        for i in range(n_full):
            outs.append(self.encoder(x[:, :, 1 + tw * i: 1 + tw * (i + 1)], st))
        if (t - 1) % tw:
            outs.append(self.encoder(x[:, :, 1 + tw * n_full:], st))
        mu, _ = self.conv1(torch.cat(outs, 2)).chunk(2, dim=1)
        return (mu - self._scale(scale[0], mu)) * self._scale(scale[1], mu)

    def decode(self, z, scale):
        st = StreamState()
        z = z / self._scale(scale[1], z) + self._scale(scale[0], z)
        x = self.conv2(z)
        out = torch.cat([self.decoder(x[:, :, i: i + 1], st) for i in range(z.shape[2])], 2)
        return unpatchify(out, 2)

    def forward(self, x, scale=(0.0, 1.0)):
        mu = self.encode(x, scale)
        return self.decode(mu, scale), mu


class Wan2pt2VAEInterface(VideoTokenizerInterface):
    def __init__(self, chunk_duration: int = 93, vae_pth: Optional[str] = None, device="cuda", dtype=torch.bfloat16,
                 temporal_window: int = 4, dim: int = 160, dec_dim: int = 256, **_unused):
        self.device, self.dtype_, self.chunk_duration = torch.device(device), dtype, chunk_duration
        self.model = Wan22VAE_(dim=dim, dec_dim=dec_dim, z_dim=48, temporal_window=temporal_window).eval().requires_grad_(False)
        if vae_pth:
            self.model.load_state_dict(torch.load(vae_pth, map_location="cpu", weights_only=False), strict=True)
        self.model.to(self.device, dtype)
        self.scale = [torch.tensor(WAN22_LATENT_MEAN, dtype=dtype, device=self.device),
                      1.0 / torch.tensor(WAN22_LATENT_STD, dtype=dtype, device=self.device)]

    @property
    def dtype(self):
        return self.dtype_

    def reset_dtype(self):
        pass

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        return self.model.encode(state.to(self.device, self.dtype_), self.scale)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        return self.model.decode(latent.to(self.device, self.dtype_), self.scale)

    def get_latent_num_frames(self, num_pixel_frames: int) -> int:
        return 1 + (num_pixel_frames - 1) // 4

    def get_pixel_num_frames(self, num_latent_frames: int) -> int:
        return (num_latent_frames - 1) * 4 + 1

    spatial_compression_factor = 16
    temporal_compression_factor = 4
    latent_ch = 48
    spatial_resolution = "720"

    @property
    def pixel_chunk_duration(self):
        return self.chunk_duration

    @property
    def latent_chunk_duration(self):
        return self.get_latent_num_frames(self.chunk_duration)

    @property
    def name(self):
        return "wan2pt2_tokenizer"
