"""Wan2.1 causal 3-D convolutional VAE (16 latent channels, 8x8 spatial / 4x temporal compression) and the
video-tokenizer interface built on it.

Parity targets: ``CausalConv3d`` / ``RMS_norm`` / ``Resample`` / ``ResidualBlock`` / ``AttentionBlock`` /
``Encoder3d`` / ``Decoder3d`` / ``WanVAE_`` / ``WanVAE`` / ``Wan2pt1VAEInterface``
(cosmos_predict2/_src/predict2/tokenizers/wan2pt1.py:40-928) and ``VideoTokenizerInterface``
(cosmos_predict2/_src/predict2/tokenizers/interface.py:25-98). Parameter names match the reference
checkpoint (``encoder.downsamples.3.residual.2.weight``, ``decoder.upsamples.7.time_conv.weight`` ...).

Streaming semantics that must be preserved: the encoder consumes 1 + k*temporal_window pixel frames per
chunk, the decoder one latent frame per step; every causal convolution carries the last two input frames of
the previous chunk; the first latent frame decodes to one pixel frame and each later one to four (the
temporal up-sampler is skipped on the first chunk); encode is deterministic (mu only) with per-channel
(mu - mean) / std scaling.

The streaming state is an explicit ``StreamState`` object keyed by module instead of a positional list that
is threaded through every forward call. On a GPU, bf16 decodes of one video run channels-last on this package's
implicit-GEMM convolution kernel (``vae_wan_cl.DecoderCL``); the module tree below is the definition, the CPU / fp32 path and
the row-sharded path, with convolutions on cuDNN through torch. Under
``vae_parallel.row_sharded`` the decoder works on a horizontal band of the frame per rank and swaps boundary
rows with its neighbours (``Wan2pt1VAEInterface.decode_parallel``).
"""

from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import vae_parallel

CACHE_T = 2

WAN21_LATENT_MEAN = [-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
                     0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921]
WAN21_LATENT_STD = [2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
                    3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160]


class StreamState:
    """Per-module carry-over between chunks of one video. ``FIRST`` marks a temporal up-sampler that has seen
    its first chunk (which it passes through unchanged)."""

    FIRST = "first-chunk-passed"

    def __init__(self):
        self.store: Dict[int, object] = {}

    def get(self, mod):
        return self.store.get(id(mod))

    def set(self, mod, value):
        self.store[id(mod)] = value


def _tail(x: torch.Tensor, prev) -> torch.Tensor:
    """Last CACHE_T frames of the stream ending with chunk ``x`` (borrowing one frame from ``prev``)."""
    c = x[:, :, -CACHE_T:].clone()
    if c.shape[2] < CACHE_T and isinstance(prev, torch.Tensor):
        c = torch.cat([prev[:, :, -1:].to(c.device), c], dim=2)
    return c


class CausalConv3d(nn.Conv3d):
    """Conv3d padded on the past side of time only; a cache of earlier frames replaces (part of) the padding."""

    def __init__(self, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self._pad = (self.padding[2], self.padding[2], self.padding[1], self.padding[1], 2 * self.padding[0], 0)
        self.padding = (0, 0, 0)

    def forward(self, x, cache_x: Optional[torch.Tensor] = None):
        pad = list(self._pad)
        if cache_x is not None and pad[4] > 0:
            x = torch.cat([cache_x.to(x.device, x.dtype), x], dim=2)
            pad[4] -= cache_x.shape[2]
        if pad[2] > 0 and vae_parallel.active() is not None:
            # row-sharded decode: the neighbours' boundary rows stand in for the padding along H
            x = vae_parallel.exchange_rows(x, 3, pad[2])
            pad[2] = pad[3] = 0
        x = F.pad(x, pad)
        return super().forward(x)

    def stream(self, x, state: Optional[StreamState]):
        if state is None:
            return self(x)
        prev = state.get(self)
        new = _tail(x, prev)
        y = self(x, prev if isinstance(prev, torch.Tensor) else None)
        state.set(self, new)
        return y


class RMS_norm(nn.Module):
    """L2-normalise over channels, scale by sqrt(C) * gamma (+ bias)."""

    def __init__(self, dim, channel_first=True, images=True, bias=False):
        super().__init__()
        bdims = (1, 1, 1) if not images else (1, 1)
        shape = (dim, *bdims) if channel_first else (dim,)
        self.channel_first = channel_first
        self.scale = dim ** 0.5
        self.gamma = nn.Parameter(torch.ones(shape))
        self.bias = nn.Parameter(torch.zeros(shape)) if bias else 0.0

    def forward(self, x):
        return F.normalize(x, dim=(1 if self.channel_first else -1)) * self.scale * self.gamma + self.bias


class Upsample(nn.Upsample):
    def forward(self, x):
        return super().forward(x.float()).type_as(x)


class Resample(nn.Module):
    def __init__(self, dim, mode):
        assert mode in ("none", "upsample2d", "upsample3d", "downsample2d", "downsample3d")
        super().__init__()
        self.dim, self.mode = dim, mode
        if mode in ("upsample2d", "upsample3d"):
            self.resample = nn.Sequential(Upsample(scale_factor=(2.0, 2.0), mode="nearest-exact"),
                                          nn.Conv2d(dim, dim // 2, 3, padding=1))
            if mode == "upsample3d":
                self.time_conv = CausalConv3d(dim, dim * 2, (3, 1, 1), padding=(1, 0, 0))
        elif mode in ("downsample2d", "downsample3d"):
            self.resample = nn.Sequential(nn.ZeroPad2d((0, 1, 0, 1)), nn.Conv2d(dim, dim, 3, stride=(2, 2)))
            if mode == "downsample3d":
                self.time_conv = CausalConv3d(dim, dim, (3, 1, 1), stride=(2, 1, 1), padding=(0, 0, 0))
        else:
            self.resample = nn.Identity()

    def forward(self, x, state: Optional[StreamState] = None):
        b, c, t, h, w = x.shape
        if self.mode == "upsample3d" and state is not None:
            prev = state.get(self)
            if prev is None:
                state.set(self, StreamState.FIRST)  # first chunk: no temporal up-sampling
            else:
                cache = x[:, :, -CACHE_T:].clone()
                if cache.shape[2] < CACHE_T:
                    head = prev[:, :, -1:].to(cache.device) if isinstance(prev, torch.Tensor) else torch.zeros_like(cache)
                    cache = torch.cat([head, cache], dim=2)
                x = self.time_conv(x) if not isinstance(prev, torch.Tensor) else self.time_conv(x, prev)
                state.set(self, cache)
                x = x.reshape(b, 2, c, t, h, w)
                x = torch.stack((x[:, 0], x[:, 1]), 3).reshape(b, c, t * 2, h, w)
        t = x.shape[2]
        x = x.permute(0, 2, 1, 3, 4).reshape(b * t, x.shape[1], h, w)
        if vae_parallel.active() is not None and self.mode in ("upsample2d", "upsample3d"):
            conv = self.resample[1]
            x = vae_parallel.exchange_rows(self.resample[0](x), 2, 1)
            x = F.conv2d(x, conv.weight, conv.bias, padding=(0, 1))
        elif vae_parallel.active() is not None and self.mode in ("downsample2d", "downsample3d"):
            # stride-2 convolution padded on the bottom / right only: output row j reads input rows 2j .. 2j+2, so an even band
            # needs exactly one row of the next rank below it (zeros at the bottom of the frame)
            assert x.shape[2] % 2 == 0, "row bands must keep an even height through every down-sampling stage"
            conv = self.resample[1]
            x = vae_parallel.exchange_rows(x, 2, 1, top=False)
            x = F.conv2d(F.pad(x, (0, 1, 0, 0)), conv.weight, conv.bias, stride=2)
        else:
            x = self.resample(x)
        x = x.reshape(b, t, *x.shape[1:]).permute(0, 2, 1, 3, 4)
        if self.mode == "downsample3d" and state is not None:
            prev = state.get(self)
            if prev is None:
                state.set(self, x.clone())
            else:
                cache = x[:, :, -1:].clone()
                x = self.time_conv(torch.cat([prev[:, :, -1:], x], 2))
                state.set(self, cache)
        return x


class ResidualBlock(nn.Module):
    def __init__(self, in_dim, out_dim, dropout=0.0):
        super().__init__()
        self.in_dim, self.out_dim = in_dim, out_dim
        self.residual = nn.Sequential(
            RMS_norm(in_dim, images=False), nn.SiLU(), CausalConv3d(in_dim, out_dim, 3, padding=1),
            RMS_norm(out_dim, images=False), nn.SiLU(), nn.Dropout(dropout), CausalConv3d(out_dim, out_dim, 3, padding=1))
        self.shortcut = CausalConv3d(in_dim, out_dim, 1) if in_dim != out_dim else nn.Identity()

    def forward(self, x, state: Optional[StreamState] = None):
        h = self.shortcut(x)
        for layer in self.residual:
            x = layer.stream(x, state) if isinstance(layer, CausalConv3d) else layer(x)
        return x + h


class AttentionBlock(nn.Module):
    """Single-head spatial self-attention applied to every frame independently."""

    def __init__(self, dim):
        super().__init__()
        self.dim = dim
        self.norm = RMS_norm(dim)
        self.to_qkv = nn.Conv2d(dim, dim * 3, 1)
        self.proj = nn.Conv2d(dim, dim, 1)
        nn.init.zeros_(self.proj.weight)

    def forward(self, x, state=None):
        identity = x
        b, c, t, h, w = x.shape
        y = x.permute(0, 2, 1, 3, 4).reshape(b * t, c, h, w)
        y = self.norm(y)
        q, k, v = self.to_qkv(y).reshape(b * t, 1, c * 3, -1).permute(0, 1, 3, 2).contiguous().chunk(3, dim=-1)
        if vae_parallel.active() is not None:  # local rows attend to the whole frame
            k, v = vae_parallel.gather_tokens(k, 2), vae_parallel.gather_tokens(v, 2)
        y = F.scaled_dot_product_attention(q, k, v)
        y = y.squeeze(1).permute(0, 2, 1).reshape(b * t, c, h, w)
        y = self.proj(y)
        y = y.reshape(b, t, c, h, w).permute(0, 2, 1, 3, 4)
        return y + identity


class Encoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(True, True, False), dropout=0.0):
        super().__init__()
        dims = [dim * u for u in [1] + list(dim_mult)]
        scale = 1.0
        self.conv1 = CausalConv3d(3, dims[0], 3, padding=1)
        downs: List[nn.Module] = []
        out_dim = dims[0]
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            for _ in range(num_res_blocks):
                downs.append(ResidualBlock(in_dim, out_dim, dropout))
                if scale in attn_scales:
                    downs.append(AttentionBlock(out_dim))
                in_dim = out_dim
            if i != len(dim_mult) - 1:
                downs.append(Resample(out_dim, mode="downsample3d" if temperal_downsample[i] else "downsample2d"))
                scale /= 2.0
        self.downsamples = nn.Sequential(*downs)
        self.middle = nn.Sequential(ResidualBlock(out_dim, out_dim, dropout), AttentionBlock(out_dim),
                                    ResidualBlock(out_dim, out_dim, dropout))
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, z_dim, 3, padding=1))

    def forward(self, x, state: Optional[StreamState] = None):
        x = self.conv1.stream(x, state)
        for layer in self.downsamples:
            x = layer(x, state)
        for layer in self.middle:
            x = layer(x, state)
        for layer in self.head:
            x = layer.stream(x, state) if isinstance(layer, CausalConv3d) else layer(x)
        return x


class Decoder3d(nn.Module):
    def __init__(self, dim=128, z_dim=4, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_upsample=(False, True, True), dropout=0.0):
        super().__init__()
        dim_mult = list(dim_mult)
        dims = [dim * u for u in [dim_mult[-1]] + dim_mult[::-1]]
        scale = 1.0 / 2 ** (len(dim_mult) - 2)
        self.conv1 = CausalConv3d(z_dim, dims[0], 3, padding=1)
        self.middle = nn.Sequential(ResidualBlock(dims[0], dims[0], dropout), AttentionBlock(dims[0]),
                                    ResidualBlock(dims[0], dims[0], dropout))
        ups: List[nn.Module] = []
        out_dim = dims[0]
        for i, (in_dim, out_dim) in enumerate(zip(dims[:-1], dims[1:])):
            if i in (1, 2, 3):
                in_dim = in_dim // 2
            for _ in range(num_res_blocks + 1):
                ups.append(ResidualBlock(in_dim, out_dim, dropout))
                if scale in attn_scales:
                    ups.append(AttentionBlock(out_dim))
                in_dim = out_dim
            if i != len(dim_mult) - 1:
                ups.append(Resample(out_dim, mode="upsample3d" if temperal_upsample[i] else "upsample2d"))
                scale *= 2.0
        self.upsamples = nn.Sequential(*ups)
        self.head = nn.Sequential(RMS_norm(out_dim, images=False), nn.SiLU(), CausalConv3d(out_dim, 3, 3, padding=1))

    def forward(self, x, state: Optional[StreamState] = None):
        x = self.conv1.stream(x, state)
        for layer in self.middle:
            x = layer(x, state)
        for layer in self.upsamples:
            x = layer(x, state)
        for layer in self.head:
            x = layer.stream(x, state) if isinstance(layer, CausalConv3d) else layer(x)
        return x


class WanVAE_(nn.Module):
    def __init__(self, dim=96, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=2, attn_scales=(),
                 temperal_downsample=(False, True, True), dropout=0.0, temporal_window=4):
        super().__init__()
        self.dim, self.z_dim = dim, z_dim
        self.temporal_window = temporal_window
        self.temperal_downsample = list(temperal_downsample)
        self.temperal_upsample = self.temperal_downsample[::-1]
        self.encoder = Encoder3d(dim, z_dim * 2, dim_mult, num_res_blocks, attn_scales, self.temperal_downsample, dropout)
        self.conv1 = CausalConv3d(z_dim * 2, z_dim * 2, 1)
        self.conv2 = CausalConv3d(z_dim, z_dim, 1)
        self.decoder = Decoder3d(dim, z_dim, dim_mult, num_res_blocks, attn_scales, self.temperal_upsample, dropout)
        self._enc_state: Optional[StreamState] = None
        self._dec_state: Optional[StreamState] = None

    def clear_cache(self):
        self._enc_state = None
        self._dec_state = None

    def encode(self, x, scale, clear_encoder_cache: bool = True):
        """x [B,3,T,H,W] in [-1,1] with T = 1 + 4k -> mu [B,z,1+k,H/8,W/8], normalised per channel."""
        if clear_encoder_cache or self._enc_state is None:
            self._enc_state = StreamState()
        st = self._enc_state
        t = x.shape[2]
        tw = self.temporal_window
        cl = self._kernel_encoder(x)
        if cl is not None:
            # channels-last encoder on this package's convolution kernel; it keeps its own stream state
            if clear_encoder_cache or cl.state is None:
                cl.reset()
            run = cl.step
        else:
            run = lambda chunk: self.encoder(chunk, st)
        outs = [run(x[:, :, :1])]
        n_full = (t - 1) // tw
        for i in range(n_full):
            outs.append(run(x[:, :, 1 + tw * i: 1 + tw * (i + 1)]))
        if (t - 1) % tw:
            outs.append(run(x[:, :, 1 + tw * n_full:]))
        if cl is not None and clear_encoder_cache:
            cl.state = None
        out = torch.cat(outs, 2)
        mu, _log_var = self.conv1(out).chunk(2, dim=1)
        mean, inv_std = scale
        if isinstance(mean, torch.Tensor):
            mu = (mu - mean.view(1, self.z_dim, 1, 1, 1).to(mu)) * inv_std.view(1, self.z_dim, 1, 1, 1).to(mu)
        else:
            mu = (mu - mean) * inv_std
        if clear_encoder_cache:
            self._enc_state = None
        return mu

    def decode(self, z, scale, clear_decoder_cache: bool = True):
        """z [B,z,T',h,w] -> pixels [B,3,1+4(T'-1),8h,8w], one latent frame per step."""
        if clear_decoder_cache or self._dec_state is None:
            self._dec_state = StreamState()
        st = self._dec_state
        mean, inv_std = scale
        if isinstance(mean, torch.Tensor):
            z = z / inv_std.view(1, self.z_dim, 1, 1, 1).to(z) + mean.view(1, self.z_dim, 1, 1, 1).to(z)
        else:
            z = z / inv_std + mean
        x = self.conv2(z)
        cl = self._kernel_decoder(x)
        if cl is not None:
            # channels-last decoder on this package's convolution kernel; it keeps its own stream state
            if clear_decoder_cache or cl.state is None:
                cl.reset()
            outs = [cl.step(x[:, :, i: i + 1]) for i in range(z.shape[2])]
            if clear_decoder_cache:
                cl.state = None
                self._dec_state = None
            return torch.cat(outs, 2)
        outs = [self.decoder(x[:, :, i: i + 1], st) for i in range(z.shape[2])]
        if clear_decoder_cache:
            self._dec_state = None
        return torch.cat(outs, 2)

    def _kernel_encoder(self, x):
        """The channels-last kernel encoder for this input, or None when the torch / cuDNN path has to serve it."""
        from ..ops import functional as F_ops
        from . import vae_wan_cl
        if F_ops.settings.conv != "native" or not vae_wan_cl.encoder_supported(x):
            return None
        sig = tuple((p.data_ptr(), p._version) for p in self.encoder.parameters())
        if getattr(self, "_enc_cl", None) is None or self._enc_cl_sig != sig:
            self._enc_cl = vae_wan_cl.EncoderCL(self.encoder, x.device)
            self._enc_cl_sig = sig
        return self._enc_cl

    def _kernel_decoder(self, x):
        """The channels-last kernel decoder for this input, or None when the torch / cuDNN path has to serve it (CPU tensors,
        fp32, batches, ``settings.conv == "cudnn"``). Weights are repacked when they change."""
        from ..ops import functional as F_ops
        from . import vae_wan_cl
        if F_ops.settings.conv != "native" or not vae_wan_cl.supported(self.decoder, x):
            return None
        sig = tuple((p.data_ptr(), p._version) for p in self.decoder.parameters())
        if getattr(self, "_dec_cl", None) is None or self._dec_cl_sig != sig:
            self._dec_cl = vae_wan_cl.DecoderCL(self.decoder, x.device)
            self._dec_cl_sig = sig
        return self._dec_cl

    def forward(self, x, scale=(0.0, 1.0)):
        mu = self.encode(x, scale)
        return self.decode(mu, scale), mu


class VideoTokenizerInterface:
    """What a model needs from a tokenizer: encode/decode and the frame / resolution arithmetic."""

    def reset_dtype(self):
        pass

    def encode(self, state: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def get_latent_num_frames(self, num_pixel_frames: int) -> int:
        raise NotImplementedError

    def get_pixel_num_frames(self, num_latent_frames: int) -> int:
        raise NotImplementedError

    spatial_compression_factor = 8
    temporal_compression_factor = 4
    spatial_resolution = 512
    latent_ch = 16
    is_chunk_overlap = False
    is_causal = True


class Wan2pt1VAEInterface(VideoTokenizerInterface):
    """bf16 Wan2.1 VAE as a tokenizer: ``encode`` pixels [-1,1] -> normalised latents, ``decode`` back."""

    def __init__(self, chunk_duration: int = 81, vae_pth: Optional[str] = None, device="cuda", dtype=torch.bfloat16,
                 temporal_window: int = 4, keep_decoder_cache: bool = False, keep_encoder_cache: bool = False,
                 load_mean_std: bool = False, dim: int = 96, **_unused):
        self.device = torch.device(device)
        self.dtype_ = dtype
        self.chunk_duration = chunk_duration
        self.keep_decoder_cache = keep_decoder_cache
        self.keep_encoder_cache = keep_encoder_cache
        self.model = WanVAE_(dim=dim, z_dim=16, temporal_window=temporal_window).eval().requires_grad_(False)
        if vae_pth:
            sd = torch.load(vae_pth, map_location="cpu", weights_only=False)
            self.model.load_state_dict(sd, strict=True)
        self.model.to(device=self.device, dtype=dtype)
        mean = torch.tensor(WAN21_LATENT_MEAN, dtype=dtype, device=self.device)
        std = torch.tensor(WAN21_LATENT_STD, dtype=dtype, device=self.device)
        self.scale = [mean, 1.0 / std]
        # optional dataset-level statistics; identity unless load_mean_std
        self.img_mean = torch.zeros(1, 16, 1, 1, 1, device=self.device, dtype=dtype)
        self.img_std = torch.ones(1, 16, 1, 1, 1, device=self.device, dtype=dtype)
        self.video_mean = torch.zeros(1, 16, 32, 1, 1, device=self.device, dtype=dtype)
        self.video_std = torch.ones(1, 16, 32, 1, 1, device=self.device, dtype=dtype)

    @property
    def dtype(self):
        return self.dtype_

    def clear_cache(self):
        self.model.clear_cache()

    def count_param(self) -> int:
        return sum(p.numel() for p in self.model.parameters())

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        lat = self.model.encode(state.to(self.device, self.dtype_), self.scale, clear_encoder_cache=not self.keep_encoder_cache)
        n = lat.shape[2]
        if n == 1:
            return (lat - self.img_mean.type_as(lat)) / self.img_std.type_as(lat)
        if n <= self.video_mean.shape[2]:
            return (lat - self.video_mean[:, :, :n].type_as(lat)) / self.video_std[:, :, :n].type_as(lat)
        return lat

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        n = latent.shape[2]
        latent = latent.to(self.device, self.dtype_)
        if n == 1:
            latent = latent * self.img_std.type_as(latent) + self.img_mean.type_as(latent)
        elif n <= self.video_mean.shape[2]:
            latent = latent * self.video_std[:, :, :n].type_as(latent) + self.video_mean[:, :, :n].type_as(latent)
        return self.model.decode(latent, self.scale, clear_decoder_cache=not self.keep_decoder_cache)

    @torch.no_grad()
    def decode_parallel(self, latent: torch.Tensor, group, dst: Optional[int] = None) -> Optional[torch.Tensor]:
        """``decode`` with the frame split into horizontal bands over ``group`` (every rank passes the same latent).
        Exact: neighbours exchange boundary rows before every spatial convolution. Falls back to ``decode`` when
        the latent rows do not divide over the group. With ``dst`` only that rank of the group gets the video."""
        if not vae_parallel.can_shard(latent.shape[3], group):
            return self.decode(latent)
        return vae_parallel.decode_row_sharded(self.decode, latent, group, dst)

    @torch.no_grad()
    def encode_parallel(self, state: torch.Tensor, group) -> torch.Tensor:
        """``encode`` with the frame split into horizontal bands over ``group`` (every rank passes the same video); exact.
        Falls back to ``encode`` when the pixel rows do not divide into bands of a multiple of 8 rows."""
        import torch.distributed as dist
        ok = group is not None and dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1 \
            and state.shape[3] % (8 * dist.get_world_size(group)) == 0
        if not ok:
            return self.encode(state)
        return vae_parallel.encode_row_sharded(self.encode, state, group)

    def get_latent_num_frames(self, num_pixel_frames: int) -> int:
        return 1 + (num_pixel_frames - 1) // 4

    def get_pixel_num_frames(self, num_latent_frames: int) -> int:
        return (num_latent_frames - 1) * 4 + 1

    @property
    def pixel_chunk_duration(self):
        return self.chunk_duration

    @property
    def latent_chunk_duration(self):
        return self.get_latent_num_frames(self.chunk_duration)

    @property
    def name(self):
        return "wan2pt1_tokenizer"


class DummyTokenizer(VideoTokenizerInterface):
    """Parameter-free stand-in with the Wan compression ratios (tests and synthetic-data runs): average pooling
    to 16 channels on encode, nearest up-sampling on decode."""

    def __init__(self, latent_ch: int = 16, spatial: int = 8, temporal: int = 4):
        self.latent_ch = latent_ch
        self.spatial_compression_factor = spatial
        self.temporal_compression_factor = temporal

    def get_latent_num_frames(self, n: int) -> int:
        return 1 + (n - 1) // self.temporal_compression_factor

    def get_pixel_num_frames(self, n: int) -> int:
        return (n - 1) * self.temporal_compression_factor + 1

    def encode(self, x: torch.Tensor) -> torch.Tensor:
        B, C, T, H, W = x.shape
        s, tc = self.spatial_compression_factor, self.temporal_compression_factor
        first = F.avg_pool2d(x[:, :, 0], s)
        parts = [first.unsqueeze(2)]
        if T > 1:
            rest = x[:, :, 1:]
            Tr = (T - 1) // tc
            rest = rest[:, :, : Tr * tc].reshape(B, C, Tr, tc, H, W).mean(3)
            parts.append(F.avg_pool3d(rest, (1, s, s)))
        lat = torch.cat(parts, 2)
        reps = (self.latent_ch + C - 1) // C
        return lat.repeat(1, reps, 1, 1, 1)[:, : self.latent_ch]

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        s, tc = self.spatial_compression_factor, self.temporal_compression_factor
        x = z[:, :3]
        first = F.interpolate(x[:, :, 0], scale_factor=s, mode="nearest").unsqueeze(2)
        if x.shape[2] == 1:
            return first
        rest = F.interpolate(x[:, :, 1:], scale_factor=(tc, s, s), mode="nearest")
        return torch.cat([first, rest], 2)
