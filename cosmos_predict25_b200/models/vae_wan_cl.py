"""Channels-last decoder of the Wan2.1 VAE on the implicit-GEMM convolution kernel (``ops/csrc/conv3d_cl.cu``).

``DecoderCL`` takes the weights of a ``vae_wan.Decoder3d`` and runs the same streaming decode - one latent frame per step,
every causal convolution carrying the last two input frames of the previous step, the temporal up-sampler skipped on the first
step (cosmos_predict2/_src/predict2/tokenizers/wan2pt1.py:40-58, 84-137, 184-215, 358-462, 543-562) - with activations kept as
``[T, H, W, C]`` bf16 tensors throughout:

  * every convolution is one launch of ``conv_cl`` (TMA boxes shifted by the tap are the im2col; out-of-range boxes are the zero
    padding; bias and the residual add of a block are its epilogue);
  * "nearest 2x up-sampling + 3 x 3 convolution" is computed as four 2 x 2 phase convolutions on the low-resolution frame with
    pre-summed weights: output pixel (2y + a, 2x + b) only ever sees a 2 x 2 neighbourhood of the input, so 4 taps replace 9 and
    the up-sampled frame is never materialised; the phases interleave through the kernel's output mapping;
  * the temporal up-sampler's channel-to-frame interleave is an output mapping too (two launches, one per output-channel half);
  * RMS-norm + SiLU in front of a convolution is one element-wise kernel.

The single-head frame attention of the middle block keeps torch's attention (head dimension 384) with its 1 x 1 projections on
this package's GEMM. Weights are repacked once (``[C_out, taps, C_in padded to 64]`` bf16, fp32 bias) when the object is built.
"""

from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from ..ops import functional as F_ops
from ..ops import native
from . import vae_parallel

CACHE_T = 2


def _n_tile(cout: int) -> int:
    if cout <= 256:
        return (cout + 15) // 16 * 16
    for t in (192, 256, 128):
        if cout % t == 0:
            return t
    return 256


class ConvCL:
    """One convolution with repacked weights. ``taps``: (dt, dh, dw) offsets added to an output coordinate to get the input
    coordinate; ``weight_taps``: [C_out, n_taps, C_in] fp32/bf16 in the same order."""

    def __init__(self, weight_taps: torch.Tensor, bias: Optional[torch.Tensor], taps: Sequence[Tuple[int, int, int]], device):
        cout, ntaps, cin = weight_taps.shape
        assert ntaps == len(taps) and cin % 16 == 0, (weight_taps.shape, len(taps))
        self.cout, self.cin, self.n_tile = cout, cin, _n_tile(cout)
        rows = (cout + self.n_tile - 1) // self.n_tile * self.n_tile
        cpad = (cin + 63) // 64 * 64
        w = torch.zeros(rows, ntaps, cpad, dtype=torch.bfloat16, device=device)
        w[:cout, :, :cin] = weight_taps.to(device=device, dtype=torch.bfloat16)
        self.w = w.view(rows, ntaps * cpad).contiguous()
        self.bias = bias.detach().to(device=device, dtype=torch.float32).contiguous() if bias is not None else None
        self.taps = [int(v) for t in taps for v in t]
        self.spatial = any(t[1] != 0 for t in taps)            # reads neighbouring rows: needs halo rows under row sharding
        self.taps_halo = [int(v) for t in taps for v in (t[0], t[1] + 1, t[2])]

    def __call__(self, x: torch.Tensor, t_out: int, out: Optional[torch.Tensor] = None, out_map: Optional[List[int]] = None,
                 resid: Optional[torch.Tensor] = None, h_out: Optional[int] = None, w_out: Optional[int] = None) -> torch.Tensor:
        """x [T_in, H, W, C_in]. Default output: a new [t_out, H, W, C_out] tensor with the identity mapping. Under row-sharded
        decoding (``vae_parallel.row_sharded``) a convolution that reads neighbouring rows first receives one boundary row from
        each neighbouring rank (zeros at the frame border) and reads its input shifted by that row."""
        _, H, W, _ = x.shape
        h_out, w_out = h_out or H, w_out or W
        taps = self.taps
        if self.spatial and vae_parallel.active() is not None:
            x = vae_parallel.exchange_rows(x, 1, 1)
            taps = self.taps_halo
        if out is None:
            out = torch.empty(t_out, h_out, w_out, self.cout, dtype=torch.bfloat16, device=x.device)
        if out_map is None:
            out_map = [1, 0, 1, 0, 1, 0, out.shape[1], out.shape[2], out.shape[3], 0]
        native.load().conv_cl(x, self.w, self.n_tile, self.cout, taps, t_out, h_out, w_out, out_map, out, resid, self.bias)
        native.count_launch()
        return out


def _causal3_taps(kt: int, kh: int, kw: int):
    """Taps of a causal convolution whose input tensor starts with the (kt - 1) frames of temporal padding / stream cache."""
    return [(it, ih - kh // 2, iw - kw // 2) for it in range(kt) for ih in range(kh) for iw in range(kw)]


def _conv3d(mod, device) -> ConvCL:
    w = mod.weight.detach().float()                      # [Cout, Cin, kt, kh, kw]
    cout, cin, kt, kh, kw = w.shape
    wt = w.permute(0, 2, 3, 4, 1).reshape(cout, kt * kh * kw, cin)
    return ConvCL(wt, mod.bias, _causal3_taps(kt, kh, kw), device)


def _upsample_conv2d_phases(conv2d, device) -> List[Tuple[ConvCL, int, int]]:
    """The four phase convolutions of nearest-2x + ``conv2d`` (3 x 3, padding 1). Phase (a, b) produces output pixels
    (2y + a, 2x + b) from input pixels (y + u - 1 + a, x + v - 1 + b), u, v in {0, 1}; rows of the 3 x 3 kernel that read the
    same input row are summed (a = 0: {0}, {1, 2}; a = 1: {0, 1}, {2})."""
    w = conv2d.weight.detach().float()                   # [Cout, Cin, 3, 3]
    groups = {0: ([0], [1, 2]), 1: ([0, 1], [2])}
    phases = []
    for a in (0, 1):
        for b in (0, 1):
            taps, mats = [], []
            for u in (0, 1):
                for v in (0, 1):
                    m = sum(w[:, :, i, j] for i in groups[a][u] for j in groups[b][v])   # [Cout, Cin]
                    mats.append(m)
                    taps.append((0, u - 1 + a, v - 1 + b))
            phases.append((ConvCL(torch.stack(mats, 1), conv2d.bias, taps, device), a, b))
    return phases


class _Stream:
    """Last two input frames of every causal convolution (keyed by the ConvCL object)."""

    def __init__(self):
        self.store = {}


def _with_cache(conv: ConvCL, x: torch.Tensor, state: _Stream, pad_frames: int = CACHE_T) -> torch.Tensor:
    """[cache | x] along time and the cache update: the convolution's input tensor with its causal padding in front."""
    prev = state.store.get(id(conv))
    if prev is None:
        prev = x.new_zeros(pad_frames, *x.shape[1:])
    full = torch.cat([prev, x], 0)
    state.store[id(conv)] = full[-pad_frames:].clone()
    return full


class _ResBlockCL:
    def __init__(self, block, device):
        res = block.residual
        self.g1 = res[0].gamma.detach().float().reshape(-1).to(device).contiguous()
        self.c1 = _conv3d(res[2], device)
        self.g2 = res[3].gamma.detach().float().reshape(-1).to(device).contiguous()
        self.c2 = _conv3d(res[6], device)
        self.short = _conv3d(block.shortcut, device) if not isinstance(block.shortcut, torch.nn.Identity) else None

    def __call__(self, x, state):
        ops = native.load()
        T = x.shape[0]
        h = self.short(x, T) if self.short is not None else x
        y = ops.rmsnorm_silu_cl(x, self.g1, True)
        y = self.c1(_with_cache(self.c1, y, state), T)
        y = ops.rmsnorm_silu_cl(y, self.g2, True)
        native.count_launch(2)
        return self.c2(_with_cache(self.c2, y, state), T, resid=h)


class _AttnCL:
    def __init__(self, block, device):
        C = block.dim
        self.C = C
        self.gamma = block.norm.gamma.detach().float().reshape(-1).to(device).contiguous()
        self.w_qkv = block.to_qkv.weight.detach().reshape(3 * C, C).to(device=device, dtype=torch.bfloat16).contiguous()
        self.b_qkv = block.to_qkv.bias.detach().to(device=device, dtype=torch.bfloat16).contiguous()
        self.w_proj = block.proj.weight.detach().reshape(C, C).to(device=device, dtype=torch.bfloat16).contiguous()
        self.b_proj = block.proj.bias.detach().to(device=device, dtype=torch.bfloat16).contiguous()

    def __call__(self, x, state):
        T, H, W, C = x.shape
        y = native.load().rmsnorm_silu_cl(x, self.gamma, False)
        native.count_launch()
        qkv = F_ops.linear(y.view(T * H * W, C), self.w_qkv, self.b_qkv).view(T, H * W, 3, C)
        q, k, v = (qkv[:, :, i].unsqueeze(1) for i in range(3))          # [T, 1, HW, C]
        if vae_parallel.active() is not None:                             # local rows attend to the whole frame
            k, v = vae_parallel.gather_tokens(k.contiguous(), 2), vae_parallel.gather_tokens(v.contiguous(), 2)
        o = F.scaled_dot_product_attention(q, k, v)                       # single head of dimension C
        o = F_ops.linear(o.squeeze(1).reshape(T * H * W, C), self.w_proj, self.b_proj)
        return o.view(T, H, W, C) + x


class _UpsampleCL:
    def __init__(self, mod, device):
        self.mode = mod.mode
        self.dim = mod.dim
        self.phases = _upsample_conv2d_phases(mod.resample[1], device)
        self.time = None
        if mod.mode == "upsample3d":
            w = mod.time_conv.weight.detach().float()        # [2C, C, 3, 1, 1]
            C = mod.dim
            b = mod.time_conv.bias
            self.time = []
            for s in (0, 1):                                 # output-channel half s becomes frame 2t + s
                wt = w[s * C:(s + 1) * C, :, :, 0, 0].permute(0, 2, 1).contiguous()   # [C, 3, C]
                self.time.append(ConvCL(wt, b[s * C:(s + 1) * C] if b is not None else None, _causal3_taps(3, 1, 1), device))
        self._key = object()

    def __call__(self, x, state):
        T, H, W, C = x.shape
        if self.time is not None:
            prev = state.store.get(id(self._key))
            if prev is None:
                state.store[id(self._key)] = "first"          # first step: no temporal up-sampling
            else:
                cache = x[-CACHE_T:].clone()
                if cache.shape[0] < CACHE_T:
                    head = prev[-1:] if isinstance(prev, torch.Tensor) else torch.zeros_like(cache[:1])
                    cache = torch.cat([head, cache], 0)
                pad = prev if isinstance(prev, torch.Tensor) else x.new_zeros(CACHE_T, H, W, C)
                full = torch.cat([pad[-CACHE_T:], x], 0)
                out = torch.empty(2 * T, H, W, C, dtype=x.dtype, device=x.device)
                for s, conv in enumerate(self.time):
                    conv(full, T, out=out, out_map=[2, s, 1, 0, 1, 0, H, W, C, 0])
                state.store[id(self._key)] = cache
                x = out
                T = 2 * T
        cout = self.phases[0][0].cout
        out = torch.empty(T, 2 * H, 2 * W, cout, dtype=x.dtype, device=x.device)
        for conv, a, b in self.phases:
            conv(x, T, out=out, out_map=[1, 0, 2, a, 2, b, 2 * H, 2 * W, cout, 0], h_out=H, w_out=W)
        return out


class DecoderCL:
    """Streaming channels-last decoder built from a ``Decoder3d`` (weights are repacked at construction)."""

    def __init__(self, decoder, device):
        self.device = torch.device(device)
        dev = self.device
        self.z_pad = 64   # the 16 latent channels travel zero-padded to one 64-channel block
        w = decoder.conv1.weight.detach().float()            # [C0, z, 3, 3, 3]
        c0, z = w.shape[:2]
        wt = torch.zeros(c0, 27, self.z_pad)
        wt[:, :, :z] = w.permute(0, 2, 3, 4, 1).reshape(c0, 27, z)
        self.z_dim = z
        self.conv1 = ConvCL(wt, decoder.conv1.bias, _causal3_taps(3, 3, 3), dev)
        self.layers = []
        from . import vae_wan
        for layer in list(decoder.middle) + list(decoder.upsamples):
            if isinstance(layer, vae_wan.ResidualBlock):
                self.layers.append(_ResBlockCL(layer, dev))
            elif isinstance(layer, vae_wan.AttentionBlock):
                self.layers.append(_AttnCL(layer, dev))
            elif isinstance(layer, vae_wan.Resample):
                self.layers.append(_UpsampleCL(layer, dev))
            else:
                raise TypeError(type(layer))
        self.head_gamma = decoder.head[0].gamma.detach().float().reshape(-1).to(dev).contiguous()
        self.head = _conv3d(decoder.head[2], dev)
        self.state: Optional[_Stream] = None

    def reset(self):
        self.state = _Stream()

    @torch.no_grad()
    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x [B=1, z, T, h, w] (already through the 1 x 1 ``conv2``) -> pixels [1, 3, T', 8h, 8w] for this chunk."""
        assert x.shape[0] == 1, "the channels-last decoder runs one video at a time"
        if self.state is None:
            self.reset()
        st = self.state
        T, h, w = x.shape[2:]
        xin = torch.zeros(T, h, w, self.z_pad, dtype=torch.bfloat16, device=self.device)
        xin[..., : self.z_dim] = x[0].permute(1, 2, 3, 0)
        y = self.conv1(_with_cache(self.conv1, xin, st), T)
        for layer in self.layers:
            y = layer(y, st)
        y = native.load().rmsnorm_silu_cl(y, self.head_gamma, True)
        native.count_launch()
        y = self.head(_with_cache(self.head, y, st), y.shape[0])
        return y.permute(3, 0, 1, 2).unsqueeze(0)


def supported(decoder, z: torch.Tensor) -> bool:
    """The kernel path serves bf16 CUDA decodes of one video (whole frames or, under ``vae_parallel.row_sharded``, row bands)."""
    return (z.is_cuda and z.dtype == torch.bfloat16 and z.shape[0] == 1 and native.available()
            and hasattr(native.load(), "conv_cl") and not native.forward_mode())


# ------------------------------------------------------------------------------------------------------------------ encoder
class _DownsampleCL:
    """``ZeroPad2d((0, 1, 0, 1)) + Conv2d(3 x 3, stride 2)`` and, for the 3-D mode, the causal ``(3, 1, 1)`` convolution with
    temporal stride 2 (wan2pt1.py:84-137), both restated as stride-1 convolutions the kernel can run:

      * space: the frame is regrouped into 2 x 2 pixel blocks ([T, H/2, W/2, 4C], channel = (row in block, column in block, c));
        output pixel (y, x) reads input pixels (2y + i, 2x + j), i, j in 0..2, which live in blocks (y, x), (y, x + 1), (y + 1, x),
        (y + 1, x + 1): a 2 x 2-tap convolution whose weights are the 3 x 3 kernel scattered over the block positions (the rest
        zero); blocks past the bottom / right edge read the kernel's out-of-range fill, which is the zero padding;
      * time: [previous last frame | chunk] is regrouped into frame pairs ([T/2 + 1, H, W, 2C]); output frame t reads input frames
        2t, 2t + 1 (pair t) and 2t + 2 (first half of pair t + 1): two taps."""

    def __init__(self, mod, device):
        conv = mod.resample[1]
        w = conv.weight.detach().float().cpu()               # [Cout, C, 3, 3]
        cout, C = w.shape[:2]
        taps, mats = [], []
        for dy in (0, 1):
            for dx in (0, 1):
                m = torch.zeros(cout, 2, 2, C)
                for a in (0, 1):
                    for b in (0, 1):
                        if 2 * dy + a < 3 and 2 * dx + b < 3:
                            m[:, a, b] = w[:, :, 2 * dy + a, 2 * dx + b]
                mats.append(m.reshape(cout, 4 * C))
                taps.append((0, dy, dx))
        self.space = ConvCL(torch.stack(mats, 1), conv.bias, taps, device)
        self.time = None
        if mod.mode == "downsample3d":
            wt = mod.time_conv.weight.detach().float().cpu()[:, :, :, 0, 0]     # [C, C, 3]
            c2 = wt.shape[0]
            m0 = torch.cat([wt[:, :, 0], wt[:, :, 1]], 1)                   # pair t: frames 2t, 2t + 1
            m1 = torch.cat([wt[:, :, 2], torch.zeros(c2, c2)], 1)          # pair t + 1: frame 2t + 2
            self.time = ConvCL(torch.stack([m0, m1], 1), mod.time_conv.bias, [(0, 0, 0), (1, 0, 0)], device)
        self._key = object()

    def __call__(self, x, state):
        T, H, W, C = x.shape
        blocks = x.view(T, H // 2, 2, W // 2, 2, C).permute(0, 1, 3, 2, 4, 5).reshape(T, H // 2, W // 2, 4 * C)
        y = self.space(blocks, T)
        if self.time is None:
            return y
        prev = state.store.get(id(self._key))
        state.store[id(self._key)] = y[-1:].clone()
        if prev is None:                                                 # first chunk: no temporal down-sampling
            return y
        full = torch.cat([prev, y], 0)                                   # T + 1 frames
        if full.shape[0] % 2:
            full = torch.cat([full, torch.zeros_like(full[:1])], 0)
        n_p, (_, h, w, c) = full.shape[0] // 2, full.shape
        pairs = full.view(n_p, 2, h, w, c).permute(0, 2, 3, 1, 4).reshape(n_p, h, w, 2 * c)
        return self.time(pairs, T // 2)


class EncoderCL:
    """Streaming channels-last encoder built from an ``Encoder3d``: the same chunked semantics (a chunk of one frame first, then
    chunks of ``temporal_window`` frames; every causal convolution carries the last two input frames; the temporal down-samplers
    pass the first chunk through), every convolution on the kernel (wan2pt1.py:270-357, 500-533)."""

    def __init__(self, encoder, device):
        self.device = torch.device(device)
        dev = self.device
        from . import vae_wan
        w = encoder.conv1.weight.detach().float().cpu()      # [C0, 3, 3, 3, 3]
        c0, cin = w.shape[:2]
        self.in_pad = 16                                     # RGB travels zero-padded to 16 channels
        wt = torch.zeros(c0, 27, self.in_pad)
        wt[:, :, :cin] = w.permute(0, 2, 3, 4, 1).reshape(c0, 27, cin)
        self.cin = cin
        self.conv1 = ConvCL(wt, encoder.conv1.bias, _causal3_taps(3, 3, 3), dev)
        self.layers = []
        for layer in list(encoder.downsamples) + list(encoder.middle):
            if isinstance(layer, vae_wan.ResidualBlock):
                self.layers.append(_ResBlockCL(layer, dev))
            elif isinstance(layer, vae_wan.AttentionBlock):
                self.layers.append(_AttnCL(layer, dev))
            elif isinstance(layer, vae_wan.Resample):
                self.layers.append(_DownsampleCL(layer, dev))
            else:
                raise TypeError(type(layer))
        self.head_gamma = encoder.head[0].gamma.detach().float().reshape(-1).to(dev).contiguous()
        self.head = _conv3d(encoder.head[2], dev)
        self.state: Optional[_Stream] = None

    def reset(self):
        self.state = _Stream()

    @torch.no_grad()
    def step(self, x: torch.Tensor) -> torch.Tensor:
        """x [1, 3, T, H, W] (one chunk) -> [1, 2 z, T', H / 8, W / 8] (input of the 1 x 1 ``conv1`` of the VAE)."""
        assert x.shape[0] == 1, "the channels-last encoder runs one video at a time"
        if self.state is None:
            self.reset()
        st = self.state
        T, H, W = x.shape[2:]
        xin = torch.zeros(T, H, W, self.in_pad, dtype=torch.bfloat16, device=self.device)
        xin[..., : self.cin] = x[0].permute(1, 2, 3, 0)
        y = self.conv1(_with_cache(self.conv1, xin, st), T)
        for layer in self.layers:
            y = layer(y, st)
        y = native.load().rmsnorm_silu_cl(y, self.head_gamma, True)
        native.count_launch()
        y = self.head(_with_cache(self.head, y, st), y.shape[0])
        return y.permute(3, 0, 1, 2).unsqueeze(0)


def encoder_supported(x: torch.Tensor) -> bool:
    """The kernel encoder serves bf16 CUDA videos, one at a time, whole frames (row-sharded encoding stays on the torch path),
    with frame sizes that survive three halvings as whole 16 x 8 pixel tiles."""
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.shape[0] == 1 and x.shape[-2] % 64 == 0 and x.shape[-1] % 128 == 0
            and vae_parallel.active() is None and native.available() and hasattr(native.load(), "conv_cl")
            and not native.forward_mode())
