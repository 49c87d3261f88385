"""Vision tower of the Reason1 / Qwen2.5-VL model: patch embedding, window + full attention blocks with 2-D rotary positions,
2 x 2 patch merger. Parameter names follow the released checkpoints (``patch_embed.proj.weight``, ``blocks.N.attn.qkv.weight``,
``merger.mlp.0.weight`` ...), so a ``visual.*`` sub-dict of a Qwen2.5-VL state dict loads with ``load_state_dict``.

Parity target: the vision encoder inside cosmos_predict2/_src/reason1/networks/qwen2_5_vl.py (the text-conditioning path of the
video model uses the language tower only; this tower serves image / video prompts of the VLM and its training stack).

Input convention (the processor's): ``pixel_patches [N, C * tp * p * p]`` - every row one (temporal patch x spatial patch) cube,
rows ordered image by image, inside an image frame-major with the patches of each ``merge x merge`` group adjacent - and
``grid_thw [n_images, 3]`` with the patch grid of every image / video. Output: ``[N / merge^2, out_hidden]`` in input order.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclass
class QwenVisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    intermediate_size: int = 3420
    num_heads: int = 16
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: List[int] = field(default_factory=lambda: [7, 15, 23, 31])
    out_hidden_size: int = 3584
    rms_eps: float = 1e-6
    rope_theta: float = 10000.0


class _RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        h = x.float()
        return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _PatchEmbed(nn.Module):
    """The released weights store the embedding as a Conv3d whose kernel covers exactly one patch cube: a linear map."""

    def __init__(self, c: QwenVisionConfig):
        super().__init__()
        k = (c.temporal_patch_size, c.patch_size, c.patch_size)
        self.proj = nn.Conv3d(c.in_channels, c.hidden_size, kernel_size=k, stride=k, bias=False)

    def forward(self, patches):
        w = self.proj.weight
        return F.linear(patches.to(w.dtype), w.reshape(w.shape[0], -1))


def _rotate_half(x):
    a, b = x[..., : x.shape[-1] // 2], x[..., x.shape[-1] // 2:]
    return torch.cat([-b, a], -1)


def segment_attention(q, k, v, cu: torch.Tensor):
    """Non-causal attention inside the segments ``[cu[i], cu[i+1])`` of a packed sequence; q, k, v: [N, heads, D]. Segments of equal
    length run as one batched call (windows of a frame have the same size except at the borders)."""
    out = torch.empty_like(q)
    starts, lens = cu[:-1].tolist(), (cu[1:] - cu[:-1]).tolist()
    by_len = {}
    for s, n in zip(starts, lens):
        if n > 0:
            by_len.setdefault(n, []).append(s)
    for n, ss in by_len.items():
        idx = (torch.tensor(ss, device=q.device)[:, None] + torch.arange(n, device=q.device)[None, :]).reshape(-1)
        qb, kb, vb = (t.index_select(0, idx).view(len(ss), n, t.shape[1], t.shape[2]).transpose(1, 2) for t in (q, k, v))
        ob = F.scaled_dot_product_attention(qb, kb, vb)
        out.index_copy_(0, idx, ob.transpose(1, 2).reshape(len(ss) * n, q.shape[1], q.shape[2]))
    return out


class _VisionAttention(nn.Module):
    def __init__(self, c: QwenVisionConfig):
        super().__init__()
        self.num_heads = c.num_heads
        self.qkv = nn.Linear(c.hidden_size, 3 * c.hidden_size, bias=True)
        self.proj = nn.Linear(c.hidden_size, c.hidden_size, bias=True)

    def forward(self, x, cu, cos, sin):
        N, D = x.shape
        q, k, v = self.qkv(x).view(N, 3, self.num_heads, D // self.num_heads).unbind(1)
        qf, kf = q.float(), k.float()
        q = (qf * cos[:, None] + _rotate_half(qf) * sin[:, None]).to(x.dtype)
        k = (kf * cos[:, None] + _rotate_half(kf) * sin[:, None]).to(x.dtype)
        return self.proj(segment_attention(q, k, v, cu).reshape(N, D))


class _VisionMLP(nn.Module):
    def __init__(self, c: QwenVisionConfig):
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=True)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=True)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=True)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class _VisionBlock(nn.Module):
    def __init__(self, c: QwenVisionConfig):
        super().__init__()
        self.norm1 = _RMSNorm(c.hidden_size, c.rms_eps)
        self.norm2 = _RMSNorm(c.hidden_size, c.rms_eps)
        self.attn = _VisionAttention(c)
        self.mlp = _VisionMLP(c)

    def forward(self, x, cu, cos, sin):
        x = x + self.attn(self.norm1(x), cu, cos, sin)
        return x + self.mlp(self.norm2(x))


class _PatchMerger(nn.Module):
    def __init__(self, c: QwenVisionConfig):
        super().__init__()
        self.unit = c.spatial_merge_size ** 2
        self.ln_q = _RMSNorm(c.hidden_size, c.rms_eps)
        d = c.hidden_size * self.unit
        self.mlp = nn.Sequential(nn.Linear(d, d), nn.GELU(), nn.Linear(d, c.out_hidden_size))

    def forward(self, x):
        return self.mlp(self.ln_q(x).view(-1, x.shape[-1] * self.unit))


class QwenVisionTower(nn.Module):
    def __init__(self, config: QwenVisionConfig):
        super().__init__()
        c = self.config = config
        self.patch_embed = _PatchEmbed(c)
        self.blocks = nn.ModuleList([_VisionBlock(c) for _ in range(c.depth)])
        self.merger = _PatchMerger(c)
        self.head_dim = c.hidden_size // c.num_heads

    # ---- index bookkeeping (host side, tiny) -----------------------------------------------------------------------------------
    def rotary_angles(self, grid_thw: torch.Tensor) -> torch.Tensor:
        """[N, head_dim / 2] rotary angles: the first half of the frequencies turns with the patch row, the second with the patch
        column; rows follow the processor's order (merge x merge groups adjacent)."""
        m = self.config.spatial_merge_size
        pos = []
        for t, h, w in grid_thw.tolist():
            hp = torch.arange(h)[:, None].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            wp = torch.arange(w)[None, :].expand(h, w).reshape(h // m, m, w // m, m).permute(0, 2, 1, 3).reshape(-1)
            pos.append(torch.stack([hp, wp], -1).repeat(t, 1))
        pos = torch.cat(pos, 0)
        dim = self.head_dim // 2
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
        table = torch.outer(torch.arange(int(grid_thw[:, 1:].max()), dtype=torch.float32), inv)       # [max side, dim / 2]
        return table[pos].flatten(1)

    def window_index(self, grid_thw: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """Order of the merged tokens window by window (every frame is cut into windows of ``window_size`` pixels), and the
        cumulative patch counts of the windows."""
        c = self.config
        m, unit = c.spatial_merge_size, c.spatial_merge_size ** 2
        side = c.window_size // m // c.patch_size                       # window side in merged tokens
        order, cu, base = [], [0], 0
        for t, h, w in grid_thw.tolist():
            gh, gw = h // m, w // m
            idx = torch.arange(t * gh * gw).view(t, gh, gw)
            ph, pw = (-gh) % side, (-gw) % side
            idx = F.pad(idx, (0, pw, 0, ph), value=-1)
            nh, nw = (gh + ph) // side, (gw + pw) // side
            win = idx.view(t, nh, side, nw, side).permute(0, 1, 3, 2, 4).reshape(t * nh * nw, side * side)
            keep = win >= 0
            order.append(win[keep] + base)
            counts = keep.sum(1)
            cu.extend((torch.cumsum(counts, 0) * unit + cu[-1]).tolist())
            base += t * gh * gw
        cu = torch.tensor(cu, dtype=torch.int64)
        cu = torch.unique_consecutive(cu)                              # windows that are all padding add nothing
        return torch.cat(order), cu

    # ---- forward -----------------------------------------------------------------------------------------------------------
    def forward(self, pixel_patches: torch.Tensor, grid_thw: torch.Tensor) -> torch.Tensor:
        c = self.config
        unit = c.spatial_merge_size ** 2
        dev = pixel_patches.device
        x = self.patch_embed(pixel_patches)
        N = x.shape[0]
        ang = self.rotary_angles(grid_thw)
        order, cu_win = self.window_index(grid_thw)
        order_d = order.to(dev)
        x = x.view(N // unit, unit, -1)[order_d].reshape(N, -1)
        ang = ang.view(N // unit, unit, -1)[order].reshape(N, -1).to(dev)
        ang = torch.cat([ang, ang], -1)
        cos, sin = ang.cos(), ang.sin()
        per_frame = (grid_thw[:, 1] * grid_thw[:, 2]).repeat_interleave(grid_thw[:, 0])
        cu_full = F.pad(torch.cumsum(per_frame, 0), (1, 0)).to(torch.int64)
        for i, blk in enumerate(self.blocks):
            x = blk(x, cu_full if i in c.fullatt_block_indexes else cu_win, cos, sin)
        y = self.merger(x)
        return y[torch.argsort(order_d)]
