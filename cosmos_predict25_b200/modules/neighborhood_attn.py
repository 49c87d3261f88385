"""Neighbourhood (sliding-window, sparse) self-attention over a T x H x W token grid.

Parity target: ``NeighborhoodAttention`` (cosmos_predict2/_src/predict2/modules/neighborhood_attn.py:57-250), which
wraps the external NATTEN package (``neighborhood_attention_generic`` with ``kernel_size / stride / dilation /
is_causal`` per axis) and its use as the sparse self-attention operator of selected DiT blocks
(cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:1739-1812). NATTEN is not a dependency here: the
operator is defined below and runs on a tile-sparse mode of this package's own tcgen05 attention kernel.

Definition used, per axis of length L with window k, stride s, dilation d (k * d <= L, s <= k):

  * dilation splits the axis into d interleaved groups (positions with equal ``i % d``); a query only sees keys of
    its own group, and everything below is in group coordinates ``i' = i // d`` with group length L';
  * stride makes every run of s consecutive queries share one window, that of its leader:
    ``leader = min((i' // s) * s + s // 2, L' - 1)`` (s = 1: every query is its own leader);
  * the window is the k positions around the leader, shifted inwards at the borders so that it never shrinks:
    ``start = clamp(leader - k // 2, 0, L' - k)``, keys ``start .. start + k - 1``;
  * a causal axis looks backwards only: ``leader = min((i' // s) * s + s - 1, L' - 1)``,
    ``start = max(leader - k + 1, 0)``, keys ``start .. i'``.

A key is visible to a query iff it is visible along all three axes (the 3-D window is the product of the 1-D ones).

Execution on the GPU (inference, bf16, head_dim 128, dilation 1, T % 4 == H % 4 == W % 8 == 0): the kernel works on
4 x 4 x 8 (t, h, w) tiles of the token grid, fetched by TMA as 5-D boxes straight from the natural [B, T*H*W, heads, D]
layout (no re-ordering pass); per pair of query tiles the host builds the list of key tiles that contain at least one
visible key; the kernel walks only that list, masks inside a tile with three small bit tables (one per axis) and writes
each output row back to its natural position. With a stride that matches the tile (e.g. (1, 4, 8)) most visited tiles are
fully visible and skip the masking. Everything else (CPU, autograd, dilation > 1, odd grid sizes) runs the dense-masked
PyTorch definition, which is also the oracle of the kernel tests.
"""

from __future__ import annotations

import math
from collections import namedtuple
from collections.abc import Mapping, Sequence
from typing import Dict, Optional, Tuple

import torch
from torch import nn

VideoSize = namedtuple("VideoSize", ["T", "H", "W"])

TILE = (4, 4, 8)  # tokens of one 128-row tile along (T, H, W)


# --------------------------------------------------------------------------------------------- definition
def axis_visibility(L: int, k: int, s: int = 1, d: int = 1, causal: bool = False) -> torch.Tensor:
    """Boolean [L, L]: entry (i, j) says whether key j is visible to query i along one axis."""
    assert 1 <= k and k * d <= L, f"window {k} x dilation {d} exceeds the axis length {L}"
    assert 1 <= s <= k, f"stride {s} must lie in [1, window {k}]"
    vis = torch.zeros(L, L, dtype=torch.bool)
    for r in range(d):
        pos = torch.arange(r, L, d)              # positions of this dilation group
        Lg = pos.numel()
        if Lg == 0:
            continue
        kk = min(k, Lg)
        i = torch.arange(Lg)
        if causal:
            leader = torch.clamp((i // s) * s + s - 1, max=Lg - 1)
            start = torch.clamp(leader - kk + 1, min=0)
            end = i + 1
        else:
            leader = torch.clamp((i // s) * s + s // 2, max=Lg - 1)
            start = torch.clamp(leader - kk // 2, min=0, max=Lg - kk)
            end = start + kk
        j = torch.arange(Lg)
        grp = (j[None, :] >= start[:, None]) & (j[None, :] < end[:, None])
        vis[pos[:, None], pos[None, :]] = grp
    return vis


def _triple(v, typ):
    if isinstance(v, typ):
        return (v, v, v)
    return tuple(v)


def neighborhood_mask(video_size, window, stride=1, dilation=1, is_causal=False) -> torch.Tensor:
    """Boolean [L, L] with L = T*H*W (token order t, h, w row-major). For tests and small problems only."""
    stride, dilation, is_causal = _triple(stride, int), _triple(dilation, int), _triple(is_causal, bool)
    mt, mh, mw = (axis_visibility(L, k, s, d, c) for L, k, s, d, c in zip(video_size, window, stride, dilation, is_causal))
    T, H, W = video_size
    m = mt[:, None, None, :, None, None] & mh[None, :, None, None, :, None] & mw[None, None, :, None, None, :]
    return m.reshape(T * H * W, T * H * W)


def neighborhood_attention_reference(q, k, v, video_size, window, stride=1, dilation=1, is_causal=False,
                                     scale: Optional[float] = None, chunk: int = 4096) -> torch.Tensor:
    """The definition in plain PyTorch: dense scores with invisible keys at -inf, fp32 softmax, query-chunked.
    q, k, v: [B, L, heads, D]; differentiable."""
    B, L, Hh, D = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    stride, dilation, is_causal = _triple(stride, int), _triple(dilation, int), _triple(is_causal, bool)
    mt, mh, mw = (axis_visibility(n, kk, s, d, c).to(q.device)
                  for n, kk, s, d, c in zip(video_size, window, stride, dilation, is_causal))
    T, H, W = video_size
    kf, vf = k.float().permute(0, 2, 1, 3), v.float().permute(0, 2, 1, 3)        # [B, heads, L, D]
    idx = torch.arange(L, device=q.device)
    it, ih, iw = idx // (H * W), (idx // W) % H, idx % W
    outs = []
    for a in range(0, L, chunk):
        b = min(L, a + chunk)
        m = mt[it[a:b]][:, it] & mh[ih[a:b]][:, ih] & mw[iw[a:b]][:, iw]             # [chunk, L]
        s = torch.matmul(q[:, a:b].float().permute(0, 2, 1, 3), kf.transpose(-1, -2)) * scale
        s = s.masked_fill(~m, float("-inf"))
        outs.append(torch.matmul(torch.softmax(s, dim=-1), vf))
    return torch.cat(outs, 2).permute(0, 2, 1, 3).to(q.dtype)


# --------------------------------------------------------------------------------------------- tile plan (GPU path)
class TilePlan:
    """Host-side schedule of the tile-sparse kernel for one (grid, window, stride, causal) combination."""

    def __init__(self, video_size, window, stride, is_causal, device):
        T, H, W = video_size
        tt, th, tw = TILE
        assert T % tt == 0 and H % th == 0 and W % tw == 0
        self.video_size = (T, H, W)
        self.n = (T // tt, H // th, W // tw)
        vis = [axis_visibility(L, k, s, 1, c) for L, k, s, c in zip(video_size, window, stride, is_causal)]
        tables, tile_any = [], []
        for m, L, t in zip(vis, video_size, TILE):
            g = m.view(L, L // t, t)                                            # [query, key tile, key in tile]
            weights = (1 << torch.arange(t)).view(1, 1, t)
            tables.append((g.long() * weights).sum(-1).to(torch.uint8))          # bit i: key i of that tile visible
            tile_any.append(g.any(-1).view(L // t, t, L // t).any(1))           # [query tile, key tile]
        nT, nH, nW = self.n
        need = (tile_any[0][:, None, None, :, None, None] & tile_any[1][None, :, None, None, :, None]
                & tile_any[2][None, None, :, None, None, :]).reshape(nT * nH * nW, nT * nH * nW)
        n_tiles = need.shape[0]
        need_all = need                                                          # [query tile, key tile], before padding
        if n_tiles % 2:
            need = torch.cat([need, torch.zeros(1, n_tiles, dtype=torch.bool)], 0)
        block_need = need[0::2] | need[1::2]                                    # a CTA serves two consecutive query tiles
        cnt = block_need.sum(1)
        max_n = int(cnt.max())
        order = torch.argsort((~block_need).to(torch.int8), dim=1, stable=True)[:, :max_n]   # needed tiles first, ascending
        last = order.gather(1, (cnt - 1).clamp(min=0)[:, None])
        pad = torch.arange(max_n)[None, :] >= cnt[:, None]
        order = torch.where(pad, last.expand_as(order), order)
        self.kv_idx = order.to(torch.int32).contiguous().to(device)
        self.kv_cnt = cnt.to(torch.int32).contiguous().to(device)
        self.bt, self.bh, self.bw = (t.contiguous().to(device) for t in tables)
        self.visited_fraction = float(cnt.sum()) / float(block_need.shape[0] * n_tiles)
        # ---- backward: a CTA owns a key tile and walks the query tiles that see it. Tables: for one key coordinate and one query
        # tile, the visibility bits of the tile's query coordinates; list entries carry the top bit when the whole pair is visible.
        tables_b, full_axis = [], []
        for m, L, t in zip(vis, video_size, TILE):
            gT = m.t().contiguous().view(L, L // t, t)                          # [key, query tile, query in tile]
            weights = (1 << torch.arange(t)).view(1, 1, t)
            tables_b.append((gT.long() * weights).sum(-1).to(torch.uint8))
            full_axis.append(m.view(L // t, t, L // t, t).permute(0, 2, 1, 3).reshape(L // t, L // t, t * t).all(-1))
        full = (full_axis[0][:, None, None, :, None, None] & full_axis[1][None, :, None, None, :, None]
                & full_axis[2][None, None, :, None, None, :]).reshape(n_tiles, n_tiles)
        need_b, full_b = need_all.t().contiguous(), full.t().contiguous()       # [key tile, query tile]
        cnt_b = need_b.sum(1)
        assert int(cnt_b.min()) >= 1                                            # every tile sees itself
        max_nb = int(cnt_b.max())
        order_b = torch.argsort((~need_b).to(torch.int8), dim=1, stable=True)[:, :max_nb]
        last_b = order_b.gather(1, (cnt_b - 1)[:, None])
        order_b = torch.where(torch.arange(max_nb)[None, :] >= cnt_b[:, None], last_b.expand_as(order_b), order_b)
        entries = torch.where(full_b.gather(1, order_b), order_b - (1 << 31), order_b)
        self.q_list = entries.to(torch.int32).contiguous().to(device)
        self.q_cnt = cnt_b.to(torch.int32).contiguous().to(device)
        self.bt_b, self.bh_b, self.bw_b = (t.contiguous().to(device) for t in tables_b)
        L = T * H * W
        self.perm = self.to_tiles(torch.arange(L).view(1, L, 1, 1)).reshape(L).to(device)   # tile-order position -> natural index

    def to_tiles(self, x: torch.Tensor) -> torch.Tensor:
        """[B, T*H*W, heads, D] in (t, h, w) order -> the same tokens tile by tile (the order in which the kernel numbers
        its rows; the kernel itself reads the natural layout, this helper serves the host-side checks)."""
        B, L, Hh, D = x.shape
        (nT, nH, nW), (tt, th, tw) = self.n, TILE
        return x.view(B, nT, tt, nH, th, nW, tw, Hh, D).permute(0, 1, 3, 5, 2, 4, 6, 7, 8).reshape(B, L, Hh, D)

    def from_tiles(self, x: torch.Tensor) -> torch.Tensor:
        B, L, Hh, D = x.shape
        (nT, nH, nW), (tt, th, tw) = self.n, TILE
        return x.view(B, nT, nH, nW, tt, th, tw, Hh, D).permute(0, 1, 4, 2, 5, 3, 6, 7, 8).reshape(B, L, Hh, D)


_plans: Dict[Tuple, TilePlan] = {}


def tile_plan(video_size, window, stride, is_causal, device) -> TilePlan:
    key = (tuple(video_size), tuple(window), tuple(stride), tuple(is_causal), str(device))
    if key not in _plans:
        _plans[key] = TilePlan(video_size, window, stride, is_causal, device)
    return _plans[key]


class _TileNeighborhoodAttention(torch.autograd.Function):
    """Tile-sparse forward kernel on the natural layout; backward on the tile-sparse single-pass kernel, which wants every
    128-row tile contiguous: the operands are brought into tile order (one copy each) and the gradients back."""

    @staticmethod
    def forward(ctx, q, k, v, plan, scale):
        from ..ops import native
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = native.load().fa_fwd_na(q, k, v, scale, plan.kv_idx, plan.kv_cnt, plan.bt, plan.bh, plan.bw)
        native.count_launch()
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.plan, ctx.scale = plan, scale
        return o

    @staticmethod
    def backward(ctx, do):
        from ..ops import native
        q, k, v, o, lse = ctx.saved_tensors
        plan = ctx.plan
        qt, kt, vt, ot, dot = (plan.to_tiles(x).contiguous() for x in (q, k, v, o, do))
        lse_t = lse.index_select(2, plan.perm).contiguous()
        dq, dk, dv = native.load().fa_bwd_na(dot, qt, kt, vt, ot, lse_t, ctx.scale, plan.q_list, plan.q_cnt,
                                             plan.bt_b, plan.bh_b, plan.bw_b)
        native.count_launch(3)
        return plan.from_tiles(dq), plan.from_tiles(dk), plan.from_tiles(dv), None, None


def tile_kernel_supported(q: torch.Tensor, video_size, dilation) -> bool:
    from ..ops import native
    T, H, W = video_size
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.shape[-1] == 128 and native.use_native(q)
            and all(d == 1 for d in dilation)
            and T % TILE[0] == 0 and H % TILE[1] == 0 and W % TILE[2] == 0
            and native.available() and hasattr(native.load(), "fa_fwd_na"))


def _tile_backward_available() -> bool:
    from ..ops import native
    return native.available() and hasattr(native.load(), "fa_bwd_na")


def _group_starts(L: int, k: int, s: int) -> torch.Tensor:
    """First visible key of every stride group of a non-causal, undilated axis (all queries of a group share the window)."""
    g = torch.arange(L // s)
    leader = torch.clamp(g * s + s // 2, max=L - 1)
    return torch.clamp(leader - k // 2, min=0, max=L - k)


def grouped_attention_supported(video_size, window, stride, dilation, is_causal) -> bool:
    return (all(d == 1 for d in dilation) and not any(is_causal)
            and all(L % s == 0 and k <= L for L, k, s in zip(video_size, window, stride)))


def neighborhood_attention_grouped(q, k, v, video_size, window, stride, scale: Optional[float] = None,
                                   max_keys_per_chunk: int = 1 << 24) -> torch.Tensor:
    """Differentiable neighbourhood attention whose cost follows the window, not the sequence: the queries of one stride group
    share one box of keys, so each group is a small dense attention over its gathered box (``scaled_dot_product_attention`` on
    [groups, heads, queries per group, keys per box]); autograd scatters the key / value gradients back through the gather.
    Non-causal, dilation 1, axis lengths divisible by the strides. Groups are processed in chunks to bound the gathered size."""
    import torch.nn.functional as F
    B, L, Hh, D = q.shape
    T, H, W = video_size
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    (kt, kh, kw), (st, sh, sw) = window, stride
    Gt, Gh, Gw = T // st, H // sh, W // sw
    dev = q.device
    it = (_group_starts(T, kt, st)[:, None] + torch.arange(kt)[None]).to(dev)        # [Gt, kt]
    ih = (_group_starts(H, kh, sh)[:, None] + torch.arange(kh)[None]).to(dev)        # [Gh, kh]
    iw = (_group_starts(W, kw, sw)[:, None] + torch.arange(kw)[None]).to(dev)        # [Gw, kw]
    q6 = q.view(B, Gt, st, Gh, sh, Gw, sw, Hh, D).permute(0, 1, 3, 5, 7, 2, 4, 6, 8)   # [B,Gt,Gh,Gw,heads,st,sh,sw,D]
    k5, v5 = k.view(B, T, H, W, Hh, D), v.view(B, T, H, W, Hh, D)
    nq, nk = st * sh * sw, kt * kh * kw
    rows_per_chunk = max(1, max_keys_per_chunk // max(1, B * Gw * nk * Hh))          # (gt, gh) pairs per chunk
    out = q.new_empty(B, Gt, Gh, Gw, Hh, nq, D)
    pairs = [(a, b) for a in range(Gt) for b in range(Gh)]
    for c0 in range(0, len(pairs), rows_per_chunk):
        chunk = pairs[c0:c0 + rows_per_chunk]
        ga = torch.tensor([a for a, _ in chunk], device=dev)
        gb = torch.tensor([b for _, b in chunk], device=dev)
        n = len(chunk)
        # key boxes of the groups (ga[i], gb[i], every gw): [B, n, Gw, kt, kh, kw, heads, D]
        tt = it[ga][:, None, :, None, None]                                          # [n,1,kt,1,1]
        hh = ih[gb][:, None, None, :, None]                                          # [n,1,1,kh,1]
        ww = iw[None, :, None, None, :]                                              # [1,Gw,1,1,kw]
        kb = k5[:, tt, hh, ww]
        vb = v5[:, tt, hh, ww]
        kb = kb.reshape(B * n * Gw, nk, Hh, D).transpose(1, 2)
        vb = vb.reshape(B * n * Gw, nk, Hh, D).transpose(1, 2)
        qb = q6[:, ga, gb].reshape(B * n * Gw, Hh, nq, D)
        ob = F.scaled_dot_product_attention(qb, kb, vb, scale=scale).view(B, n, Gw, Hh, nq, D)
        out[:, ga, gb] = ob
    o = out.view(B, Gt, Gh, Gw, Hh, st, sh, sw, D).permute(0, 1, 5, 2, 6, 3, 7, 4, 8)
    return o.reshape(B, L, Hh, D)


def neighborhood_attention(q, k, v, video_size, window, stride=1, dilation=1, is_causal=False,
                           scale: Optional[float] = None) -> torch.Tensor:
    """q, k, v: [B, T*H*W, heads, D] -> [B, T*H*W, heads, D]."""
    stride, dilation, is_causal = _triple(stride, int), _triple(dilation, int), _triple(is_causal, bool)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    needs_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad)
    if not tile_kernel_supported(q, video_size, dilation) or (needs_grad and not _tile_backward_available()):
        # training / CPU: gather the shared key box of every stride group when the configuration allows it (cost follows the
        # window), otherwise the dense-masked definition
        if grouped_attention_supported(video_size, window, stride, dilation, is_causal) and q.shape[1] > 4096:
            return neighborhood_attention_grouped(q, k, v, video_size, window, stride, scale)
        return neighborhood_attention_reference(q, k, v, video_size, window, stride, dilation, is_causal, scale)
    from ..ops import native
    plan = tile_plan(video_size, window, stride, is_causal, q.device)
    if needs_grad:
        return _TileNeighborhoodAttention.apply(q, k, v, plan, scale)
    o, _ = native.load().fa_fwd_na(q.contiguous(), k.contiguous(), v.contiguous(), scale, plan.kv_idx, plan.kv_cnt,
                                   plan.bt, plan.bh, plan.bw)
    native.count_launch()
    return o


# --------------------------------------------------------------------------------------------- module
class NeighborhoodAttention(nn.Module):
    """Sparse self-attention operator of a DiT block. ``natten_parameters``: dict with ``window_size`` (3 ints; an
    entry <= 1 means the whole axis) and ``layer_id``, optional ``stride``, ``dilation``, ``is_causal`` (int / bool or
    3 of them) and ``base_size`` (grid the window was chosen for; other grids scale window, stride and dilation).
    Single-frame inputs (T == 1) go to ``base_attn_op`` (dense attention)."""

    def __init__(self, natten_parameters, base_attn_op=None):
        super().__init__()
        self.base_attn_op = base_attn_op
        if not isinstance(natten_parameters, Mapping) or "window_size" not in natten_parameters or "layer_id" not in natten_parameters:
            raise ValueError(f"expected a dict with at least `window_size` and `layer_id`, got {natten_parameters!r}")
        self.natten_parameters = dict(natten_parameters)
        self.layer_id = natten_parameters["layer_id"]
        self.window_size = natten_parameters["window_size"]
        self.stride = natten_parameters.get("stride", 1)
        self.dilation = natten_parameters.get("dilation", 1)
        self.is_causal = natten_parameters.get("is_causal", False)
        self.base_size = natten_parameters.get("base_size")
        if not isinstance(self.window_size, Sequence) or len(self.window_size) != 3:
            raise ValueError(f"window_size must have 3 entries, got {self.window_size}")
        for name, val, typ in (("stride", self.stride, int), ("dilation", self.dilation, int), ("is_causal", self.is_causal, bool)):
            if not isinstance(val, typ) and not (isinstance(val, Sequence) and len(val) == 3):
                raise ValueError(f"{name} must be a {typ.__name__} or 3 of them, got {val}")
        if self.base_size is not None and (not isinstance(self.base_size, Sequence) or len(self.base_size) != 3):
            raise ValueError(f"base_size must have 3 entries or be None, got {self.base_size}")

    @staticmethod
    def get_adaptive_parameters(window_size, stride, dilation, is_causal, input_shape, base_size=None):
        """Resolve whole-axis windows and rescale (window, stride, dilation) from ``base_size`` to ``input_shape``
        (neighborhood_attn.py:142-174 of the reference)."""
        window_size = tuple(w if w > 1 else x for x, w in zip(input_shape, window_size))
        stride, dilation, is_causal = _triple(stride, int), _triple(dilation, int), _triple(is_causal, bool)
        if base_size is not None:
            base = tuple(b if b > 0 else x for x, b in zip(input_shape, base_size))
            ratio = tuple(x / b for x, b in zip(input_shape, base))
            window_size = tuple(min(max(2, round(w * r)), x) for w, r, x in zip(window_size, ratio, input_shape))
            stride = tuple(min(max(1, round(s * r)), w) for w, r, s in zip(window_size, ratio, stride))
            max_d = tuple(x // w for x, w in zip(input_shape, window_size))
            dilation = tuple(min(max(1, round(d * r)), m) for d, r, m in zip(dilation, ratio, max_d))
        assert all(x >= w * d for x, w, d in zip(input_shape, window_size, dilation))
        assert all(w >= s for w, s in zip(window_size, stride))
        return window_size, stride, dilation, is_causal

    def forward(self, q_B_L_H_D, k_B_L_H_D, v_B_L_H_D, video_size: Optional[VideoSize] = None):
        if not (q_B_L_H_D.shape == k_B_L_H_D.shape == v_B_L_H_D.shape):
            raise ValueError("neighbourhood attention needs q, k, v of one shape")
        T, H, W = video_size
        if q_B_L_H_D.shape[1] != T * H * W:
            raise ValueError(f"sequence length {q_B_L_H_D.shape[1]} does not match video_size {tuple(video_size)}")
        if T == 1:
            if self.base_attn_op is not None:
                return self.base_attn_op(q_B_L_H_D, k_B_L_H_D, v_B_L_H_D)
            from ..ops import functional as ops
            return ops.attention(q_B_L_H_D, k_B_L_H_D, v_B_L_H_D)
        window, stride, dilation, causal = self.get_adaptive_parameters(self.window_size, self.stride, self.dilation,
                                                                        self.is_causal, (T, H, W), self.base_size)
        return neighborhood_attention(q_B_L_H_D, k_B_L_H_D, v_B_L_H_D, (T, H, W), window, stride, dilation, causal)
