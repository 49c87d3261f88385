"""Neighbourhood attention: definition, tile schedule of the GPU kernel (emulated on the host), module, DiT wiring."""

import pytest
import torch

from cosmos_predict25_b200.modules import neighborhood_attn as na
from cosmos_predict25_b200.ops import ref


def test_axis_visibility_window_is_never_smaller_than_k():
    m = na.axis_visibility(12, 5)
    assert (m.sum(1) == 5).all()
    assert m[0, :5].all() and m[11, 7:].all()          # shifted inwards at the borders
    assert m[6, 4:9].all() and m.diagonal().all()


def test_axis_visibility_stride_groups_share_a_window():
    m = na.axis_visibility(16, 8, s=4)
    for g in range(4):
        rows = m[4 * g: 4 * g + 4]
        assert (rows == rows[0]).all() and rows[0].sum() == 8
    assert m.diagonal().all()                         # a query always sees itself (s <= k)


def test_axis_visibility_causal_and_dilation():
    m = na.axis_visibility(10, 3, causal=True)
    assert not torch.triu(m, 1).any() and m.diagonal().all()
    assert m[0].sum() == 1 and m[1].sum() == 2 and (m[2:].sum(1) == 3).all()
    d = na.axis_visibility(12, 3, d=2)
    i = torch.arange(12)
    assert not d[(i[:, None] % 2) != (i[None, :] % 2)].any()      # only keys of the own dilation group
    assert (d.sum(1) == 3).all()


def test_reference_with_whole_axis_windows_is_dense_attention():
    torch.manual_seed(0)
    vs = (2, 3, 4)
    q, k, v = (torch.randn(2, 24, 2, 16) for _ in range(3))
    got = na.neighborhood_attention_reference(q, k, v, vs, vs)
    want = ref.attention(q, k, v, 16 ** -0.5)[0]
    assert torch.allclose(got, want, atol=1e-5)


@pytest.mark.parametrize("window,stride,causal", [((4, 4, 8), 1, False), ((8, 4, 16), (1, 4, 8), False),
                                                  ((5, 7, 9), (2, 3, 4), (True, False, False)), ((8, 12, 8), 1, False)])
def test_tile_plan_reproduces_the_mask(window, stride, causal):
    """What the kernel computes from the tile lists and bit tables equals the definition."""
    vs = (8, 12, 16)
    stride3, causal3 = na._triple(stride, int), na._triple(causal, bool)
    plan = na.TilePlan(vs, window, stride3, causal3, "cpu")
    mask = na.neighborhood_mask(vs, window, stride3, 1, causal3)
    L = mask.shape[0]
    idx = torch.arange(L).view(1, L, 1, 1)
    perm = plan.to_tiles(idx).view(L)                 # tile-ordered position -> original token
    assert torch.equal(plan.from_tiles(plan.to_tiles(idx)), idx)
    mask_t = mask[perm][:, perm]                      # mask in tile order
    nT, nH, nW = plan.n
    got = torch.zeros_like(mask_t)
    lt, lh, lw = torch.arange(128) >> 5, (torch.arange(128) >> 3) & 3, torch.arange(128) & 7
    for row in range(L):
        blk, qt, loc = row // 256, row // 128, row % 128
        qT, qH, qW = qt // (nH * nW), (qt // nW) % nH, qt % nW
        tq, hq, wq = qT * 4 + (loc >> 5), qH * 4 + ((loc >> 3) & 3), qW * 8 + (loc & 7)
        for j in range(int(plan.kv_cnt[blk])):
            kt = int(plan.kv_idx[blk, j])
            mt, mh, mw = int(plan.bt[tq, kt // (nH * nW)]), int(plan.bh[hq, (kt // nW) % nH]), int(plan.bw[wq, kt % nW])
            vis = ((mt >> lt) & 1) & ((mh >> lh) & 1) & ((mw >> lw) & 1)
            got[row, kt * 128: kt * 128 + 128] = vis.bool()
    assert torch.equal(got, mask_t)
    assert (plan.kv_cnt >= 1).all() and plan.visited_fraction <= 1.0
    lists = [plan.kv_idx[b, : int(plan.kv_cnt[b])] for b in range(plan.kv_idx.shape[0])]
    assert all((l[1:] > l[:-1]).all() for l in lists)          # ascending, no duplicates


def test_module_parameters_and_single_frame_path():
    with pytest.raises(ValueError):
        na.NeighborhoodAttention({"window_size": (4, 4)})
    with pytest.raises(ValueError):
        na.NeighborhoodAttention({"window_size": (4, 4, 4), "layer_id": 0, "stride": (1, 2)})
    op = na.NeighborhoodAttention({"window_size": (-1, 4, 8), "layer_id": 3, "stride": (1, 2, 4), "base_size": (-1, 8, 16)})
    w, s, d, c = op.get_adaptive_parameters(op.window_size, op.stride, op.dilation, op.is_causal, (6, 16, 32), op.base_size)
    assert w == (6, 8, 16) and s == (1, 4, 8) and d == (1, 2, 2) and c == (False, False, False)  # dilation scales with the grid too
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 12, 2, 8) for _ in range(3))
    one = op(q, k, v, na.VideoSize(1, 3, 4))                     # image input: dense attention
    assert torch.allclose(one, ref.attention(q, k, v, 8 ** -0.5)[0], atol=1e-5)
    q, k, v = (torch.randn(1, 2 * 8 * 16, 2, 8, requires_grad=True) for _ in range(3))
    out = op(q, k, v, na.VideoSize(2, 8, 16))
    out.sum().backward()
    assert q.grad is not None and torch.isfinite(q.grad).all()


def test_dit_blocks_switch_to_sparse_attention():
    from cosmos_predict25_b200.models.dit import NET_PRESETS, CosmosDiT, replace_selfattn_op_with_sparse_attn_op
    torch.manual_seed(0)
    cfg = NET_PRESETS["tiny"]()
    net = CosmosDiT(cfg).eval()
    net.init_weights()
    x = torch.randn(1, cfg.in_channels, 4, 16, 16)
    mask = torch.zeros(1, 1, 4, 16, 16)
    args = dict(timesteps_B_T=torch.tensor([[0.5]]), crossattn_emb=torch.randn(1, 8, cfg.crossattn_proj_in_channels
                                                                               if cfg.use_crossattn_projection else cfg.crossattn_emb_channels),
                condition_video_input_mask_B_C_T_H_W=mask, fps=torch.tensor([16.0]), padding_mask=torch.zeros(1, 1, 16, 16))
    with torch.no_grad():
        dense = net(x, **args)
        # whole-axis windows: the sparse operator must reproduce dense attention exactly
        replace_selfattn_op_with_sparse_attn_op(net, 1, {"window_size": (-1, -1, -1)})
        n_sparse = sum(b.self_attn.sparse_op is not None for b in net.blocks)
        assert n_sparse == len(net.blocks) - 1 and net.blocks[len(net.blocks) // 2].self_attn.sparse_op is None
        same = net(x, **args)
        assert torch.allclose(same, dense, atol=1e-4)
        for b in net.blocks:
            if b.self_attn.sparse_op is not None:
                b.self_attn.sparse_op.window_size = (2, 4, 4)
        local = net(x, **args)
        assert local.shape == dense.shape and torch.isfinite(local).all() and not torch.allclose(local, dense, atol=1e-4)
    with pytest.raises(ValueError):
        replace_selfattn_op_with_sparse_attn_op(net, 0, None)


@pytest.mark.parametrize("window,stride", [((4, 4, 8), (1, 1, 1)), ((8, 4, 16), (1, 4, 8)), ((5, 7, 9), (2, 3, 4)), ((8, 12, 16), (2, 2, 2))])
def test_grouped_gather_path_matches_definition_with_gradients(window, stride):
    torch.manual_seed(4)
    vs = (8, 12, 16)
    assert na.grouped_attention_supported(vs, window, stride, (1, 1, 1), (False, False, False))
    L = vs[0] * vs[1] * vs[2]
    q, k, v = (torch.randn(1, L, 2, 8, dtype=torch.float64, requires_grad=True) for _ in range(3))
    go = torch.randn(1, L, 2, 8, dtype=torch.float64)
    got = na.neighborhood_attention_grouped(q, k, v, vs, window, stride, max_keys_per_chunk=1 << 14)   # several chunks
    g1 = torch.autograd.grad(got, (q, k, v), go)
    want = na.neighborhood_attention_reference(q, k, v, vs, window, stride)
    g2 = torch.autograd.grad(want, (q, k, v), go)
    assert torch.allclose(got, want.double(), atol=1e-5)
    for a, b in zip(g1, g2):
        assert torch.allclose(a, b.double(), atol=1e-4), (a - b).abs().max()
    assert not na.grouped_attention_supported(vs, window, stride, (1, 1, 1), (True, False, False))
    assert not na.grouped_attention_supported((9, 12, 16), (4, 4, 8), (2, 1, 1), (1, 1, 1), (False, False, False))
