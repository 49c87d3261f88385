"""The vision tower against the transformers implementation of Qwen2.5-VL's vision encoder with the same random weights."""

import pytest
import torch

from cosmos_predict25_b200.models.qwen_vision import QwenVisionConfig, QwenVisionTower, segment_attention


def _hf():
    mod = pytest.importorskip("transformers.models.qwen2_5_vl.modeling_qwen2_5_vl")
    cfg_mod = pytest.importorskip("transformers.models.qwen2_5_vl.configuration_qwen2_5_vl")
    return mod, cfg_mod


@pytest.mark.parametrize("grids", [[(1, 8, 12)], [(2, 12, 20), (1, 4, 4)]])
def test_vision_tower_matches_transformers(grids):
    mod, cfg_mod = _hf()
    kw = dict(depth=4, hidden_size=64, intermediate_size=96, num_heads=4, in_channels=3, patch_size=14, temporal_patch_size=2,
              spatial_merge_size=2, window_size=112, fullatt_block_indexes=[1, 3], out_hidden_size=80)
    hf_cfg = cfg_mod.Qwen2_5_VLVisionConfig(**kw, hidden_act="silu")
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    hf = mod.Qwen2_5_VisionTransformerPretrainedModel(hf_cfg).eval().float()
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05) if p.dim() > 1 else torch.nn.init.normal_(p, mean=0.5, std=0.2)
    ours = QwenVisionTower(QwenVisionConfig(**kw)).eval()
    missing, unexpected = ours.load_state_dict(hf.state_dict(), strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    grid = torch.tensor(grids)
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum())
    patches = torch.randn(n, 3 * 2 * 14 * 14)
    with torch.no_grad():
        want = hf(patches, grid_thw=grid)
        want = want if isinstance(want, torch.Tensor) else (getattr(want, "pooler_output", None) if getattr(want, "pooler_output", None) is not None else want[0])
        got = ours(patches, grid)
    assert got.shape == (n // 4, 80)
    if want.shape != got.shape:        # newer transformers return the un-merged hidden states first
        pytest.skip(f"transformers returned {tuple(want.shape)}")
    assert torch.allclose(got, want, atol=2e-4, rtol=2e-3), (got - want).abs().max()


def test_segment_attention_equals_masked_attention():
    torch.manual_seed(1)
    cu = torch.tensor([0, 5, 5, 12, 17, 22])
    q, k, v = (torch.randn(22, 2, 8) for _ in range(3))
    seg = torch.bucketize(torch.arange(22), cu[1:], right=True)
    mask = seg[:, None] == seg[None, :]
    want = torch.nn.functional.scaled_dot_product_attention(q.transpose(0, 1), k.transpose(0, 1), v.transpose(0, 1), attn_mask=mask)
    assert torch.allclose(segment_attention(q, k, v, cu), want.transpose(0, 1), atol=1e-5)
