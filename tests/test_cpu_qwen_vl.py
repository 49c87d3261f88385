"""The vision-language wrapper against the transformers implementation of Qwen2.5-VL on the same random weights."""

import pytest
import torch

from cosmos_predict25_b200.models.qwen_vision import QwenVisionConfig
from cosmos_predict25_b200.models.qwen_vl import QwenVLConfig, QwenVLModel, multimodal_positions
from cosmos_predict25_b200.models.text_encoder import QwenConfig

IMG, VID, START = 151655, 151656, 151652


def _cfg():
    text = QwenConfig(vocab_size=152064, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2)
    vis = QwenVisionConfig(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, out_hidden_size=64, fullatt_block_indexes=[1])
    return QwenVLConfig(text=text, vision=vis, mrope_section=(2, 3, 3))


def test_multimodal_positions_by_hand():
    cfg = _cfg()
    # 2 text tokens, an image of 1 x 4 x 4 patches (2 x 2 merged tokens), 2 text tokens
    ids = torch.tensor([[11, START, IMG, IMG, IMG, IMG, 12, 13]])
    pos = multimodal_positions(ids, torch.tensor([[1, 4, 4]]), None, None, None, cfg)
    assert pos[:, 0, :2].tolist() == [[0, 1]] * 3
    assert pos[0, 0, 2:6].tolist() == [2, 2, 2, 2]               # t: an image has one temporal step
    assert pos[1, 0, 2:6].tolist() == [2, 2, 3, 3]               # rows
    assert pos[2, 0, 2:6].tolist() == [2, 3, 2, 3]               # columns
    assert pos[:, 0, 6:].tolist() == [[4, 5]] * 3                # text continues after the largest position
    # text only, left padding
    ids = torch.tensor([[0, 0, 5, 6, 7]])
    pos = multimodal_positions(ids, None, None, None, torch.tensor([[0, 0, 1, 1, 1]]), cfg)
    assert pos[0, 0].tolist() == [1, 1, 0, 1, 2]


def test_vision_language_model_matches_transformers():
    mod = pytest.importorskip("transformers.models.qwen2_5_vl.modeling_qwen2_5_vl")
    cmod = pytest.importorskip("transformers.models.qwen2_5_vl.configuration_qwen2_5_vl")
    cfg = _cfg()
    t, v = cfg.text, cfg.vision
    try:
        hf_cfg = cmod.Qwen2_5_VLConfig(
            text_config=dict(vocab_size=t.vocab_size, hidden_size=t.hidden_size, intermediate_size=t.intermediate_size,
                             num_hidden_layers=t.num_hidden_layers, num_attention_heads=t.num_attention_heads,
                             num_key_value_heads=t.num_key_value_heads, rms_norm_eps=t.rms_norm_eps, rope_theta=t.rope_theta,
                             rope_scaling={"type": "mrope", "mrope_section": list(cfg.mrope_section)}, max_position_embeddings=4096,
                             use_sliding_window=False),
            vision_config=dict(depth=v.depth, hidden_size=v.hidden_size, intermediate_size=v.intermediate_size, num_heads=v.num_heads,
                               out_hidden_size=v.out_hidden_size, fullatt_block_indexes=v.fullatt_block_indexes, hidden_act="silu"),
            image_token_id=IMG, video_token_id=VID, vision_start_token_id=START)
        hf_cfg._attn_implementation = "eager"
        torch.manual_seed(0)
        hf = mod.Qwen2_5_VLModel(hf_cfg).eval().float()
    except Exception as e:   # the configuration schema of this wrapper differs between transformers releases
        pytest.skip(f"cannot build the transformers model: {e!r}")
    for p in hf.parameters():
        torch.nn.init.normal_(p, std=0.05) if p.dim() > 1 else torch.nn.init.normal_(p, mean=0.5, std=0.2)
    ours = QwenVLModel(cfg).eval()
    ours.load_hf_state_dict(hf.state_dict())
    grid = torch.tensor([[1, 4, 8]])
    n_img = 1 * 2 * 4
    ids = torch.tensor([[21, 22, START] + [IMG] * n_img + [23, 24, 25]])
    patches = torch.randn(32, 3 * 2 * 14 * 14)
    with torch.no_grad():
        # The positions are passed in explicitly: the rule under test is the reference's (an image's temporal component is the
        # position where its block starts, cosmos_reason1 qwen2_5_vl.py:1692-1728; checked by hand in the test above), and
        # transformers releases differ from one another in that component. Everything else - feature scatter, rotary
        # sections, both towers - is compared.
        pos = multimodal_positions(ids, grid, None, None, None, cfg)
        try:
            want = hf(input_ids=ids, pixel_values=patches, image_grid_thw=grid, position_ids=pos, output_hidden_states=True)
        except Exception as e:
            pytest.skip(f"the transformers forward does not take these arguments: {e!r}")
        got = ours(ids, pixel_values=patches, image_grid_thw=grid)
    hs = want.hidden_states
    assert len(hs) == len(got)
    for i, (a, b) in enumerate(zip(got, hs)):
        assert torch.allclose(a, b, atol=2e-4, rtol=2e-3), (i, (a - b).abs().max())
