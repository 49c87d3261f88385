"""T5 encoder tower and OpenAI-CLIP image tower against the transformers implementations on the same random weights."""

import pytest
import torch


@pytest.mark.parametrize("ff", ["relu", "gated-gelu"])
def test_t5_encoder_matches_transformers(ff):
    transformers = pytest.importorskip("transformers")
    from cosmos_predict25_b200.models.t5_xxl import T5Config, T5Encoder, T5EncoderTower
    torch.manual_seed(0)
    hf_cfg = transformers.T5Config(vocab_size=100, d_model=32, d_kv=8, num_heads=4, d_ff=64, num_layers=3, relative_attention_num_buckets=8,
                                   relative_attention_max_distance=16, feed_forward_proj=ff, dropout_rate=0.0)
    hf = transformers.T5EncoderModel(hf_cfg).eval()
    tower = T5EncoderTower(T5Config(vocab_size=100, d_model=32, d_kv=8, num_heads=4, d_ff=64, num_layers=3, num_buckets=8, max_distance=16,
                                    feed_forward=ff))
    tower.load_hf_state_dict(hf.state_dict())
    ids = torch.randint(0, 100, (2, 12))
    mask = torch.ones(2, 12, dtype=torch.long)
    mask[1, 7:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got = tower(ids, mask)
    assert torch.allclose(got[0], want[0], atol=1e-5) and torch.allclose(got[1, :7], want[1, :7], atol=1e-5)

    class _Tok:
        def __call__(self, texts, **kw):
            return {"input_ids": ids, "attention_mask": mask}
    emb, m = T5Encoder(tower, _Tok(), max_seq_len=10, model_seq_len=12).encode(["a", "b"])
    assert emb.shape == (2, 10, 32) and m.shape == (2, 10) and emb[1, 7:].abs().max() == 0 and torch.allclose(emb[0], want[0, :10], atol=1e-5)


def _openai_names(hf_sd, layers_v, layers_t):
    """transformers CLIPModel state dict -> the names of the released OpenAI checkpoints."""
    sd = {}

    def blocks(src, dst, n):
        for i in range(n):
            s, d = f"{src}.encoder.layers.{i}", f"{dst}.resblocks.{i}"
            sd[f"{d}.attn.in_proj_weight"] = torch.cat([hf_sd[f"{s}.self_attn.{p}_proj.weight"] for p in "qkv"])
            sd[f"{d}.attn.in_proj_bias"] = torch.cat([hf_sd[f"{s}.self_attn.{p}_proj.bias"] for p in "qkv"])
            for a, b in (("self_attn.out_proj", "attn.out_proj"), ("layer_norm1", "ln_1"), ("layer_norm2", "ln_2"), ("mlp.fc1", "mlp.c_fc"),
                         ("mlp.fc2", "mlp.c_proj")):
                for w in ("weight", "bias"):
                    sd[f"{d}.{b}.{w}"] = hf_sd[f"{s}.{a}.{w}"]
    blocks("vision_model", "visual.transformer", layers_v)
    blocks("text_model", "transformer", layers_t)
    sd["visual.conv1.weight"] = hf_sd["vision_model.embeddings.patch_embedding.weight"]
    sd["visual.class_embedding"] = hf_sd["vision_model.embeddings.class_embedding"]
    sd["visual.positional_embedding"] = hf_sd["vision_model.embeddings.position_embedding.weight"]
    for a, b in (("pre_layrnorm", "ln_pre"), ("post_layernorm", "ln_post")):
        for w in ("weight", "bias"):
            sd[f"visual.{b}.{w}"] = hf_sd[f"vision_model.{a}.{w}"]
    sd["visual.proj"] = hf_sd["visual_projection.weight"].t()
    sd["token_embedding.weight"] = hf_sd["text_model.embeddings.token_embedding.weight"]
    sd["positional_embedding"] = hf_sd["text_model.embeddings.position_embedding.weight"]
    for w in ("weight", "bias"):
        sd[f"ln_final.{w}"] = hf_sd[f"text_model.final_layer_norm.{w}"]
    sd["text_projection"] = hf_sd["text_projection.weight"].t()
    sd["logit_scale"] = hf_sd["logit_scale"]
    return sd


def test_openai_clip_matches_transformers():
    transformers = pytest.importorskip("transformers")
    from cosmos_predict25_b200.models.clip_openai import build_model
    torch.manual_seed(0)
    cfg = transformers.CLIPConfig(
        text_config=dict(vocab_size=99, hidden_size=64, intermediate_size=256, num_hidden_layers=2, num_attention_heads=1,
                         max_position_embeddings=16, hidden_act="quick_gelu", eos_token_id=98, bos_token_id=97, pad_token_id=0),
        vision_config=dict(hidden_size=128, intermediate_size=512, num_hidden_layers=2, num_attention_heads=2, image_size=32, patch_size=8,
                           hidden_act="quick_gelu"),
        projection_dim=48)
    hf = transformers.CLIPModel(cfg).eval()
    hf_sd = {k: v for k, v in hf.state_dict().items() if "position_ids" not in k}
    model = build_model({k: v.clone() for k, v in _openai_names(hf_sd, 2, 2).items()})
    assert model.visual.input_resolution == 32 and model.context_length == 16 and len(model.visual.transformer.resblocks) == 2
    image = torch.randn(2, 3, 32, 32)
    text = torch.randint(1, 97, (2, 16))
    text[0, 9], text[1, 15] = 98, 98                    # end-of-text = the largest id
    with torch.no_grad():
        want_i = hf.get_image_features(pixel_values=image)
        want_t = hf.get_text_features(input_ids=text)
        want_i = getattr(want_i, "pooler_output", want_i)
        want_t = getattr(want_t, "pooler_output", want_t)
        got_i, got_t = model.encode_image(image), model.encode_text(text)
        li, lt = model(image, text)
    assert torch.allclose(got_i, want_i, atol=1e-4), (got_i - want_i).abs().max()
    assert torch.allclose(got_t, want_t, atol=1e-4), (got_t - want_t).abs().max()
    assert li.shape == (2, 2) and torch.allclose(li, lt.t())


def test_t5_embedding_helper_matches_transformers(tmp_path):
    """``CosmosT5TextEncoder`` on a checkpoint directory written by transformers: embeddings equal the transformers encoder's,
    padded positions are zero, the mask comes back on request, an empty list is refused."""
    import pytest
    import sentencepiece as spm
    from transformers import T5Config as HFConfig, T5EncoderModel, T5TokenizerFast
    from cosmos_predict25_b200.pipeline.get_t5_emb import CosmosT5TextEncoder, get_text_embedding
    d = tmp_path / "t5"
    d.mkdir()
    (d / "c.txt").write_text("\n".join(["a red car drives", "the robot arm moves left", "people walk in the rain"] * 30))
    spm.SentencePieceTrainer.train(input=str(d / "c.txt"), model_prefix=str(d / "spiece"), vocab_size=48, model_type="unigram", pad_id=0,
                                   eos_id=1, unk_id=2, bos_id=-1, hard_vocab_limit=False, minloglevel=2)
    tok = T5TokenizerFast(vocab_file=str(d / "spiece.model"), extra_ids=0)
    tok.save_pretrained(str(d))
    torch.manual_seed(0)
    hf = T5EncoderModel(HFConfig(vocab_size=64, d_model=64, d_kv=8, num_heads=4, d_ff=128, num_layers=2, feed_forward_proj="gated-gelu")).eval()
    hf.save_pretrained(str(d))
    enc = CosmosT5TextEncoder(model_name=str(d), device="cpu")
    prompts = ["a red car drives in the rain", "people walk"]
    out, mask = enc.encode_prompts(prompts, max_length=24, return_mask=True)
    ids = tok(prompts, return_tensors="pt", padding="max_length", max_length=24, truncation=True)
    with torch.no_grad():
        want = hf(**ids).last_hidden_state * ids["attention_mask"].unsqueeze(-1)
    assert out.shape == (2, 24, 64) and mask.dtype == torch.bool and torch.equal(mask, ids["attention_mask"].bool())
    assert torch.allclose(out, want, atol=1e-5) and out[1, int(mask[1].sum()):].abs().max() == 0
    assert torch.equal(get_text_embedding("people walk", encoder=enc, device="cpu", max_length=24), out[1:2])
    with pytest.raises(ValueError, match="empty"):
        enc.encode_prompts([])
    with pytest.raises(FileNotFoundError):
        CosmosT5TextEncoder(model_name="no/such-model", device="cpu", local_files_only=True)
