"""Wan2.1 network and model (CPU)."""
import torch

from cosmos_predict25_b200.models import wan2pt1 as wan


def test_interleaved_rope_is_a_rotation_and_relative():
    torch.manual_seed(0)
    rope = wan.WanRope3D(32)
    ang = rope.generate(2, 3, 3, "cpu")
    assert ang.shape == (18, 16)
    q, k = torch.randn(1, 18, 2, 32), torch.randn(1, 18, 2, 32)
    qr, kr = wan.rope_apply_interleaved(q, ang), wan.rope_apply_interleaved(k, ang)
    assert torch.allclose(qr.norm(dim=-1), q.norm(dim=-1), atol=1e-4)
    # same position -> inner product unchanged
    assert torch.allclose((qr * kr).sum(-1), (q * k).sum(-1), atol=1e-4)
    # complex-number formulation (pairs (2i, 2i+1))
    z = torch.view_as_complex(q.float().reshape(1, 18, 2, 16, 2)) * torch.polar(torch.ones_like(ang), ang)[None, :, None, :]
    assert torch.allclose(torch.view_as_real(z).flatten(3), qr, atol=1e-5)


def test_wan_t2v_forward_backward_and_names():
    torch.manual_seed(0)
    net = wan.WanModel(wan.wan_tiny())
    net.init_weights()
    keys = set(net.state_dict())
    for k in ("patch_embedding.weight", "text_embedding.0.weight", "time_embedding.2.bias", "time_projection.1.weight",
              "blocks.0.self_attn.q.weight", "blocks.0.self_attn.norm_q.weight", "blocks.1.cross_attn.o.bias", "blocks.0.norm3.weight",
              "blocks.0.ffn.0.weight", "blocks.0.modulation", "head.head.weight", "head.modulation"):
        assert k in keys, k
    x = torch.randn(2, 16, 3, 8, 8)
    y = net(x, torch.tensor([[100.0], [900.0]]), torch.randn(2, 512, 64))
    assert y.shape == x.shape
    y.square().mean().backward()
    assert all(p.grad is not None for p in net.parameters())


def test_wan_i2v_uses_image_tokens():
    torch.manual_seed(0)
    net = wan.WanModel(wan.wan_tiny(model_type="i2v", in_dim=36))
    net.init_weights()
    x, yc = torch.randn(1, 16, 2, 8, 8), torch.randn(1, 20, 2, 8, 8)
    t, txt = torch.tensor([[500.0]]), torch.randn(1, 512, 64)
    img = torch.randn(1, 257, 1280)
    with torch.no_grad():
        a = net(x, t, txt, frame_cond_crossattn_emb_B_L_D=img, y_B_C_T_H_W=yc)
        b = net(x, t, txt, frame_cond_crossattn_emb_B_L_D=img + 1.0, y_B_C_T_H_W=yc)
    assert a.shape == x.shape and (a - b).abs().max() > 1e-6


def test_wan_rf_model_training_and_sampling():
    torch.manual_seed(0)
    cfg = wan.WanRFConfig(net=wan.wan_tiny(), precision="float32")
    m = wan.WANDiffusionModel(cfg, device=torch.device("cpu"))
    batch = {"latents": torch.randn(1, 16, 2, 8, 8), "t5_text_embeddings": torch.randn(1, 512, 64), "fps": torch.tensor([16.0]),
             "padding_mask": torch.zeros(1, 1, 8, 8)}
    out, loss = m.training_step(dict(batch), 0)
    assert torch.isfinite(loss)
    loss.backward()
    x = m.generate_samples_from_batch(dict(batch), guidance=2.0, num_steps=2)
    assert x.shape == (1, 16, 2, 8, 8) and torch.isfinite(x).all()


def test_clip_vision_tower_and_i2v_embedder():
    from cosmos_predict25_b200.models import wan_encoders as we
    torch.manual_seed(0)
    clip = we.XLMRobertaCLIP(embed_dim=32, image_size=28, patch_size=14, vision_dim=1280, vision_heads=4, vision_layers=2,
                             text_dim=32, text_heads=4, text_layers=1, vocab_size=100, max_text_len=20)
    assert "visual.transformer.0.attn.to_qkv.weight" in clip.state_dict() and "textual.blocks.0.attn.q.weight" in clip.state_dict()
    cm = we.CLIPModel(dtype=torch.float32, model=clip)
    tok = cm.visual(torch.rand(2, 3, 40, 56) * 2 - 1)
    assert tok.shape == (2, 5, 1280)
    img, txt = clip(torch.randn(1, 3, 28, 28), torch.tensor([[0, 5, 6, 2, 1, 1]]))
    assert img.shape == (1, 32) and txt.shape == (1, 32)
    emb = we.Wan2pt1CLIPEmb(num_token=5, dtype="float32", clip_model=cm)
    out = emb(None, torch.rand(1, 3, 5, 28, 28), torch.randn(1, 16, 2, 4, 4))
    assert out["y_B_C_T_H_W"].shape == (1, 20, 2, 4, 4) and out["y_B_C_T_H_W"][0, :4, 0].min() == 1 and out["y_B_C_T_H_W"][0, :4, 1].max() == 0
    assert out["frame_cond_crossattn_emb_B_L_D"].shape == (1, 5, 1280)
    out_img = emb(torch.rand(1, 3, 1, 28, 28), None, torch.randn(1, 16, 1, 4, 4))
    assert out_img["frame_cond_crossattn_emb_B_L_D"].abs().sum() == 0


def test_umt5_encoder_masks_padding():
    from cosmos_predict25_b200.models import wan_encoders as we
    torch.manual_seed(0)
    enc = we.UMT5Encoder(vocab=50, dim=32, dim_attn=32, dim_ffn=64, num_heads=4, num_layers=2, num_buckets=8)
    ids = torch.tensor([[3, 4, 5, 0, 0, 0]])
    mask = torch.tensor([[1, 1, 1, 0, 0, 0]])
    a = enc(ids, mask)
    ids2 = ids.clone()
    ids2[0, 4] = 7                       # a padded position must not influence valid positions
    b = enc(ids2, mask)
    assert torch.allclose(a[:, :3], b[:, :3], atol=1e-6)
    rel = we.T5RelativeEmbedding(8, 4)
    assert rel(5, 5).shape == (1, 4, 5, 5)
    assert "blocks.0.pos_embedding.embedding.weight" in enc.state_dict() and "blocks.1.ffn.gate.0.weight" in enc.state_dict()
