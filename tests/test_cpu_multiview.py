"""Multiview DiT / model (CPU)."""
import pytest
import torch

from cosmos_predict25_b200.models import multiview as mv
from cosmos_predict25_b200.models.multiview_dit import MultiViewDiT, multiview_dit_tiny


def _batch(B=1, V=3, state_t=2, H=8, W=8, M=8, ctx=256):
    return {"latents": torch.randn(B, 16, V * state_t, H, W), "t5_text_embeddings": torch.randn(B, V * M, ctx),
            "fps": torch.full((B,), 10.0), "padding_mask": torch.zeros(B, 1, H, W)}


def _model(**kw):
    cfg = mv.MultiviewRFConfig(net=multiview_dit_tiny(), precision="float32", state_t=2, tokens_per_view=8, **kw)
    return mv.MultiviewVid2VidModelRectifiedFlow(cfg, device=torch.device("cpu"))


def test_cross_attention_is_per_view():
    torch.manual_seed(0)
    net = MultiViewDiT(multiview_dit_tiny())
    net.init_weights()
    for blk in net.blocks:
        for m in (blk.adaln_modulation_self_attn, blk.adaln_modulation_cross_attn, blk.adaln_modulation_mlp):
            torch.nn.init.normal_(m[-1].weight, std=0.05)
    b = _batch(V=2)
    x, ctx = b["latents"], b["t5_text_embeddings"]
    t = torch.full((1, 1), 300.0)
    with torch.no_grad():
        y0 = net(x, t, ctx, fps=b["fps"], padding_mask=b["padding_mask"])
        ctx2 = ctx.clone()
        ctx2[:, 8:] += 1.0            # change the caption of view 1 only
        blk = net.blocks[0]
        h = torch.randn(1, 2 * 2 * 16, 256)
        o0 = blk.cross_attn(h, ctx)
        o1 = blk.cross_attn(h, ctx2)
    assert torch.allclose(o0[:, :32], o1[:, :32], atol=1e-6)      # view 0 tokens do not see view 1's caption
    assert (o0[:, 32:] - o1[:, 32:]).abs().max() > 1e-4
    assert y0.shape == x.shape


def test_rope_restarts_per_camera():
    net = MultiViewDiT(multiview_dit_tiny())
    r = net._rope(6, 4, 4, None)          # 3 views x 2 frames
    per = 2 * 16
    assert r.shape[0] == 3 * per
    assert torch.equal(r[:per], r[per:2 * per]) and torch.equal(r[:per], r[2 * per:])


def test_condition_locations():
    c = mv.MultiViewCondition(ref_cam_view_idx_sample_position=torch.tensor([1]),
                              view_indices_B_T=torch.arange(3).repeat_interleave(2)[None])
    gt = torch.randn(2, 16, 6, 4, 4)
    m = c.set_video_condition(2, gt, ["first_random_n"], num_conditional_frames_per_view=1).condition_video_input_mask_B_C_T_H_W
    assert m[:, 0, :, 0, 0].tolist() == [[1, 0, 1, 0, 1, 0]] * 2
    m = c.set_video_condition(2, gt, ["ref_cam"]).condition_video_input_mask_B_C_T_H_W
    assert m[0, 0, :, 0, 0].tolist() == [0, 0, 1, 1, 0, 0]
    m = c.set_video_condition(2, gt, ["any_cam", "first_random_n"], 1, 1, condition_cam_idx=2).condition_video_input_mask_B_C_T_H_W
    assert m[0, 0, :, 0, 0].tolist() == [1, 0, 1, 0, 1, 1]
    with pytest.raises(ValueError):
        mv.validate_condition_locations(["no_cam", "ref_cam"])
    with pytest.raises(ValueError):
        mv.validate_condition_locations(["any_cam", "ref_cam"])


def test_apg_reduces_to_cfg():
    c, u = torch.randn(2, 4, 3, 5, 5), torch.randn(2, 4, 3, 5, 5)
    out = mv.adaptive_projected_guidance(c, u, 3.0, eta=1.0)
    assert torch.allclose(out, c + 2.0 * (c - u), atol=1e-5)
    out0 = mv.adaptive_projected_guidance(c, u, 3.0, eta=0.0)
    par, orth = mv.project(c - u, c)
    assert torch.allclose(out0, c + 2.0 * orth, atol=1e-5)
    assert abs(float((orth * c).sum())) < 1e-3


def test_multiview_training_and_sampling():
    torch.manual_seed(0)
    m = _model()
    out, loss = m.training_step(_batch(B=2), 0)
    assert torch.isfinite(loss)
    loss.backward()
    assert m.net.view_embeddings.weight.grad is not None
    b = _batch(B=1)
    b["num_conditional_frames"] = 1
    x = m.generate_samples_from_batch(b, guidance=3.0, num_steps=3)
    assert x.shape == (1, 16, 6, 8, 8)
    # the first latent frame of every view is the clean condition
    for v in range(3):
        assert torch.allclose(x[:, :, 2 * v], b["latents"][:, :, 2 * v], atol=5e-3)
    m2 = _model(use_apg=True)
    x2 = m2.generate_samples_from_batch(b, guidance=3.0, num_steps=2)
    assert torch.isfinite(x2).all()


def test_view_subsampling():
    m = _model(train_sample_views_range=(2, 2))
    b = _batch(B=1)
    b.update(sample_n_views=torch.tensor(3), num_video_frames_per_view=torch.tensor(5),
             view_indices=torch.arange(3).repeat_interleave(5)[None], ai_caption=["a -- b -- c"])
    out = m.with_latent_view_indices(b)
    assert out["latents"].shape[2] == 4 and out["t5_text_embeddings"].shape[1] == 16
    assert out["ai_caption"] == ["a -- b"] and out["latent_view_indices_B_T"].tolist() == [[0, 0, 1, 1]]


def test_multiview_public_api_end_to_end(tmp_path):
    """experiment name -> model -> local per-camera files -> sample -> mp4, with a stand-in decoder (no codec needed)."""
    import numpy as np

    from cosmos_predict25_b200.multiview import MultiviewInference
    from cosmos_predict25_b200.multiview_config import MultiviewInferenceArguments, MultiviewSetupArguments
    from cosmos_predict25_b200.pipeline.multiview import Vid2VidInference

    pipe = Vid2VidInference("tiny_multiview_cpu", None, device=torch.device("cpu"))
    assert type(pipe.model).__name__ == "MultiviewVid2VidModelRectifiedFlow"
    files = {}
    for cam in ("front_wide", "cross_right", "rear_right"):
        p = tmp_path / f"{cam}.mp4"
        p.write_bytes(cam.encode())
        files[cam] = {"video_path": str(p)}
    setup = MultiviewSetupArguments(output_dir=tmp_path / "out", experiment="tiny_multiview_cpu", checkpoint_path="none",
                                    context_parallel_size=1)
    args = MultiviewInferenceArguments(prompt="a drive through town", n_views=3, num_input_frames=1, num_steps=2, guidance=3, **files)

    def fake_decode(raw: bytes):
        rng = np.random.default_rng(len(raw))
        return rng.integers(0, 255, size=(12, 36, 64, 3), dtype=np.uint8), 30.0

    torch.manual_seed(0)
    grad_was = torch.is_grad_enabled()
    try:
        outs = MultiviewInference(setup, pipe=pipe).generate(args, decode_fn=fake_decode)
    finally:
        torch.set_grad_enabled(grad_was)
    assert len(outs) == 1 and (tmp_path / "out" / "config.yaml").exists()


def test_multiview_experiments_registered():
    from cosmos_predict25_b200.configs import multiview as cfgmod
    from cosmos_predict25_b200.utils.checkpoint_db import get_checkpoint_by_uuid
    from cosmos_predict25_b200.utils.config import override
    ck = get_checkpoint_by_uuid("6b9d7548-33bb-4517-b5e8-60caf47edba7")
    cfg = override(cfgmod.make_config(), ["--", f"experiment={ck.experiment}"])
    assert cfg["model"]["config"]["state_t"] == 8
    assert cfg["model"]["config"]["net"]["rope_enable_fps_modulation"] is False
    assert cfg["model_parallel"]["context_parallel_size"] == 8


def test_noise_level_multiview_model_trains_samples_and_switches_to_projected_guidance():
    """The EDM-era multi-camera model: loss and gradients, sampling with every view's first latent frame given (returned at the
    model's data scale), and a batch that asks for projected guidance takes that route (its result differs from plain guidance
    and, with momentum 0 / eta 1 / no norm limit, equals plain guidance with scale g - 1)."""
    torch.manual_seed(0)
    cfg = mv.MultiviewVid2VidModelConfig(net=multiview_dit_tiny(), precision="float32", state_t=2, tokens_per_view=8,
                                         condition_locations=["first_random_n"])
    m = mv.MultiviewVid2VidModel(cfg, device=torch.device("cpu"))
    with torch.no_grad():
        for p in m.net.parameters():
            if p.abs().max() == 0:
                p.normal_(0, 0.05)
    out, loss = m.training_step(_batch(B=2), 0)
    assert torch.isfinite(loss) and out["model_pred"].shape == (2, 16, 6, 8, 8)
    loss.backward()
    assert m.net.view_embeddings.weight.grad is not None
    b = _batch(B=1)
    b["num_conditional_frames"] = 1
    x = m.generate_samples_from_batch(dict(b), guidance=2.0, num_steps=3, seed=5)
    assert x.shape == (1, 16, 6, 8, 8)
    for v in range(3):
        assert torch.allclose(x[:, :, 2 * v], b["latents"][:, :, 2 * v] * m.sigma_data, atol=1e-4)
    xa = m.generate_samples_from_batch({**b, "use_apg": True}, guidance=2.0, num_steps=3, seed=5)
    assert torch.isfinite(xa).all() and (xa - x).abs().max() > 1e-5
    m.config.apg_momentum, m.config.apg_eta, m.config.apg_norm_threshold = 0.0, 1.0, 0.0
    xb = m.generate_samples_from_batch({**b, "use_apg": True}, guidance=3.0, num_steps=3, seed=5)
    assert torch.allclose(xb, x, atol=1e-4)


def test_prompt_embeddings_computed_online_per_view():
    """One caption: the front camera's slot gets the prompt, the others the blank prompt; the negative prompt goes to the same
    slot. V captions joined by `` -- ``: one per view, and the negative prompt for every view."""
    from cosmos_predict25_b200.models.text_encoder import HashTextEncoder
    enc = HashTextEncoder(256, 8, dtype=torch.float32)
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    m = _model(text_encoder=enc, tokenizer=DummyTokenizer())
    fpv = m._pixel_frames_per_view()
    blank, neg = m.empty_string_text_embeddings, m.neg_text_embeddings
    assert blank.shape == neg.shape == (1, 8, 256)
    batch = {"video": torch.zeros(2, 3, 3 * fpv, 8, 8, dtype=torch.uint8), "num_video_frames_per_view": torch.tensor(fpv),
             "ai_caption": ["a red car", "a bus"], "front_cam_view_idx_sample_position": torch.tensor([1, 2])}
    pos, negative, dropped = m.compute_text_embeddings_online_multiview(batch)
    assert pos.shape == negative.shape == dropped.shape == (2, 24, 256)
    want = enc.compute_text_embeddings_online({"ai_caption": ["a red car", "a bus"]})
    assert torch.equal(pos[0, 8:16], want[0]) and torch.equal(pos[1, 16:24], want[1])
    assert torch.equal(pos[0, :8], blank[0]) and torch.equal(pos[1, :8], blank[0]) and torch.equal(pos[0, 16:], blank[0])
    assert torch.equal(negative[0, 8:16], neg[0]) and torch.equal(negative[0, :8], blank[0])
    assert dropped.abs().max() == 0                                   # the text embedder drops to zeros unless told otherwise
    m.conditioner.embedders["text"].use_empty_string = True
    assert torch.equal(m.compute_text_embeddings_online_multiview(batch)[2], blank.repeat(2, 3, 1))
    one = {**batch, "video": batch["video"][:1], "ai_caption": ["front -- left -- right"]}
    pos, negative, _ = m.compute_text_embeddings_online_multiview(one)
    per_view = torch.cat([enc.compute_text_embeddings_online({"ai_caption": [c]}) for c in ("front", "left", "right")], 1)
    assert torch.equal(pos, per_view) and torch.equal(negative, neg.repeat(1, 3, 1))
    m.inplace_compute_text_embeddings_online(one)
    assert torch.equal(one["t5_text_embeddings"], per_view) and one["t5_text_mask"].shape == (1, 24)
    with pytest.raises(AssertionError):
        m.compute_text_embeddings_online_multiview({**one, "ai_caption": ["a -- b"]})


def test_text_dropout_to_the_blank_prompt():
    from cosmos_predict25_b200.models.conditioner import TextAttr, TextAttrEmptyStringDrop
    torch.manual_seed(0)
    x, blank = torch.randn(64, 4, 8), torch.randn(1, 4, 8)
    t = TextAttr(dropout_rate=0.5, use_empty_string=True)
    with pytest.raises(ValueError):
        t.random_dropout_input(x)
    t.set_empty_string_embeddings(blank)
    y = t.random_dropout_input(x)
    kept = (y == x).flatten(1).all(1)
    assert 10 < kept.sum() < 54 and torch.equal(y[~kept], blank.expand(int((~kept).sum()), -1, -1))
    assert t.random_dropout_input(x, key="t5_text_mask") is x          # masks are never dropped
    d = TextAttrEmptyStringDrop(dropout_rate=1.0)
    d.set_empty_string_embeddings(blank[0])                           # a 2-d file content is given its batch axis
    assert torch.equal(d.random_dropout_input(x), blank.expand(64, -1, -1))
    z = TextAttr(dropout_rate=1.0).random_dropout_input(x)
    assert z.abs().max() == 0


def test_noise_level_multiview_experiments_and_model_groups():
    """The predict2.1-era experiment names resolve to the noise-level model with the base run's settings; the tiny twin builds from
    its config and takes a training step on the mock multi-camera data; the model groups swap the model class."""
    from cosmos_predict25_b200.configs import multiview as cfgmod
    from cosmos_predict25_b200.utils.config import override
    from cosmos_predict25_b200.utils.lazy_config import instantiate
    name = "buttercup_predict2p1_2b_mv_7views_res720p_fps10_t8_from23klr1x_jointalpamayov2mads720p_lr2x"
    cfg = override(cfgmod.make_config(), ["--", f"experiment={name}"])
    mc = cfg["model"]["config"]
    assert mc["scaling"] == "rectified_flow" and mc["sigma_data"] == 1.0 and mc["rectified_flow_loss_weight_uniform"] is False
    assert mc["net"]["timestep_scale"] == 1.0 and mc["net"]["n_cameras_emb"] == 7 and cfg["optimizer"]["lr"] == 2 ** -13.5
    assert "MultiviewVid2VidModel" in str(cfg["model"]["_target_"]) and "RectifiedFlow" not in str(cfg["model"]["_target_"])
    cfg = override(cfgmod.make_config(), ["--", "model=fsdp_multiview"])
    assert cfg["model"]["config"]["fsdp_shard_size"] == 8 and cfg["trainer"]["distributed_parallelism"] == "fsdp"
    cfg = override(cfgmod.make_config(), ["--", "model=fsdp_rectified_flow_multiview"])
    assert "RectifiedFlow" in str(cfg["model"]["_target_"])
    cfg = override(cfgmod.make_config(), ["--", "experiment=tiny_multiview_edm_cpu"])
    model = instantiate(cfg["model"])
    assert type(model).__name__ == "MultiviewVid2VidModel"
    loader = instantiate(cfg["dataloader_train"])
    batch = next(iter(loader))
    torch.manual_seed(0)
    _, loss = model.training_step(batch, 0)
    assert torch.isfinite(loss)
