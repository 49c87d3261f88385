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
