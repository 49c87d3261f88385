"""Numerical parity with the reference implementation's own code, run unmodified as the oracle (skipped where no copy of the
reference is present or a module of it cannot be imported)."""

import torch

from reference_oracle import import_reference


def test_wan_vae_encode_decode_match_the_reference():
    """Same random weights in the reference's causal video VAE and this package's: latents and reconstructions agree, for a clip
    that needs two streaming chunks and for a single image."""
    ref_mod = import_reference("cosmos_predict2._src.predict2.tokenizers.wan2pt1")
    from cosmos_predict25_b200.models.vae_wan import WanVAE_
    torch.manual_seed(0)
    kw = dict(dim=16, z_dim=4, dim_mult=[1, 2, 4, 4], num_res_blocks=1, attn_scales=[], temperal_downsample=[False, True, True], dropout=0.0)
    ref = ref_mod.WanVAE_(**kw).eval()
    ours = WanVAE_(**kw).eval()
    missing = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not missing.missing_keys and not missing.unexpected_keys
    scale = [torch.linspace(-0.5, 0.5, 4), 1.0 / torch.linspace(0.5, 2.0, 4)]
    with torch.no_grad():
        for T in (9, 1):
            x = torch.randn(1, 3, T, 32, 32)
            mu_ref = ref.encode(x, scale)
            mu = ours.encode(x, scale)
            assert mu.shape == mu_ref.shape == (1, 4, 1 + (T - 1) // 4, 4, 4)
            assert torch.allclose(mu, mu_ref, atol=1e-4), (mu - mu_ref).abs().max()
            rec_ref = ref.decode(mu_ref, scale)
            rec = ours.decode(mu_ref, scale)
            assert rec.shape == rec_ref.shape == x.shape
            assert torch.allclose(rec, rec_ref, atol=1e-4), (rec - rec_ref).abs().max()


def _net_pair(**extra):
    from reference_oracle import reference_network_modules
    from cosmos_predict25_b200.models.dit import CosmosDiT, DiTConfig
    lvg, _ = reference_network_modules()
    torch.manual_seed(0)
    kw = dict(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
              concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, crossattn_emb_channels=64,
              use_crossattn_projection=True, crossattn_proj_in_channels=96, pos_emb_cls="rope3d", use_adaln_lora=True, adaln_lora_dim=32,
              rope_h_extrapolation_ratio=3.0, rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0,
              rope_enable_fps_modulation=False, use_wan_fp32_strategy=True, timestep_scale=0.001)
    kw.update(extra)
    ref = lvg.MinimalV1LVGDiT(atten_backend="minimal_a2a", **kw)
    ours = CosmosDiT(DiTConfig(**kw))
    with torch.no_grad():
        for p in ref.parameters():                       # the reference zero-initialises its output layers: make every weight count
            if p.abs().max() == 0:
                p.normal_(0, 0.02)
    res = ours.load_state_dict(ref.state_dict(), strict=True)      # same names, shapes and dtypes, buffers included
    assert not res.missing_keys and not res.unexpected_keys
    return ref, ours


def test_dit_forward_and_gradients_match_the_reference_network():
    """The reference's Video2World network (its file, unmodified) and this package's, same state dict, fp32 on the CPU: the
    velocity and the gradient of every parameter agree; with and without conditioning frames, image and video shapes."""
    ref, ours = _net_pair()
    torch.manual_seed(1)
    for T, n_cond in ((4, 1), (1, 0), (3, 2)):
        x = torch.randn(2, 16, T, 16, 12)
        t = torch.tensor([[600.0], [35.0]])
        ctx = torch.randn(2, 8, 96)
        mask = torch.zeros(2, 1, T, 16, 12)
        mask[:, :, :n_cond] = 1
        pad = torch.zeros(2, 1, 16, 12)
        y = ref(x, t, ctx, condition_video_input_mask_B_C_T_H_W=mask, fps=None, padding_mask=pad)
        z = ours(x, t, crossattn_emb=ctx, condition_video_input_mask_B_C_T_H_W=mask, padding_mask=pad)
        assert y.shape == z.shape == x.shape
        assert (y - z).abs().max().item() < 2e-5 * max(1.0, y.abs().max().item()), (y - z).abs().max()
    g = torch.randn_like(y)
    ref.zero_grad()
    ours.zero_grad()
    (y * g).sum().backward()
    (z * g).sum().backward()
    ref_grads = {n.replace("_checkpoint_wrapped_module.", ""): p.grad for n, p in ref.named_parameters()}
    n_checked = 0
    for n, p in ours.named_parameters():
        want = ref_grads[n]
        assert (p.grad is None) == (want is None), n
        if want is not None:
            assert (p.grad - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item()), (n, (p.grad - want).abs().max())
            n_checked += 1
    assert n_checked > 40


def test_unipc_solver_matches_the_reference_solver():
    """Same velocities fed to the reference's flow UniPC scheduler and to this package's solver: identical sigma tables and the same
    trajectory, for the production setting (35 steps, shift 5), a short run where the order drops at the end, and Karras sigmas."""
    import pytest
    from reference_oracle import install_diffusers_standins
    from cosmos_predict25_b200.models.schedulers import FlowUniPCSolver
    install_diffusers_standins()
    ref_mod = import_reference("cosmos_predict2._src.predict2.models.fm_solvers_unipc")
    for steps, shift, karras in ((35, 5.0, False), (4, 3.0, False), (12, 5.0, True)):
        ref = ref_mod.FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        ref.set_timesteps(steps, device="cpu", shift=shift, use_kerras_sigma=karras)
        ours = FlowUniPCSolver(1000, shift=1.0)
        ours.set_timesteps(steps, device="cpu", shift=shift, use_kerras_sigma=karras)
        assert torch.allclose(torch.as_tensor(ours.sigmas, dtype=torch.float32), ref.sigmas.float(), atol=1e-6)
        assert torch.allclose(torch.as_tensor(ours.timesteps).float(), ref.timesteps.float(), atol=1e-3)
        g = torch.Generator().manual_seed(steps)
        x_ref = x = torch.randn(1, 4, 3, 8, 8, generator=g)
        for t_ref, t in zip(ref.timesteps, torch.as_tensor(ours.timesteps).tolist()):
            v = torch.randn(x.shape, generator=g) + 0.3 * x_ref
            x_ref = ref.step(v, t_ref, x_ref, return_dict=False)[0]
            x = ours.step(v, t, x)
        err = (x - x_ref).abs().max().item()
        assert err < 2e-4 * max(1.0, x_ref.abs().max().item()), (steps, shift, karras, err)


def test_edm_scaling_sde_and_samplers_match_the_reference():
    """EDM-era pieces against the reference's files: preconditioning coefficients, noise marginal, the Karras grid, and whole
    sampling trajectories of the multistep ("2ab") and Runge-Kutta ("1euler", "2mid") solvers on a closed-form denoiser."""
    from cosmos_predict25_b200.models import edm
    ref_scale = import_reference("cosmos_predict2._src.common.modules.denoiser_scaling")
    ref_sde = import_reference("cosmos_predict2._src.common.modules.edm_sde")
    ref_samp = import_reference("cosmos_predict2._src.common.modules.res_sampler")
    sigma = torch.tensor([0.002, 0.3, 1.0, 7.5, 80.0])
    for a, b in zip(edm.EDMScaling(0.5)(sigma), ref_scale.EDMScaling(0.5)(sigma)):
        assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)
    for kw in (dict(sigma_data=1.0, t_scaling_factor=1.0, loss_weight_uniform=True), dict(sigma_data=1.0, t_scaling_factor=1000.0,
                                                                                        loss_weight_uniform=False)):
        ours, ref = edm.RectifiedFlowScaling(**kw), ref_scale.RectifiedFlowScaling(**kw)
        for a, b in zip(ours(sigma), ref(sigma)):
            assert torch.allclose(a, b, rtol=1e-6, atol=1e-7)
        assert torch.allclose(ours.sigma_loss_weights(sigma), ref.sigma_loss_weights(sigma), rtol=1e-6)
    x0 = torch.randn(5, 2, 3)
    for a, b in zip(edm.EDMSDE(-1.2, 1.2, 80.0, 0.002).marginal_prob(x0, sigma), ref_sde.EDMSDE(-1.2, 1.2, 80.0, 0.002).marginal_prob(x0, sigma)):
        assert torch.allclose(torch.as_tensor(a), torch.as_tensor(b))
    assert torch.allclose(torch.as_tensor(edm.get_rev_ts(0.002, 80.0, 9, 7.0)), ref_samp.get_rev_ts(0.002, 80.0, 9, 7.0).double(), rtol=1e-6)

    target = torch.randn(2, 4, 3, 3)

    def x0_fn(x, s):                                      # the exact denoiser of a Gaussian around ``target`` with unit prior variance
        w = 1.0 / (1.0 + s.view(-1, 1, 1, 1).to(x.dtype) ** 2)
        return w * x + (1 - w) * target.to(x.dtype)
    noise = torch.randn(2, 4, 3, 3) * 80.0
    for solver, steps in (("2ab", 12), ("1euler", 9), ("2mid", 10)):
        want = ref_samp.Sampler()(x0_fn, noise, num_steps=steps, sigma_max=80.0, sigma_min=0.002, solver_option=solver)
        got = edm.RESSampler()(x0_fn, noise, num_steps=steps, sigma_max=80.0, sigma_min=0.002, solver_option=solver)
        assert torch.allclose(got, want, atol=1e-5), (solver, (got - want).abs().max())


def test_lr_schedules_guidance_and_camera_math_match_the_reference():
    from cosmos_predict25_b200.models.multiview import MomentumBuffer, adaptive_projected_guidance
    from cosmos_predict25_b200.modules import camera as cam
    from cosmos_predict25_b200.modules import volume_render as vr
    from cosmos_predict25_b200.trainer import optim
    ref_lr = import_reference("cosmos_predict2._src.common.functional.lr_scheduler")
    args = dict(warm_up_steps=[10, 5], f_min=[0.1, 0.2], f_max=[1.0, 0.8], f_start=[0.01, 0.3], cycle_lengths=[50, 40])
    for name in ("LambdaLinearScheduler", "LambdaWarmUpCosineScheduler"):
        ours, ref = getattr(optim, name)(**args), getattr(ref_lr, name)(**args)
        for n in range(0, 90):
            assert abs(ours(n) - ref(n)) < 1e-9, (name, n, ours(n), ref(n))

    ref_cfg = import_reference("cosmos_predict2._src.predict2_multiview.models.cfg")
    torch.manual_seed(0)
    buf, ref_buf = MomentumBuffer(-0.5), ref_cfg.MomentumBuffer(-0.5)
    for _ in range(3):
        c, u = torch.randn(2, 4, 3, 5, 5), torch.randn(2, 4, 3, 5, 5)
        got = adaptive_projected_guidance(c, u, 4.0, buf, eta=0.3, norm_threshold=2.5)
        want = ref_cfg.adaptive_projected_guidance(c, u, 4.0, ref_buf, eta=0.3, norm_threshold=2.5)
        assert torch.allclose(got, want, atol=1e-6)

    ref_cam = import_reference("cosmos_predict2._src.imaginaire.modules.camera")
    q = ref_cam.Quaternion.normalize(torch.randn(6, 4))
    assert torch.allclose(cam.Quaternion.normalize(q * 3), q, atol=1e-6)
    R = ref_cam.Quaternion.to_rotation_matrix(q)
    assert torch.allclose(cam.Quaternion.to_rotation_matrix(q), R, atol=1e-6)
    assert torch.allclose(cam.Quaternion.from_rotation_matrix(R), ref_cam.Quaternion.from_rotation_matrix(R), atol=1e-5)
    assert torch.allclose(cam.Quaternion.multiply(q, q.flip(0)), ref_cam.Quaternion.multiply(q, q.flip(0)), atol=1e-6)
    pose = torch.cat([R, torch.randn(6, 3, 1)], -1)
    intr = torch.tensor([[[50.0, 0, 16], [0, 55.0, 12], [0, 0, 1]]]).repeat(6, 1, 1)
    assert torch.allclose(cam.Camera.invert_pose(pose), ref_cam.Camera.invert_pose(pose), atol=1e-5)
    assert torch.allclose(cam.Camera.compose_poses([pose, pose.flip(0)]), ref_cam.Camera.compose_poses([pose, pose.flip(0)]), atol=1e-5)
    for a, b in zip(cam.Camera.get_camera_rays(pose, intr, (24, 32)), ref_cam.Camera.get_camera_rays(pose, intr, (24, 32))):
        assert torch.allclose(a, b, atol=1e-5)
    assert torch.allclose(cam.Camera.get_plucker_rays(pose, intr, (24, 32)), ref_cam.Camera.get_plucker_rays(pose, intr, (24, 32)), atol=1e-5)
    assert torch.allclose(cam.Camera.get_relative_poses_wrt_frame0(pose), ref_cam.Camera.get_relative_poses_wrt_frame0(pose), atol=1e-5)
    params = ref_cam.Camera.extrinsic_matrices_to_params(pose)
    assert torch.allclose(cam.Camera.extrinsic_matrices_to_params(pose), params, atol=1e-5)
    assert torch.allclose(cam.Camera.extrinsic_params_to_matrices(params), ref_cam.Camera.extrinsic_params_to_matrices(params), atol=1e-5)
    assert torch.allclose(cam.Camera.intrinsic_matrices_to_params(intr), ref_cam.Camera.intrinsic_matrices_to_params(intr))

    ref_vr = import_reference("cosmos_predict2._src.imaginaire.modules.volume_render")
    near, far = torch.full((2, 7, 1), 0.5), torch.full((2, 7, 1), 4.0)
    dists = ref_vr.sample_dists(near, far, 9)
    assert torch.allclose(vr.sample_dists(near, far, 9), dists, atol=1e-6)
    dens = torch.rand(2, 7, 9, 1) * 3
    for dist_far in (None, torch.full((2, 7, 1, 1), 4.0)):
        alphas = ref_vr.volume_rendering_alphas(dens, dists[..., None], dist_far)
        assert torch.allclose(vr.volume_rendering_alphas(dens, dists[..., None], dist_far), alphas, atol=1e-6)
    w = ref_vr.alpha_compositing_weights(alphas)
    assert torch.allclose(vr.alpha_compositing_weights(alphas), w, atol=1e-6)
    rgb = torch.rand(2, 7, 9, 3)
    assert torch.allclose(vr.composite(rgb, w), ref_vr.composite(rgb, w), atol=1e-6)

    class _Field(torch.nn.Module):                        # a radiance field in closed form
        def forward(self, points, ray_unit):
            return torch.sigmoid(points), points.norm(dim=-1, keepdim=True)
    center, ray = torch.randn(2, 7, 3), torch.nn.functional.normalize(torch.randn(2, 7, 3), dim=-1)
    for a, b in zip(vr.volume_render_rays(_Field(), center, ray, near, far, 9), ref_vr.volume_render_rays(_Field(), center, ray, near, far, 9)):
        assert torch.allclose(a, b, atol=1e-5)


def test_wan22_vae_matches_the_reference():
    ref_mod = import_reference("cosmos_predict2._src.predict2.tokenizers.wan2pt2")
    from cosmos_predict25_b200.models.vae_wan22 import Wan22VAE_
    torch.manual_seed(0)
    kw = dict(dim=16, dec_dim=16, z_dim=8, dim_mult=[1, 2, 4, 4], num_res_blocks=1, attn_scales=[], temperal_downsample=[False, True, True])
    ref = ref_mod.WanVAE_(**kw).eval()
    ours = Wan22VAE_(**kw).eval()
    res = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    scale = [torch.linspace(-0.3, 0.3, 8), 1.0 / torch.linspace(0.5, 2.0, 8)]
    with torch.no_grad():
        for T in (5, 1):
            x = torch.randn(1, 3, T, 32, 32)
            mu_ref = ref.encode(x, scale)
            mu = ours.encode(x, scale)
            assert mu.shape == mu_ref.shape and torch.allclose(mu, mu_ref, atol=1e-4), (mu - mu_ref).abs().max()
            rec_ref = ref.decode(mu_ref, scale)
            rec = ours.decode(mu_ref, scale)
            assert rec.shape == rec_ref.shape == x.shape and torch.allclose(rec, rec_ref, atol=1e-4), (rec - rec_ref).abs().max()


def test_multiview_dit_matches_the_reference_network():
    """The multi-camera network: views stacked along time, per-view cross-attention over each view's own caption, camera embedding
    channels, per-camera rotary positions. Same state dict, same output and gradients as the reference's file."""
    from reference_oracle import install_transformer_engine_standins, reference_network_modules
    from cosmos_predict25_b200.models.multiview_dit import MultiViewDiT, MultiViewDiTConfig
    install_transformer_engine_standins()
    mv = import_reference("cosmos_predict2._src.predict2_multiview.networks.multiview_dit")
    reference_network_modules()
    mv.parallel_state.is_initialized = lambda: False          # the absent process-group registry: no model parallelism here
    torch.manual_seed(0)
    V, state_t = 3, 2
    ref = mv.MultiViewDiT(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
                          concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, atten_backend="minimal_a2a",
                          crossattn_emb_channels=64, use_crossattn_projection=False, pos_emb_cls="rope3d", use_adaln_lora=True,
                          adaln_lora_dim=32, rope_h_extrapolation_ratio=3.0, rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0,
                          rope_enable_fps_modulation=False, use_wan_fp32_strategy=True, timestep_scale=0.001, state_t=state_t,
                          n_cameras_emb=4, view_condition_dim=4, concat_view_embedding=True)
    ours = MultiViewDiT(MultiViewDiTConfig(max_img_h=32, max_img_w=32, max_frames=16, model_channels=128, num_blocks=2, num_heads=2,
                                           crossattn_emb_channels=64, use_crossattn_projection=False, adaln_lora_dim=32, state_t=state_t,
                                           n_cameras_emb=4, view_condition_dim=4, concat_view_embedding=True))
    with torch.no_grad():
        for p in ref.parameters():
            if p.abs().max() == 0:
                p.normal_(0, 0.02)
    res = ours.load_state_dict(ref.state_dict(), strict=True)
    assert not res.missing_keys and not res.unexpected_keys
    x = torch.randn(1, 16, V * state_t, 16, 12)
    t = torch.full((1, 1), 420.0)
    ctx = torch.randn(1, V * 512, 64)                                      # 512 caption tokens per view
    mask = torch.zeros(1, 1, V * state_t, 16, 12)
    mask[:, :, ::state_t] = 1                                              # first frame of every view is given
    views = torch.tensor([[0, 0, 2, 2, 1, 1]])
    pad = torch.zeros(1, 1, 16, 12)
    y = ref(x, t, ctx, condition_video_input_mask_B_C_T_H_W=mask, fps=None, padding_mask=pad, view_indices_B_T=views)
    z = ours(x, t, crossattn_emb=ctx, condition_video_input_mask_B_C_T_H_W=mask, padding_mask=pad, view_indices_B_T=views)
    assert (y - z).abs().max().item() < 2e-5 * max(1.0, y.abs().max().item()), (y - z).abs().max()
    g = torch.randn_like(y)
    (y * g).sum().backward()
    (z * g).sum().backward()
    ref_grads = {n.replace("_checkpoint_wrapped_module.", ""): p.grad for n, p in ref.named_parameters()}
    for n, p in ours.named_parameters():
        want = ref_grads[n]
        assert (p.grad is None) == (want is None), n
        if want is not None:
            assert (p.grad - want).abs().max().item() < 1e-4 * max(1.0, want.abs().max().item()), n


def test_dit_variants_match_the_reference_network():
    """Options of the network beyond the released 2B / 14B setting: learnable per-block position embedding, frame-rate modulated
    rotary positions, an extra image context for the cross-attention, plain AdaLN without the low-rank branch, no text projection,
    temporal patches of 2."""
    import pytest
    cases = [
        dict(extra_per_block_abs_pos_emb=True),
        dict(rope_enable_fps_modulation=True),
        dict(extra_image_context_dim=48),
        dict(use_adaln_lora=False),
        dict(use_crossattn_projection=False, crossattn_emb_channels=96),
        dict(patch_temporal=2, rope_t_extrapolation_ratio=2.0),
        dict(use_wan_fp32_strategy=False),
    ]
    for extra in cases:
        try:
            ref, ours = _net_pair(**extra)
        except TypeError as e:                      # an option this package does not have would show up here, not pass silently
            pytest.fail(f"{extra}: {e}")
        torch.manual_seed(2)
        x = torch.randn(1, 16, 4, 16, 12)
        t = torch.tensor([[250.0]])
        ctx = torch.randn(1, 8, 96)
        mask = torch.zeros(1, 1, 4, 16, 12)
        mask[:, :, :1] = 1
        kw = dict(condition_video_input_mask_B_C_T_H_W=mask, padding_mask=torch.zeros(1, 1, 16, 12))
        if extra.get("rope_enable_fps_modulation"):
            kw["fps"] = torch.tensor([24.0])
        if "extra_image_context_dim" in extra:
            kw["img_context_emb"] = torch.randn(1, 6, 48)
        with torch.no_grad():
            y = ref(x, t, ctx, **kw)
            z = ours(x, t, crossattn_emb=ctx, **kw)
        assert (y - z).abs().max().item() < 2e-5 * max(1.0, y.abs().max().item()), (extra, (y - z).abs().max())


def test_wan21_network_matches_the_reference(monkeypatch):
    """Wan2.1 text-to-video and image-to-video networks against the reference's file (same state dict): interleaved rotary
    positions, cross-attention over text (+ CLIP image tokens), 6-way modulation."""
    from reference_oracle import install_transformer_engine_standins, reference_network_modules
    from cosmos_predict25_b200.models.wan2pt1 import WanConfig, WanModel
    install_transformer_engine_standins()
    wan = import_reference("cosmos_predict2._src.predict2.networks.wan2pt1")
    reference_network_modules()

    def rotary_interleaved(x, cos, sin, interleaved=True, inplace=False):
        # documented semantics of the fused rotary kernel the reference calls: pairs (x[2i], x[2i+1]) turn by angle i
        a, b = x[..., 0::2], x[..., 1::2]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)
    wan.flash_apply_rotary_emb = rotary_interleaved
    a2a = import_reference("cosmos_predict2._src.predict2.networks.a2a_cp")
    wan.attention = a2a.attention                           # the fp32 / math-back-end form prepared by reference_network_modules
    monkeypatch.setattr(torch.Tensor, "cuda", lambda self, *a, **k: self)       # its position tables are placed with .cuda()
    for model_type in ("t2v", "i2v"):
        torch.manual_seed(0)
        kw = dict(model_type=model_type, patch_size=(1, 2, 2), text_len=512, in_dim=16 if model_type == "t2v" else 36, dim=128, ffn_dim=256,
                  freq_dim=64, text_dim=96, out_dim=16, num_heads=2, num_layers=2, qk_norm=True, cross_attn_norm=True, eps=1e-6)
        ref = wan.WanModel(**kw, attention_backend="minimal_a2a", cp_comm_type="a2a")
        ours = WanModel(WanConfig(**kw))
        with torch.no_grad():
            for p in ref.parameters():
                if p.abs().max() == 0:
                    p.normal_(0, 0.02)
        res = ours.load_state_dict(ref.state_dict(), strict=True)
        assert not res.missing_keys and not res.unexpected_keys
        x = torch.randn(2, 16, 3, 16, 12)
        t = torch.tensor([[700.0], [20.0]])
        ctx = torch.randn(2, 512, 96)
        extra = {}
        if model_type == "i2v":
            extra = dict(frame_cond_crossattn_emb_B_L_D=torch.randn(2, 257, 1280), y_B_C_T_H_W=torch.randn(2, 20, 3, 16, 12))
        with torch.no_grad():
            y = ref(x, t, ctx, **extra)
            z = ours(x, t, ctx, **extra)
        assert y.shape == z.shape == x.shape
        assert (y - z).abs().max().item() < 3e-5 * max(1.0, y.abs().max().item()), (model_type, (y - z).abs().max())


def test_checkpoint_written_in_the_reference_layout_resumes_here(tmp_path):
    """A checkpoint written with the reference's own state-dict wrappers (torch's flattened optimizer state, its scheduler and
    trainer records, ``iter_%09d/{model,optim,scheduler,trainer}``) is read by this package's checkpointer: weights, EMA, Adam
    moments, step count, schedule position and iteration all arrive."""
    import copy
    import torch.distributed.checkpoint as dcp
    from torch.distributed.checkpoint import FileSystemWriter
    ref_ck = import_reference("cosmos_predict2._src.predict2.checkpointer.dcp")
    from cosmos_predict25_b200.checkpoint.dcp import DistributedCheckpointer
    from cosmos_predict25_b200.models.dit import CosmosDiT, dit_tiny
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    torch.manual_seed(0)

    class RefStyleModel(torch.nn.Module):                       # what the reference's model object looks like to its checkpointer
        def __init__(self):
            super().__init__()
            self.net = CosmosDiT(dit_tiny())
            self.net_ema = copy.deepcopy(self.net).requires_grad_(False)
            self.config = type("C", (), {"use_lora": False})()
    src = RefStyleModel()
    with torch.no_grad():
        for p in src.net_ema.parameters():
            p.add_(0.01 * torch.randn_like(p))
    opt = torch.optim.AdamW([p for p in src.net.parameters()], lr=1e-3, betas=(0.9, 0.999), weight_decay=0.01)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda n: 1.0)
    x = torch.randn(1, 16, 4, 16, 16)
    for _ in range(3):
        src.net(x, torch.full((1, 1), 500.0), crossattn_emb=torch.randn(1, 32, 256)).pow(2).mean().backward()
        opt.step()
        sched.step()
        opt.zero_grad()
    parts = {"model": ref_ck.ModelWrapper(src).state_dict(), "optim": ref_ck.OptimizerWrapper(src, opt).state_dict(),
             "scheduler": sched.state_dict(), "trainer": {"grad_scaler": torch.amp.GradScaler("cpu", enabled=False).state_dict(), "iteration": 3}}
    root = tmp_path / "checkpoints" / "iter_000000003"
    for k, sd in parts.items():
        dcp.save(sd, storage_writer=FileSystemWriter(str(root / k)))
    (tmp_path / "checkpoints" / "latest_checkpoint.txt").write_text("iter_000000003\n")

    m = Video2WorldModelRectifiedFlow(Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4), device=torch.device("cpu"))
    o, s = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="constant"))
    it = DistributedCheckpointer({}, str(tmp_path)).load(m, o, s)
    assert it == 3 and s.last_epoch == 3 and o.engine.step_count == 3
    for (n, a), (_, b) in zip(src.net.named_parameters(), m.net.named_parameters()):
        assert torch.equal(a, b), n
    names = [n for n, _ in src.net.named_parameters()]
    ema = {n: t for n, (t, _, _) in m.engine.sharded_state("ema").items()}
    exp_avg = {n: t for n, (t, _, _) in m.engine.sharded_state("exp_avg").items()}
    exp_avg_sq = {n: t for n, (t, _, _) in m.engine.sharded_state("exp_avg_sq").items()}
    ref_state = opt.state_dict()["state"]
    for i, (n, p) in enumerate(src.net.named_parameters()):
        assert torch.equal(ema[n].view(-1), dict(src.net_ema.named_parameters())[n].view(-1)), n
        assert torch.equal(exp_avg[n].view(-1), ref_state[i]["exp_avg"].view(-1)), n
        assert torch.equal(exp_avg_sq[n].view(-1), ref_state[i]["exp_avg_sq"].view(-1)), n
    assert len(names) == len(exp_avg)


def test_conditioner_matches_the_reference():
    """Embedder registry of the reference's conditioner against this package's: conditioned / unconditioned pair, the
    negative-prompt pair, and random dropout drawn from the same generator state."""
    from reference_oracle import install_omegaconf_standins
    install_omegaconf_standins()
    rc = import_reference("cosmos_predict2._src.predict2.conditioner")
    from cosmos_predict25_b200.models import conditioner as oc
    ref = rc.VideoConditioner(fps=rc.ReMapkey(input_key="fps", output_key="fps", dropout_rate=0.0),
                              padding_mask=rc.ReMapkey(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
                              text=rc.TextAttr(input_key=["t5_text_embeddings"], dropout_rate=0.2))
    ours = oc.VideoConditioner(fps=oc.ReMapkey("fps", "fps", 0.0), padding_mask=oc.ReMapkey("padding_mask", "padding_mask", 0.0),
                               text=oc.TextAttr("t5_text_embeddings", 0.2))
    torch.manual_seed(0)
    batch = {"fps": torch.tensor([16.0, 24.0, 30.0, 10.0]), "padding_mask": torch.zeros(4, 1, 8, 8), "t5_text_embeddings": torch.randn(4, 6, 16),
             "neg_t5_text_embeddings": torch.randn(4, 6, 16)}

    def same(a, b):
        for k in ("crossattn_emb", "fps", "padding_mask"):
            assert torch.equal(getattr(a, k), getattr(b, k)), k
    for fn in ("get_condition_uncondition", "get_condition_with_negative_prompt"):
        (c_ref, u_ref), (c, u) = getattr(ref, fn)(batch), getattr(ours, fn)(batch)
        same(c, c_ref)
        same(u, u_ref)
    assert u.crossattn_emb.abs().max() > 0 and torch.equal(u.crossattn_emb, batch["neg_t5_text_embeddings"])
    for seed in range(4):                                      # training-time dropout: same draws, same rows dropped
        torch.manual_seed(seed)
        a = ref(batch)
        torch.manual_seed(seed)
        b = ours(batch)
        same(b, a)


def test_input_preprocessing_and_resolution_tables_match_the_reference(tmp_path):
    """What reaches the tokenizer from an input image: same resize (antialiased, ceil of the scaled size), centre crop, zero frames
    after the first, uint8 layout [1, C, T, H, W]; and the resolution tables of datasets and pipelines."""
    import numpy as np
    from PIL import Image
    from reference_oracle import install_diffusers_standins, install_omegaconf_standins, install_transformer_engine_standins
    install_diffusers_standins(), install_omegaconf_standins(), install_transformer_engine_standins()
    ref = import_reference("cosmos_predict2._src.predict2.inference.video2world")
    ref_du = import_reference("cosmos_predict2._src.predict2.datasets.utils")
    from cosmos_predict25_b200.data import utils as du
    from cosmos_predict25_b200.utils import video_io
    assert du.IMAGE_RES_SIZE_INFO == ref_du.IMAGE_RES_SIZE_INFO and du.VIDEO_RES_SIZE_INFO == ref_du.VIDEO_RES_SIZE_INFO
    rng = np.random.RandomState(0)
    for (h, w), res in (((90, 200), (64, 96)), ((333, 127), (48, 80)), ((64, 96), (64, 96))):
        path = str(tmp_path / f"in_{h}x{w}.png")
        Image.fromarray((rng.rand(h, w, 3) * 255).astype(np.uint8)).save(path)
        want = ref.read_and_process_image(path, list(res), 5)
        got = video_io.read_and_process_image(path, res, 5)
        assert got.dtype == want.dtype == torch.uint8 and got.shape == want.shape == (1, 3, 5, *res)
        assert torch.equal(got, want), (h, w, res, (got.int() - want.int()).abs().max())
        vid = torch.from_numpy((rng.rand(4, 3, h, w) * 255).astype(np.uint8))
        assert torch.equal(video_io.resize_input(vid, res), ref.resize_input(vid, list(res)))


def test_easy_io_files_interoperate_with_the_reference(tmp_path):
    """Every local file format written by one side is read back identically by the other."""
    import numpy as np
    ref = import_reference("cosmos_predict2._src.imaginaire.utils.easy_io.easy_io")
    from cosmos_predict25_b200.utils.easy_io import easy_io as own
    objs = {"a.json": {"x": [1, 2, {"y": "z"}], "f": 1.5}, "b.yaml": {"k": [1, 2], "n": {"m": True}}, "c.pkl": {"t": (1, 2)},
            "d.txt": "hello\nworld\n", "e.npy": np.arange(6).reshape(2, 3), "f.pt": {"w": torch.arange(4.0)}, "g.jsonl": [{"a": 1}, {"b": 2}],
            "h.csv": [["a", "b"], ["1", "2"]]}
    for name, obj in objs.items():
        for writer, reader, tag in ((own, ref, "own_ref"), (ref, own, "ref_own")):
            path = str(tmp_path / f"{tag}_{name}")
            writer.dump(obj, path)
            back = reader.load(path)
            if isinstance(obj, np.ndarray):
                assert np.array_equal(back, obj), (name, tag)
            elif name.endswith(".pt"):
                assert torch.equal(back["w"], obj["w"]), (name, tag)
            else:
                assert back == obj, (name, tag, back)
    assert own.exists(str(tmp_path / "own_ref_a.json")) and ref.exists(str(tmp_path / "own_ref_a.json"))


def test_video_condition_matches_the_reference():
    """Conditioning-frame masks of the Video2World condition: fixed count, per-batch categorical draw and uniform draw from the same
    generator states, image batches, the inference edit of both guidance branches, and the second version of the condition."""
    import random
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  install_transformer_engine_standins)
    install_omegaconf_standins(), install_diffusers_standins(), install_transformer_engine_standins(), install_import_time_patches()
    ref = import_reference("cosmos_predict2._src.predict2.configs.video2world.defaults.conditioner")
    from cosmos_predict25_b200.models import conditioner as oc
    gt = torch.randn(4, 16, 6, 4, 4)
    flags = torch.tensor([True, True, False, True])
    for ref_cls, own_cls in ((ref.Video2WorldCondition, oc.Video2WorldCondition), (ref.Video2WorldConditionV2, oc.Video2WorldConditionV2)):
        def pair(**kw):
            a = ref_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flags.clone())
            b = own_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flags.clone())
            random.seed(5), torch.manual_seed(5)
            a = a.set_video_condition(gt, **kw)
            random.seed(5), torch.manual_seed(5)
            b = b.set_video_condition(gt, **kw)
            return a, b
        v2 = ref_cls is ref.Video2WorldConditionV2
        cases = [dict(random_min_num_conditional_frames=0, random_max_num_conditional_frames=2, num_conditional_frames=2)]
        if not v2:          # the second version overrides the count by its (scalar) flag: only the fixed-count form applies to a batch of flags
            cases += [dict(random_min_num_conditional_frames=0, random_max_num_conditional_frames=2, conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25}),
                      dict(random_min_num_conditional_frames=1, random_max_num_conditional_frames=3)]
        for kw in cases:
            if v2:
                continue
            a, b = pair(**kw)
            assert torch.equal(a.condition_video_input_mask_B_C_T_H_W, b.condition_video_input_mask_B_C_T_H_W), kw
            assert torch.equal(a.gt_frames, b.gt_frames)
        if not v2:
            a, b = pair(random_min_num_conditional_frames=0, random_max_num_conditional_frames=2, num_conditional_frames=1)
            for cond_branch in (True, False):
                ea, eb = a.edit_for_inference(cond_branch, 2), b.edit_for_inference(cond_branch, 2)
                assert torch.equal(ea.condition_video_input_mask_B_C_T_H_W, eb.condition_video_input_mask_B_C_T_H_W)
                assert torch.equal(torch.as_tensor(ea.use_video_condition), torch.as_tensor(eb.use_video_condition))
            img = torch.randn(4, 16, 1, 4, 4)
            ia = ref_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flags.clone()).set_video_condition(img, 0, 2, num_conditional_frames=2)
            ib = own_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flags.clone()).set_video_condition(img, 0, 2, num_conditional_frames=2)
            assert ia.condition_video_input_mask_B_C_T_H_W.sum() == ib.condition_video_input_mask_B_C_T_H_W.sum() == 0
        else:               # scalar flag, as the second version expects
            for flag in (True, False):
                a = ref_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flag).set_video_condition(gt, 0, 2, num_conditional_frames=2)
                b = own_cls(crossattn_emb=torch.zeros(4, 2, 8), use_video_condition=flag).set_video_condition(gt, 0, 2, num_conditional_frames=2)
                assert torch.equal(a.condition_video_input_mask_B_C_T_H_W, b.condition_video_input_mask_B_C_T_H_W), flag
                ea, eb = a.edit_for_inference(False, 1), b.edit_for_inference(False, 1)
                assert torch.equal(ea.condition_video_input_mask_B_C_T_H_W, eb.condition_video_input_mask_B_C_T_H_W)


def _reference_v2w_model(net_kw, conditional_frame_timestep=-1.0, high_sigma=False):
    """The reference's Video2World rectified-flow model object with its own network, conditioner, training schedule and sampler,
    assembled without its constructor (which needs the lazy-config / sharding stack): every method that runs below is the
    reference's, unmodified."""
    import types
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  reference_network_modules)
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    install_omegaconf_standins(), install_diffusers_standins(), install_import_time_patches()
    lvg, _ = reference_network_modules()
    ref_v2w = import_reference("cosmos_predict2._src.predict2.models.video2world_model_rectified_flow")
    ref_t2w = import_reference("cosmos_predict2._src.predict2.models.text2world_model_rectified_flow")
    ref_rf = import_reference("cosmos_predict2._src.predict2.schedulers.rectified_flow")
    ref_unipc = import_reference("cosmos_predict2._src.predict2.models.fm_solvers_unipc")
    ref_cond = import_reference("cosmos_predict2._src.predict2.configs.video2world.defaults.conditioner")
    rc = import_reference("cosmos_predict2._src.predict2.conditioner")
    for mod in (ref_v2w, ref_t2w):
        mod.parallel_state.is_initialized = lambda: False          # the absent process-group registry: no model parallelism
    m = ref_v2w.Video2WorldModelRectifiedFlow.__new__(ref_v2w.Video2WorldModelRectifiedFlow)
    torch.nn.Module.__init__(m)
    m.config = types.SimpleNamespace(
        text_encoder_config=None, use_high_sigma_strategy=high_sigma, high_sigma_ratio=0.5, high_sigma_timesteps_min=850,
        high_sigma_timesteps_max=1000, min_num_conditional_frames=0, max_num_conditional_frames=2,
        conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25}, conditional_frame_timestep=conditional_frame_timestep,
        denoise_replace_gt_frames=True, state_ch=16, use_kerras_sigma_at_inference=False)
    torch.manual_seed(0)
    m.net = lvg.MinimalV1LVGDiT(atten_backend="minimal_a2a", **net_kw)
    with torch.no_grad():
        for p in m.net.parameters():
            if p.abs().max() == 0:
                p.normal_(0, 0.02)
    m.net.disable_context_parallel = lambda: None                 # it would create a CUDA stream
    m.conditioner = ref_cond.Video2WorldConditioner(
        fps=rc.ReMapkey(input_key="fps", output_key="fps", dropout_rate=0.0),
        padding_mask=rc.ReMapkey(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
        text=rc.TextAttr(input_key=["t5_text_embeddings"], dropout_rate=0.2),
        use_video_condition=rc.BooleanFlag(input_key="fps", output_key="use_video_condition", dropout_rate=0.0))
    m.rectified_flow = ref_rf.RectifiedFlow(velocity_field=m.net, train_time_distribution="logitnormal", use_dynamic_shift=False, shift=5,
                                            device=torch.device("cpu"), dtype=torch.float32)
    m.sample_scheduler = ref_unipc.FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
    m.tokenizer = DummyTokenizer()
    m.tensor_kwargs = m.tensor_kwargs_fp32 = {"device": "cpu", "dtype": torch.float32}
    m.input_data_key, m.input_image_key, m.input_caption_key, m.data_parallel_size = "video", "images", "ai_caption", 1
    m.text_encoder = None
    return m


def _own_v2w_model(ref, net_kw, conditional_frame_timestep=-1.0, high_sigma=False):
    from cosmos_predict25_b200.models.conditioner import default_video2world_conditioner
    from cosmos_predict25_b200.models.dit import DiTConfig
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    cfg = Video2WorldRFConfig(net=DiTConfig(**net_kw), tokenizer=DummyTokenizer(), conditioner=default_video2world_conditioner(0.2),
                              precision="float32", state_t=4, shift=5.0, train_time_distribution="logitnormal",
                              min_num_conditional_frames=0, max_num_conditional_frames=2, conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25},
                              conditional_frame_timestep=conditional_frame_timestep, use_high_sigma_strategy=high_sigma, high_sigma_ratio=0.5,
                              high_sigma_timesteps_min=850, high_sigma_timesteps_max=1000)
    m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"))
    m.net.load_state_dict(ref.net.state_dict(), strict=True)
    return m


_NET_KW = dict(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
               concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, crossattn_emb_channels=64,
               use_crossattn_projection=True, crossattn_proj_in_channels=96, pos_emb_cls="rope3d", use_adaln_lora=True, adaln_lora_dim=32,
               rope_h_extrapolation_ratio=3.0, rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0,
               rope_enable_fps_modulation=False, use_wan_fp32_strategy=True, timestep_scale=0.001)


def _batch(seed, B=2):
    g = torch.Generator().manual_seed(seed)
    return {"video": torch.randint(0, 256, (B, 3, 13, 32, 32), generator=g, dtype=torch.uint8), "fps": torch.full((B,), 16.0),
            "t5_text_embeddings": torch.randn(B, 8, 96, generator=g), "neg_t5_text_embeddings": torch.randn(B, 8, 96, generator=g),
            "padding_mask": torch.zeros(B, 1, 32, 32)}


def test_training_step_matches_the_reference_model():
    """Whole training step (pixels -> tokenizer -> conditioner with dropout -> conditioning frames -> noise / time sampling ->
    interpolation -> network with frame replacement -> loss) of the reference's Video2World model object and this package's, with
    the same weights and the same seeds: the same loss, for the plain setting, with a noise level given to conditioning frames, and
    with the high-noise re-sampling strategy."""
    import random
    for kw in (dict(), dict(conditional_frame_timestep=0.1), dict(high_sigma=True)):
        ref = _reference_v2w_model(_NET_KW, **kw)
        own = _own_v2w_model(ref, _NET_KW, **kw)
        for seed in (0, 1, 2):
            B = 1 if "conditional_frame_timestep" in kw else 2      # the reference's per-frame timestep broadcast holds for one sample
            random.seed(seed), torch.manual_seed(seed)
            out_ref, loss_ref = ref.training_step(_batch(10 + seed, B), seed)
            random.seed(seed), torch.manual_seed(seed)
            out, loss = own.training_step(_batch(10 + seed, B), seed)
            assert torch.allclose(out["xt"], out_ref["xt"], atol=1e-5), (kw, seed)
            assert torch.allclose(out["sigma"].view(-1), out_ref["sigma"].view(-1)), (kw, seed)
            assert abs(loss.item() - loss_ref.item()) < 2e-5 * max(1.0, abs(loss_ref.item())), (kw, seed, loss.item(), loss_ref.item())


def test_sampling_matches_the_reference_model():
    """Latents sampled by the reference's model object and by this package's from the same conditioning clip, prompt embeddings,
    weights and seed (UniPC, classifier-free guidance with and without a negative prompt, one and two conditioning frames). The
    reference evaluates the two guidance branches one after the other, this package in one batch of two."""
    ref = _reference_v2w_model(_NET_KW)
    own = _own_v2w_model(ref, _NET_KW)
    for n_cond, neg, guidance in ((1, True, 3.0), (2, False, 1.5)):
        b1, b2 = _batch(21, 1), _batch(21, 1)
        b1["num_conditional_frames"] = b2["num_conditional_frames"] = n_cond
        with torch.no_grad():
            want = ref.generate_samples_from_batch(b1, guidance=guidance, seed=7, is_negative_prompt=neg, num_steps=5, shift=5.0)
            got = own.generate_samples_from_batch(b2, guidance=guidance, seed=7, is_negative_prompt=neg, num_steps=5, shift=5.0)
        assert got.shape == want.shape == (1, 16, 4, 4, 4)
        assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item()), (n_cond, neg, (got - want).abs().max())


def test_edm_training_step_and_sampling_match_the_reference_model(monkeypatch):
    """Noise-level (EDM) parameterised Video2World model of the reference against this package's: same loss for the same seeds with
    EDM and with rectified-flow preconditioning, the video noise multiplier, latents scaled by sigma_data, conditioning frames
    with their own noise conditioning, and each high-noise strategy. The reference places its draws with ``device="cuda"``; here
    those land on the CPU."""
    import random
    import types
    import numpy as np
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  reference_network_modules)
    from cosmos_predict25_b200.models import edm
    from cosmos_predict25_b200.models.conditioner import default_video2world_conditioner
    from cosmos_predict25_b200.models.dit import DiTConfig
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    install_omegaconf_standins(), install_diffusers_standins(), install_import_time_patches()
    lvg, _ = reference_network_modules()
    ref_mod = import_reference("cosmos_predict2._src.predict2.models.video2world_model")
    ref_t2w = import_reference("cosmos_predict2._src.predict2.models.text2world_model")
    ref_cond = import_reference("cosmos_predict2._src.predict2.configs.video2world.defaults.conditioner")
    ref_scale = import_reference("cosmos_predict2._src.common.modules.denoiser_scaling")
    ref_sde = import_reference("cosmos_predict2._src.common.modules.edm_sde")
    rc = import_reference("cosmos_predict2._src.predict2.conditioner")
    for mod in (ref_mod, ref_t2w):
        mod.parallel_state.is_initialized = lambda: False
    # device="cuda" in the reference's draws -> the CPU
    for name in ("randn", "rand", "tensor"):
        orig = getattr(torch, name)
        monkeypatch.setattr(torch, name, (lambda f: lambda *a, **k: f(*a, **{**k, "device": "cpu"} if k.get("device") == "cuda" else k))(orig))
    orig_to = torch.Tensor.to
    monkeypatch.setattr(torch.Tensor, "to", lambda self, *a, **k: orig_to(self, *a, **({**k, "device": "cpu"} if k.get("device") == "cuda" else k)))

    net_kw = dict(_NET_KW, timestep_scale=1.0)
    cases = [dict(scaling="edm", sigma_data=0.5, strat="none"), dict(scaling="rectified_flow", sigma_data=1.0, strat="none"),
             dict(scaling="edm", sigma_data=0.5, strat="uniform80_2000"), dict(scaling="edm", sigma_data=0.5, strat="LOGUNIFORM200_100000"),
             dict(scaling="rectified_flow", sigma_data=1.0, strat="shift24"), dict(scaling="edm", sigma_data=0.5, strat="balanced_two_heads_v1"),
             dict(scaling="edm", sigma_data=0.5, strat="hardcoded_20steps")]
    for case in cases:
        m = ref_mod.Video2WorldModel.__new__(ref_mod.Video2WorldModel)
        torch.nn.Module.__init__(m)
        m.config = types.SimpleNamespace(
            text_encoder_config=None, scaling=case["scaling"], sigma_data=case["sigma_data"], use_wan_fp32_strategy=False,
            min_num_conditional_frames=1, max_num_conditional_frames=2, conditional_frames_probs=None, sigma_conditional=0.0001,
            denoise_replace_gt_frames=True, high_sigma_strategy=case["strat"], high_sigma_ratio=0.5, low_sigma_ratio=0.3, state_t=4)
        torch.manual_seed(0)
        m.net = lvg.MinimalV1LVGDiT(atten_backend="minimal_a2a", **net_kw)
        with torch.no_grad():
            for p in m.net.parameters():
                if p.abs().max() == 0:
                    p.normal_(0, 0.02)
        m.net.disable_context_parallel = lambda: None
        m.conditioner = ref_cond.Video2WorldConditioner(
            fps=rc.ReMapkey(input_key="fps", output_key="fps", dropout_rate=0.0),
            padding_mask=rc.ReMapkey(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
            text=rc.TextAttr(input_key=["t5_text_embeddings"], dropout_rate=0.2),
            use_video_condition=rc.BooleanFlag(input_key="fps", output_key="use_video_condition", dropout_rate=0.0))
        m.sde = ref_sde.EDMSDE(p_mean=0.0, p_std=1.0, sigma_max=80, sigma_min=0.0002)
        m.sigma_data = case["sigma_data"]
        m.scaling = ref_scale.EDMScaling(0.5) if case["scaling"] == "edm" else ref_scale.RectifiedFlowScaling(1.0, 1.0, True)
        m.tokenizer = DummyTokenizer()
        m.tensor_kwargs = m.tensor_kwargs_fp32 = {"device": "cpu", "dtype": torch.float32}
        m.input_data_key, m.input_image_key, m.input_caption_key, m.data_parallel_size = "video", "images", "ai_caption", 1
        m.loss_reduce, m.loss_scale, m.video_noise_multiplier, m.text_encoder = "mean", 10.0, 2.0, None

        own = edm.Video2WorldModel(edm.EDMConfig(
            net=DiTConfig(**net_kw), tokenizer=DummyTokenizer(), conditioner=default_video2world_conditioner(0.2), precision="float32",
            state_t=4, scaling=case["scaling"], sigma_data=case["sigma_data"], p_mean=0.0, p_std=1.0, sigma_max=80.0, sigma_min=0.0002,
            loss_scale=10.0, adjust_video_noise=True, min_num_conditional_frames=1, max_num_conditional_frames=2, sigma_conditional=0.0001,
            high_sigma_strategy=case["strat"], high_sigma_ratio=0.5, low_sigma_ratio=0.3), device=torch.device("cpu"))
        own.net.load_state_dict(m.net.state_dict(), strict=True)
        for seed in (0, 1):
            random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
            out_ref, loss_ref = m.training_step(_batch(30 + seed), seed)
            random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
            out, loss = own.training_step(_batch(30 + seed), seed)
            assert torch.allclose(out["sigma"].view(-1), out_ref["sigma"].view(-1), rtol=1e-5), (case, seed, out["sigma"], out_ref["sigma"])
            assert torch.allclose(out["xt"], out_ref["xt"], rtol=1e-4, atol=1e-4), (case, seed)
            assert abs(loss.item() - loss_ref.item()) < 1e-4 * max(1.0, abs(loss_ref.item())), (case, seed, loss.item(), loss_ref.item())
        if case["strat"] != "none":
            continue
        # sampling: noise-level sampler ("2ab", "2mid") and the flow UniPC route, guidance with a negative prompt
        ref_samp = import_reference("cosmos_predict2._src.common.modules.res_sampler")
        m.sampler = ref_samp.Sampler()
        m.config.state_ch = 16
        for flow, solver in ((False, "2ab"), (False, "2mid"), (True, "2ab")):
            m.config.use_flowunipc_scheduler = own.config.use_flowunipc_scheduler = flow
            b1, b2 = _batch(50, 1), _batch(50, 1)
            b1["num_conditional_frames"] = b2["num_conditional_frames"] = 1
            with torch.no_grad():
                want = m.generate_samples_from_batch(b1, guidance=2.0, seed=3, is_negative_prompt=True, num_steps=6, solver_option=solver)
                got = own.generate_samples_from_batch(b2, guidance=2.0, seed=3, is_negative_prompt=True, num_steps=6, solver_option=solver)
            assert got.shape == want.shape == (1, 16, 4, 4, 4)
            assert (got - want).abs().max().item() < 5e-4 * max(1.0, want.abs().max().item()), (case, flow, solver, (got - want).abs().max())


def test_multiview_condition_matches_the_reference():
    """Conditioning masks of the multi-camera condition for every location rule (reference camera, any camera, first n frames of
    every view, their combinations, view dropout), from the same generator states."""
    import random
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  install_transformer_engine_standins)
    install_omegaconf_standins(), install_diffusers_standins(), install_transformer_engine_standins(), install_import_time_patches()
    ref = import_reference("cosmos_predict2._src.predict2_multiview.configs.vid2vid.defaults.conditioner")
    from cosmos_predict25_b200.models import multiview as om
    B, V, state_t = 2, 3, 4
    gt = torch.randn(B, 16, V * state_t, 4, 4)
    views = torch.tensor([[2] * state_t + [0] * state_t + [1] * state_t] * B)
    base = dict(crossattn_emb=torch.zeros(B, 2, 8), use_video_condition=torch.tensor([True, True]), view_indices_B_T=views,
                ref_cam_view_idx_sample_position=torch.tensor([1, 1]))
    L = ref.ConditionLocation
    cases = [
        ([L.FIRST_RANDOM_N], ["first_random_n"], dict(num_conditional_frames_per_view=2)),
        ([L.FIRST_RANDOM_N], ["first_random_n"], dict(random_min_num_conditional_frames_per_view=0, random_max_num_conditional_frames_per_view=3)),
        ([L.FIRST_RANDOM_N], ["first_random_n"], dict(conditional_frames_probs={0: 0.3, 1: 0.3, 2: 0.4}, random_min_num_conditional_frames_per_view=0,
                                                      random_max_num_conditional_frames_per_view=2)),
        ([L.REF_CAM], ["ref_cam"], dict()),
        ([L.REF_CAM, L.FIRST_RANDOM_N], ["ref_cam", "first_random_n"], dict(num_conditional_frames_per_view=1, view_condition_dropout_max=2)),
        ([L.ANY_CAM], ["any_cam"], dict(condition_cam_idx=2)),
        ([L.ANY_CAM], ["any_cam"], dict()),
        ([L.ANY_CAM, L.FIRST_RANDOM_N], ["any_cam", "first_random_n"], dict(random_min_num_conditional_frames_per_view=1,
                                                                            random_max_num_conditional_frames_per_view=2, view_condition_dropout_max=1)),
    ]
    for ref_locs, own_locs, kw in cases:
        for seed in (0, 1, 2):
            random.seed(seed), torch.manual_seed(seed)
            a = ref.MultiViewCondition(**base).set_video_condition(state_t=state_t, gt_frames=gt, condition_locations=ref.ConditionLocationList(ref_locs), **kw)
            random.seed(seed), torch.manual_seed(seed)
            b = om.MultiViewCondition(**base).set_video_condition(state_t=state_t, gt_frames=gt, condition_locations=own_locs, **kw)
            assert torch.equal(a.condition_video_input_mask_B_C_T_H_W, b.condition_video_input_mask_B_C_T_H_W), (own_locs, kw, seed)
    a = ref.MultiViewCondition(**base).set_video_condition(state_t=state_t, gt_frames=gt, condition_locations=ref.ConditionLocationList([L.FIRST_RANDOM_N]),
                                                           num_conditional_frames_per_view=1)
    b = om.MultiViewCondition(**base).set_video_condition(state_t=state_t, gt_frames=gt, condition_locations=["first_random_n"], num_conditional_frames_per_view=1)
    for cond_branch in (True, False):
        ea = a.edit_for_inference(ref.ConditionLocationList([L.FIRST_RANDOM_N]), cond_branch, 2)
        eb = b.edit_for_inference(["first_random_n"], cond_branch, 2)
        assert torch.equal(ea.condition_video_input_mask_B_C_T_H_W, eb.condition_video_input_mask_B_C_T_H_W)
        assert torch.equal(torch.as_tensor(ea.use_video_condition), torch.as_tensor(eb.use_video_condition))


def test_multiview_training_step_matches_the_reference_model():
    """Multi-camera model object of the reference (its network, conditioner, per-view tokenisation, latent view indices) against
    this package's: the same loss for the same seeds and weights."""
    import random
    import types
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  install_transformer_engine_standins, reference_network_modules)
    from cosmos_predict25_b200.models import multiview as om
    from cosmos_predict25_b200.models.multiview_dit import MultiViewDiTConfig
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    install_omegaconf_standins(), install_diffusers_standins(), install_transformer_engine_standins(), install_import_time_patches()
    mvnet = import_reference("cosmos_predict2._src.predict2_multiview.networks.multiview_dit")
    reference_network_modules()
    ref_mod = import_reference("cosmos_predict2._src.predict2_multiview.models.multiview_vid2vid_model_rectified_flow")
    ref_t2w = import_reference("cosmos_predict2._src.predict2.models.text2world_model_rectified_flow")
    ref_v2w = import_reference("cosmos_predict2._src.predict2.models.video2world_model_rectified_flow")
    ref_rf = import_reference("cosmos_predict2._src.predict2.schedulers.rectified_flow")
    ref_cond = import_reference("cosmos_predict2._src.predict2_multiview.configs.vid2vid.defaults.conditioner")
    rc = import_reference("cosmos_predict2._src.predict2.conditioner")
    for mod in (ref_mod, ref_t2w, ref_v2w, mvnet):
        mod.parallel_state.is_initialized = lambda: False
    ref_mod.parallel_state.get_context_parallel_group = lambda: None
    ref_mod.get_process_group_ranks = lambda g: [0]                  # one rank: views are tokenised one after the other
    V, state_t = 3, 2
    net_kw = dict(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
                  concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, crossattn_emb_channels=64,
                  use_crossattn_projection=False, pos_emb_cls="rope3d", use_adaln_lora=True, adaln_lora_dim=32, rope_h_extrapolation_ratio=3.0,
                  rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0, rope_enable_fps_modulation=False, use_wan_fp32_strategy=True,
                  timestep_scale=0.001, state_t=state_t, n_cameras_emb=4, view_condition_dim=4, concat_view_embedding=True)
    m = ref_mod.MultiviewVid2VidModelRectifiedFlow.__new__(ref_mod.MultiviewVid2VidModelRectifiedFlow)
    torch.nn.Module.__init__(m)
    L = ref_cond.ConditionLocation
    m.config = types.SimpleNamespace(
        text_encoder_config=None, use_high_sigma_strategy=False, state_t=state_t, train_sample_views_range=None,
        condition_locations=ref_cond.ConditionLocationList([L.FIRST_RANDOM_N]), min_num_conditional_frames_per_view=0,
        max_num_conditional_frames_per_view=1, view_condition_dropout_max=0, conditional_frames_probs=None,
        conditional_frame_timestep=-1.0, denoise_replace_gt_frames=True)
    m.state_t = state_t
    torch.manual_seed(0)
    m.net = mvnet.MultiViewDiT(atten_backend="minimal_a2a", **net_kw)
    with torch.no_grad():
        for p in m.net.parameters():
            if p.abs().max() == 0:
                p.normal_(0, 0.02)
    m.net.disable_context_parallel = lambda: None
    m.conditioner = ref_cond.MultiViewConditioner(
        fps=rc.ReMapkey(input_key="fps", output_key="fps", dropout_rate=0.0),
        padding_mask=rc.ReMapkey(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
        text=rc.TextAttr(input_key=["t5_text_embeddings"], dropout_rate=0.2),
        use_video_condition=rc.BooleanFlag(input_key="fps", output_key="use_video_condition", dropout_rate=0.0),
        view_indices_B_T=rc.ReMapkey(input_key="latent_view_indices_B_T", output_key="view_indices_B_T", dropout_rate=0.0),
        ref_cam_view_idx_sample_position=rc.ReMapkey(input_key="ref_cam_view_idx_sample_position",
                                                     output_key="ref_cam_view_idx_sample_position", dropout_rate=0.0))
    m.rectified_flow = ref_rf.RectifiedFlow(velocity_field=m.net, train_time_distribution="logitnormal", use_dynamic_shift=False, shift=5,
                                            device=torch.device("cpu"), dtype=torch.float32)
    m.tokenizer = DummyTokenizer()
    m.tensor_kwargs = m.tensor_kwargs_fp32 = {"device": "cpu", "dtype": torch.float32}
    m.input_data_key, m.input_image_key, m.input_caption_key, m.data_parallel_size, m.text_encoder = "video", "images", "ai_caption", 1, None

    own_net_kw = {k: v for k, v in net_kw.items() if k not in ("in_channels", "out_channels", "patch_spatial", "patch_temporal", "concat_padding_mask",
                                                                "pos_emb_cls", "use_adaln_lora")}
    own = om.MultiviewVid2VidModelRectifiedFlow(om.MultiviewRFConfig(
        net=MultiViewDiTConfig(**own_net_kw), tokenizer=DummyTokenizer(), precision="float32", state_t=state_t, shift=5.0,
        train_time_distribution="logitnormal", condition_locations=["first_random_n"], min_num_conditional_frames_per_view=0,
        max_num_conditional_frames_per_view=1, text_dropout=0.2), device=torch.device("cpu"))
    own.net.load_state_dict(m.net.state_dict(), strict=True)
    fpv = DummyTokenizer().get_pixel_num_frames(state_t)

    def batch(seed):
        g = torch.Generator().manual_seed(seed)
        return {"video": torch.randint(0, 256, (1, 3, V * fpv, 32, 32), generator=g, dtype=torch.uint8), "fps": torch.full((1,), 16.0),
                "t5_text_embeddings": torch.randn(1, V * 512, 64, generator=g), "padding_mask": torch.zeros(1, 1, 32, 32),
                "view_indices": torch.tensor([2, 0, 1]).repeat_interleave(fpv)[None], "num_video_frames_per_view": torch.tensor(fpv),
                "sample_n_views": torch.tensor(V), "ref_cam_view_idx_sample_position": torch.tensor([-1])}
    for seed in (0, 1, 2):
        random.seed(seed), torch.manual_seed(seed)
        out_ref, loss_ref = m.training_step(batch(40 + seed), seed)
        random.seed(seed), torch.manual_seed(seed)
        out, loss = own.training_step(batch(40 + seed), seed)
        assert torch.allclose(out["xt"], out_ref["xt"], atol=1e-5), seed
        assert abs(loss.item() - loss_ref.item()) < 2e-5 * max(1.0, abs(loss_ref.item())), (seed, loss.item(), loss_ref.item())

    # sampling: every view's first latent frame given, classifier-free guidance on the other frames (the reference runs the two
    # guidance branches one after the other and draws the conditioning mask before it overwrites it for inference)
    ref_unipc = import_reference("cosmos_predict2._src.predict2.models.fm_solvers_unipc")
    m.sample_scheduler = ref_unipc.FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
    m.config.state_ch, m.config.use_kerras_sigma_at_inference = 16, False
    shape = (16, V * state_t, 4, 4)                                  # callers pass the shape of the tokenised views
    for n_cond, guidance in ((1, 2.0), (0, 0.5)):
        b1, b2 = batch(50), batch(50)
        b1["num_conditional_frames"] = b2["num_conditional_frames"] = n_cond
        with torch.no_grad():
            random.seed(3), torch.manual_seed(3)
            want = m.generate_samples_from_batch(b1, guidance=guidance, seed=11, state_shape=shape, num_steps=4, shift=5.0)
            random.seed(3), torch.manual_seed(3)
            got = own.generate_samples_from_batch(b2, guidance=guidance, seed=11, state_shape=shape, num_steps=4, shift=5.0)
        assert got.shape == want.shape == (1, 16, V * state_t, 4, 4)
        assert (got - want).abs().max().item() < 2e-4 * max(1.0, want.abs().max().item()), (n_cond, (got - want).abs().max())


def test_noise_level_multiview_model_matches_the_reference_model(monkeypatch):
    """The reference's EDM-era multi-camera model object against this package's: training loss, and sampling with classifier-free
    and with adaptive projected guidance (requested through the batch)."""
    import random
    import types
    import numpy as np
    from reference_oracle import (install_diffusers_standins, install_import_time_patches, install_omegaconf_standins,
                                  install_transformer_engine_standins, reference_network_modules)
    from cosmos_predict25_b200.models import multiview as om
    from cosmos_predict25_b200.models.multiview_dit import MultiViewDiTConfig
    from cosmos_predict25_b200.models.vae_wan import DummyTokenizer
    install_omegaconf_standins(), install_diffusers_standins(), install_transformer_engine_standins(), install_import_time_patches()
    mvnet = import_reference("cosmos_predict2._src.predict2_multiview.networks.multiview_dit")
    reference_network_modules()
    ref_mod = import_reference("cosmos_predict2._src.predict2_multiview.models.multiview_vid2vid_model")
    ref_v2w = import_reference("cosmos_predict2._src.predict2.models.video2world_model")
    ref_t2w = import_reference("cosmos_predict2._src.predict2.models.text2world_model")
    ref_cond = import_reference("cosmos_predict2._src.predict2_multiview.configs.vid2vid.defaults.conditioner")
    ref_scale = import_reference("cosmos_predict2._src.common.modules.denoiser_scaling")
    ref_sde = import_reference("cosmos_predict2._src.common.modules.edm_sde")
    ref_samp = import_reference("cosmos_predict2._src.common.modules.res_sampler")
    rc = import_reference("cosmos_predict2._src.predict2.conditioner")
    for mod in (ref_mod, ref_v2w, ref_t2w, mvnet):
        mod.parallel_state.is_initialized = lambda: False
    for name in ("randn", "rand", "tensor"):                         # device="cuda" in the reference's draws -> the CPU
        orig = getattr(torch, name)
        monkeypatch.setattr(torch, name, (lambda f: lambda *a, **k: f(*a, **{**k, "device": "cpu"} if k.get("device") == "cuda" else k))(orig))
    orig_to = torch.Tensor.to
    monkeypatch.setattr(torch.Tensor, "to", lambda self, *a, **k: orig_to(self, *a, **({**k, "device": "cpu"} if k.get("device") == "cuda" else k)))
    V, state_t = 3, 2
    net_kw = dict(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
                  concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, crossattn_emb_channels=64,
                  use_crossattn_projection=False, pos_emb_cls="rope3d", use_adaln_lora=True, adaln_lora_dim=32, rope_h_extrapolation_ratio=3.0,
                  rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0, rope_enable_fps_modulation=False, use_wan_fp32_strategy=False,
                  timestep_scale=1.0, state_t=state_t, n_cameras_emb=4, view_condition_dim=4, concat_view_embedding=True)
    m = ref_mod.MultiviewVid2VidModel.__new__(ref_mod.MultiviewVid2VidModel)
    torch.nn.Module.__init__(m)
    L = ref_cond.ConditionLocation
    m.config = types.SimpleNamespace(
        text_encoder_config=None, scaling="edm", sigma_data=0.5, use_wan_fp32_strategy=False, state_t=state_t, state_ch=16,
        train_sample_views_range=None, condition_locations=ref_cond.ConditionLocationList([L.FIRST_RANDOM_N]),
        min_num_conditional_frames_per_view=0, max_num_conditional_frames_per_view=1, view_condition_dropout_max=0,
        conditional_frames_probs=None, sigma_conditional=0.0001, denoise_replace_gt_frames=True, high_sigma_strategy="none",
        high_sigma_ratio=0.05, low_sigma_ratio=0.05, apg_momentum=-0.75, apg_eta=0.0, apg_norm_threshold=7.5, use_flowunipc_scheduler=False)
    m.state_t = state_t
    torch.manual_seed(0)
    m.net = mvnet.MultiViewDiT(atten_backend="minimal_a2a", **net_kw)
    with torch.no_grad():
        for p in m.net.parameters():
            if p.abs().max() == 0:
                p.normal_(0, 0.02)
    m.net.disable_context_parallel = lambda: None
    m.conditioner = ref_cond.MultiViewConditioner(
        fps=rc.ReMapkey(input_key="fps", output_key="fps", dropout_rate=0.0),
        padding_mask=rc.ReMapkey(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
        text=rc.TextAttr(input_key=["t5_text_embeddings"], dropout_rate=0.2),
        use_video_condition=rc.BooleanFlag(input_key="fps", output_key="use_video_condition", dropout_rate=0.0),
        view_indices_B_T=rc.ReMapkey(input_key="latent_view_indices_B_T", output_key="view_indices_B_T", dropout_rate=0.0),
        ref_cam_view_idx_sample_position=rc.ReMapkey(input_key="ref_cam_view_idx_sample_position",
                                                     output_key="ref_cam_view_idx_sample_position", dropout_rate=0.0))
    m.sde = ref_sde.EDMSDE(p_mean=0.0, p_std=1.0, sigma_max=80, sigma_min=0.0002)
    m.sigma_data, m.scaling, m.sampler = 0.5, ref_scale.EDMScaling(0.5), ref_samp.Sampler()
    m.tokenizer = DummyTokenizer()
    m.tensor_kwargs = m.tensor_kwargs_fp32 = {"device": "cpu", "dtype": torch.float32}
    m.input_data_key, m.input_image_key, m.input_caption_key, m.data_parallel_size = "video", "images", "ai_caption", 1
    m.loss_reduce, m.loss_scale, m.video_noise_multiplier, m.text_encoder = "mean", 10.0, state_t ** 0.5, None

    own_net_kw = {k: v for k, v in net_kw.items() if k not in ("in_channels", "out_channels", "patch_spatial", "patch_temporal", "concat_padding_mask",
                                                                "pos_emb_cls", "use_adaln_lora")}
    own = om.MultiviewVid2VidModel(om.MultiviewVid2VidModelConfig(
        net=MultiViewDiTConfig(**own_net_kw), tokenizer=DummyTokenizer(), precision="float32", state_t=state_t, scaling="edm", sigma_data=0.5,
        p_mean=0.0, p_std=1.0, sigma_max=80.0, sigma_min=0.0002, loss_scale=10.0, adjust_video_noise=True, sigma_conditional=0.0001,
        condition_locations=["first_random_n"], min_num_conditional_frames_per_view=0, max_num_conditional_frames_per_view=1,
        text_dropout=0.2), device=torch.device("cpu"))
    own.net.load_state_dict(m.net.state_dict(), strict=True)
    fpv = DummyTokenizer().get_pixel_num_frames(state_t)

    def batch(seed):
        g = torch.Generator().manual_seed(seed)
        return {"video": torch.randint(0, 256, (1, 3, V * fpv, 32, 32), generator=g, dtype=torch.uint8), "fps": torch.full((1,), 16.0),
                "t5_text_embeddings": torch.randn(1, V * 512, 64, generator=g), "padding_mask": torch.zeros(1, 1, 32, 32),
                "view_indices": torch.tensor([2, 0, 1]).repeat_interleave(fpv)[None], "num_video_frames_per_view": torch.tensor(fpv),
                "sample_n_views": torch.tensor(V), "ref_cam_view_idx_sample_position": torch.tensor([-1])}
    for seed in (0, 1):
        random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
        out_ref, loss_ref = m.training_step(batch(60 + seed), seed)
        random.seed(seed), np.random.seed(seed), torch.manual_seed(seed)
        out, loss = own.training_step(batch(60 + seed), seed)
        assert torch.allclose(out["xt"], out_ref["xt"], rtol=1e-4, atol=1e-4), seed
        assert abs(loss.item() - loss_ref.item()) < 1e-4 * max(1.0, abs(loss_ref.item())), (seed, loss.item(), loss_ref.item())
    shape = (16, V * state_t, 4, 4)
    for apg in (False, True):
        b1, b2 = batch(70), batch(70)
        for b in (b1, b2):
            b["num_conditional_frames"] = 1
            if apg:
                b["use_apg"] = True
        with torch.no_grad():
            random.seed(3), torch.manual_seed(3)
            want = m.generate_samples_from_batch(b1, guidance=2.5, seed=4, state_shape=shape, num_steps=5)
            random.seed(3), torch.manual_seed(3)
            got = own.generate_samples_from_batch(b2, guidance=2.5, seed=4, state_shape=shape, num_steps=5)
        assert got.shape == want.shape == (1,) + shape
        assert (got - want).abs().max().item() < 5e-4 * max(1.0, want.abs().max().item()), (apg, (got - want).abs().max())
