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
    ref = lvg.MinimalV1LVGDiT(max_img_h=32, max_img_w=32, max_frames=16, in_channels=16, out_channels=16, patch_spatial=2, patch_temporal=1,
                              concat_padding_mask=True, model_channels=128, num_blocks=2, num_heads=2, atten_backend="minimal_a2a",
                              crossattn_emb_channels=64, use_crossattn_projection=True, crossattn_proj_in_channels=96, pos_emb_cls="rope3d",
                              use_adaln_lora=True, adaln_lora_dim=32, rope_h_extrapolation_ratio=3.0, rope_w_extrapolation_ratio=3.0,
                              rope_t_extrapolation_ratio=1.0, rope_enable_fps_modulation=False, use_wan_fp32_strategy=True,
                              timestep_scale=0.001, **extra)
    ours = CosmosDiT(DiTConfig(max_img_h=32, max_img_w=32, max_frames=16, model_channels=128, num_blocks=2, num_heads=2,
                               crossattn_emb_channels=64, crossattn_proj_in_channels=96, adaln_lora_dim=32, **extra))
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
