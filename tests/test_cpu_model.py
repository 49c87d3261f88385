"""CPU (fp32) tests of the model stack: tiny DiT, rectified-flow training step, conditioning, samplers."""

import math

import numpy as np
import pytest
import torch

from cosmos_predict25_b200.models import schedulers
from cosmos_predict25_b200.models.conditioner import DataType, Video2WorldCondition, default_video2world_conditioner
from cosmos_predict25_b200.models.dit import CosmosDiT, dit_tiny
from cosmos_predict25_b200.models.rectified_flow import (Text2WorldModelRectifiedFlow, Text2WorldRFConfig,
                                                          Video2WorldModelRectifiedFlow, Video2WorldRFConfig)
from cosmos_predict25_b200.ops import ref
from cosmos_predict25_b200.trainer.optim import LambdaLinearScheduler, OptimizerConfig, SchedulerConfig

CPU = torch.device("cpu")


def _batch(B=1, T=4, H=16, W=16, ctx=256, n_cond=1):
    return {"latents": torch.randn(B, 16, T, H, W), "t5_text_embeddings": torch.randn(B, 32, ctx),
            "fps": torch.full((B,), 16.0), "padding_mask": torch.zeros(B, 1, H, W), "num_conditional_frames": n_cond}


def test_dit_state_dict_names_match_reference_layout():
    net = CosmosDiT(dit_tiny())
    keys = set(net.state_dict().keys())
    for k in ["x_embedder.proj.1.weight", "pos_embedder.seq", "pos_embedder.dim_spatial_range", "pos_embedder.dim_temporal_range",
              "t_embedder.1.linear_1.weight", "t_embedder.1.linear_2.weight", "t_embedding_norm.weight",
              "blocks.0.self_attn.q_proj.weight", "blocks.0.self_attn.q_norm.weight", "blocks.0.self_attn.output_proj.weight",
              "blocks.1.cross_attn.k_proj.weight", "blocks.1.cross_attn.v_proj.weight", "blocks.0.mlp.layer1.weight",
              "blocks.0.mlp.layer2.weight", "blocks.0.adaln_modulation_self_attn.1.weight",
              "blocks.0.adaln_modulation_cross_attn.2.weight", "blocks.0.adaln_modulation_mlp.2.weight",
              "final_layer.linear.weight", "final_layer.adaln_modulation.1.weight", "final_layer.adaln_modulation.2.weight",
              "accum_video_sample_counter", "accum_iteration"]:
        assert k in keys, k
    sd = net.state_dict()
    assert sd["x_embedder.proj.1.weight"].shape == (256, 18 * 4)
    assert sd["final_layer.linear.weight"].shape == (64, 256)
    assert sd["blocks.0.adaln_modulation_mlp.2.weight"].shape == (3 * 256, 64)
    full = CosmosDiT.__new__(CosmosDiT)  # 2B shapes without allocating: check the config arithmetic only
    from cosmos_predict25_b200.models.dit import dit_2b
    c = dit_2b()
    assert c.head_dim == 128 and c.model_channels * int(c.mlp_ratio) == 8192


def test_dit_identity_at_init_and_shapes():
    torch.manual_seed(0)
    net = CosmosDiT(dit_tiny())
    net.init_weights()
    torch.nn.init.zeros_(net.t_embedder[1].linear_2.weight)  # silence the shared AdaLN-LoRA term as well
    x = torch.randn(2, 16, 4, 16, 16)
    t = torch.tensor([[500.0], [20.0]])
    ctx = torch.randn(2, 32, 256)
    mask = torch.zeros(2, 1, 4, 16, 16)
    out = net(x, t, ctx, condition_video_input_mask_B_C_T_H_W=mask, padding_mask=torch.zeros(2, 1, 16, 16))
    assert out.shape == x.shape
    # AdaLN output projections are zero-initialised (and the LoRA term zeroed above): gates are 0, so blocks are identity and the final
    # modulation is LN(x) with scale 0 / shift 0; the output then only depends on x_embedder + final linear
    emb = net._embed(x, mask, torch.zeros(2, 1, 16, 16)).view(2, 4, 64, 256)
    want = net.unpatchify(torch.nn.functional.linear(ref.ln_modulate(emb, torch.zeros(2, 4, 256), torch.zeros(2, 4, 256)),
                                                     net.final_layer.linear.weight).view(2, 4, 8, 8, 64))
    assert torch.allclose(out, want, atol=1e-4)


def test_patchify_unpatchify_roundtrip_orders():
    net = CosmosDiT(dit_tiny())
    x = torch.arange(2 * 3 * 2 * 4 * 6, dtype=torch.float32).view(2, 3, 2, 4, 6)
    p = net.x_embedder.proj[0](x)  # b t h w (c r m n)
    assert p.shape == (2, 2, 2, 3, 12)
    assert p[0, 1, 1, 2].tolist() == [x[0, c, 1, 2 + m, 4 + n].item() for c in range(3) for m in range(2) for n in range(2)]
    y = torch.randn(1, 2, 3, 4, 2 * 2 * 1 * 16)
    u = net.unpatchify(y)  # B C (T t) (H p1) (W p2) from (p1 p2 t C)
    assert u.shape == (1, 16, 2, 6, 8)
    assert torch.equal(u[0, 5, 1, 2 * 2 + 1, 3 * 2 + 0], y[0, 1, 2, 3].view(2, 2, 1, 16)[1, 0, 0, 5])


def test_rope_table_layout():
    net = CosmosDiT(dit_tiny())
    ang = net.pos_embedder.generate(3, 4, 5)
    hd = 64
    dim_h = hd // 6 * 2
    dim_t = hd - 2 * dim_h
    assert ang.shape == (60, hd)
    assert torch.equal(ang[:, : hd // 2], ang[:, hd // 2:])
    tok = (2 * 4 + 1) * 5 + 3  # t=2, h=1, w=3
    t_freq = 1.0 / (10000.0 ** (torch.arange(0, dim_t, 2).float() / dim_t))
    assert torch.allclose(ang[tok, : dim_t // 2], 2 * t_freq)
    h_theta = 10000.0 * 3.0 ** (dim_h / (dim_h - 2))
    h_freq = 1.0 / (h_theta ** (torch.arange(0, dim_h, 2).float() / dim_h))
    assert torch.allclose(ang[tok, dim_t // 2: dim_t // 2 + dim_h // 2], 1 * h_freq)
    assert torch.allclose(ang[tok, dim_t // 2 + dim_h // 2: hd // 2], 3 * h_freq)


def test_training_step_reduces_loss_and_updates_ema():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=CPU)
    opt, sch = m.init_optimizer_scheduler(OptimizerConfig(lr=2e-3, max_grad_norm=1.0), SchedulerConfig(kind="constant"))
    batch = _batch()
    torch.manual_seed(1)
    losses = []
    for it in range(8):
        torch.manual_seed(100)  # same noise / time every step: the loss must go down
        _, loss = m.training_step(dict(batch), it)
        loss.backward()
        opt.ema_beta = m.ema_beta(it + 1)
        opt.step()
        sch.step()
        losses.append(loss.item())
    assert all(math.isfinite(l) for l in losses)
    assert losses[-1] < losses[0]
    u = m.engine.units[0]
    assert not torch.equal(u.ema, u.master)
    with m.ema_scope():
        p_ema = next(m.net.parameters()).detach().clone()
    p_reg = next(m.net.parameters()).detach().clone()
    assert not torch.equal(p_ema, p_reg)


def test_ema_beta_schedule():
    m = Text2WorldModelRectifiedFlow(Text2WorldRFConfig(net=dit_tiny(), precision="float32"), device=CPU)
    assert abs(m.ema_exp_coefficient - 6.94) < 0.01
    assert m.ema_beta(0) == 0.0
    assert abs(m.ema_beta(1) - 0.5 ** (m.ema_exp_coefficient + 1)) < 1e-12
    assert m.ema_beta(10 ** 6) > 0.99999


def test_video2world_conditioning_mask_and_velocity_replacement():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4, conditional_frame_timestep=0.1)
    m = Video2WorldModelRectifiedFlow(cfg, device=CPU)
    batch = _batch(n_cond=2)
    _, x0, cond = m.get_data_and_condition(dict(batch))
    assert isinstance(cond, Video2WorldCondition)
    mask = cond.condition_video_input_mask_B_C_T_H_W
    assert mask.shape == (1, 1, 4, 16, 16) and mask[0, 0, :2].min() == 1 and mask[0, 0, 2:].max() == 0
    eps = torch.randn_like(x0)
    v = m.denoise(eps, torch.randn_like(x0), torch.tensor([[700.0]]), cond)
    assert torch.allclose(v[:, :, :2], (eps - x0)[:, :, :2], atol=1e-5)  # exact velocity on clean frames
    img = {"images": torch.rand(1, 3, 16, 16) * 2 - 1, "t5_text_embeddings": torch.randn(1, 32, 256), "fps": torch.tensor([16.0]),
           "padding_mask": torch.zeros(1, 1, 16, 16)}

    class Tok:
        spatial_compression_factor = 1

        def encode(self, x):
            return x.repeat(1, 6, 1, 1, 1)[:, :16]
    m.tokenizer = Tok()
    _, x0i, condi = m.get_data_and_condition(img)
    assert condi.data_type == DataType.IMAGE and condi.condition_video_input_mask_B_C_T_H_W.sum() == 0


def test_conditioner_dropout_and_negative_prompt():
    c = default_video2world_conditioner(0.2)
    batch = {"t5_text_embeddings": torch.ones(4, 8, 16), "neg_t5_text_embeddings": torch.full((4, 8, 16), 2.0),
             "fps": torch.ones(4), "padding_mask": torch.zeros(4, 1, 4, 4)}
    cond, uncond = c.get_condition_uncondition(batch)
    assert cond.crossattn_emb.eq(1).all() and uncond.crossattn_emb.eq(0).all()
    cond, uncond = c.get_condition_with_negative_prompt(batch)
    assert cond.crossattn_emb.eq(1).all() and uncond.crossattn_emb.eq(2).all()
    torch.manual_seed(0)
    drops = sum(int((c(batch).crossattn_emb.flatten(1).abs().sum(1) == 0).sum()) for _ in range(200))
    assert 100 < drops < 220  # ~20 % of 800 samples


def test_rectified_flow_schedule_table():
    s = schedulers.RectifiedFlowSchedule(shift=5.0)
    tau = np.linspace(1, 1 / 1000, 1000)
    want = 5 * tau / (1 + 4 * tau)
    assert np.allclose(s.sigmas.numpy(), want, atol=1e-6)
    assert abs(float(s.timesteps[0]) - 1000.0) < 1e-3
    u = torch.tensor([0.0, 0.5, 0.9995])
    assert s.indices(u).tolist() == [0, 500, 999]
    x0, eps = torch.randn(3, 2), torch.randn(3, 2)
    xt, v = s.interpolate(eps, x0, torch.tensor([0.0, 0.3, 1.0]))
    assert torch.allclose(xt[0], x0[0]) and torch.allclose(xt[2], eps[2]) and torch.allclose(v, eps - x0)


def test_unipc_timesteps_and_exactness_on_linear_velocity():
    sol = schedulers.FlowUniPCSolver(1000, shift=1.0)
    sol.set_timesteps(35, shift=5.0)
    assert len(sol.timesteps) == 35 and sol.timesteps.dtype == torch.int64
    sig = np.linspace(0.999, 0.0, 36)[:-1]
    sig = 5 * sig / (1 + 4 * sig)
    assert np.allclose(sol.sigmas[:-1], sig, atol=1e-6) and sol.sigmas[-1] == 0
    assert sol.timesteps[0].item() == int(1000 * sig[0])
    # if the model predicts the exact velocity of a straight path x_t = sigma*eps + (1-sigma)*x0, every
    # data prediction equals x0 and any consistent solver must land on x0
    torch.manual_seed(0)
    x0, eps = torch.randn(2, 3, 4), torch.randn(2, 3, 4)
    for solver in (schedulers.FlowUniPCSolver(1000, shift=1.0), schedulers.FlowEulerSolver(1000, shift=1.0)):
        solver.set_timesteps(12, shift=3.0)
        x = float(solver.sigmas[0]) * eps + (1 - float(solver.sigmas[0])) * x0
        for t in solver.timesteps.tolist():
            x = solver.step(eps - x0, t, x)
        assert torch.allclose(x, x0, atol=1e-4), type(solver).__name__


def test_unipc_is_more_accurate_than_euler_on_curved_path():
    """Velocity field whose data prediction drifts with sigma: higher-order UniPC beats Euler."""
    torch.manual_seed(0)
    x_start = torch.randn(64)

    def v_of(x, sigma):  # dx/dsigma = -x * 2 sigma  => x(sigma) = x(s0) * exp(s0^2 - sigma^2)
        return -2.0 * sigma * x

    errs = {}
    for name, solver in (("unipc", schedulers.FlowUniPCSolver(1000, shift=1.0)), ("euler", schedulers.FlowEulerSolver(1000, shift=1.0))):
        solver.set_timesteps(10, shift=1.0)
        x = x_start.clone()
        s0 = float(solver.sigmas[0])
        for i, t in enumerate(solver.timesteps.tolist()):
            x = solver.step(v_of(x, float(solver.sigmas[i])), t, x)
        exact = x_start * math.exp(s0 ** 2 - 0.0)
        errs[name] = (x - exact).abs().max().item()
    assert errs["unipc"] < errs["euler"]


def test_karras_sigma_override():
    sol = schedulers.FlowUniPCSolver(1000, shift=1.0)
    sol.set_timesteps(35, shift=5.0, use_kerras_sigma=True)
    assert len(sol.timesteps) == 36  # 36 evaluations
    assert abs(sol.sigmas[0] - 200 / 201) < 1e-6 and abs(sol.sigmas[-2] - 0.01 / 1.01) < 1e-6


def test_sampling_euler_and_unipc_run_and_are_deterministic():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=CPU).eval()
    b = _batch()
    s1 = m.generate_samples_from_batch(dict(b), guidance=3.0, seed=7, num_steps=4, solver="euler")
    s2 = m.generate_samples_from_batch(dict(b), guidance=3.0, seed=7, num_steps=4, solver="euler")
    s3 = m.generate_samples_from_batch(dict(b), guidance=3.0, seed=8, num_steps=4, solver="unipc")
    assert s1.shape == (1, 16, 4, 16, 16) and torch.equal(s1, s2) and torch.isfinite(s3).all()
    # the conditioning frame is reproduced exactly by the sampler (velocity replaced by eps - x0)
    assert torch.allclose(s1[:, :, 0], b["latents"][:, :, 0], atol=1e-3)


def test_batched_cfg_equals_two_separate_forwards():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=CPU).eval()
    for p in m.net.parameters():  # leave the zero-init so the network is not an identity
        if p.abs().sum() == 0:
            torch.nn.init.normal_(p, std=0.02)
    b = _batch()
    b["neg_t5_text_embeddings"] = torch.randn(1, 32, 256)
    fn = m.get_velocity_fn_from_batch(dict(b), guidance=7.0, is_negative_prompt=True)
    noise, x, t = torch.randn(1, 16, 4, 16, 16), torch.randn(1, 16, 4, 16, 16), torch.tensor([[400.0]])
    with torch.no_grad():
        v = fn(noise, x, t)
        cond, uncond = m._conditions_for_sampling(dict(b), True)
        x0 = b["latents"]
        cond = cond.set_video_condition(x0, 0, 0, num_conditional_frames=1).edit_for_inference(True, 1)
        uncond = uncond.set_video_condition(x0, 0, 0, num_conditional_frames=1).edit_for_inference(False, 1)
        vc, vu = m.denoise(noise, x, t, cond), m.denoise(noise, x, t, uncond)
    assert torch.allclose(v, vc + 7.0 * (vc - vu), atol=1e-4)


def test_lr_schedule_warmup_then_linear():
    f = LambdaLinearScheduler([10], [0.1], [1.0], [0.0], [110])
    assert f(0) == 0.0 and abs(f(5) - 0.5) < 1e-9 and f(10) == 1.0
    assert abs(f(60) - (0.1 + 0.9 * 50 / 100)) < 1e-9 and abs(f(110) - 0.1) < 1e-9


def test_state_dict_roundtrip_with_ema_prefixes():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=CPU)
    m.on_train_start()
    sd = m.state_dict()
    assert any(k.startswith("net.") for k in sd) and any(k.startswith("net_ema.") for k in sd)
    sd["net.blocks.0.self_attn._extra_state"] = torch.zeros(1)  # TE-style key that loaders must skip
    m2 = Video2WorldModelRectifiedFlow(cfg, device=CPU)
    m2.on_train_start()
    m2.load_state_dict(sd, strict=False)
    for (n1, p1), (n2, p2) in zip(m.net.named_parameters(), m2.net.named_parameters()):
        assert torch.equal(p1, p2), n1


def test_batched_adaln_equals_per_mlp_modulation():
    """All modulation MLPs in one call (the few-row batched GEMM front-end; its torch fallback on CPU) equal the per-MLP path,
    with and without the LoRA bottleneck, for the 3-chunk block MLPs and the 2-chunk final layer; gradients reach every weight."""
    from cosmos_predict25_b200.models.dit import _adaln_mlp, _run_adaln, run_adaln_many
    torch.manual_seed(0)
    D, r = 64, 16
    emb = torch.randn(2, 3, D)
    for use_lora, chunks in ((True, 3), (False, 3), (True, 2)):
        mlps = [_adaln_mlp(D, r, chunks, use_lora) for _ in range(4)]
        lora = torch.randn(2, 3, chunks * D, requires_grad=True) if use_lora else None
        many = run_adaln_many(mlps, emb, lora, True)
        assert many.shape == (4, 2, 3, chunks * D)
        for z, mlp in enumerate(mlps):
            assert torch.allclose(many[z], _run_adaln(mlp, emb, lora, True), atol=1e-5)
        many.square().sum().backward()
        assert all(p.grad is not None and p.grad.abs().sum() > 0 for m in mlps for p in m.parameters())
        assert lora is None or lora.grad is not None


def test_neighborhood_backward_plan_matches_dense_mask():
    """Host plan of the tile-sparse backward kernel (query-tile lists per key tile, transposed per-axis bit tables) rebuilt into a
    dense mask equals the definition."""
    from cosmos_predict25_b200.modules.neighborhood_attn import TilePlan, neighborhood_mask
    vs, win, st, causal = (8, 8, 16), (3, 5, 9), (1, 2, 3), (True, False, False)
    plan = TilePlan(vs, win, st, causal, torch.device("cpu"))
    L = vs[0] * vs[1] * vs[2]
    nT, nH, nW = plan.n
    want = neighborhood_mask(vs, win, st, 1, causal)[plan.perm][:, plan.perm]          # [query, key] in tile order
    got = torch.zeros_like(want)
    row = torch.arange(128)
    col = torch.arange(128)
    for kt in range(L // 128):
        k_t, k_h, k_w = (kt // (nH * nW)) * 4 + (row >> 5), ((kt // nW) % nH) * 4 + ((row >> 3) & 3), (kt % nW) * 8 + (row & 7)
        for i in range(int(plan.q_cnt[kt])):
            e = int(plan.q_list[kt, i])
            qt = e & 0x7FFFFFFF
            bt = plan.bt_b[k_t, qt // (nH * nW)].long()[:, None]
            bh = plan.bh_b[k_h, (qt // nW) % nH].long()[:, None]
            bw = plan.bw_b[k_w, qt % nW].long()[:, None]
            vis = ((bt >> (col >> 5)[None]) & (bh >> ((col >> 3) & 3)[None]) & (bw >> (col & 7)[None]) & 1).bool()   # [key row, query col]
            assert not e < 0 or bool(vis.all())
            got[qt * 128:(qt + 1) * 128, kt * 128:(kt + 1) * 128] = vis.t()
    assert torch.equal(got, want)


def _conv_cl_on_cpu(self, x, t_out, out=None, out_map=None, resid=None, h_out=None, w_out=None):
    """What the convolution kernel computes, in plain torch: out[t, y, x] = sum over taps of W_tap x[t + dt, y + dh, x + dw] with
    zeros outside the tensor (default output mapping only)."""
    T, H, W, C = x.shape
    h_out, w_out = h_out or H, w_out or W
    ntaps = len(self.taps) // 3
    cpad = self.w.shape[1] // ntaps
    w = self.w.float().view(-1, ntaps, cpad)[: self.cout, :, :C]
    xp = torch.nn.functional.pad(x.float(), (0, 0, 2, 2, 2, 2, 0, 2))            # W, H by 2 each side; T by 2 at the end
    acc = torch.zeros(t_out, h_out, w_out, self.cout)
    for i in range(ntaps):
        dt, dh, dw = self.taps[3 * i: 3 * i + 3]
        acc += xp[dt: dt + t_out, 2 + dh: 2 + dh + h_out, 2 + dw: 2 + dw + w_out] @ w[:, i].t()
    if self.bias is not None:
        acc += self.bias
    return acc.to(torch.bfloat16) if resid is None else (acc + resid.float()).to(torch.bfloat16)


def test_kernel_encoder_downsampling_restatements(monkeypatch):
    """Stride-2 spatial convolution as a 2 x 2-tap convolution on 2 x 2 pixel blocks, and the stride-2 causal time convolution as
    a 2-tap convolution on frame pairs, against the torch ``Resample`` module chunk by chunk (streaming state included)."""
    from cosmos_predict25_b200.models import vae_wan, vae_wan_cl
    monkeypatch.setattr(vae_wan_cl.ConvCL, "__call__", _conv_cl_on_cpu)
    torch.manual_seed(0)
    for mode in ("downsample2d", "downsample3d"):
        mod = vae_wan.Resample(16, mode).float()
        cl = vae_wan_cl._DownsampleCL(mod, "cpu")
        st_t, st_c = vae_wan.StreamState(), vae_wan_cl._Stream()
        for T in (1, 4, 4, 2):
            x = torch.randn(1, 16, T, 8, 12).bfloat16().float()
            want = mod(x, st_t)                                                      # [1, C, T', 4, 6]
            got = cl(x[0].permute(1, 2, 3, 0).contiguous().bfloat16(), st_c)         # [T', 4, 6, C]
            assert got.shape == (want.shape[2], 4, 6, 16), (mode, T, got.shape, want.shape)
            err = (got.float().permute(3, 0, 1, 2) - want[0]).abs().max().item()
            assert err < 3e-2, (mode, T, err)


def test_kernel_encoder_matches_torch_encoder_on_cpu(monkeypatch):
    """The whole channels-last encoder (with the kernel replaced by its torch definition) against ``Encoder3d`` over a 1 + 4 + 4
    frame video: same chunking, caches and down-sampling skips."""
    from cosmos_predict25_b200.models import vae_wan, vae_wan_cl
    from cosmos_predict25_b200.ops import native
    monkeypatch.setattr(vae_wan_cl.ConvCL, "__call__", _conv_cl_on_cpu)

    class _Ops:
        @staticmethod
        def rmsnorm_silu_cl(x, gamma, silu):
            y = torch.nn.functional.normalize(x.float(), dim=-1) * (x.shape[-1] ** 0.5) * gamma
            return (torch.nn.functional.silu(y) if silu else y).to(torch.bfloat16)

    monkeypatch.setattr(native, "load", lambda: _Ops)
    torch.manual_seed(1)
    enc = vae_wan.Encoder3d(dim=16, z_dim=8, dim_mult=(1, 2, 2), num_res_blocks=1, temperal_downsample=(False, True)).float()
    cl = vae_wan_cl.EncoderCL(enc, "cpu")
    st = vae_wan.StreamState()
    x = torch.randn(1, 3, 9, 16, 32).bfloat16().float()
    for lo, hi in ((0, 1), (1, 5), (5, 9)):
        want = enc(x[:, :, lo:hi], st)
        got = cl.step(x[:, :, lo:hi].bfloat16())
        assert got.shape == want.shape, (got.shape, want.shape)
        scale = want.abs().mean().item()
        assert (got.float() - want).abs().mean().item() < 0.05 * scale + 1e-3, (lo, hi)


def test_sampler_state_update_definitions():
    """The torch definitions behind the sampling-loop kernels: a linear combination equals the term-by-term arithmetic, the frame
    replacement keeps conditioning frames (scaled by the per-sample flag) or their velocity and everything else untouched."""
    from cosmos_predict25_b200.ops import functional as F
    torch.manual_seed(0)
    xs = [torch.randn(2, 3, 4, 5, 8) for _ in range(3)]
    out = F.lincomb(xs, [1.0, -0.25, 2.0])
    assert torch.allclose(out, xs[0] - 0.25 * xs[1] + 2.0 * xs[2], atol=1e-6)
    x, gt, noise = xs
    mask = torch.zeros(2, 1, 4, 5, 8)
    mask[:, :, 0] = 1
    flag = torch.tensor([1.0, 0.0]).view(2, 1, 1, 1, 1)
    a = F.frame_blend(x, gt, None, mask, flag)
    assert torch.equal(a[0, :, 0], gt[0, :, 0]) and torch.equal(a[1, :, 0], torch.zeros_like(gt[1, :, 0])) and torch.equal(a[:, :, 1:], x[:, :, 1:])
    b = F.frame_blend(x, gt, noise, mask, out_dtype=torch.bfloat16)
    assert b.dtype == torch.bfloat16 and torch.equal(b[:, :, 0], (noise - gt)[:, :, 0].bfloat16()) and torch.equal(b[:, :, 1:], x[:, :, 1:].bfloat16())


def test_condition_v2_and_fourier_features():
    from dataclasses import replace
    from cosmos_predict25_b200.models.conditioner import Video2WorldCondition, Video2WorldConditionV2
    from cosmos_predict25_b200.models.dit import FourierFeatures
    gt = torch.randn(2, 4, 5, 6, 6)
    base = dict(crossattn_emb=torch.zeros(2, 3, 8))
    flags = torch.tensor([True, False])
    v1 = Video2WorldCondition(**base, use_video_condition=flags).set_video_condition(gt, 0, 0, num_conditional_frames=2)
    v2 = Video2WorldConditionV2(**base, use_video_condition=flags).set_video_condition(gt, 0, 0, num_conditional_frames=2)
    m1, m2 = v1.condition_video_input_mask_B_C_T_H_W, v2.condition_video_input_mask_B_C_T_H_W
    assert m1[:, 0, :, 0, 0].sum(1).tolist() == [2, 2] and m2[:, 0, :, 0, 0].sum(1).tolist() == [2, 0]
    inf = replace(v2, use_video_condition=False).edit_for_inference(is_cfg_conditional=False, num_conditional_frames=1)
    assert inf.condition_video_input_mask_B_C_T_H_W[:, 0, :, 0, 0].sum(1).tolist() == [1, 1]
    f1, f2 = FourierFeatures(16, bandwidth=0.5, normalize=True), FourierFeatures(16, bandwidth=0.5, normalize=True)
    x = torch.tensor([0.0, 0.3, -1.2])
    y = f1(x)
    assert y.shape == (3, 16) and torch.equal(y, f2(x)) and torch.allclose(y[0], math.sqrt(2) * f1.phases.cos(), atol=1e-6)
    assert set(f1.state_dict()) == {"freqs", "phases"}
