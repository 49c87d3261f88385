"""EDM-era samplers/models and LoRA adapters (CPU)."""
import math

import numpy as np
import pytest
import torch

from cosmos_predict25_b200.models import edm
from cosmos_predict25_b200.models.dit import NET_PRESETS
from cosmos_predict25_b200.models.lora import LoRALinear, add_lora, lora_state_dict, merge_lora, unmerge_lora


def test_scalings():
    s = torch.tensor([0.5, 2.0, 80.0])
    c_skip, c_out, c_in, c_noise = edm.EDMScaling(0.5)(s)
    assert torch.allclose(c_skip, 0.25 / (s ** 2 + 0.25))
    assert torch.allclose(c_noise, 0.25 * s.log())
    # variance preserving input: Var[c_in * (x0 + sigma eps)] = 1 when Var[x0] = sigma_data^2
    assert torch.allclose(c_in ** 2 * (0.25 + s ** 2), torch.ones(3))
    c_skip, c_out, c_in, c_noise = edm.RectifiedFlowScaling()(s)
    t = s / (1 + s)
    assert torch.allclose(c_skip, 1 - t) and torch.allclose(c_out, -t) and torch.allclose(c_noise, t)
    # x_sigma * c_in is the rectified-flow interpolant (1 - t) x0 + t eps
    x0, eps = torch.randn(3), torch.randn(3)
    assert torch.allclose((x0 + s * eps) * c_in, (1 - t) * x0 + t * eps, atol=1e-6)


def test_karras_grid():
    g = edm.get_rev_ts(0.002, 80.0, 35, 7.0)
    assert len(g) == 36 and abs(g[0] - 80) < 1e-9 and abs(g[-1] - 0.002) < 1e-12
    assert np.all(np.diff(g) < 0)
    with pytest.raises(ValueError):
        edm.get_rev_ts(1.0, 0.5, 4)


def _gauss_denoiser(sd):
    return lambda x, sigma: x * (sd ** 2 / (sd ** 2 + sigma.view(-1, 1) ** 2))


@pytest.mark.parametrize("solver", ["2ab", "1euler", "2mid", "2heun"])
def test_res_sampler_gaussian_ode(solver):
    """For N(0, sd^2) data the probability-flow ODE has the closed form x(s) = x(S) sqrt((sd^2+s^2)/(sd^2+S^2))."""
    sd, S, smin = 0.5, 80.0, 0.002
    x = torch.randn(4, 8, dtype=torch.float64) * S
    out = edm.RESSampler()(_gauss_denoiser(sd), x, num_steps=36, sigma_min=smin, sigma_max=S, solver_option=solver,
                           sample_clean=False)
    exact = x * math.sqrt((sd ** 2 + smin ** 2) / (sd ** 2 + S ** 2))
    err = (out - exact).abs().max().item() / exact.abs().max().item()
    assert err < {"1euler": 0.15, "2heun": 0.08}.get(solver, 0.03), err


def test_second_order_beats_euler():
    sd, S, smin = 0.5, 80.0, 0.002
    x = torch.randn(2, 16, dtype=torch.float64) * S
    exact = x * math.sqrt((sd ** 2 + smin ** 2) / (sd ** 2 + S ** 2))
    errs = {}
    for solver in ("1euler", "2ab"):
        out = edm.RESSampler()(_gauss_denoiser(sd), x, num_steps=20, sigma_min=smin, sigma_max=S, solver_option=solver,
                               sample_clean=False)
        errs[solver] = (out - exact).abs().max().item()
    assert errs["2ab"] < 0.7 * errs["1euler"], errs


def test_point_mass_and_edm_euler():
    c = torch.full((2, 5), 0.7)
    fn = lambda x, s: c.to(x.dtype)
    x = torch.randn(2, 5) * 80
    assert torch.allclose(edm.RESSampler()(fn, x, num_steps=10), c, atol=1e-5)
    assert torch.allclose(edm.EDMEulerSampler()(fn, x, num_steps=10), c, atol=1e-5)


def _edm_cfg(cls_cfg=edm.EDMConfig, **kw):
    return cls_cfg(net=NET_PRESETS["tiny"](), precision="float32", **kw)


def _batch(B=2, T=3, H=8, W=8, ctx=None):
    net = NET_PRESETS["tiny"]()
    d = net.crossattn_proj_in_channels if net.use_crossattn_projection else net.crossattn_emb_channels
    return {"latents": torch.randn(B, 16, T, H, W), "t5_text_embeddings": torch.randn(B, 8, d), "fps": torch.full((B,), 16.0),
            "padding_mask": torch.zeros(B, 1, H, W)}


def test_edm_training_step_and_sampling():
    torch.manual_seed(0)
    m = edm.Video2WorldModel(_edm_cfg(high_sigma_strategy=edm.HighSigmaStrategy.UNIFORM80_2000, high_sigma_ratio=0.5),
                             device=torch.device("cpu"))
    out, loss = m.training_step(_batch(), 0)
    assert torch.isfinite(loss) and out["model_pred"].shape == (2, 16, 3, 8, 8)
    loss.backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in m.net.parameters())
    b = _batch(B=1)
    b["num_conditional_frames"] = 1
    x = m.generate_samples_from_batch(b, guidance=2.0, num_steps=4)
    assert x.shape == (1, 16, 3, 8, 8) and torch.isfinite(x).all()
    # conditioning frame comes back unchanged
    assert torch.allclose(x[:, :, 0], b["latents"][:, :, 0] * m.sigma_data, atol=1e-4)      # samples live at the model's data scale


def test_high_sigma_strategies():
    for strat in ("uniform80_2000", "loguniform200_100000", "shift24", "balanced_two_heads_v1", "hardcoded_20steps"):
        m = edm.Video2WorldModel(_edm_cfg(high_sigma_strategy=strat, high_sigma_ratio=1.0), device=torch.device("cpu"))
        s = m.draw_training_sigma(64, True)
        assert torch.isfinite(s).all() and (s > 0).all()
        if strat == "uniform80_2000":
            assert (s >= 80).all() and (s <= 2000).all()
        if strat == "loguniform200_100000":
            assert (s >= 200).all() and (s <= 100000 * 1.001).all()


def test_lora_identity_merge_and_freeze():
    from cosmos_predict25_b200.models.dit import CosmosDiT
    torch.manual_seed(0)
    net = CosmosDiT(NET_PRESETS["tiny"]())
    net.init_weights()
    # make the blocks non-trivial
    for blk in net.blocks:
        for mlp in (blk.adaln_modulation_self_attn, blk.adaln_modulation_cross_attn, blk.adaln_modulation_mlp):
            torch.nn.init.normal_(mlp[-1].weight, std=0.05)
    b = _batch(B=1)
    args = (b["latents"], torch.full((1, 1), 0.3))
    kw = dict(crossattn_emb=b["t5_text_embeddings"], fps=b["fps"], padding_mask=b["padding_mask"])
    with torch.no_grad():
        y0 = net(*args, **kw)
    add_lora(net, 4, 8)
    wrapped = [m for m in net.modules() if isinstance(m, LoRALinear)]
    assert len(wrapped) == len(net.blocks) * 10   # 4 + 4 attention projections, 2 MLP layers per block
    assert all(("lora_" in n) == p.requires_grad for n, p in net.named_parameters())
    keys = list(lora_state_dict(net))
    assert any(k.endswith("self_attn.q_proj.lora_A.default.weight") for k in keys)
    assert any(k.endswith("mlp.layer2.base_layer.weight") for k in net.state_dict())
    with torch.no_grad():
        assert torch.allclose(net(*args, **kw), y0, atol=1e-5)     # B = 0 -> identity
        for m in wrapped:
            torch.nn.init.normal_(m.lora_B["default"].weight, std=0.05)
        y1 = net(*args, **kw)
        assert (y1 - y0).abs().max() > 1e-4
        merge_lora(net)
        y2 = net(*args, **kw)
        assert torch.allclose(y1, y2, atol=2e-4), (y1 - y2).abs().max()
        unmerge_lora(net)
        assert torch.allclose(net(*args, **kw), y1, atol=2e-4)
    # gradients reach only adapters
    net(*args, **kw).sum().backward()
    assert all((p.grad is not None) == ("lora_" in n) for n, p in net.named_parameters())
