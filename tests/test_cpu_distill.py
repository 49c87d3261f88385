"""Consistency distillation (sCM / rCM) on the tiny DiT (CPU)."""
import torch

from cosmos_predict25_b200.models import distill
from cosmos_predict25_b200.models.dit import CosmosDiT, NET_PRESETS


def _batch(B=2, T=3, H=8, W=8):
    return {"latents": torch.randn(B, 16, T, H, W), "t5_text_embeddings": torch.randn(B, 8, 256), "fps": torch.full((B,), 16.0),
            "padding_mask": torch.zeros(B, 1, H, W)}


def _nontrivial(net):
    for blk in net.blocks:
        for m in (blk.adaln_modulation_self_attn, blk.adaln_modulation_cross_attn, blk.adaln_modulation_mlp):
            torch.nn.init.normal_(m[-1].weight, std=0.05)
    torch.nn.init.normal_(net.final_layer.linear.weight, std=0.05)


def test_network_jvp_matches_finite_difference_and_func_jvp():
    torch.manual_seed(0)
    net = CosmosDiT(NET_PRESETS["tiny"]()).double()
    net.init_weights()
    _nontrivial(net)
    x = torch.randn(1, 16, 2, 8, 8, dtype=torch.float64)
    t = torch.full((1, 1), 400.0, dtype=torch.float64)
    tx, tt = torch.randn_like(x), torch.full_like(t, 1000.0)
    kw = dict(crossattn_emb=torch.randn(1, 8, 256, dtype=torch.float64), fps=torch.tensor([16.0]), padding_mask=torch.zeros(1, 1, 8, 8, dtype=torch.float64))
    F, dF = distill.network_jvp(net, x, t, tx, tt, **kw)
    e = 2e-3      # the network computes its time embedding and norms in fp32: keep the step well above fp32 noise
    with torch.no_grad():
        fd = (net(x + e * tx, t + e * tt, **kw) - net(x - e * tx, t - e * tt, **kw)) / (2 * e)
        assert torch.allclose(F, net(x, t, **kw))
    assert dF.abs().max() > 1e-3
    assert (dF - fd).abs().max() < 2e-2 * max(1.0, float(fd.abs().max())), (dF - fd).abs().max()
    _, dF2 = torch.func.jvp(lambda a, b: net(a, b, **kw), (x, t), (tx, tt))
    assert torch.allclose(dF, dF2.detach(), rtol=1e-5, atol=1e-6)


def _model(**kw):
    cfg = distill.DistillConfig(net=NET_PRESETS["tiny"](), precision="float32", tangent_warmup_iters=10, student_sample_steps=2, **kw)
    m = distill.ConsistencyDistillModel(cfg, device=torch.device("cpu"))
    _nontrivial(m.net)
    m.load_teacher_state_dict(m.net.state_dict())
    return m


def test_scm_step_trains_student_only_and_jvp_equals_fd():
    torch.manual_seed(1)
    m = _model()
    assert all(not p.requires_grad for p in m.teacher.parameters())
    out, loss = m.training_step(_batch(), iteration=5)
    assert torch.isfinite(loss) and 0.0 < float(out["scm/warmup"]) <= 1.0
    loss.backward()
    assert any(p.grad is not None and p.grad.abs().sum() > 0 for p in m.net.parameters())
    assert all(p.grad is None for p in m.teacher.parameters())
    # the finite-difference variant of the tangent gives the same loss value for the same random draws
    torch.manual_seed(3)
    _, l_jvp = m.training_step(_batch(), iteration=10)
    m.config.use_jvp = False
    torch.manual_seed(3)
    _, l_fd = m.training_step(_batch(), iteration=10)
    assert abs(float(l_jvp) - float(l_fd)) < 2e-2 * max(1.0, abs(float(l_jvp))), (float(l_jvp), float(l_fd))


def test_consistency_fixed_point_has_zero_tangent():
    """If the student equals the teacher and the teacher's ODE is followed, f is constant along it up to the student's own
    t-dependence: with warm-up 0 the tangent is  -t (v_T - F) = 0  and the loss is exactly 0."""
    torch.manual_seed(2)
    m = _model()
    m.config.tangent_warmup_iters = 10 ** 9
    out, loss = m.training_step(_batch(), iteration=0)
    assert float(loss) < 1e-10


def test_rcm_phases_and_sampling():
    torch.manual_seed(4)
    m = _model(dmd_weight=0.5)
    assert m.fake_score is not None
    out, loss = m.training_step(_batch(B=1), iteration=3)
    assert "dmd_loss" in out and torch.isfinite(loss)
    loss.backward()
    assert all(p.grad is None for p in m.fake_score.parameters())          # the student phase does not touch the critic
    m.zero_grad(set_to_none=True)
    m.set_phase("critic")
    out, loss = m.training_step(_batch(B=1), iteration=4)
    assert "critic_loss" in out
    loss.backward()
    assert any(p.grad is not None for p in m.fake_score.parameters()) and all(p.grad is None for p in m.net.parameters())
    assert distill.DistillTrainerMixin.phase_of(0, 2, True) == "student" and distill.DistillTrainerMixin.phase_of(1, 2, True) == "critic"
    b = _batch(B=1)
    b["num_conditional_frames"] = 1
    x = m.generate_samples_from_batch(b, num_steps=2)
    assert x.shape == (1, 16, 3, 8, 8) and torch.allclose(x[:, :, 0], b["latents"][:, :, 0], atol=1e-5)
