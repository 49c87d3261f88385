"""Training pieces of the language tower: labels, loss (token normalisation, z-loss), part-wise optimisers, schedule."""

import math

import torch

from cosmos_predict25_b200.models.text_encoder import QwenConfig
from cosmos_predict25_b200.models import vlm_train as vt


def _tiny():
    torch.manual_seed(0)
    cfg = QwenConfig(vocab_size=48, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2)
    return vt.QwenForCausalLM(cfg)


def test_labels_supervise_assistant_tokens_only():
    ids = torch.tensor([[5, 6, 7, 8, 9]])
    assistant = torch.tensor([[0, 0, 1, 1, 0]])
    labels = vt.build_labels(ids, assistant)
    assert labels.tolist() == [[-100, 7, 8, -100, -100]]


def test_loss_matches_manual_cross_entropy_and_z_loss():
    torch.manual_seed(1)
    logits = torch.randn(2, 5, 11)
    labels = torch.tensor([[-100, 3, 4, -100, 1], [2, -100, -100, -100, -100]])
    loss, stats = vt.causal_lm_loss(logits, labels)
    lp = torch.log_softmax(logits, -1)
    want = -(lp[0, 1, 3] + lp[0, 2, 4] + lp[0, 4, 1] + lp[1, 0, 2]) / 4
    assert torch.allclose(loss, want, atol=1e-6) and int(stats["num_supervised_tokens"]) == 4
    lz, sz = vt.causal_lm_loss(logits, labels, z_loss_coeff=0.1)
    lse = torch.logsumexp(logits, -1)
    z = 0.1 * torch.stack([lse[0, 1], lse[0, 2], lse[0, 4], lse[1, 0]]).pow(2).mean()
    assert torch.allclose(lz, want + z, atol=1e-6) and torch.allclose(sz["z_loss"], z, atol=1e-6)
    ln, _ = vt.causal_lm_loss(logits, labels, token_normalization=True)     # one rank: average count == own count
    assert torch.allclose(ln, want, atol=1e-6)
    empty, _ = vt.causal_lm_loss(logits, torch.full_like(labels, -100), z_loss_coeff=0.1)
    assert float(empty) == 0.0


def test_schedule_warmup_then_cosine_or_linear():
    cfg = vt.VLMOptimizerConfig(lr=1e-3, init_lr=1e-5, end_lr=1e-4, warmup_steps=10, total_steps=110, decay="cosine")
    f = vt.lr_lambda(cfg)
    assert math.isclose(f(0) * cfg.lr, 1e-5) and math.isclose(f(10), 1.0) and math.isclose(f(5) * cfg.lr, (1e-5 + 1e-3) / 2)
    assert math.isclose(f(110) * cfg.lr, 1e-4) and math.isclose(f(60) * cfg.lr, (1e-3 + 1e-4) / 2, rel_tol=1e-6)
    cfg.decay = "linear"
    assert math.isclose(vt.lr_lambda(cfg)(60) * cfg.lr, (1e-3 + 1e-4) / 2, rel_tol=1e-6)


def test_part_optimisers_multipliers_freeze_and_training_reduces_loss():
    model = _tiny()
    cfg = vt.VLMOptimizerConfig(lr=1e-2, init_lr=1e-2, end_lr=1e-2, warmup_steps=0, decay="none",
                                lr_multipliers={"lm_head": 0.5}, frozen_parts=("embed",))
    parts = vt.model_parts(model)
    assert set(parts) == {"embed", "llm", "lm_head"}
    opts, scheds = vt.build_part_optimizers(model, cfg)
    assert set(opts) == {"llm", "lm_head"} and not model.model.embed_tokens.weight.requires_grad
    assert math.isclose(opts["lm_head"].param_groups[0]["lr"], 5e-3) and math.isclose(opts["llm"].param_groups[0]["lr"], 1e-2)
    assert opts["llm"].param_groups[1]["weight_decay"] == 0.0          # norm weights and biases are not decayed
    torch.manual_seed(3)
    ids = torch.randint(0, 48, (4, 12))
    batch = {"input_ids": ids, "attention_mask": torch.ones_like(ids), "assistant_mask": (torch.arange(12) >= 4).expand(4, 12).long()}
    embed_before = model.model.embed_tokens.weight.clone()
    losses = [vt.train_step(model, batch, opts, scheds, z_loss_coeff=1e-4)["loss"] for _ in range(25)]
    assert losses[-1] < 0.5 * losses[0]
    assert torch.equal(model.model.embed_tokens.weight, embed_before)


def test_tied_embedding_is_one_parameter():
    cfg = QwenConfig(vocab_size=16, hidden_size=8, intermediate_size=16, num_hidden_layers=1, num_attention_heads=2,
                     num_key_value_heads=1, tie_word_embeddings=True)
    m = vt.QwenForCausalLM(cfg)
    assert m.lm_head.weight is m.model.embed_tokens.weight
    assert "lm_head" not in vt.model_parts(m)
