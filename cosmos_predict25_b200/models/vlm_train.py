"""Training pieces of the vision-language (Reason1 / Qwen) stack: causal-LM head, loss, per-part optimisers, LR schedule.

Parity targets (the reference's VLM package; only its inference forward is used by the world model, the training side is
reproduced here for completeness):

  * training step = next-token cross-entropy with ``ignore_index=-100`` on non-assistant tokens, optional per-token
    normalisation by the average number of supervised tokens over the data-parallel group, optional z-loss
    ``coeff * mean(logsumexp(logits)^2)`` (cosmos_predict2/_src/reason1/models/vlm_base.py:271-411);
  * one optimiser per model part (embedding, decoder layers, final norm, ``lm_head``, optional vision parts) with per-part
    learning-rate multipliers and freeze flags; AdamW betas (0.9, 0.95), weight decay 0.1
    (cosmos_predict2/_src/reason1/models/vlm_qwen.py and configs/default/model_config.py:24-323);
  * LR = linear warm-up from ``init_lr`` to ``lr``, then linear decay or cosine cool-down to ``end_lr``.

The decoder itself is ``QwenLanguageModel`` (text_encoder.py); this module only adds what training needs.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from .text_encoder import QwenConfig, QwenLanguageModel

IGNORE_INDEX = -100


class QwenForCausalLM(nn.Module):
    """Decoder + ``lm_head`` (tied to the embedding when the config says so). ``forward`` runs with autograd."""

    def __init__(self, config: QwenConfig):
        super().__init__()
        self.config = config
        self.model = QwenLanguageModel(config)
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)
        if config.tie_word_embeddings:
            self.lm_head.weight = self.model.embed_tokens.weight

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        m = self.model
        x = m.embed_tokens(input_ids)
        B, S, _ = x.shape
        cos, sin = m.rope(S, x.device, x.dtype)
        mask = None
        if attention_mask is not None:
            causal = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
            mask = causal[None, None] & attention_mask[:, None, None, :].bool()
        for layer in m.layers:
            x = layer(x, cos, sin, mask)
        return self.lm_head(m.norm(x))


def build_labels(input_ids: torch.Tensor, assistant_mask: torch.Tensor) -> torch.Tensor:
    """Next-token labels: position i is supervised with token i+1 iff token i+1 belongs to an assistant turn."""
    labels = torch.full_like(input_ids, IGNORE_INDEX)
    labels[:, :-1] = torch.where(assistant_mask[:, 1:].bool(), input_ids[:, 1:], torch.full_like(input_ids[:, 1:], IGNORE_INDEX))
    return labels


def causal_lm_loss(logits: torch.Tensor, labels: torch.Tensor, z_loss_coeff: float = 0.0, token_normalization: bool = False,
                   group=None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
    """Cross-entropy over supervised positions (+ z-loss). Default: mean over this rank's supervised tokens. With
    ``token_normalization`` the sum is divided by the *average* supervised-token count over ``group`` instead, so that
    after the gradient all-reduce (mean) every supervised token of the global batch has the same weight."""
    V = logits.shape[-1]
    flat, tgt = logits.float().reshape(-1, V), labels.reshape(-1)
    n_tok = (tgt != IGNORE_INDEX).sum()
    ce_sum = F.cross_entropy(flat, tgt, ignore_index=IGNORE_INDEX, reduction="sum")
    if token_normalization:
        avg = n_tok.float().clone()
        if group is not None and dist.is_available() and dist.is_initialized():
            dist.all_reduce(avg, group=group)
            avg = avg / dist.get_world_size(group)
        denom = avg.clamp(min=1.0)
    else:
        denom = n_tok.clamp(min=1).float()
    ce = ce_sum / denom
    out = {"ce_loss": ce.detach(), "num_supervised_tokens": n_tok}
    loss = ce
    if z_loss_coeff > 0:
        sup = tgt != IGNORE_INDEX
        lse = torch.logsumexp(flat, dim=-1)
        z = z_loss_coeff * (lse[sup] ** 2).mean() if bool(sup.any()) else flat.sum() * 0.0
        out["z_loss"] = z.detach()
        loss = loss + z
    return loss, out


@dataclass
class VLMOptimizerConfig:
    lr: float = 3e-4
    init_lr: float = 1e-5
    end_lr: float = 2.5e-5
    betas: Tuple[float, float] = (0.9, 0.95)
    weight_decay: float = 0.1
    eps: float = 1e-8
    warmup_steps: int = 1000
    total_steps: int = 400_000
    decay: str = "cosine"                  # linear | cosine | none
    lr_multipliers: Dict[str, float] = field(default_factory=lambda: {"vision": 0.1})
    frozen_parts: Tuple[str, ...] = ()


def model_parts(model: nn.Module) -> Dict[str, List[nn.Parameter]]:
    """Parameters grouped into the parts that get their own optimiser: ``embed``, ``llm`` (decoder layers + final norm),
    ``lm_head``, and ``vision`` / ``projector`` when the model has such sub-modules."""
    parts: Dict[str, List[nn.Parameter]] = {}
    seen = set()
    for name, p in model.named_parameters():
        if id(p) in seen:
            continue
        seen.add(id(p))
        if "embed_tokens" in name:
            key = "embed"
        elif name.startswith("lm_head"):
            key = "lm_head"
        elif "vision" in name or "visual" in name:
            key = "vision"
        elif "projector" in name or "merger" in name:
            key = "projector"
        else:
            key = "llm"
        parts.setdefault(key, []).append(p)
    return parts


def lr_lambda(cfg: VLMOptimizerConfig):
    """Multiplier of ``cfg.lr`` at a given step."""
    lo, hi, end = cfg.init_lr / cfg.lr, 1.0, cfg.end_lr / cfg.lr

    def f(step: int) -> float:
        if step < cfg.warmup_steps:
            return lo + (hi - lo) * step / max(1, cfg.warmup_steps)
        if cfg.decay == "none":
            return hi
        t = min(1.0, (step - cfg.warmup_steps) / max(1, cfg.total_steps - cfg.warmup_steps))
        if cfg.decay == "linear":
            return hi + (end - hi) * t
        return end + (hi - end) * 0.5 * (1.0 + math.cos(math.pi * t))

    return f


def build_part_optimizers(model: nn.Module, cfg: VLMOptimizerConfig):
    """One AdamW + LambdaLR per trainable part. Returns ({part: optimizer}, {part: scheduler}); frozen parts get
    ``requires_grad=False`` and no optimiser."""
    opts, scheds = {}, {}
    for part, params in model_parts(model).items():
        if part in cfg.frozen_parts:
            for p in params:
                p.requires_grad_(False)
            continue
        lr = cfg.lr * cfg.lr_multipliers.get(part, 1.0)
        decay = [p for p in params if p.ndim >= 2]
        no_decay = [p for p in params if p.ndim < 2]
        opt = torch.optim.AdamW([{"params": decay, "weight_decay": cfg.weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
                                lr=lr, betas=cfg.betas, eps=cfg.eps)
        opts[part] = opt
        scheds[part] = torch.optim.lr_scheduler.LambdaLR(opt, lr_lambda(cfg))
    return opts, scheds


def train_step(model: QwenForCausalLM, batch: Dict[str, torch.Tensor], opts, scheds, z_loss_coeff: float = 0.0,
               token_normalization: bool = False, max_grad_norm: float = 1.0, group=None) -> Dict[str, float]:
    """One optimisation step on ``batch`` = {input_ids, attention_mask, assistant_mask}."""
    labels = build_labels(batch["input_ids"], batch["assistant_mask"])
    logits = model(batch["input_ids"], batch.get("attention_mask"))
    loss, stats = causal_lm_loss(logits, labels, z_loss_coeff, token_normalization, group)
    for o in opts.values():
        o.zero_grad(set_to_none=True)
    loss.backward()
    params = [p for o in opts.values() for g in o.param_groups for p in g["params"] if p.grad is not None]
    gn = torch.nn.utils.clip_grad_norm_(params, max_grad_norm) if params else torch.tensor(0.0)
    for o in opts.values():
        o.step()
    for s in scheds.values():
        s.step()
    return {"loss": float(loss.detach()), "grad_norm": float(gn), **{k: float(v) for k, v in stats.items()}}
