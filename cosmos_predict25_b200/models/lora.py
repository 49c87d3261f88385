"""LoRA adapters for the DiT.

Parity target: ``Text2WorldModelRectifiedFlow.add_lora`` (cosmos_predict2/_src/predict2/models/text2world_model_rectified_flow.py:833-919),
which injects PEFT adapters into every module whose name contains one of the comma-separated targets, freezes the
rest of the network and keeps the adapter weights in fp32. This file does the same without PEFT and keeps PEFT's
parameter names (``<name>.base_layer.weight``, ``<name>.lora_A.default.weight``, ``<name>.lora_B.default.weight``) so
adapter checkpoints interchange.

The low-rank term is evaluated as two skinny GEMMs beside the base GEMM: ``y = W x + (alpha / r) * B (A x)``.
``merge_lora`` folds it into the base weight for inference so sampling runs the unmodified fused path.
"""

from __future__ import annotations

import math
from typing import Iterable, List

import torch
import torch.nn as nn

from ..utils import log

DEFAULT_TARGETS = "q_proj,k_proj,v_proj,output_proj,mlp.layer1,mlp.layer2"


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, rank: int, alpha: float, init_lora_weights: bool = True, adapter: str = "default"):
        super().__init__()
        self.base_layer = base
        self.rank, self.alpha, self.adapter = rank, alpha, adapter
        self.scaling = alpha / rank
        dev = base.weight.device
        self.lora_A = nn.ModuleDict({adapter: nn.Linear(base.in_features, rank, bias=False, device=dev, dtype=torch.float32)})
        self.lora_B = nn.ModuleDict({adapter: nn.Linear(rank, base.out_features, bias=False, device=dev, dtype=torch.float32)})
        self.merged = False
        self.reset_lora_parameters(init_lora_weights)

    @property
    def in_features(self):
        return self.base_layer.in_features

    @property
    def out_features(self):
        return self.base_layer.out_features

    @property
    def weight(self):
        return self.base_layer.weight

    @property
    def bias(self):
        return self.base_layer.bias

    def reset_lora_parameters(self, init_lora_weights: bool = True):
        a, b = self.lora_A[self.adapter].weight, self.lora_B[self.adapter].weight
        nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        if init_lora_weights:
            nn.init.zeros_(b)          # adapter starts as the identity
        else:
            nn.init.normal_(b, std=0.02)

    def delta_weight(self) -> torch.Tensor:
        return self.scaling * (self.lora_B[self.adapter].weight.float() @ self.lora_A[self.adapter].weight.float())

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self.base_layer(x)
        if self.merged:
            return y
        a, b = self.lora_A[self.adapter].weight, self.lora_B[self.adapter].weight
        # the activation of a fused-GELU base layer applies to the base product only when the adapter is the identity;
        # targets with an activation are therefore evaluated pre-activation
        act = getattr(self.base_layer, "act", "none")
        low = torch.nn.functional.linear(torch.nn.functional.linear(x.to(a.dtype), a), b) * self.scaling
        if act == "none":
            return y + low.to(y.dtype)
        pre = torch.nn.functional.linear(x, self.base_layer.weight, self.base_layer.bias)
        return torch.nn.functional.gelu(pre.float() + low.float()).to(y.dtype)

    @torch.no_grad()
    def merge(self):
        if not self.merged:
            self.base_layer.weight.add_(self.delta_weight().to(self.base_layer.weight.dtype))
            self.merged = True

    @torch.no_grad()
    def unmerge(self):
        if self.merged:
            self.base_layer.weight.sub_(self.delta_weight().to(self.base_layer.weight.dtype))
            self.merged = False


def _targets(spec) -> List[str]:
    items = spec.split(",") if isinstance(spec, str) else list(spec)
    items = [t.strip() for t in items if t.strip()]
    if not items:
        raise ValueError("LoRA target_modules cannot be empty")
    return items


def add_lora(network: nn.Module, lora_rank: int = 4, lora_alpha: float = 4, lora_target_modules=DEFAULT_TARGETS,
             init_lora_weights: bool = True) -> nn.Module:
    """Wrap every ``nn.Linear`` whose qualified name ends with a target; freeze everything else."""
    if lora_rank <= 0:
        raise ValueError(f"LoRA rank must be positive, got {lora_rank}")
    if lora_alpha <= 0:
        raise ValueError(f"LoRA alpha must be positive, got {lora_alpha}")
    targets = _targets(lora_target_modules)
    names = [n for n, _ in network.named_modules()]
    missing = [t for t in targets if not any(t in n for n in names)]
    if missing:
        log.warning(f"LoRA target modules not found in model: {missing}")
    for p in network.parameters():
        p.requires_grad_(False)
    n_wrapped = 0
    for name, mod in list(network.named_modules()):
        if not isinstance(mod, nn.Linear) or isinstance(mod, LoRALinear):
            continue
        if ".lora_A." in name or ".lora_B." in name or name.endswith("base_layer"):
            continue
        if not any(name == t or name.endswith("." + t) for t in targets):
            continue
        parent_name, _, child = name.rpartition(".")
        parent = network.get_submodule(parent_name) if parent_name else network
        setattr(parent, child, LoRALinear(mod, lora_rank, lora_alpha, init_lora_weights))
        n_wrapped += 1
    lora_params = sum(p.numel() for p in network.parameters() if p.requires_grad)
    total = sum(p.numel() for p in network.parameters())
    log.info(f"LoRA: wrapped {n_wrapped} projections, {lora_params:,} trainable of {total:,} parameters "
             f"({100 * lora_params / max(total, 1):.3f}%)")
    return network


def lora_modules(network: nn.Module) -> Iterable[LoRALinear]:
    return (m for m in network.modules() if isinstance(m, LoRALinear))


def merge_lora(network: nn.Module):
    for m in lora_modules(network):
        m.merge()


def unmerge_lora(network: nn.Module):
    for m in lora_modules(network):
        m.unmerge()


def lora_state_dict(network: nn.Module):
    """Only the adapter tensors (what a LoRA post-training run needs to save)."""
    return {k: v for k, v in network.state_dict().items() if ".lora_A." in k or ".lora_B." in k}
