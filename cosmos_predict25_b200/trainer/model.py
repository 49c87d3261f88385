"""Base class of trainable models: the hooks the trainer calls
(contract of cosmos_predict2/_src/imaginaire/model.py:23-129). The video models of this package implement the same methods
without deriving from it; it exists for user models and for code written against the reference."""

from __future__ import annotations

from typing import Any, Dict, Tuple

import torch


class ImaginaireModel(torch.nn.Module):
    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        """(optimizer, scheduler) for this model's trainable parameters."""
        from ..utils.lazy_config import instantiate, is_lazy
        if is_lazy(optimizer_config):
            # the reference's form: lazy calls whose ``params`` / ``optimizer`` arguments are filled in here
            # (imaginaire/model.py:40-56 there)
            optimizer = instantiate(optimizer_config, params=[p for p in self.parameters() if p.requires_grad])
            return optimizer, instantiate(scheduler_config, optimizer=optimizer)
        from .optim import build_scheduler
        opt = torch.optim.AdamW([p for p in self.parameters() if p.requires_grad], lr=optimizer_config.lr, betas=tuple(optimizer_config.betas),
                                eps=optimizer_config.eps, weight_decay=optimizer_config.weight_decay)
        for g in opt.param_groups:
            g.setdefault("initial_lr", g["lr"])
        return opt, build_scheduler(scheduler_config, opt)

    def training_step(self, data_batch: Dict[str, torch.Tensor], iteration: int) -> Tuple[Dict[str, torch.Tensor], torch.Tensor]:
        raise NotImplementedError

    @torch.no_grad()
    def validation_step(self, data_batch: Dict[str, torch.Tensor], iteration: int) -> Tuple[Dict[str, torch.Tensor], torch.Tensor]:
        raise NotImplementedError

    @torch.inference_mode()
    def forward(self, *args: Any, **kwargs: Any) -> Any:
        raise NotImplementedError

    def on_train_start(self, memory_format: torch.memory_format = torch.preserve_format) -> None:
        pass

    def on_before_zero_grad(self, optimizer, scheduler, iteration: int) -> None:
        pass

    def on_after_backward(self, iteration: int = 0) -> None:
        pass
