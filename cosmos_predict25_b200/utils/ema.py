"""Exponential-moving-average weights kept outside the sharded engine.

The video models of this package keep their EMA inside the optimizer kernel (``parallel/fsdp.py``: one pass updates masters,
moments and the EMA shard). These classes serve everything else - small models, the VLM stack, scripts written against the
reference - with the API of cosmos_predict2/_src/imaginaire/utils/ema.py:

* ``FastEmaModelUpdater``: stateless; updates a target module (fp32) from a source module with ``torch._foreach`` ops.
* ``EMAModelTracker``: a module whose buffers are the EMA weights, named like the parameters with ``.`` replaced by ``-``
  (buffers cannot have dots), so that they travel in the model's state dict; ``update_average`` / ``copy_to`` / ``cache`` /
  ``restore``.
* ``PowerEMATracker``: the power-function schedule of the EDM2 paper: beta_i = (1 - 1/(i+1))^(gamma+1) with gamma chosen so that
  the averaging profile has relative width ``s``.
* ``ema_scope``: run a block with the EMA weights in place of the regular ones.
"""

from __future__ import annotations

import contextlib
from typing import Any, Iterable, List, Optional

import numpy as np
import torch


class FastEmaModelUpdater:
    def __init__(self):
        self.is_cached = False
        self.collected_params: List[torch.Tensor] = []

    @torch.no_grad()
    def update_average(self, src_model: torch.nn.Module, tgt_model: torch.nn.Module, beta: float = 0.9999) -> None:
        tgt = list(tgt_model.parameters())
        src = [p.data for p in src_model.parameters()]
        for t in tgt:
            assert t.dtype == torch.float32, f"EMA model only works in FP32 dtype, got {t.dtype} instead."
        if tgt:
            torch._foreach_mul_(tgt, beta)
            torch._foreach_add_(tgt, [s.to(t.dtype) for s, t in zip(src, tgt)], alpha=1.0 - beta)

    @torch.no_grad()
    def copy_to(self, src_model: torch.nn.Module, tgt_model: torch.nn.Module) -> None:
        for t, s in zip(tgt_model.parameters(), src_model.parameters()):
            t.data.copy_(s.data)

    def cache(self, parameters: Iterable[torch.Tensor], is_cpu: bool = False) -> None:
        assert not self.is_cached, "EMA cache is already taken. Did you forget to restore it?"
        self.collected_params = [p.detach().clone().cpu() if is_cpu else p.detach().clone() for p in parameters]
        self.is_cached = True

    @torch.no_grad()
    def restore(self, parameters: Iterable[torch.Tensor]) -> None:
        assert self.is_cached, "EMA cache is not taken yet."
        for c, p in zip(self.collected_params, parameters):
            p.data.copy_(c.data.to(p.device).type_as(p.data))
        self.collected_params, self.is_cached = [], False


def get_buffer_name(param_name: str, torch_compile_buffer_renaming: bool = False) -> str:
    name = param_name.replace(".", "-")
    return name.replace("_orig_mod-", "") if torch_compile_buffer_renaming else name


class EMAModelTracker(torch.nn.Module):
    def __init__(self, model: torch.nn.Module, beta: float = 0.9999, torch_compile_buffer_renaming: bool = False):
        super().__init__()
        self.torch_compile_buffer_renaming = torch_compile_buffer_renaming
        self.beta = beta
        self.collected_params: List[torch.Tensor] = []
        for name, p in model.named_parameters():
            if p.requires_grad:
                self.register_buffer(get_buffer_name(name, torch_compile_buffer_renaming), p.detach().clone().float())

    def _pairs(self, model: torch.nn.Module):
        bufs = dict(self.named_buffers())
        for name, p in model.named_parameters():
            if p.requires_grad:
                yield p, bufs[get_buffer_name(name, self.torch_compile_buffer_renaming)]

    @torch.no_grad()
    def update_average(self, model: torch.nn.Module, iteration: Optional[int] = None) -> None:
        del iteration
        params, emas = zip(*self._pairs(model))
        torch._foreach_mul_(list(emas), self.beta)
        torch._foreach_add_(list(emas), [p.data.to(e.dtype) for p, e in zip(params, emas)], alpha=1.0 - self.beta)

    @torch.no_grad()
    def copy_to(self, model: torch.nn.Module) -> None:
        for p, e in self._pairs(model):
            p.data.copy_(e.data.to(p.dtype))

    def cache(self, parameters: Iterable[torch.Tensor]) -> None:
        self.collected_params = [p.detach().clone() for p in parameters]

    @torch.no_grad()
    def restore(self, parameters: Iterable[torch.Tensor]) -> None:
        for c, p in zip(self.collected_params, parameters):
            p.data.copy_(c.data)
        self.collected_params = []

    @classmethod
    def initialize_multi_rank_ema(cls, model: torch.nn.Module, rate: float, num: int, enabled: bool = True):
        """One tracker per rank; rank r < ``num`` uses ``rate / 2^r`` (several averaging widths from one run)."""
        if not enabled:
            return None
        import torch.distributed as dist
        rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        return cls(model, rate / (2 ** rank) if rank < num else rate)


class PowerEMATracker(EMAModelTracker):
    def __init__(self, model: torch.nn.Module, s: float = 0.1, torch_compile_buffer_renaming: bool = False):
        super().__init__(model, beta=0.0, torch_compile_buffer_renaming=torch_compile_buffer_renaming)
        self.exp = float(np.roots([1, 7, 16 - s ** -2, 12 - s ** -2]).real.max())

    @torch.no_grad()
    def update_average(self, model: torch.nn.Module, iteration: Optional[int] = None) -> None:
        self.beta = 0.0 if not iteration else (1 - 1 / (iteration + 1)) ** (self.exp + 1)
        super().update_average(model, iteration)


@contextlib.contextmanager
def ema_scope(model: Any, enabled: bool = False):
    """Run the body with ``model.ema``'s weights in ``model``; the regular weights come back afterwards."""
    if enabled:
        params = [p for p in model.parameters() if p.requires_grad]
        model.ema.cache(params)
        model.ema.copy_to(model)
    try:
        yield None
    finally:
        if enabled:
            model.ema.restore([p for p in model.parameters() if p.requires_grad])
