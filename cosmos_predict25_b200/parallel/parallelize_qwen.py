"""Parallelisation recipe for the Qwen language tower (the text encoder / VLM side).

Parity target: ``parallelize_qwen`` and its steps ``apply_tp`` / ``apply_ac`` / ``apply_compile`` / ``apply_fsdp`` / ``apply_ddp``
(cosmos_predict2/_src/reason1/parallelisms/parallelize_qwen.py:48-400). Tensor parallelism uses DTensor plans: q/k/v and
gate/up projections column-wise, o / down projections row-wise (one all-reduce per attention and per MLP); with
``sequence_parallel`` the residual stream is sharded on the sequence axis between blocks and the norms run
sequence-parallel. Activation checkpointing wraps every (or every n-th) layer. FSDP / DDP use torch's composable APIs on the
``dp_shard_cp`` / ``dp`` mesh views. ``torch.compile`` is not part of this framework's execution model, so ``apply_compile`` only
validates its argument.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from ..utils import log
from .parallel_dims import ParallelDims


def apply_tp(model: nn.Module, tp_mesh, sequence_parallel: bool = False, loss_parallel: bool = False, enable_float8: bool = False,
             enable_async_tp: bool = False) -> nn.Module:
    from torch.distributed.tensor import Replicate, Shard
    from torch.distributed.tensor.parallel import (ColwiseParallel, PrepareModuleInput, RowwiseParallel, SequenceParallel,
                                                   parallelize_module)
    if enable_async_tp:
        # the reference's asynchronous tensor parallelism is a torch.compile pass over symmetric memory; this framework's
        # counterpart for weights that arrive over NVLink is the all-gather fused into the GEMM kernel of the video model
        log.warning("async tensor parallelism relies on torch.compile; running the synchronous plan")
    cfg = model.config
    tp = tp_mesh.size()
    assert cfg.num_attention_heads % tp == 0 and cfg.num_key_value_heads % tp == 0, \
        f"tp={tp} must divide the attention ({cfg.num_attention_heads}) and key/value ({cfg.num_key_value_heads}) head counts"
    if sequence_parallel:
        parallelize_module(model, tp_mesh, {
            "embed_tokens": RowwiseParallel(input_layouts=Replicate(), output_layouts=Shard(1)),
            "norm": SequenceParallel(),
        })
    for layer in model.layers:
        if sequence_parallel:
            plan = {
                "input_layernorm": SequenceParallel(),
                "self_attn": PrepareModuleInput(input_layouts=(Shard(1), None, None, None), desired_input_layouts=(Replicate(), None, None, None)),
                "self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(), "self_attn.v_proj": ColwiseParallel(),
                "self_attn.o_proj": RowwiseParallel(output_layouts=Shard(1)),
                "post_attention_layernorm": SequenceParallel(),
                "mlp": PrepareModuleInput(input_layouts=(Shard(1),), desired_input_layouts=(Replicate(),)),
                "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(),
                "mlp.down_proj": RowwiseParallel(output_layouts=Shard(1)),
            }
        else:
            plan = {
                "self_attn.q_proj": ColwiseParallel(), "self_attn.k_proj": ColwiseParallel(), "self_attn.v_proj": ColwiseParallel(),
                "self_attn.o_proj": RowwiseParallel(),
                "mlp.gate_proj": ColwiseParallel(), "mlp.up_proj": ColwiseParallel(), "mlp.down_proj": RowwiseParallel(),
            }
        parallelize_module(layer, tp_mesh, plan)
    log.info(f"applied tensor parallelism (tp={tp}, sequence_parallel={sequence_parallel})")
    return model


class _Checkpointed(nn.Module):
    def __init__(self, inner: nn.Module):
        super().__init__()
        self.inner = inner

    def forward(self, *args, **kwargs):
        from torch.utils.checkpoint import checkpoint
        if torch.is_grad_enabled():
            return checkpoint(self.inner, *args, use_reentrant=False, **kwargs)
        return self.inner(*args, **kwargs)


def apply_ac(model: nn.Module, mode: str = "full", selective_option: str = "2") -> nn.Module:
    """``full``: every layer; ``selective`` with an integer option n: every n-th layer; ``none``."""
    if mode == "none":
        return model
    if mode not in ("full", "selective"):
        raise ValueError(f"invalid activation-checkpoint mode {mode!r}")
    every = 1 if mode == "full" else int(selective_option)
    for i, layer in enumerate(list(model.layers)):
        if i % every == 0:
            model.layers[i] = _Checkpointed(layer)
    return model


def apply_float8(model: nn.Module, keep_high_precision=("lm_head", "embed_tokens")) -> int:
    """Run the linear layers of the tower on 8-bit GEMM operands (dynamic tensor-wise scaling, e4m3 forward / e5m2 gradients:
    ``modules/float8.py``). Applied BEFORE the tensor-parallel plan: the converted layers are still ``nn.Linear`` modules, so the
    column- / row-wise plans shard them as usual and the 8-bit products run on the local shards."""
    from ..modules.float8 import convert_to_float8
    n = convert_to_float8(model, lambda name, m: not any(k in name for k in keep_high_precision))
    log.info(f"float8: {n} linear layers converted")
    return n


def apply_compile(model: nn.Module, enabled: bool = False) -> nn.Module:
    if enabled:
        raise NotImplementedError("torch.compile is not used by this framework: hot operators are hand-written kernels")
    return model


def apply_fsdp(model: nn.Module, dp_mesh, param_dtype=torch.bfloat16, reduce_dtype=torch.float32, reshard_after_forward: bool = True,
               cpu_offload: bool = False) -> nn.Module:
    from torch.distributed.fsdp import CPUOffloadPolicy, MixedPrecisionPolicy, fully_shard
    kw = dict(mesh=dp_mesh, mp_policy=MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype))
    if cpu_offload:
        kw["offload_policy"] = CPUOffloadPolicy()
    n = len(model.layers)
    for i, layer in enumerate(model.layers):
        fully_shard(layer, **kw, reshard_after_forward=reshard_after_forward and i < n - 1)   # the last layer is needed again at once
    fully_shard(model, **kw, reshard_after_forward=reshard_after_forward)
    return model


def apply_ddp(model: nn.Module, dp_mesh) -> nn.Module:
    from torch.distributed._composable.replicate import replicate
    replicate(model, device_mesh=dp_mesh, bucket_cap_mb=100)
    return model


def parallelize_qwen(model: nn.Module, world_mesh, parallel_dims: ParallelDims, ac_mode: str = "none", sequence_parallel: bool = False,
                     enable_float8: bool = False, enable_async_tp: bool = False, compile: bool = False, data_parallel: str = "fsdp",
                     param_dtype=torch.bfloat16, reduce_dtype=torch.float32) -> nn.Module:
    """(float8 conversion) -> TP -> activation checkpointing -> (compile) -> FSDP / DDP, in that order."""
    if enable_float8:
        apply_float8(model)
    if parallel_dims.tp_enabled:
        apply_tp(model, world_mesh["tp"], sequence_parallel, parallel_dims.loss_parallel_enabled, enable_float8, enable_async_tp)
    apply_ac(model, ac_mode)
    apply_compile(model, compile)
    if parallel_dims.dp_shard_enabled or parallel_dims.cp_enabled:
        apply_fsdp(model, world_mesh["dp_shard_cp"], param_dtype, reduce_dtype)
    elif parallel_dims.dp_replicate_enabled and data_parallel == "ddp":
        apply_ddp(model, world_mesh["dp_replicate"])
    return model
