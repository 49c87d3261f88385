"""Activation checkpointing of DiT blocks.

Modes (names of the reference's ``CheckpointMode`` they correspond to in parentheses;
cosmos_predict2/_src/predict2/networks/selective_activation_checkpoint.py:34-73,
cosmos_predict2/_src/predict2/networks/minimal_v4_dit.py:53-198):

  none            keep every activation ("none")
  block_wise      keep only each block's input, recompute the whole block in backward ("block_wise")
  save_attention  recompute everything except attention outputs, which are kept
                  ("predict2_2b_720_aggressive": at 84k tokens attention is ~85 % of a block's
                  FLOPs, so this costs ~1.15x forward instead of 2x)
  mm_only         keep matmul outputs, recompute the element-wise ops ("mm_only")
  save_attention_some_mm   attention outputs + a fraction of the GEMM outputs
                  ("predict2_14b_720_aggressive": 3 of every 16 matmuls)
"""

from __future__ import annotations

import functools
from typing import Optional

import torch
from torch.utils.checkpoint import CheckpointPolicy, checkpoint, create_selective_checkpoint_contexts

from ..ops import native

CHECKPOINT_MODES = ("none", "block_wise", "save_attention", "mm_only", "save_attention_some_mm")

# reference mode names accepted as aliases
MODE_ALIASES = {
    "predict2_2b_720": "save_attention",
    "predict2_2b_720_aggressive": "save_attention",
    "predict2_14b_720": "save_attention_some_mm",
    "predict2_14b_720_aggressive": "save_attention_some_mm",
    "predict2_14b_720_aggressive_v2": "save_attention_some_mm",
    "linear_selfattn": "mm_only",
}


def _attention_ops():
    names = []
    aten = torch.ops.aten
    for n in ("_scaled_dot_product_cudnn_attention", "_scaled_dot_product_flash_attention",
              "_scaled_dot_product_efficient_attention", "_scaled_dot_product_flash_attention_for_cpu"):
        if hasattr(aten, n):
            names.append(getattr(aten, n).default)
    for n in ("fa_fwd", "fa_fwd_na"):
        try:
            names.append(getattr(torch.ops.cosmos_b200, n).default)
        except (AttributeError, RuntimeError):
            pass
    return set(names)


def _mm_ops():
    aten = torch.ops.aten
    s = {aten.mm.default, aten.addmm.default, aten.bmm.default}
    for name in ("gemm_bf16", "gemm_bf16_gelu_pre", "gemm_bf16_gate_residual", "gemm_bf16_gate_residual_pre", "gemm_bf16_gather"):
        try:
            s.add(getattr(torch.ops.cosmos_b200, name).default)
        except (AttributeError, RuntimeError):
            pass
    return s


def _make_policy(mode: str):
    attn, mm = _attention_ops(), _mm_ops()
    own = {op for op in (attn | mm) if "cosmos_b200" in str(op)}   # operators whose front-ends count kernel launches
    counter = {False: 0, True: 0}  # forward pass / recompute pass must take identical decisions

    def decide(ctx, op):
        if mode in ("save_attention", "save_attention_some_mm") and op in attn:
            return CheckpointPolicy.MUST_SAVE
        if mode == "mm_only" and (op in mm or op in attn):
            return CheckpointPolicy.MUST_SAVE
        if mode == "save_attention_some_mm" and op in mm:
            counter[bool(ctx.is_recompute)] += 1
            if counter[bool(ctx.is_recompute)] % 16 in (1, 6, 11):
                return CheckpointPolicy.MUST_SAVE
        return CheckpointPolicy.PREFER_RECOMPUTE

    def policy(ctx, op, *args, **kwargs):
        d = decide(ctx, op)
        if d == CheckpointPolicy.MUST_SAVE and ctx.is_recompute and op in own:
            # the recompute pass takes this result from the cache: the front-end still counted a launch that never happens
            native.count_launch(-1)
        return d

    return policy


def run_block(block, mode: str, *args):
    """Run ``block(*args)`` under the activation-checkpoint ``mode``."""
    mode = MODE_ALIASES.get(mode, mode)
    if mode == "none" or not torch.is_grad_enabled():
        return block(*args)
    if mode == "block_wise":
        return checkpoint(block, *args, use_reentrant=False)
    if mode not in CHECKPOINT_MODES:
        raise ValueError(f"unknown checkpoint mode {mode!r}; expected one of {CHECKPOINT_MODES}")
    ctx_fn = functools.partial(create_selective_checkpoint_contexts, _make_policy(mode))
    return checkpoint(block, *args, use_reentrant=False, context_fn=ctx_fn)
