"""Float8 training of linear layers (the language / vision towers of the VLM stack).

Recipe (dynamic, tensor-wise scaling; what the reference enables through torchao in
cosmos_predict2/_src/reason1/parallelisms/parallelize_qwen.py:114-176, ``enable_float8``):

* forward   y = x W^T      x, W quantised to e4m3 with one scale each (448 / amax), fp32 accumulation, output in the input dtype
* backward  dx = g W       g quantised to e5m2 (57344 / amax), W e4m3
            dW = g^T x     g e5m2, x e4m3 (the quantised x of the forward is what is kept for the backward: half the bytes of bf16)

The master weights stay in their own dtype; only the GEMM operands are 8-bit. On a GPU the three products are fp8 tensor-core
GEMMs of the vendor library (``torch._scaled_mm``: plain library GEMMs, nothing is fused around them); on the CPU the same
quantised operands are multiplied in fp32, which is the oracle of the tests.

Tensor parallelism: when the weight is a DTensor sharded by ``ColwiseParallel`` / ``RowwiseParallel``, the product runs on the
local shards with per-shard scales (every partial product is de-quantised before it is summed, so no scale has to be agreed
between ranks) and the result is handed back as a DTensor with the placement the plan expects (sharded on the last dimension,
or partial sums).
"""

from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.nn as nn

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2
_FMAX = {E4M3: 448.0, E5M2: 57344.0}


def quantize(t: torch.Tensor, dtype=E4M3):
    """(8-bit tensor, scale): ``t ~= q.float() / scale`` with ``scale = fmax / amax(t)`` (an fp32 scalar tensor on t's device)."""
    amax = t.detach().abs().amax().float().clamp_(min=1e-12)
    scale = _FMAX[dtype] / amax
    q = (t.detach().float() * scale).clamp_(-_FMAX[dtype], _FMAX[dtype]).to(dtype).contiguous()
    return q, scale


def scaled_mm(a8: torch.Tensor, sa: torch.Tensor, b8: torch.Tensor, sb: torch.Tensor, out_dtype) -> torch.Tensor:
    """``(a8 / sa) @ (b8 / sb)^T`` for row-major ``a8 [M, K]`` and ``b8 [N, K]``."""
    if a8.is_cuda:
        K = a8.shape[1]
        if K % 16:                      # the contraction length of the weight gradient is the token count: pad with zero rows
            pad = 16 - K % 16
            a8 = torch.nn.functional.pad(a8.view(torch.uint8), (0, pad)).view(a8.dtype)
            b8 = torch.nn.functional.pad(b8.view(torch.uint8), (0, pad)).view(b8.dtype)
        if b8.shape[0] % 16 == 0:
            return torch._scaled_mm(a8, b8.t(), scale_a=sa.reciprocal(), scale_b=sb.reciprocal(), out_dtype=out_dtype)
        return ((a8.to(torch.bfloat16) @ b8.to(torch.bfloat16).t()).float() / (sa * sb)).to(out_dtype)
    return ((a8.float() @ b8.float().t()) / (sa * sb)).to(out_dtype)


class _Float8Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        x8, sx = quantize(x2)
        w8, sw = quantize(w)
        ctx.save_for_backward(x8, sx, w8, sw)
        ctx.x_shape, ctx.x_dtype, ctx.w_dtype = x.shape, x.dtype, w.dtype
        return scaled_mm(x8, sx, w8, sw, x.dtype).reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, g: torch.Tensor):
        x8, sx, w8, sw = ctx.saved_tensors
        g8, sg = quantize(g.reshape(-1, g.shape[-1]), E5M2)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = scaled_mm(g8, sg, w8.t().contiguous(), sw, ctx.x_dtype).reshape(ctx.x_shape)           # [M, N] x [K, N]^T
        if ctx.needs_input_grad[1]:
            acc = torch.float32 if not g.is_cuda or ctx.w_dtype == torch.float32 else ctx.w_dtype
            dw = scaled_mm(g8.t().contiguous(), sg, x8.t().contiguous(), sx, acc).to(ctx.w_dtype)      # [N, M] x [K, M]^T
        return dx, dw


def float8_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = _Float8Linear.apply(x, w)
    return y if bias is None else y + bias.to(y.dtype)


def _supported(in_features: int, out_features: int) -> bool:
    return in_features % 16 == 0 and out_features % 16 == 0        # the fp8 tensor-core GEMM's size rule


class Float8Linear(nn.Linear):
    """``nn.Linear`` whose three GEMMs run on 8-bit operands; parameters, state dict and initialisation are nn.Linear's."""

    @classmethod
    def from_linear(cls, lin: nn.Linear) -> "Float8Linear":
        new = cls.__new__(cls)
        nn.Module.__init__(new)
        new.in_features, new.out_features = lin.in_features, lin.out_features
        new.weight, new.bias = lin.weight, lin.bias
        return new

    def forward(self, x):
        from torch.distributed.tensor import DTensor
        w = self.weight
        if not isinstance(w, DTensor):
            return float8_linear(x, w, self.bias)
        from torch.distributed.tensor import Partial, Shard
        assert len(w.placements) == 1 and isinstance(w.placements[0], Shard), "float8 expects a weight sharded over one mesh dimension"
        mesh, col = w.device_mesh, w.placements[0].dim == 0
        if isinstance(x, DTensor):
            # column-wise: x is replicated, each rank's input gradient is a partial sum; row-wise: x is sharded on its last dimension
            x = x.to_local(grad_placements=[Partial()] if col else [Shard(x.dim() - 1)])
        y = _Float8Linear.apply(x, w.to_local())
        if col:
            if self.bias is not None:
                y = y + self.bias.to_local().to(y.dtype)
            return DTensor.from_local(y, mesh, [Shard(y.dim() - 1)], run_check=False)
        assert self.bias is None, "a row-wise sharded float8 linear cannot add its bias before the partial sums are reduced"
        return DTensor.from_local(y, mesh, [Partial()], run_check=False)


def convert_to_float8(model: nn.Module, module_filter: Optional[Callable[[str, nn.Linear], bool]] = None) -> int:
    """Swap every ``nn.Linear`` of ``model`` (exact type, sizes multiples of 16, accepted by ``module_filter(name, module)``) for a
    ``Float8Linear`` that shares its parameters. Returns the number of layers converted. The usual filter keeps the output head
    and anything feeding a softmax over the vocabulary in high precision."""
    n = 0
    for name, mod in list(model.named_modules()):
        for child_name, child in list(mod.named_children()):
            full = f"{name}.{child_name}" if name else child_name
            if type(child) is nn.Linear and _supported(child.in_features, child.out_features) and (
                    module_filter is None or module_filter(full, child)):
                setattr(mod, child_name, Float8Linear.from_linear(child))
                n += 1
    return n
