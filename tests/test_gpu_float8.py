"""Float8 linear on the GPU (fp8 tensor-core GEMMs of the vendor library) against the CPU emulation of the same quantised product."""

import pytest
import torch

from cosmos_predict25_b200.modules.float8 import float8_linear


@pytest.mark.gpu
def test_float8_linear_gpu_matches_the_emulated_product():
    torch.manual_seed(0)
    x = torch.randn(2, 50, 128)                    # 100 tokens: the weight gradient's contraction length is padded to 112
    w = torch.randn(256, 128) / 11
    g = torch.randn(2, 50, 256)
    outs = []
    for dev in ("cpu", "cuda"):
        xd = x.to(dev, torch.bfloat16).requires_grad_()
        wd = w.to(dev, torch.bfloat16).requires_grad_()
        y = float8_linear(xd, wd)
        y.backward(g.to(dev, torch.bfloat16))
        outs.append([t.float().cpu() for t in (y, xd.grad, wd.grad)])
    for a, b, name in zip(outs[0], outs[1], ("output", "input gradient", "weight gradient")):
        rel = ((a - b).norm() / a.norm()).item()
        assert rel < 2e-2, (name, rel)            # same 8-bit operands; only accumulation order and the bf16 rounding differ
    ref = torch.nn.functional.linear(x, w)
    assert ((outs[1][0] - ref).norm() / ref.norm()).item() < 0.06
