"""Float8 linear layers: quantisation round trip, forward / backward against fp32 within the 8-bit error, model conversion."""

import torch
import torch.nn as nn

from cosmos_predict25_b200.modules.float8 import E4M3, E5M2, Float8Linear, convert_to_float8, float8_linear, quantize


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm()).item()


def test_quantize_round_trip():
    torch.manual_seed(0)
    t = torch.randn(64, 48) * 3
    for dtype, tol in ((E4M3, 0.04), (E5M2, 0.08)):
        q, s = quantize(t, dtype)
        assert q.dtype == dtype and _rel(q.float() / s, t) < tol
    q, s = quantize(torch.zeros(4, 16))
    assert torch.isfinite(s) and q.float().abs().max() == 0


def test_float8_linear_forward_and_gradients_are_close_to_fp32():
    torch.manual_seed(1)
    x = torch.randn(3, 20, 64, requires_grad=True)
    w = (torch.randn(96, 64) / 8).requires_grad_()
    b = torch.randn(96, requires_grad=True)
    y = float8_linear(x, w, b)
    g = torch.randn_like(y)
    y.backward(g)
    x2, w2, b2 = (t.detach().clone().requires_grad_() for t in (x, w, b))
    y2 = torch.nn.functional.linear(x2, w2, b2)
    y2.backward(g)
    assert _rel(y, y2) < 0.05 and _rel(x.grad, x2.grad) < 0.08 and _rel(w.grad, w2.grad) < 0.08
    assert torch.allclose(b.grad, b2.grad, atol=1e-5)


def test_convert_swaps_supported_linears_and_shares_parameters():
    torch.manual_seed(2)
    model = nn.Sequential(nn.Linear(32, 64), nn.GELU(), nn.Linear(64, 30), nn.Linear(30, 16), nn.Linear(16, 16))
    first = model[0].weight
    n = convert_to_float8(model, module_filter=lambda name, m: name != "4")      # "2", "3": sizes not multiples of 16; "4": filtered
    assert n == 1 and isinstance(model[0], Float8Linear) and all(type(model[i]) is nn.Linear for i in (2, 3, 4))
    assert model[0].weight is first and list(model.state_dict())[:2] == ["0.weight", "0.bias"]
    out = model(torch.randn(5, 32))
    out.sum().backward()
    assert model[0].weight.grad is not None and out.shape == (5, 16)
