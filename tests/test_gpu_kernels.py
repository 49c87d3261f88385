"""Numerics of every sm_100a kernel against the plain PyTorch fp32 oracle of the same op."""

import math

import pytest
import torch

from cosmos_predict25_b200.ops import functional as F_ops
from cosmos_predict25_b200.ops import native, ref

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _ops():
    return native.load()


def _close(a, b, atol, rtol, name="", cap=8.0):
    """At most 1e-4 of the elements may miss the tolerance (bf16 rounding outliers), and NO element may miss it by more
    than ``cap`` times: a wrong tail row or a dropped tile fails even when it is a tiny share of the tensor."""
    a, b = a.float(), b.float()
    assert a.shape == b.shape, f"{name}: shape {tuple(a.shape)} vs {tuple(b.shape)}"
    assert torch.isfinite(a).all(), f"{name}: non-finite values"
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    worst = (err / tol).max().item()
    assert bad < 1e-4, f"{name}: {bad * 100:.3f}% elements out of tolerance, max err {err.max().item():.4g}"
    assert worst < cap, f"{name}: an element misses the tolerance {worst:.1f}-fold (max err {err.max().item():.4g})"


def _no_kernel_error():
    torch.cuda.synchronize()
    code = _ops().kernel_error(torch.cuda.current_device(), True)
    assert code == 0, f"a kernel reported bounded-wait error code {code}"


@pytest.mark.parametrize("D,L,T", [(256, 12, 3), (2048, 40, 2), (5120, 7, 2)])
def test_ln_modulate_fwd_bwd(D, L, T):
    torch.manual_seed(0)
    B = 2
    x = torch.randn(B, T, L, D, device=DEV).bfloat16().requires_grad_(True)
    shift = (0.1 * torch.randn(B, T, D, device=DEV)).requires_grad_(True)
    scale = (0.1 * torch.randn(B, T, D, device=DEV)).requires_grad_(True)
    y = F_ops.ln_modulate(x, shift, scale)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    sr = shift.detach().clone().requires_grad_(True)
    cr = scale.detach().clone().requires_grad_(True)
    yr = ref.ln_modulate(xr, sr, cr)
    yr.backward(dy.float())
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(x.grad, xr.grad, 3e-2, 3e-2, "dx")
    _close(shift.grad, sr.grad, 5e-2 * math.sqrt(L), 2e-2, "dshift")
    _close(scale.grad, cr.grad, 5e-2 * math.sqrt(L), 2e-2, "dscale")


@pytest.mark.parametrize("D,L", [(256, 9), (2048, 33)])
def test_gate_residual_fwd_bwd(D, L):
    torch.manual_seed(1)
    B, T = 2, 3
    x = torch.randn(B, T, L, D, device=DEV).bfloat16().requires_grad_(True)
    y = torch.randn(B, T, L, D, device=DEV).bfloat16().requires_grad_(True)
    g = torch.randn(B, T, D, device=DEV).requires_grad_(True)
    out = F_ops.gate_residual(x, g, y)
    do = torch.randn_like(out)
    out.backward(do)
    xr, yr, gr = (t.detach().float().requires_grad_(True) for t in (x, y, g))
    outr = ref.gate_residual(xr, gr, yr)
    outr.backward(do.float())
    _close(out, outr, 2e-2, 2e-2, "out")
    _close(x.grad, xr.grad, 1e-2, 1e-2, "dx")
    _close(y.grad, yr.grad, 2e-2, 2e-2, "dy")
    _close(g.grad, gr.grad, 5e-2 * math.sqrt(L), 2e-2, "dgate")


@pytest.mark.parametrize("HD,use_rope", [(128, True), (128, False), (64, True)])
def test_rmsnorm_rope_fwd_bwd(HD, use_rope):
    torch.manual_seed(2)
    B, S, H = 2, 37, 3
    x = torch.randn(B, S, H, HD, device=DEV).bfloat16().requires_grad_(True)
    w = (1 + 0.1 * torch.randn(HD, device=DEV)).requires_grad_(True)
    half = torch.rand(S, HD // 2, device=DEV) * 50
    angles = torch.cat([half, half], -1)
    rope = F_ops.RopeTable(angles) if use_rope else None
    y = F_ops.rmsnorm_rope(x, w, rope)
    dy = torch.randn_like(y)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    wr = w.detach().clone().requires_grad_(True)
    yr = ref.rmsnorm_rope(xr, wr, angles if use_rope else None)
    yr.backward(dy.float())
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(x.grad, xr.grad, 3e-2, 3e-2, "dx")
    _close(w.grad, wr.grad, 0.3, 3e-2, "dw")


def test_gelu_and_cfg():
    torch.manual_seed(3)
    x = (2 * torch.randn(1000, 64, device=DEV)).bfloat16()
    y = _ops().gelu_fwd(x)
    _close(y, torch.nn.functional.gelu(x.float()), 2e-2, 1e-2, "gelu")
    dy = torch.randn_like(x)
    dx = _ops().gelu_bwd(dy, x)
    xr = x.float().requires_grad_(True)
    torch.nn.functional.gelu(xr).backward(dy.float())
    _close(dx, xr.grad, 2e-2, 2e-2, "dgelu")
    c, u = torch.randn(3, 777, device=DEV), torch.randn(3, 777, device=DEV)
    _close(F_ops.cfg_combine(c, u, 7.0), c + 7.0 * (c - u), 1e-5, 1e-5, "cfg")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (384, 512, 256), (1000, 2048, 512), (4096, 64, 2048), (333 * 8, 2048, 72 * 8)])
def test_gemm_nt(M, N, K):
    torch.manual_seed(4)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    c = _ops().gemm_bf16(a, b, None, 0, False, False)
    _no_kernel_error()
    _close(c, a.float() @ b.float().T, 2e-2, 2e-2, "gemm_nt")


def test_gemm_transposed_operands():
    torch.manual_seed(5)
    M, N, K = 512, 768, 1024
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    want = a.float() @ b.float().T
    c = _ops().gemm_bf16(a, b.T.contiguous(), None, 0, False, True)   # B stored [K, N]
    _no_kernel_error()
    _close(c, want, 2e-2, 2e-2, "gemm trans_b")
    c = _ops().gemm_bf16(a.T.contiguous(), b, None, 0, True, False)   # A stored [K, M]
    _no_kernel_error()
    _close(c, want, 2e-2, 2e-2, "gemm trans_a")
    c = _ops().gemm_bf16(a.T.contiguous(), b.T.contiguous(), None, 0, True, True)
    _no_kernel_error()
    _close(c, want, 2e-2, 2e-2, "gemm trans_a trans_b")


@pytest.fixture
def gemm_pairs():
    """Run the GEMM on CTA pairs (256 x 256 tile per cluster of two) for the duration of a test."""
    prev = _ops().gemm_pair_mode(1)
    yield
    _ops().gemm_pair_mode(prev)


@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (512, 512, 256), (1000, 2048, 512), (4096, 64, 2048), (333 * 8, 2048, 72 * 8),
                                   (8192 + 128, 1024, 1024)])
def test_gemm_cta_pairs(M, N, K, gemm_pairs):
    """tcgen05 cta_group::2 tiles: all operand-major combinations, ragged edges (a pair whose second CTA has no rows, a last
    N tile narrower than 256), many tiles per pair; bitwise equal to the single-CTA kernel (same products, same order)."""
    torch.manual_seed(4)
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    want = a.float() @ b.float().T
    got = {}
    for ta, tb in ((False, False), (False, True), (True, False), (True, True)):
        aa = a.T.contiguous() if ta else a
        bb = b.T.contiguous() if tb else b
        c = _ops().gemm_bf16(aa, bb, None, 0, ta, tb)
        _no_kernel_error()
        _close(c, want, 2e-2, 2e-2, f"pair gemm trans_a={ta} trans_b={tb}")
        got[(ta, tb)] = c
    _ops().gemm_pair_mode(0)
    single = _ops().gemm_bf16(a, b, None, 0, False, False)
    _no_kernel_error()
    _close(single, want, 2e-2, 2e-2, "single-CTA gemm")
    assert torch.equal(single, got[(False, False)])


@pytest.mark.parametrize("M,N,L", [(640, 1024, 40), (600, 1000, 40)])
def test_gemm_cta_pairs_epilogues(M, N, L, gemm_pairs):
    test_gemm_epilogues(M, N, L)


@pytest.mark.parametrize("M,N,L", [(640, 1024, 40), (600, 1024, 40), (600, 1000, 40)])   # full, ragged rows, ragged rows + columns
def test_gemm_epilogues(M, N, L):
    torch.manual_seed(6)
    K = 512
    a = torch.randn(M, K, device=DEV).bfloat16()
    b = (torch.randn(N, K, device=DEV) / math.sqrt(K)).bfloat16()
    bias = torch.randn(N, device=DEV).bfloat16()
    base = a.float() @ b.float().T
    c = _ops().gemm_bf16(a, b, bias, 1, False, False)
    _close(c, torch.nn.functional.gelu(base + bias.float()), 2e-2, 2e-2, "bias+gelu")
    c, pre = _ops().gemm_bf16_gelu_pre(a, b, None)
    _close(pre, base, 2e-2, 2e-2, "pre")
    _close(c, torch.nn.functional.gelu(base), 2e-2, 2e-2, "gelu")
    resid = torch.randn(M, N, device=DEV).bfloat16()
    gate = torch.randn(M // L, N, device=DEV)
    c = _ops().gemm_bf16_gate_residual(a, b, resid, gate, L)
    want = resid.float() + gate.repeat_interleave(L, 0) * base
    _close(c, want, 3e-2, 2e-2, "gate residual")
    _no_kernel_error()


def test_linear_autograd_matches_reference():
    torch.manual_seed(7)
    x = torch.randn(2, 264, 512, device=DEV).bfloat16().requires_grad_(True)
    w = (torch.randn(1024, 512, device=DEV) / math.sqrt(512)).bfloat16().requires_grad_(True)
    y = F_ops.linear(x, w, None, "gelu")
    dy = torch.randn_like(y)
    y.backward(dy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = torch.nn.functional.gelu(xr @ wr.T)
    yr.backward(dy.float())
    _no_kernel_error()
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(x.grad, xr.grad, 3e-2, 3e-2, "dx")
    _close(w.grad, wr.grad, 0.3, 3e-2, "dw")


@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 256, 256, 2), (2, 512, 384, 3), (1, 1000, 999, 2), (1, 300, 15, 4), (1, 2048, 4096, 2)])
def test_flash_attention_fwd(B, Sq, Skv, H):
    torch.manual_seed(8)
    q = torch.randn(B, Sq, H, 128, device=DEV).bfloat16()
    k = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    v = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(128)
    o, lse = _ops().fa_fwd(q, k, v, scale)
    _no_kernel_error()
    orf, lser = ref.attention(q.float(), k.float(), v.float(), scale)
    _close(lse, lser, 2e-2, 1e-3, "lse")
    _close(o, orf, 2e-2, 2e-2, "o")


@pytest.mark.parametrize("vs,window,stride,causal", [
    ((8, 8, 16), (4, 4, 8), 1, False),                       # 8 tiles, every visited tile partly masked
    ((4, 12, 24), (4, 8, 16), (1, 4, 8), False),             # 9 tiles (odd: last CTA has one query tile), stride = tile
    ((8, 8, 16), (3, 5, 7), (1, 2, 3), (True, False, False)),  # causal in time, odd windows
    ((4, 4, 8), (4, 4, 8), 1, False),                        # one tile, whole-axis windows = dense attention
])
def test_neighborhood_attention_kernel(vs, window, stride, causal):
    from cosmos_predict25_b200.modules import neighborhood_attn as na
    torch.manual_seed(12)
    L, H = vs[0] * vs[1] * vs[2], 3
    q, k, v = (torch.randn(2, L, H, 128, device=DEV).bfloat16() for _ in range(3))
    with torch.no_grad():
        assert na.tile_kernel_supported(q, vs, (1, 1, 1))
        got = na.neighborhood_attention(q, k, v, vs, window, stride, 1, causal)
        _no_kernel_error()
        want = na.neighborhood_attention_reference(q.float(), k.float(), v.float(), vs, window, stride, 1, causal)
    _close(got, want, 2e-2, 2e-2, "neighbourhood attention")


@pytest.mark.parametrize("vs,window,stride,causal", [
    ((8, 8, 16), (4, 4, 8), 1, False),                       # every visited tile pair partly masked
    ((4, 12, 24), (4, 8, 16), (1, 4, 8), False),             # 9 tiles, stride = tile
    ((8, 8, 16), (3, 5, 7), (1, 2, 3), (True, False, False)),  # causal in time, odd windows
    ((4, 4, 8), (4, 4, 8), 1, False),                        # one tile, whole-axis windows = dense attention (fully visible pair)
    ((8, 16, 32), (8, 12, 24), 1, False),                    # 32 tiles, wide windows: fully visible pairs beside masked ones
])
def test_neighborhood_attention_backward_kernel(vs, window, stride, causal):
    """Gradients of the tile-sparse kernels (forward + single-pass tile-sparse backward) against autograd through the dense-masked
    fp32 definition."""
    from cosmos_predict25_b200.modules import neighborhood_attn as na
    torch.manual_seed(12)
    L, H = vs[0] * vs[1] * vs[2], 2
    q, k, v = (torch.randn(1, L, H, 128, device=DEV).bfloat16().requires_grad_(True) for _ in range(3))
    assert na.tile_kernel_supported(q, vs, (1, 1, 1)) and na._tile_backward_available()
    before = native.launches()
    got = na.neighborhood_attention(q, k, v, vs, window, stride, 1, causal)
    do = torch.randn_like(got)
    gq, gk, gv = torch.autograd.grad(got, (q, k, v), do)
    assert native.launches() - before >= 4, "the tile-sparse kernels did not serve forward and backward"
    _no_kernel_error()
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    want = na.neighborhood_attention_reference(qr, kr, vr, vs, window, stride, 1, causal)
    wq, wk, wv = torch.autograd.grad(want, (qr, kr, vr), do.float())
    _close(got, want, 2e-2, 2e-2, "o")
    for name, a, b in (("dq", gq, wq), ("dk", gk, wk), ("dv", gv, wv)):
        _close(a, b, 3e-2 * b.abs().max().item() + 1e-3, 3e-2, name)


# tuning variants of the forward kernel: 1 = all exponentials on the special-function unit, whole-row hand-off; 2-6 = polynomial
# share 0..3 of 4 pairs with / without the half-row hand-off; 7, 8 = one query tile per CTA (short key sequences);
# 9-11 = with register re-division between the warpgroups
@pytest.mark.parametrize("variant", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11])
@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 256, 256, 2), (2, 512, 384, 3), (1, 1000, 999, 2), (1, 300, 15, 4), (1, 300, 70, 2),
                                        (1, 2048, 4096, 2)])
def test_flash_attention_fwd_variants(B, Sq, Skv, H, variant):
    torch.manual_seed(9)
    q = torch.randn(B, Sq, H, 128, device=DEV).bfloat16() * 2      # larger scores: the running maximum moves
    k = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    v = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(128)
    o, lse = _ops().fa_fwd_variant(q, k, v, scale, variant)
    _no_kernel_error()
    orf, lser = ref.attention(q.float(), k.float(), v.float(), scale)
    _close(lse, lser, 2e-2, 1e-3, "lse")
    _close(o, orf, 2e-2, 2e-2, "o")


def test_forward_kernels_are_bitwise_repeatable():
    """The forward has no atomics: two runs on the same inputs must agree bit for bit (default shape choice for long and for
    short key sequences)."""
    torch.manual_seed(3)
    scale = 1.0 / math.sqrt(128)
    for Sq, Skv in ((1500, 1400), (900, 512)):
        q = torch.randn(1, Sq, 3, 128, device=DEV).bfloat16()
        k, v = (torch.randn(1, Skv, 3, 128, device=DEV).bfloat16() for _ in range(2))
        o1, l1 = _ops().fa_fwd(q, k, v, scale)
        o2, l2 = _ops().fa_fwd(q, k, v, scale)
        assert torch.equal(o1, o2) and torch.equal(l1, l2)
    _no_kernel_error()


def test_flash_attention_large_scores_rescale():
    """Rows whose maximum keeps growing across key tiles exercise the TMEM rescale path."""
    torch.manual_seed(9)
    B, S, H = 1, 1024, 2
    q = torch.randn(B, S, H, 128, device=DEV).bfloat16()
    k = torch.randn(B, S, H, 128, device=DEV)
    k = (k * torch.linspace(0.2, 6.0, S, device=DEV).view(1, S, 1, 1)).bfloat16()
    v = torch.randn(B, S, H, 128, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(128)
    o, lse = _ops().fa_fwd(q, k, v, scale)
    _no_kernel_error()
    orf, lser = ref.attention(q.float(), k.float(), v.float(), scale)
    _close(lse, lser, 3e-2, 2e-3, "lse")
    _close(o, orf, 3e-2, 3e-2, "o")


@pytest.mark.parametrize("variant", [1, 2, 3])
@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 256, 128, 2), (2, 512, 384, 3), (1, 1000, 999, 2), (1, 300, 15, 2), (1, 2048, 2048, 2),
                                        (1, 1664, 640, 1)])
def test_flash_attention_bwd(B, Sq, Skv, H, variant):
    torch.manual_seed(12)
    q = torch.randn(B, Sq, H, 128, device=DEV).bfloat16()
    k = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    v = torch.randn(B, Skv, H, 128, device=DEV).bfloat16()
    do = torch.randn(B, Sq, H, 128, device=DEV).bfloat16()
    scale = 1.0 / math.sqrt(128)
    o, lse = _ops().fa_fwd(q, k, v, scale)
    dq, dk, dv = _ops().fa_bwd_variant(do, q, k, v, o, lse, scale, variant)
    _no_kernel_error()
    qr, kr, vr = (t.float().requires_grad_(True) for t in (q, k, v))
    orf, _ = ref.attention(qr, kr, vr, scale)
    orf.backward(do.float())
    _close(dv, vr.grad, 3e-2, 3e-2, "dv")
    _close(dk, kr.grad, 3e-2, 3e-2, "dk")
    _close(dq, qr.grad, 3e-2, 3e-2, "dq")


def test_backward_repeatability():
    """The two-kernel backward has no atomics and must repeat bit for bit; the single-pass kernels add dQ partials with
    fp32 reductions whose order is not fixed, so dK / dV repeat exactly and dQ may drift by rounding only."""
    torch.manual_seed(5)
    B, S, H = 1, 1536, 2
    q, k, v, do = (torch.randn(B, S, H, 128, device=DEV).bfloat16() for _ in range(4))
    scale = 1.0 / math.sqrt(128)
    o, lse = _ops().fa_fwd(q, k, v, scale)
    a = _ops().fa_bwd_variant(do, q, k, v, o, lse, scale, 1)
    b = _ops().fa_bwd_variant(do, q, k, v, o, lse, scale, 1)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    for variant in (2, 3):
        a = _ops().fa_bwd_variant(do, q, k, v, o, lse, scale, variant)
        b = _ops().fa_bwd_variant(do, q, k, v, o, lse, scale, variant)
        assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
        drift = (a[0].float() - b[0].float()).abs().max().item()
        assert drift <= 2 ** -7 * a[0].float().abs().max().item(), f"variant {variant}: dQ drifts by {drift}"
    _no_kernel_error()


@pytest.mark.parametrize("B,Sq,Skv,H", [(1, 256, 128, 2), (2, 384, 512, 3), (1, 1000, 999, 2), (1, 300, 15, 2), (1, 2048, 2048, 2)])
def test_flash_attention_jvp(B, Sq, Skv, H):
    torch.manual_seed(14)
    q, tq = (torch.randn(B, Sq, H, 128, device=DEV).bfloat16() for _ in range(2))
    k, v, tk, tv = (torch.randn(B, Skv, H, 128, device=DEV).bfloat16() for _ in range(4))
    scale = 1.0 / math.sqrt(128)
    o, to, lse = _ops().fa_jvp(q, k, v, tq, tk, tv, scale)
    _no_kernel_error()
    orf, tor, lser = ref.attention_jvp(q.float(), k.float(), v.float(), tq.float(), tk.float(), tv.float(), scale)
    _close(o, orf, 3e-2, 3e-2, "o")
    _close(lse, lser, 3e-2, 2e-3, "lse")
    _close(to, tor, 4e-2, 4e-2, "to")
    # cross-check against autograd's forward-mode on the fp32 reference
    import torch.autograd.forward_ad as fwAD
    with fwAD.dual_level():
        qd, kd, vd = (fwAD.make_dual(a.float(), t.float()) for a, t in ((q, tq), (k, tk), (v, tv)))
        od, _ = ref.attention(qd, kd, vd, scale)
        to_ad = fwAD.unpack_dual(od).tangent
    _close(to, to_ad, 4e-2, 4e-2, "to vs forward-mode autograd")


def test_attention_autograd():
    torch.manual_seed(10)
    B, S, H = 1, 384, 2
    q, k, v = (torch.randn(B, S, H, 128, device=DEV).bfloat16().requires_grad_(True) for _ in range(3))
    o = F_ops.attention(q, k, v)
    do = torch.randn_like(o)
    o.backward(do)
    qr, kr, vr = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    orf, _ = ref.attention(qr, kr, vr)
    orf.backward(do.float())
    _no_kernel_error()
    _close(o, orf, 2e-2, 2e-2, "o")
    _close(q.grad, qr.grad, 3e-2, 3e-2, "dq")
    _close(k.grad, kr.grad, 3e-2, 3e-2, "dk")
    _close(v.grad, vr.grad, 3e-2, 3e-2, "dv")


@pytest.mark.parametrize("Z,R,K,N,wdtype,shared,silu,add_cols", [
    (3, 24, 2048, 256, torch.bfloat16, True, True, 0),         # AdaLN-LoRA first stage of one block
    (3, 24, 256, 6144, torch.bfloat16, False, False, 6144),    # second stage + shared LoRA term
    (1, 48, 256, 4096, torch.bfloat16, False, False, 4096),    # final layer: 2 chunks
    (5, 7, 100, 70, torch.float32, True, False, 33),           # ragged everything, fp32 weights, partial add
    (2, 130, 96, 200, torch.bfloat16, False, True, 0),         # more rows than one tile
])
def test_skinny_linears_fwd_bwd(Z, R, K, N, wdtype, shared, silu, add_cols):
    """The few-row batched fp32 GEMM (forward, input gradient, weight gradient, shared-term gradient) against torch fp32."""
    torch.manual_seed(0)
    ws = [(torch.randn(N, K, device=DEV) / math.sqrt(K)).to(wdtype).requires_grad_(True) for _ in range(Z)]
    a = torch.randn(*((R, K) if shared else (Z, R, K)), device=DEV).requires_grad_(True)
    add = torch.randn(R, add_cols, device=DEV).requires_grad_(True) if add_cols else None
    before = native.launches()
    out = F_ops.skinny_linears(a, ws, silu=silu, add=add)
    assert native.launches() == before + 1, "the skinny GEMM kernel did not serve the call"
    dout = torch.randn_like(out)
    out.backward(dout)
    ar = a.detach().clone().requires_grad_(True)
    wr = [w.detach().float().requires_grad_(True) for w in ws]
    addr = add.detach().clone().requires_grad_(True) if add is not None else None
    h = torch.nn.functional.silu(ar) if silu else ar
    outs = []
    for z in range(Z):
        o = (h if shared else h[z]) @ wr[z].t()
        if addr is not None:
            o = torch.cat([o[:, :add_cols] + addr, o[:, add_cols:]], 1)
        outs.append(o)
    want = torch.stack(outs)
    want.backward(dout)
    assert out.dtype == torch.float32
    _close(out, want, 1e-4, 1e-4, "out")
    _close(a.grad, ar.grad, 1e-3, 1e-3, "da")
    gtol = 2e-2 if wdtype == torch.bfloat16 else 1e-4
    for z in range(Z):
        assert ws[z].grad.dtype == wdtype
        _close(ws[z].grad, wr[z].grad, gtol * math.sqrt(R), gtol, f"dW[{z}]")
    if add is not None:
        _close(add.grad, addr.grad, 1e-4, 1e-4, "dadd")
    again = F_ops.skinny_linears(a, ws, silu=silu, add=add)
    assert torch.equal(out, again), "the skinny GEMM is not bitwise repeatable"


def test_optimizer_kernels():
    torch.manual_seed(11)
    n = 100_003 * 8
    g16 = torch.randn(n, device=DEV).bfloat16()
    g16[5] = float("nan")
    g16[77] = float("inf")
    g32 = torch.empty(n, device=DEV)
    sumsq = torch.zeros(1, device=DEV)
    _ops().grad_cast_norm(g16, g32, sumsq, 0.5)
    want = torch.nan_to_num(g16.float() * 0.5, nan=0.0, posinf=0.0, neginf=0.0)
    _close(g32, want, 1e-6, 1e-6, "g32")
    assert abs(sumsq.item() - want.pow(2).sum().item()) / want.pow(2).sum().item() < 1e-4
    master = torch.randn(n, device=DEV)
    m = torch.zeros(n, device=DEV)
    v = torch.zeros(n, device=DEV)
    ema = master.clone()
    out16 = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    mr, mm, vv = master.clone(), m.clone(), v.clone()
    clip = torch.tensor([0.7], device=DEV)
    for step in (1, 2):
        _ops().adamw_ema_shard(master, g32, m, v, ema, out16, clip, 1e-2, 0.9, 0.99, 1e-8, 0.1, step, 0.5)
        ref.adamw_step(mr, g32 * 0.7, mm, vv, lr=1e-2, beta1=0.9, beta2=0.99, eps=1e-8, weight_decay=0.1, step=step)
    _close(master, mr, 1e-5, 1e-4, "master")
    _close(out16, mr, 1e-2, 1e-2, "bf16 params")


def test_network_jvp_uses_attention_jvp_kernel(monkeypatch):
    """Forward-mode through the DiT on the GPU: attention goes through the JVP kernel; everything else through torch ops.
    Compared with the same forward-mode pass that uses the explicit-softmax reference attention."""
    from cosmos_predict25_b200.models.distill import network_jvp
    from cosmos_predict25_b200.models.dit import CosmosDiT, dit_mini
    from cosmos_predict25_b200.ops import functional as F_ops
    torch.manual_seed(0)
    net = CosmosDiT(dit_mini(crossattn_proj_in_channels=256)).to(DEV)
    net.init_weights()
    for blk in net.blocks:
        for m in (blk.adaln_modulation_self_attn, blk.adaln_modulation_cross_attn, blk.adaln_modulation_mlp):
            torch.nn.init.normal_(m[-1].weight, std=0.05)
    torch.nn.init.normal_(net.final_layer.linear.weight, std=0.05)
    net = net.bfloat16()
    x = torch.randn(1, 16, 2, 16, 16, device=DEV).bfloat16()
    t = torch.full((1, 1), 400.0, device=DEV)
    tx, tt = torch.randn_like(x), torch.full_like(t, 1000.0)
    kw = dict(crossattn_emb=torch.randn(1, 16, 256, device=DEV).bfloat16(), fps=torch.tensor([16.0], device=DEV),
              padding_mask=torch.zeros(1, 1, 16, 16, device=DEV))
    before = native.launches()
    F1, dF1 = network_jvp(net, x, t, tx, tt, **kw)
    assert native.launches() - before >= 2 * len(net.blocks) * 2        # forward + tangent kernels for self- and cross-attention
    _no_kernel_error()
    monkeypatch.setattr(F_ops, "native_attention_supported", lambda q, k: False)
    F2, dF2 = network_jvp(net, x, t, tx, tt, **kw)
    _close(F1, F2, 5e-2, 5e-2, "F")
    _close(dF1, dF2, 8e-2, 8e-2, "dF")
    assert dF2.float().abs().max() > 1e-2


@pytest.mark.parametrize("D,L,T", [(256, 12, 3), (2048, 40, 2), (5120, 7, 2)])
def test_ln_modulate_tangent_kernel(D, L, T):
    """Value and directional derivative of LayerNorm-modulate in one pass against torch.func.jvp of the fp32 definition."""
    torch.manual_seed(0)
    B = 2
    x, tx = torch.randn(B, T, L, D, device=DEV).bfloat16(), torch.randn(B, T, L, D, device=DEV).bfloat16()
    sh, sc, tsh, tsc = (0.3 * torch.randn(B, T, D, device=DEV) for _ in range(4))
    y, ty = _ops().ln_modulate_jvp(x.view(-1, D), tx.view(-1, D), sh.view(-1, D), sc.view(-1, D), tsh.view(-1, D), tsc.view(-1, D), L, 1e-6)
    assert ty.data_ptr() == y.data_ptr() + y.numel() * 2, "value and tangent must be adjacent for the stacked GEMM"
    yr, tyr = torch.func.jvp(lambda a, b, c: ref.ln_modulate(a, b, c), (x.float(), sh, sc), (tx.float(), tsh, tsc))
    _close(y.view(B, T, L, D), yr, 2e-2, 2e-2, "y")
    _close(ty.view(B, T, L, D), tyr, 3e-2, 3e-2, "ty")
    y0, ty0 = _ops().ln_modulate_jvp(x.view(-1, D), tx.view(-1, D), sh.view(-1, D), sc.view(-1, D), None, None, L, 1e-6)
    _, tyr0 = torch.func.jvp(lambda a: ref.ln_modulate(a, sh, sc), (x.float(),), (tx.float(),))
    _close(ty0.view(B, T, L, D), tyr0, 3e-2, 3e-2, "ty without modulation tangents")
    _no_kernel_error()


@pytest.mark.parametrize("HD,rope", [(128, True), (128, False), (64, True)])
def test_rmsnorm_rope_tangent_kernel(HD, rope):
    torch.manual_seed(0)
    B, S, H = 2, 37, 3
    x, tx = torch.randn(B, S, H, HD, device=DEV).bfloat16(), torch.randn(B, S, H, HD, device=DEV).bfloat16()
    w = 1 + 0.1 * torch.randn(HD, device=DEV)
    half = torch.randn(S, HD // 2, device=DEV)
    table = F_ops.RopeTable(torch.cat([half, half], -1)) if rope else None
    cos, sin = table.cos_sin() if rope else (None, None)
    y, ty = _ops().rmsnorm_rope_jvp(x, tx, w, cos, sin, 1e-6)
    yr, tyr = torch.func.jvp(lambda a: ref.rmsnorm_rope(a, w, table.angles if rope else None, 1e-6), (x.float(),), (tx.float(),))
    _close(y, yr, 2e-2, 2e-2, "y")
    _close(ty, tyr, 3e-2, 3e-2, "ty")
    _no_kernel_error()


def test_network_jvp_runs_on_native_kernels(monkeypatch):
    """Forward-mode through the DiT with every block op on this package's kernels (tangent kernels, GEMMs on stacked value /
    tangent rows, JVP attention, few-row GEMM) against the same pass on torch ops (library GEMMs, eager element-wise)."""
    from cosmos_predict25_b200.models.distill import network_jvp
    from cosmos_predict25_b200.models.dit import CosmosDiT, dit_mini
    torch.manual_seed(0)
    net = CosmosDiT(dit_mini(crossattn_proj_in_channels=256)).to(DEV)
    net.init_weights()
    for blk in net.blocks:
        for m in blk.adaln_mlps():
            torch.nn.init.normal_(m[-1].weight, std=0.05)
    torch.nn.init.normal_(net.final_layer.linear.weight, std=0.05)
    net = net.bfloat16()
    x = torch.randn(1, 16, 2, 16, 16, device=DEV).bfloat16()
    t = torch.full((1, 1), 400.0, device=DEV)
    tx, tt = torch.randn_like(x), torch.full_like(t, 1000.0)
    kw = dict(crossattn_emb=torch.randn(1, 16, 256, device=DEV).bfloat16(), fps=torch.tensor([16.0], device=DEV),
              padding_mask=torch.zeros(1, 1, 16, 16, device=DEV))
    before = native.launches()
    F1, dF1 = network_jvp(net, x, t, tx, tt, **kw)
    per_block = 3 + 4 + 2 + 2 + 3 + 2          # LN tangent, GEMMs (stacked q/k/v + out), norm tangent, attention, ... (lower bound)
    assert native.launches() - before >= len(net.blocks) * per_block, native.launches() - before
    _no_kernel_error()
    monkeypatch.setattr(F_ops.settings, "gemm", "cublas")        # switches the forward-mode fast paths off
    mid = native.launches()
    F2, dF2 = network_jvp(net, x, t, tx, tt, **kw)
    assert native.launches() - mid < (native.launches() - before) // 2
    _close(F1, F2, 5e-2, 5e-2, "F")
    _close(dF1, dF2, 1e-1, 1e-1, "dF")
    assert dF2.float().abs().max() > 1e-2


def test_linear_gate_residual_training_path():
    """One GEMM with the gated residual in its epilogue and the product as second output: forward and all four gradients against
    the fp32 composition; the unfused pair (GEMM + gated-residual kernel) must give the same result."""
    torch.manual_seed(8)
    B, T, L, D, K = 1, 3, 88, 512, 256
    h = torch.randn(B, T * L, K, device=DEV).bfloat16().requires_grad_(True)
    w = (torch.randn(D, K, device=DEV) / math.sqrt(K)).bfloat16().requires_grad_(True)
    resid = torch.randn(B, T, L, D, device=DEV).bfloat16().requires_grad_(True)
    gate = torch.randn(B, T, D, device=DEV).requires_grad_(True)
    before = native.launches()
    out = F_ops.linear_gate_residual(h, w, resid, gate)
    assert native.launches() == before + 1, "the fused two-output GEMM did not serve the training path"
    do = torch.randn_like(out)
    got = torch.autograd.grad(out, (h, w, resid, gate), do)
    hr, wr, rr, gr = (t.detach().float().requires_grad_(True) for t in (h, w, resid, gate))
    want_out = rr + gr.unsqueeze(2) * (hr @ wr.t()).view(B, T, L, D)
    want = torch.autograd.grad(want_out, (hr, wr, rr, gr), do.float())
    _close(out, want_out, 3e-2, 2e-2, "out")
    for name, a, b in zip(("dh", "dw", "dresid", "dgate"), got, want):
        _close(a, b, 3e-2 * b.abs().max().item() + 1e-3, 3e-2, name)
    _no_kernel_error()


@pytest.mark.gpu
def test_sampler_state_update_and_frame_replacement_kernels():
    """One-pass kernels of the sampling loop against their torch definitions: linear combination of up to 6 fp32 tensors (ragged
    tail included) and the replacement of conditioning frames (both forms, fp32 and bf16 output)."""
    from cosmos_predict25_b200.ops import functional as F, ref
    torch.manual_seed(0)
    for n_ops, shape in ((1, (1027,)), (2, (2, 16, 3, 10, 12)), (4, (1, 16, 24, 88, 160)), (6, (3, 5, 7))):
        xs = [torch.randn(shape, device="cuda") for _ in range(n_ops)]
        cs = [0.37 * (k + 1) * (-1) ** k for k in range(n_ops)]
        out = F.lincomb(xs, cs)
        want = sum(c * x.double() for c, x in zip(cs, xs))
        assert out.dtype == torch.float32 and (out.double() - want).abs().max().item() < 1e-5
    B, C, T, H, W = 2, 16, 6, 10, 12
    x, gt, noise = (torch.randn(B, C, T, H, W, device="cuda") for _ in range(3))
    mask = torch.zeros(B, 1, T, H, W, device="cuda")
    mask[:, :, :2] = 1
    flag = torch.tensor([1.0, 0.0], device="cuda").view(B, 1, 1, 1, 1)
    before = F.native.launches()
    a = F.frame_blend(x, gt, None, mask, flag)
    assert torch.equal(a, ref.frame_blend(x, gt, None, mask, flag))
    a16 = F.frame_blend(x, gt, None, mask, flag, out_dtype=torch.bfloat16)
    assert a16.dtype == torch.bfloat16 and torch.equal(a16, ref.frame_blend(x, gt, None, mask, flag).bfloat16())
    b = F.frame_blend(x, gt, noise, mask)
    assert torch.equal(b, ref.frame_blend(x, gt, noise, mask))
    soft = torch.rand(B, 1, T, H, W, device="cuda")                # a fractional mask: fused multiply-add rounding only
    assert (F.frame_blend(x, gt, noise, soft) - ref.frame_blend(x, gt, noise, soft)).abs().max().item() < 1e-5
    assert F.native.launches() >= before + 4, "the sampler kernels did not run"


@pytest.mark.gpu
def test_unipc_on_the_state_update_kernel_matches_the_host_arithmetic():
    from cosmos_predict25_b200.models.schedulers import FlowUniPCSolver
    torch.manual_seed(1)
    x_dev = torch.randn(1, 16, 4, 8, 12, device="cuda")
    x_cpu = x_dev.cpu()
    s_dev, s_cpu = FlowUniPCSolver(1000), FlowUniPCSolver(1000)
    for s in (s_dev, s_cpu):
        s.set_timesteps(6, device="cpu", shift=5.0)
    for t in s_dev.timesteps.tolist():
        v = torch.randn_like(x_cpu)
        x_cpu = s_cpu.step(v, t, x_cpu)
        x_dev = s_dev.step(v.cuda(), t, x_dev)
    assert (x_dev.cpu() - x_cpu).abs().max().item() < 1e-4 * x_cpu.abs().max().item()
