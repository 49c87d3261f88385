"""The channels-last implicit-GEMM convolution kernel against ``F.conv3d`` / ``F.conv2d`` in fp32, and the channels-last VAE
decoder built on it against the torch decoder it restates."""

import pytest
import torch
import torch.nn.functional as F

from cosmos_predict25_b200.ops import functional as F_ops
from cosmos_predict25_b200.ops import native

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(a, b, atol, rtol, name=""):
    a, b = a.float(), b.float()
    assert a.shape == b.shape, (a.shape, b.shape)
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    assert bad < 1e-4 and (err / tol).max().item() < 8, f"{name}: {bad * 100:.3f}% out of tolerance, max err {err.max().item():.4g}"


def _no_kernel_error():
    torch.cuda.synchronize()
    code = native.load().kernel_error(torch.cuda.current_device(), True)
    assert code == 0, f"a kernel reported bounded-wait error code {code}"


# (T, H, W, Cin, Cout): whole tiles; ragged frame (H, W not multiples of 8 / 16); 96 channels (a half-filled channel block);
# more output channels than one N tile; an N tile of 16 with 3 real channels (the decoder head)
@pytest.mark.parametrize("T,H,W,Cin,Cout", [(2, 16, 32, 64, 64), (3, 11, 20, 128, 192), (2, 24, 48, 96, 96), (1, 8, 16, 192, 384),
                                            (2, 9, 17, 96, 3), (2, 8, 16, 64, 768)])
def test_causal_conv3d_matches_torch(T, H, W, Cin, Cout):
    from cosmos_predict25_b200.models import vae_wan, vae_wan_cl
    torch.manual_seed(0)
    conv = vae_wan.CausalConv3d(Cin, Cout, 3, padding=1).to(DEV)
    conv.weight.data = conv.weight.data.bfloat16().float()
    x = torch.randn(1, Cin, T, H, W, device=DEV).bfloat16()
    cache = torch.randn(1, Cin, 2, H, W, device=DEV).bfloat16()
    want = conv(x.float(), cache.float())                                        # [1, Cout, T, H, W]
    cl = vae_wan_cl._conv3d(conv, DEV)
    xin = torch.cat([cache, x], 2)[0].permute(1, 2, 3, 0).contiguous()           # [T + 2, H, W, Cin]
    resid = torch.randn(T, H, W, Cout, device=DEV).bfloat16() if Cout % 8 == 0 else None
    got = cl(xin, T, resid=resid)
    _no_kernel_error()
    ref = want[0].permute(1, 2, 3, 0)
    if resid is not None:
        ref = ref + resid.float()
    _close(got, ref, 2e-2 * (27 * Cin) ** 0.5 / 8, 2e-2, "conv3d")


def test_upsample_phase_convolutions_match_nearest_then_conv():
    from cosmos_predict25_b200.models import vae_wan, vae_wan_cl
    torch.manual_seed(1)
    mod = vae_wan.Resample(128, "upsample2d").to(DEV)
    conv = mod.resample[1]
    conv.weight.data = conv.weight.data.bfloat16().float()
    T, H, W = 2, 12, 20
    x = torch.randn(T, H, W, 128, device=DEV).bfloat16()
    up = vae_wan_cl._UpsampleCL(mod, DEV)
    got = up(x, vae_wan_cl._Stream())
    _no_kernel_error()
    want = conv(F.interpolate(x.float().permute(0, 3, 1, 2), scale_factor=2.0, mode="nearest-exact")).permute(0, 2, 3, 1)
    _close(got, want, 6e-2, 3e-2, "upsample + conv2d")


def test_rmsnorm_silu_channels_last():
    torch.manual_seed(2)
    x = torch.randn(5, 7, 9, 96, device=DEV).bfloat16()
    g = (1 + 0.1 * torch.randn(96, device=DEV)).float()
    got = native.load().rmsnorm_silu_cl(x, g, True)
    want = F.silu(F.normalize(x.float(), dim=-1) * 96 ** 0.5 * g)
    _close(got, want, 2e-2, 2e-2, "rmsnorm+silu")


def test_channels_last_decoder_matches_torch_decoder():
    """Whole streaming decode (3 latent frames -> 9 pixel frames) on the kernel path against the torch modules in fp32."""
    from cosmos_predict25_b200.models.vae_wan import WanVAE_
    torch.manual_seed(3)
    vae = WanVAE_(dim=32, z_dim=16).eval().requires_grad_(False).to(DEV)
    for p in vae.parameters():
        p.data = p.data.bfloat16().float()
    z = torch.randn(1, 16, 3, 16, 32, device=DEV)
    F_ops.settings.conv = "cudnn"
    try:
        want = vae.decode(z, (0.0, 1.0))
    finally:
        F_ops.settings.conv = "native"
    vae16 = vae.to(torch.bfloat16)
    got = vae16.decode(z.bfloat16(), (0.0, 1.0))
    _no_kernel_error()
    assert got.shape == want.shape == (1, 3, 9, 128, 256)
    assert getattr(vae16, "_dec_cl", None) is not None, "the kernel decoder did not serve the bf16 decode"
    err = (got.float() - want).abs()
    scale = want.abs().mean().item()
    assert err.mean().item() < 0.03 * scale + 1e-3 and err.max().item() < 0.5 * want.abs().max().item() + 0.05, \
        f"mean err {err.mean().item():.4g} (signal {scale:.4g}), max err {err.max().item():.4g}"


def test_channels_last_encoder_matches_torch_encoder():
    """Whole streaming encode (1 + 4 + 4 pixel frames -> 3 latent frames) on the kernel path against the torch modules in fp32."""
    from cosmos_predict25_b200.models.vae_wan import WanVAE_
    torch.manual_seed(4)
    vae = WanVAE_(dim=32, z_dim=16).eval().requires_grad_(False).to(DEV)
    for p in vae.parameters():
        p.data = p.data.bfloat16().float()
    x = torch.randn(1, 3, 9, 128, 256, device=DEV).clamp(-1, 1)
    F_ops.settings.conv = "cudnn"
    try:
        want = vae.encode(x, (0.0, 1.0))
    finally:
        F_ops.settings.conv = "native"
    vae16 = vae.to(torch.bfloat16)
    before = native.launches()
    got = vae16.encode(x.bfloat16(), (0.0, 1.0))
    _no_kernel_error()
    assert got.shape == want.shape == (1, 16, 3, 16, 32)
    assert getattr(vae16, "_enc_cl", None) is not None and native.launches() - before > 30, "the kernel encoder did not serve the bf16 encode"
    err = (got.float() - want).abs()
    scale = want.abs().mean().item()
    assert err.mean().item() < 0.03 * scale + 1e-3 and err.max().item() < 0.5 * want.abs().max().item() + 0.05, \
        f"mean err {err.mean().item():.4g} (signal {scale:.4g}), max err {err.max().item():.4g}"
