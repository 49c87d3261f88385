"""Wan2.2 VAE (CPU)."""
import torch
from einops import rearrange

from cosmos_predict25_b200.models import vae_wan22 as v22


def test_patchify_roundtrip_and_layout():
    x = torch.randn(2, 3, 5, 8, 12)
    p = v22.patchify(x, 2)
    assert torch.equal(p, rearrange(x, "b c f (h q) (w r) -> b (c r q) f h w", q=2, r=2))
    assert torch.equal(v22.unpatchify(p, 2), x)
    y = torch.randn(2, 3, 8, 12)
    assert torch.equal(v22.unpatchify(v22.patchify(y, 2), 2), y)


def test_shortcuts():
    x = torch.randn(1, 8, 3, 4, 4)
    d = v22.AvgDown3D(8, 16, factor_t=2, factor_s=2)(x)
    assert d.shape == (1, 16, 2, 2, 2)
    # the first output frame averages (zero pad, frame 0)
    xp = torch.nn.functional.pad(x, (0, 0, 0, 0, 1, 0))
    ref = rearrange(xp, "b c (t a) (h p) (w q) -> b (c a p q) t h w", a=2, p=2, q=2).view(1, 16, 4, 2, 2, 2).mean(2)
    assert torch.allclose(d, ref, atol=1e-6)
    u = v22.DupUp3D(16, 8, factor_t=2, factor_s=2)
    z = torch.randn(1, 16, 2, 2, 2)
    assert u(z).shape == (1, 8, 4, 4, 4) and u(z, first_chunk=True).shape == (1, 8, 3, 4, 4)


def test_vae22_shapes_causality_and_names():
    torch.manual_seed(0)
    vae = v22.Wan22VAE_(dim=8, dec_dim=8, z_dim=4).eval()
    x = torch.randn(1, 3, 9, 32, 32)
    with torch.no_grad():
        z = vae.encode(x, (0.0, 1.0))
        assert z.shape == (1, 4, 3, 2, 2)
        y = vae.decode(z, (0.0, 1.0))
        assert y.shape == x.shape
        # causal: the first latent frame depends only on the first pixel frame, the first pixel frame only on the first latent
        x2 = x.clone()
        x2[:, :, 1:] += 1.0
        assert torch.allclose(vae.encode(x2, (0.0, 1.0))[:, :, :1], z[:, :, :1], atol=1e-5)
        z2 = z.clone()
        z2[:, :, 1:] += 1.0
        assert torch.allclose(vae.decode(z2, (0.0, 1.0))[:, :, :1], y[:, :, :1], atol=1e-5)
    keys = set(vae.state_dict())
    for k in ("encoder.conv1.weight", "encoder.downsamples.0.downsamples.0.residual.2.weight", "encoder.downsamples.1.downsamples.2.time_conv.weight",
              "decoder.upsamples.0.upsamples.3.resample.1.weight", "decoder.head.2.bias", "conv1.weight", "conv2.weight"):
        assert k in keys, k
    assert vae.encoder.conv1.in_channels == 12 and vae.decoder.head[2].out_channels == 12


def test_vae22_interface():
    tok = v22.Wan2pt2VAEInterface(device="cpu", dtype=torch.float32, dim=8, dec_dim=8)
    assert tok.get_latent_num_frames(93) == 24 and tok.get_pixel_num_frames(24) == 93
    assert tok.spatial_compression_factor == 16 and tok.latent_ch == 48
    z = tok.encode(torch.rand(1, 3, 5, 32, 32) * 2 - 1)
    assert z.shape == (1, 48, 2, 2, 2) and tok.decode(z).shape == (1, 3, 5, 32, 32)
