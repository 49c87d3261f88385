"""Wan2.1-style causal VAE: shapes, streaming equivalence and tokenizer arithmetic (small widths, CPU)."""

import torch

from cosmos_predict25_b200.models.vae_wan import (CausalConv3d, DummyTokenizer, StreamState, Wan2pt1VAEInterface, WanVAE_)


def test_causal_conv_streaming_equals_one_shot():
    torch.manual_seed(0)
    conv = CausalConv3d(4, 6, 3, padding=1)
    x = torch.randn(1, 4, 7, 5, 5)
    full = conv(x)
    st = StreamState()
    parts = [conv.stream(x[:, :, :1], st), conv.stream(x[:, :, 1:5], st), conv.stream(x[:, :, 5:], st)]
    assert torch.allclose(torch.cat(parts, 2), full, atol=1e-5)
    # causality: output frame t does not depend on later frames
    x2 = x.clone()
    x2[:, :, 4:] += 1.0
    assert torch.allclose(conv(x2)[:, :, :4], full[:, :, :4], atol=1e-6)


def test_vae_shapes_and_frame_arithmetic():
    torch.manual_seed(0)
    vae = WanVAE_(dim=8, z_dim=16, temporal_window=4).eval()
    x = torch.rand(1, 3, 9, 32, 32) * 2 - 1
    with torch.no_grad():
        mu = vae.encode(x, (0.0, 1.0))
        assert mu.shape == (1, 16, 3, 4, 4)
        y = vae.decode(mu, (0.0, 1.0))
        assert y.shape == (1, 3, 9, 32, 32)
        # image: one frame in, one latent, one frame out
        mi = vae.encode(x[:, :, :1], (0.0, 1.0))
        assert mi.shape == (1, 16, 1, 4, 4) and vae.decode(mi, (0.0, 1.0)).shape == (1, 3, 1, 32, 32)
        # the first latent frame only depends on the first pixel frame (causal encoder)
        x2 = x.clone()
        x2[:, :, 1:] = 0
        assert torch.allclose(vae.encode(x2, (0.0, 1.0))[:, :, :1], mu[:, :, :1], atol=1e-5)


def test_decoder_cache_carries_over_between_calls():
    torch.manual_seed(1)
    vae = WanVAE_(dim=8, z_dim=16).eval()
    z = torch.randn(1, 16, 3, 4, 4)
    with torch.no_grad():
        full = vae.decode(z, (0.0, 1.0))
        a = vae.decode(z[:, :, :2], (0.0, 1.0), clear_decoder_cache=False)
        b = vae.decode(z[:, :, 2:], (0.0, 1.0), clear_decoder_cache=False)
        vae.clear_cache()
    assert torch.allclose(torch.cat([a, b], 2), full, atol=1e-5)


def test_parameter_names_follow_reference_checkpoint_layout():
    vae = WanVAE_(dim=8, z_dim=16)
    keys = set(vae.state_dict())
    for k in ["encoder.conv1.weight", "encoder.downsamples.0.residual.0.gamma", "encoder.downsamples.0.residual.2.weight",
              "encoder.downsamples.2.resample.1.weight", "encoder.middle.1.to_qkv.weight", "encoder.head.2.weight", "conv1.weight",
              "conv2.weight", "decoder.conv1.weight", "decoder.middle.0.residual.6.bias", "decoder.upsamples.3.time_conv.weight",
              "decoder.upsamples.4.shortcut.weight", "decoder.head.0.gamma", "decoder.head.2.weight"]:
        assert k in keys, k


def test_tokenizer_interface_and_dummy():
    tok = Wan2pt1VAEInterface(device="cpu", dtype=torch.float32, dim=8)
    assert tok.get_latent_num_frames(93) == 24 and tok.get_pixel_num_frames(24) == 93
    assert tok.spatial_compression_factor == 8 and tok.temporal_compression_factor == 4 and tok.latent_ch == 16
    x = torch.rand(1, 3, 5, 16, 16) * 2 - 1
    z = tok.encode(x)
    assert z.shape == (1, 16, 2, 2, 2) and tok.decode(z).shape == (1, 3, 5, 16, 16)
    d = DummyTokenizer()
    assert d.encode(torch.rand(2, 3, 9, 32, 32)).shape == (2, 16, 3, 4, 4)
    assert d.decode(torch.rand(2, 16, 3, 4, 4)).shape == (2, 3, 9, 32, 32)
