"""Forward CUDA-graph helper: pass-through on CPU, capture / replay equals eager on the GPU."""

import pytest
import torch

from cosmos_predict25_b200.utils import cuda_graphs as cg


def test_cpu_inputs_pass_through():
    lin = torch.nn.Linear(4, 4)
    same = cg.make_graphed_callables_forward(lin, (torch.randn(2, 4),))
    assert same is lin
    a, b = cg.make_graphed_callables_forward((lin, lin), ((torch.randn(2, 4),), (torch.randn(2, 4),)))
    assert a is lin and b is lin
    assert cg.is_graph_capturing() is False
    storage = {}
    blocks = torch.nn.ModuleList([torch.nn.Identity()])
    key = cg.create_cuda_graph(storage, blocks, torch.randn(1, 2, 3, 4), torch.randn(1, 2, 4), torch.randn(1, 5, 4))
    assert key == "1_2_3_4_1_2_4_1_5_4" and storage[key][0] is blocks[0]


@pytest.mark.gpu
def test_graph_replay_matches_eager():
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(64, 128), torch.nn.GELU(), torch.nn.Linear(128, 32)).to(dev)
    seen = []

    def fn(x, scale=1.0):
        seen.append(cg.is_graph_capturing())
        return {"y": net(x) * scale, "n": x.shape[0]}

    g = cg.make_graphed_callables_forward(fn, (torch.randn(8, 64, device=dev),), sample_kwargs={"scale": 2.0})
    assert isinstance(g, cg.GraphedForward) and all(seen)
    for _ in range(3):
        x = torch.randn(8, 64, device=dev)
        out = g(x, scale=2.0)
        with torch.no_grad():
            want = net(x) * 2.0
        assert out["n"] == 8 and torch.allclose(out["y"], want, atol=1e-5)
    assert not g.matches((torch.randn(4, 64, device=dev),), {"scale": 2.0})


@pytest.mark.gpu
def test_dit_blocks_replay_through_graphs():
    """The blocks of a DiT (tcgen05 GEMMs, attention, fused element-wise kernels) captured per block and replayed."""
    from cosmos_predict25_b200.models.dit import NET_PRESETS, CosmosDiT
    from cosmos_predict25_b200.ops import functional as F_ops
    from cosmos_predict25_b200.ops import native
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    cfg = NET_PRESETS["mini"]()
    net = CosmosDiT(cfg).to(dev).bfloat16().eval()
    net.init_weights()
    B, T, L, D = 1, 2, 128, cfg.model_channels
    x = torch.randn(B, T, L, D, device=dev).bfloat16()
    emb = torch.randn(B, T, D, device=dev).bfloat16()
    lora = torch.randn(B, T, 3 * D, device=dev).bfloat16() if cfg.use_adaln_lora else None
    ctx = torch.randn(B, 64, cfg.crossattn_emb_channels, device=dev).bfloat16()
    half = torch.rand(T * L, cfg.head_dim // 2, device=dev) * 10
    rope = F_ops.RopeTable(torch.cat([half, half], -1))
    storage = {}
    with torch.no_grad():
        key = cg.create_cuda_graph(storage, net.blocks, x, emb, ctx, rope, lora)
        assert cg.create_cuda_graph(storage, net.blocks, x, emb, ctx, rope, lora) == key and len(storage) == 1
        y_g, y_e = x, x
        for i, block in enumerate(net.blocks):
            y_g = storage[key][i](y_g, emb, ctx, rope, lora, None).clone()
            y_e = block(y_e, emb, ctx, rope, lora, None)
    assert native.load().kernel_error(0, True) == 0
    assert torch.isfinite(y_g.float()).all()
    assert (y_g.float() - y_e.float()).abs().max() <= 2e-2 * max(1.0, y_e.float().abs().max().item())
