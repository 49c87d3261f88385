"""Legacy .pt checkpointers: plain, model-parallel (per-rank files) and model-parallel with EMA."""

import os

import torch

from cosmos_predict25_b200.checkpoint.simple import (DummyCheckpointer, ModelParallelEmaPtCheckpointer, ModelParallelPtCheckpointer,
                                                     PtCheckpointer, broadcast_object)


def _setup():
    torch.manual_seed(0)
    net = torch.nn.Linear(4, 3)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-2)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: 1.0 / (1 + s))
    net(torch.randn(2, 4)).sum().backward()
    opt.step()
    sched.step()
    return net, opt, sched


def test_plain_roundtrip_and_latest_pointer(tmp_path):
    net, opt, sched = _setup()
    ck = PtCheckpointer({}, str(tmp_path))
    ck.save(net, opt, sched, 7)
    ck.finalize()
    assert (tmp_path / "checkpoints" / "latest_checkpoint.txt").read_text().strip() == "iter_000000007"
    net2, opt2, sched2 = _setup()
    with torch.no_grad():
        net2.weight.add_(1.0)
    it = PtCheckpointer({}, str(tmp_path)).load(net2, opt2, sched2)
    assert it == 7 and torch.equal(net2.weight, net.weight)
    assert DummyCheckpointer().load(net2) == 0 and broadcast_object({"a": 1}) == {"a": 1}


def test_model_parallel_files_per_rank(tmp_path):
    net, opt, sched = _setup()
    for r in (0, 1):
        ck = ModelParallelPtCheckpointer({}, str(tmp_path), mp_rank=lambda r=r: r)
        ck.save(net, opt, sched, 3)
        ck.finalize()
    files = sorted(os.listdir(tmp_path / "checkpoints"))
    assert "iter_000000003_model_mp_0.pt" in files and "iter_000000003_model_mp_1.pt" in files
    assert "iter_000000003_optim_mp_1.pt" in files and "iter_000000003_scheduler.pt" in files and "iter_000000003.pt" in files
    other = ModelParallelPtCheckpointer({}, str(tmp_path), dp_rank=lambda: 1)      # not the first replica: writes nothing
    other.save(net, opt, sched, 9)
    other.finalize()
    assert not any(f.startswith("iter_000000009") for f in os.listdir(tmp_path / "checkpoints"))
    net2, opt2, sched2 = _setup()
    with torch.no_grad():
        net2.bias.zero_()
    assert ModelParallelPtCheckpointer({}, str(tmp_path), mp_rank=lambda: 1).load(net2, opt2, sched2) == 3
    assert torch.equal(net2.bias, net.bias)


def test_model_parallel_ema_key(tmp_path):
    net, opt, sched = _setup()
    ema = {k: v.clone() * 0.5 for k, v in net.state_dict().items()}
    got = {}
    ck = ModelParallelEmaPtCheckpointer({}, str(tmp_path), get_ema=lambda m: ema, set_ema=lambda m, sd: got.update(sd))
    ck.save(net, opt, sched, 1)
    ck.finalize()
    raw = torch.load(tmp_path / "checkpoints" / "iter_000000001_model_mp_0.pt", weights_only=False)
    assert "ema" in raw and torch.equal(raw["ema"]["weight"], ema["weight"])
    net2, opt2, sched2 = _setup()
    assert ck.load(net2, opt2, sched2) == 1
    assert torch.equal(got["weight"], ema["weight"]) and torch.equal(net2.weight, net.weight)
