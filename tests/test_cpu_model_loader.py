"""Model loader: experiment name -> model, consolidated .pt with net.* / net_ema.* keys, EMA-as-regular load."""

import torch

from cosmos_predict25_b200.utils import distributed as D
from cosmos_predict25_b200.utils.model_loader import load_model_from_checkpoint, load_model_state_dict_from_checkpoint


def test_load_model_from_experiment_and_consolidated_checkpoint(tmp_path):
    torch.manual_seed(0)
    model, config = load_model_from_checkpoint("tiny_video2world_cpu", None, device=torch.device("cpu"))
    assert config["dataloader_train"] is None and not model.training
    sd = {k: v.clone() for k, v in model.state_dict().items()}
    net_keys = [k for k in sd if k.startswith("net.")]
    assert net_keys, "the model state dict uses net.* keys"
    # a checkpoint whose EMA weights differ from the regular ones
    ck = dict(sd)
    for k in net_keys:
        if sd[k].is_floating_point():
            ck["net_ema." + k[len("net."):]] = sd[k] + 1.0
    path = tmp_path / "model.pt"
    torch.save({"model": ck}, path)
    probe = next(k for k in net_keys if sd[k].is_floating_point() and sd[k].numel() > 1)

    fresh, _ = load_model_from_checkpoint("tiny_video2world_cpu", str(path), device=torch.device("cpu"))
    assert torch.equal(fresh.state_dict()[probe], sd[probe])
    as_ema, _ = load_model_from_checkpoint("tiny_video2world_cpu", str(path), device=torch.device("cpu"), load_ema_to_reg=True)
    assert torch.allclose(as_ema.state_dict()[probe], sd[probe] + 1.0)

    # non-strict load tolerates a missing and an unexpected key
    partial = {k: v for k, v in ck.items() if k != probe}
    partial["net.not_a_real_key"] = torch.zeros(1)
    torch.save(partial, tmp_path / "partial.pt")
    load_model_state_dict_from_checkpoint(fresh, str(tmp_path / "partial.pt"), strict=False)


def test_single_process_distributed_helpers():
    assert D.get_rank() == 0 and D.get_world_size() == 1 and D.is_rank0()
    D.barrier()
    t = torch.arange(3.0)
    assert D.all_gather_tensor(t)[0] is t and D.dist_reduce_tensor(t) is t
    D.sync_model_states(torch.nn.Linear(2, 2))
    D.destroy()
