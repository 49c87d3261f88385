"""Checkpointer of the vision-language training stack: full save / resume, per-part export at iteration 0 under Hugging Face names,
asynchronous saves through the writer process."""

import os

import torch

from cosmos_predict25_b200.checkpoint.vlm import VLMCheckpointer, from_hf_parts, to_hf_parts
from cosmos_predict25_b200.models.text_encoder import QwenConfig
from cosmos_predict25_b200.models.vlm_train import QwenForCausalLM


def _model(seed):
    torch.manual_seed(seed)
    return QwenForCausalLM(QwenConfig(vocab_size=97, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2))


def test_part_names_round_trip():
    sd = {"model.layers.0.mlp.up_proj.weight": torch.zeros(1), "lm_head.weight": torch.zeros(1), "visual.blocks.0.attn.qkv.weight": torch.zeros(1),
          "visual.merger.mlp.0.weight": torch.zeros(1), "language_model.norm.weight": torch.zeros(1)}
    parts = to_hf_parts(sd)
    assert set(parts["llm"]) == {"model.layers.0.mlp.up_proj.weight", "lm_head.weight", "model.norm.weight"}
    assert set(parts["vision_encoder"]) == {"visual.blocks.0.attn.qkv.weight"} and set(parts["mm_projector"]) == {"visual.merger.mlp.0.weight"}
    back = from_hf_parts(parts, list(sd))
    assert set(back) == set(sd)


def test_save_resume_and_part_export(tmp_path):
    m = _model(0)
    opt = {"llm": torch.optim.AdamW(m.parameters(), lr=1e-3)}
    sched = {"llm": torch.optim.lr_scheduler.LambdaLR(opt["llm"], lambda s: 1.0)}
    ids = torch.randint(0, 97, (2, 9))
    for _ in range(2):
        m(ids).float().pow(2).mean().backward()
        opt["llm"].step()
        sched["llm"].step()
        opt["llm"].zero_grad()
    ck = VLMCheckpointer(str(tmp_path))
    ck.save(m, opt, sched, iteration=0)
    root = tmp_path / "checkpoints" / "iter_000000000"
    assert (root / "llm" / ".metadata").exists() and not (root / "vision_encoder").exists()
    ck.save(m, opt, sched, iteration=2)
    assert ck.latest() == "iter_000000002" and not (tmp_path / "checkpoints" / "iter_000000002" / "llm").exists()
    # full resume: parameters, moments and the schedule position come back
    m2 = _model(1)
    opt2 = {"llm": torch.optim.AdamW(m2.parameters(), lr=1e-3)}
    sched2 = {"llm": torch.optim.lr_scheduler.LambdaLR(opt2["llm"], lambda s: 1.0)}
    assert VLMCheckpointer(str(tmp_path)).load(m2, opt2, sched2) == 2
    for (n, a), (_, b) in zip(m.state_dict().items(), m2.state_dict().items()):
        assert torch.equal(a, b), n
    s1, s2 = opt["llm"].state_dict()["state"], opt2["llm"].state_dict()["state"]
    assert s1.keys() == s2.keys() and all(torch.equal(s1[k]["exp_avg"], s2[k]["exp_avg"]) for k in s1)
    assert sched2["llm"].last_epoch == sched["llm"].last_epoch
    m(ids).float().pow(2).mean().backward()
    m2(ids).float().pow(2).mean().backward()
    opt["llm"].step()
    opt2["llm"].step()
    assert all(torch.equal(a, b) for a, b in zip(m.parameters(), m2.parameters()))
    # seeding another run from the exported language-model part
    m3 = _model(2)
    assert VLMCheckpointer(str(tmp_path)).load(m3, name="iter_000000000", parts_only=True) == 0
    m0 = _model(0)
    assert not torch.equal(m3.lm_head.weight, m0.lm_head.weight)       # iteration 0 was written after two steps of training


def test_asynchronous_save_through_the_writer_process(tmp_path):
    m = _model(0)
    ck = VLMCheckpointer(str(tmp_path), async_mode=True)
    ck.save(m, iteration=0)
    ck.close()
    assert ck.last_error is None and ck.latest() == "iter_000000000"
    m2 = _model(5)
    assert VLMCheckpointer(str(tmp_path)).load(m2) == 0
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
