"""Public API, config composition, inference pipeline, checkpointing and guardrails on CPU with the tiny network."""

import json
import os

import numpy as np
import pytest
import torch

from cosmos_predict25_b200.config import InferenceArguments, ModelKey, MODEL_CHECKPOINTS, SetupArguments
from cosmos_predict25_b200.configs import video2world as v2w_cfg
from cosmos_predict25_b200.guardrail import presets
from cosmos_predict25_b200.guardrail.blocklist import Blocklist
from cosmos_predict25_b200.utils.config import ConfigStore, override
from cosmos_predict25_b200.utils.lazy_config import L, LazyConfig, instantiate


@pytest.fixture(autouse=True)
def _grad_on():
    """``Inference`` switches autograd off process-wide (as the reference does); give every test a clean state."""
    torch.set_grad_enabled(True)
    yield
    torch.set_grad_enabled(True)


def test_model_key_names_and_registry():
    names = {k.name for k in MODEL_CHECKPOINTS}
    assert {"2B/pre-trained", "2B/post-trained", "14B/pre-trained", "2B/auto/multiview", "2B/robot/multiview"} <= names
    assert ModelKey().name == "2B/post-trained"
    s = SetupArguments(output_dir="/tmp/x")
    assert s.experiment == MODEL_CHECKPOINTS[ModelKey()].experiment and s.context_parallel_size == 1 and s.enable_guardrails


def test_inference_arguments_from_file(tmp_path):
    (tmp_path / "p.txt").write_text("a robot pours water\n")
    (tmp_path / "in.jpg").write_bytes(b"x")
    (tmp_path / "a.json").write_text(json.dumps({"inference_type": "image2world",
                                                 "samples": {"s0": {"prompt_path": "p.txt", "input_path": "in.jpg"}}}))
    a = InferenceArguments.from_file(tmp_path / "a.json")
    assert a.samples["s0"].prompt == "a robot pours water" and a.num_input_frames == 1 and a.guidance == 7 and a.seed == 1
    with pytest.raises(Exception):
        InferenceArguments(inference_type="video2world", samples={"s": {"prompt": "x"}})
    assert InferenceArguments(inference_type="text2world", samples={"s": {"prompt": "x"}}).num_input_frames == 0


def test_lazy_call_and_overrides():
    node = L(torch.nn.Linear)(in_features=3, out_features=L(int)())
    node["out_features"] = 5
    lin = instantiate(node)
    assert isinstance(lin, torch.nn.Linear) and lin.out_features == 5 and lin.bias is not None
    c = override(v2w_cfg.make_config(), ["--", "experiment=tiny_video2world_cpu", "trainer.max_iter=7", "+job.tag=abc", "~dataloader_val",
                                         "optimizer.lr=0.5", "net=mini_net"])
    assert c["trainer"]["max_iter"] == 7 and c["job"]["tag"] == "abc" and "dataloader_val" not in c
    assert c["optimizer"]["lr"] == 0.5 and c["model"]["config"]["net"]["model_channels"] == 1024
    with pytest.raises(KeyError):
        override(v2w_cfg.make_config(), ["trainer.no_such_key=1"])
    y = LazyConfig.to_yaml(c)
    assert "_target_: cosmos_predict25_b200.models.rectified_flow.Video2WorldModelRectifiedFlow" in y
    c.freeze()
    with pytest.raises(AttributeError):
        c["job"] = {}
    assert "predict2_video2world_training_2b_cosmos_nemo_assets" in ConfigStore.instance().names("experiment")


def test_pipeline_generates_and_saves_video(tmp_path):
    from cosmos_predict25_b200.inference import Inference
    from cosmos_predict25_b200.pipeline.video2world import Video2WorldInference
    from PIL import Image
    torch.manual_seed(0)
    Image.fromarray((np.random.rand(40, 64, 3) * 255).astype(np.uint8)).save(tmp_path / "in.png")
    pipe = Video2WorldInference("tiny_video2world_cpu", None, device=torch.device("cpu"))
    vid = pipe.generate_vid2world("a test prompt", str(tmp_path / "in.png"), guidance=3, num_latent_conditional_frames=1,
                                  resolution="32,32", seed=3, num_steps=3)
    assert vid.shape == (1, 3, 13, 32, 32) and vid.abs().max() <= 1.0
    setup = SetupArguments(output_dir=tmp_path / "out", experiment="tiny_video2world_cpu", checkpoint_path="none",
                           disable_guardrails=False)
    inf = Inference(setup, pipe=pipe)
    args = InferenceArguments(inference_type="text2world", samples={"clip": {"prompt": "waves on a beach"}}, resolution="32,32")
    paths = inf.generate(args, tmp_path / "out")
    assert os.path.exists(paths[0]) and paths[0].endswith(".mp4") and os.path.getsize(paths[0]) > 0


def test_dcp_checkpoint_roundtrip_and_resume(tmp_path):
    from cosmos_predict25_b200.checkpoint.dcp import DistributedCheckpointer, convert_distcp_to_pt
    from cosmos_predict25_b200.models.dit import dit_tiny
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    batch = {"latents": torch.randn(1, 16, 4, 16, 16), "t5_text_embeddings": torch.randn(1, 32, 256), "fps": torch.tensor([16.0]),
             "padding_mask": torch.zeros(1, 1, 16, 16)}

    def make():
        m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"))
        o, s = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="lambdalinear", warm_up_steps=(10,),
                                                                                     cycle_lengths=(100,), f_start=(0.1,), f_max=(1.0,), f_min=(0.5,)))
        return m, o, s

    m, o, s = make()
    for it in range(2):
        _, loss = m.training_step(dict(batch), it)
        loss.backward()
        o.ema_beta = m.ema_beta(it + 1)
        o.step()
        s.step()
    ck = DistributedCheckpointer({"save_iter": 1}, str(tmp_path))
    ck.save(m, o, s, iteration=2)
    assert (tmp_path / "checkpoints" / "latest_checkpoint.txt").read_text().strip() == "iter_000000002"
    for key in ("model", "optim", "scheduler", "trainer"):
        assert (tmp_path / "checkpoints" / "iter_000000002" / key / ".metadata").exists()
    m2, o2, s2 = make()
    it = DistributedCheckpointer({}, str(tmp_path)).load(m2, o2, s2)
    assert it == 2 and o2.engine.step_count == 2 and s2.last_epoch == s.last_epoch
    for (n, a), (_, b) in zip(m.net.named_parameters(), m2.net.named_parameters()):
        assert torch.equal(a, b), n
    for ua, ub in zip(m.engine.units, m2.engine.units):
        assert torch.equal(ua.master, ub.master) and torch.equal(ua.exp_avg, ub.exp_avg) and torch.equal(ua.ema, ub.ema)
    # bit-exact continuation
    torch.manual_seed(5)
    _, l1 = m.training_step(dict(batch), 2)
    torch.manual_seed(5)
    _, l2 = m2.training_step(dict(batch), 2)
    assert torch.equal(l1, l2)
    # consolidated export: EMA weights renamed to net.*
    paths = convert_distcp_to_pt(str(tmp_path / "checkpoints" / "iter_000000002" / "model"), str(tmp_path / "export"))
    ema = torch.load(paths["ema_bf16"], weights_only=False)
    assert "net.blocks.0.self_attn.q_proj.weight" in ema and ema["net.final_layer.linear.weight"].dtype == torch.bfloat16
    # load_ema_to_reg through load_path on a fresh job dir
    m3, _, _ = make()
    DistributedCheckpointer({"load_path": str(tmp_path / "checkpoints"), "load_ema_to_reg": True}, str(tmp_path / "new")).load(m3)
    got = dict(m3.net.named_parameters())["blocks.0.self_attn.q_proj.weight"]
    assert torch.allclose(got, m.engine.full_state_dict("ema")["blocks.0.self_attn.q_proj.weight"])


def test_guardrails():
    b = Blocklist(terms=["forbidden thing", "badword"])
    assert b.is_safe("a calm lake at dawn")[0]
    assert not b.is_safe("show me the Forbidden, things!")[0]
    assert not b.is_safe("badwords everywhere")[0]
    r = presets.create_text_guardrail_runner(with_llm=False)
    assert presets.run_text_guardrail("a robot arm welding", r)
    vr = presets.create_video_guardrail_runner()
    frames = (np.random.rand(3, 32, 32, 3) * 255).astype(np.uint8)
    out = presets.run_video_guardrail(frames, vr)
    assert out is not None and out.shape == frames.shape


def test_folder_monitor_and_text2image(tmp_path):
    from cosmos_predict25_b200.pipeline.online import FolderMonitor, Text2ImageInference
    from cosmos_predict25_b200.pipeline.video2world import Video2WorldInference
    pipe = Video2WorldInference("tiny_video2world_cpu", None, device=torch.device("cpu"))
    prompts, results = tmp_path / "prompts", tmp_path / "results"
    mon = FolderMonitor(pipe, str(prompts), str(results), guidance=3.0, num_video_frames=13, resolution="32,32", seed=5, num_steps=2)
    (prompts / "a_cat.txt").write_text("a cat walking")
    (prompts / "empty.txt").write_text("   ")
    assert mon.run_once() == 2
    out = results / "a_cat"
    assert (out / "prompt.txt").read_text() == "a cat walking" and "Seed: 5" in (out / "generation_info.txt").read_text()
    assert mon.existing_video("a_cat") is not None and not (results / "empty").exists()
    assert mon.run_once() == 0                                     # nothing new
    mon.processed_files.clear()
    assert mon.process_prompt_file(prompts / "a_cat.txt") is None    # output exists -> skipped
    (prompts / "STOP").write_text("")
    mon.run()                                                        # returns at once
    img = Text2ImageInference("tiny_video2world_cpu", None, pipe=pipe).generate_image("a dog", resolution="32,32", num_steps=2, guidance=2.0)
    assert img.shape[0] == 1 and img.shape[2] == 1 and torch.isfinite(img).all()


def test_sparse_attention_experiments_resolve_and_build():
    """The sparse experiments: schedules have one entry per block of their network, the chosen 2B schedule resolves through the
    config system into the network's two sparse fields, and the tiny sparse experiment builds a model whose first block attends
    through the neighbourhood operator (second block dense) and still trains a step."""
    from cosmos_predict25_b200.configs import sparse
    for name, sched in sparse.SCHEDULES.items():
        assert len(sched) == (28 if name.startswith("2B") else 36) and set(sched) <= set(sparse.LAYER_KINDS) | {"-"}
    assert 0.5 < sparse.skipped_fraction("2B_comb02") < 0.9
    cfg = override(v2w_cfg.make_config(), ["--", f"experiment={sparse.SPARSE_2B}"])
    net = cfg["model"]["config"]["net"]
    assert net["n_dense_blocks"] == 0 and len(net["natten_parameters"]) == 28
    assert tuple(net["natten_parameters"][0]["dilation"]) == (1, 11, 5) and cfg["optimizer"]["weight_decay"] == 0.1
    cfg = override(v2w_cfg.make_config(), ["--", "experiment=tiny_video2world_sparse_cpu"])
    model = instantiate(cfg["model"])
    assert model.net.blocks[0].self_attn.sparse_op is not None and model.net.blocks[1].self_attn.sparse_op is None
    out = model.net(torch.randn(1, 16, 4, 16, 16), torch.full((1, 1), 500.0), crossattn_emb=torch.randn(1, 32, 256))
    assert out.shape == (1, 16, 4, 16, 16) and bool(out.isfinite().all())
