"""The reference's entry objects on this package's loop: whole-config trainer, user model class, lazy optimizer / scheduler
configs, the ``.pt`` checkpointer's calling convention and the global parallel-state accessors (CPU, one rank)."""
import os

import pytest
import torch
import torch.distributed as dist

from cosmos_predict25_b200.checkpoint.ddp import Checkpointer
from cosmos_predict25_b200.parallel import parallel_state
from cosmos_predict25_b200.trainer.callbacks import Callback
from cosmos_predict25_b200.trainer.model import ImaginaireModel
from cosmos_predict25_b200.trainer.trainer import ImaginaireTrainer
from cosmos_predict25_b200.utils.config import CheckpointConfig, Config, JobConfig, ObjectStoreConfig
from cosmos_predict25_b200.utils.lazy_config import L


class Regressor(ImaginaireModel):
    def __init__(self):
        super().__init__()
        self.fc = torch.nn.Linear(10, 5)

    def forward(self, x):
        return self.fc(x)

    def training_step(self, data_batch, iteration):
        pred = self(data_batch["x"])
        loss = torch.nn.functional.mse_loss(pred, data_batch["y"])
        return {"pred": pred}, loss


class Count(Callback):
    steps = saves = 0

    def on_training_step_end(self, model, data, output, loss, iteration=0):
        Count.steps += 1

    def on_save_checkpoint_start(self, model, iteration=0):
        Count.saves += 1


@pytest.fixture
def single_rank(tmp_path, monkeypatch):
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    for k, v in dict(RANK="0", WORLD_SIZE="1", LOCAL_RANK="0", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                     IMAGINAIRE_OUTPUT_ROOT=str(tmp_path)).items():
        monkeypatch.setenv(k, v)
    yield tmp_path
    if dist.is_initialized():
        dist.destroy_process_group()
    parallel_state.destroy_model_parallel()


def _config(max_iter):
    c = Config(model=L(Regressor)(), optimizer=L(torch.optim.SGD)(params=None, lr=0.05),
               scheduler=L(torch.optim.lr_scheduler.StepLR)(optimizer=None, step_size=2, gamma=0.5), dataloader_train=None, dataloader_val=None)
    c["job"] = JobConfig(project="p", group="g", name="toy")
    c["trainer"].update(max_iter=max_iter, logging_iter=1, callbacks=dict(count=L(Count)()))
    c["checkpoint"].update(save_iter=2)
    return c


def test_whole_config_trainer_runs_a_user_model_and_resumes(single_rank):
    torch.manual_seed(0)
    data = [{"x": torch.randn(8, 10), "y": torch.randn(8, 5)} for _ in range(3)]
    Count.steps = Count.saves = 0
    config = _config(4)
    trainer = ImaginaireTrainer(config)
    assert trainer.output_dir == os.path.join(str(single_rank), "p", "g", "toy") and dist.is_initialized()
    model = Regressor()
    w0 = model.fc.weight.detach().clone()
    trainer.train(model, data)
    assert Count.steps == 4 and Count.saves == 2 and not torch.equal(model.fc.weight, w0)
    ckpt_dir = os.path.join(trainer.output_dir, "checkpoints")
    assert open(os.path.join(ckpt_dir, "latest_checkpoint.txt")).read().strip() == "iter_000000004"
    assert isinstance(trainer.inner.optimizer, torch.optim.SGD) and trainer.inner.scheduler.get_last_lr() == [0.05 * 0.25]
    # a second run of the same job resumes at iteration 4 with the saved weights and goes on to 6
    trainer2 = ImaginaireTrainer(_config(6))
    model2 = Regressor()
    trainer2.train(model2, data)
    assert trainer2.inner.iteration == 6 and Count.steps == 6
    assert trainer2.inner.scheduler.get_last_lr() == [0.05 * 0.125]


def test_checkpointer_calling_convention_and_parallel_state(single_rank):
    trainer = ImaginaireTrainer(_config(1))
    parallel_state.initialize_model_parallel(context_parallel_size=1)
    assert parallel_state.is_initialized() and parallel_state.get_context_parallel_world_size() == 1
    assert parallel_state.get_data_parallel_rank(with_context_parallel=True) == 0 and parallel_state.get_model_parallel_group().size() == 1
    assert parallel_state.get_pipeline_model_parallel_world_size() == parallel_state.get_expert_model_parallel_world_size() == 1
    with pytest.raises(NotImplementedError):
        parallel_state.destroy_model_parallel()
        parallel_state.initialize_model_parallel(tensor_model_parallel_size=2)
    store = ObjectStoreConfig(enabled=False, bucket="b", credentials="c")
    cc = CheckpointConfig(save_to_object_store=store, load_from_object_store=store, strict_resume=True, load_path=None,
                          load_training_state=True, only_load_scheduler_state=False)
    job = JobConfig(project="p", group="g", name="convention")
    ck = Checkpointer(cc, job, trainer.callbacks)
    assert ck.checkpoint_dir_local == os.path.join(str(single_rank), "p", "g", "convention", "checkpoints")
    model = Regressor()
    opt = torch.optim.Adam(model.parameters(), lr=1e-2)
    sch = torch.optim.lr_scheduler.StepLR(opt, step_size=1, gamma=0.1)
    scaler = torch.amp.GradScaler("cpu", enabled=False)
    model(torch.randn(4, 10)).sum().backward()
    opt.step(), sch.step()
    ck.save(model, opt, sch, scaler, iteration=7)
    ck.finalize()
    model2 = Regressor()
    opt2 = torch.optim.Adam(model2.parameters(), lr=1e-2)
    sch2 = torch.optim.lr_scheduler.StepLR(opt2, step_size=1, gamma=0.1)
    assert Checkpointer(cc, job, trainer.callbacks).load(model2, opt2, sch2, scaler) == 7
    assert torch.equal(model2.fc.weight, model.fc.weight) and sch2.get_last_lr() == sch.get_last_lr()
    s1, s2 = opt.state_dict()["state"], opt2.state_dict()["state"]
    assert all(torch.equal(s1[k]["exp_avg"], s2[k]["exp_avg"]) for k in s1)


def test_model_config_from_named_default_objects():
    """The reference's spelling: a model config assembled from module-level default objects (lazy calls), for the rectified-flow
    and the noise-level Video2World models; the tiny network keeps this a CPU test."""
    from cosmos_predict25_b200.configs.defaults import (DummyJointImageVideoConfig, PowerEMAConfig, VideoPredictionConditioner, mini_net,
                                                        tiny_net)
    from cosmos_predict25_b200.models import edm
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    assert mini_net["model_channels"] == 1024 and mini_net["num_blocks"] == 2 and mini_net["num_heads"] == 8
    batch = {"video": torch.randint(0, 255, (1, 3, 5, 32, 32), dtype=torch.uint8), "t5_text_embeddings": torch.randn(1, 16, 256),
             "fps": torch.full((1,), 16.0), "padding_mask": torch.zeros(1, 1, 32, 32)}
    for cls, cfg_cls in ((Video2WorldModelRectifiedFlow, Video2WorldRFConfig), (edm.Video2WorldModel, edm.EDMConfig)):
        cfg = cfg_cls(tokenizer=DummyJointImageVideoConfig, conditioner=VideoPredictionConditioner, net=tiny_net, ema=PowerEMAConfig,
                      precision="float32", state_t=2)
        model = cls(cfg, device=torch.device("cpu"))
        model.on_train_start()
        assert type(model.tokenizer).__name__ == "DummyTokenizer" and model.config.ema.enabled and model.config.ema.rate == 0.1
        _, loss = model.training_step(dict(batch), 1)
        loss.backward()
        assert torch.isfinite(loss)


def test_runif_and_run_command():
    from cosmos_predict25_b200.utils.helper_test import RunIf, get_gpu_architecture, run_command
    ok = RunIf(min_torch="1.8", min_python="3.8", requires_package="torch")
    assert ok.name == "skipif" and ok.kwargs["condition"] is False
    no = RunIf(min_gpus=64, max_torch="1.0", requires_file="/no/such/file", requires_package=["no_such_package_xyz"], supported_arch="Z999")
    assert no.kwargs["condition"] is True
    for part in ("GPUs>=64", "torch<1.0", "requires file=/no/such/file", "no_such_package_xyz", "arch=Z999"):
        assert part in no.kwargs["reason"]
    assert get_gpu_architecture() in ("B200", "H100", "A100", "L40S", "Other")
    assert run_command("echo hello").stdout.strip() == "hello"
    assert run_command("exit 3", max_retry_counter=0, is_raise=False).returncode == 3
    with pytest.raises(RuntimeError, match="exit 3"):
        run_command("exit 3", max_retry_counter=0)
