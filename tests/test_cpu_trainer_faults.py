"""Host-side failure tests of the training loop: a hung step trips the watchdog, a failing dataloader surfaces, and no alarm
is left armed afterwards."""

import signal
import time

import pytest
import torch

from cosmos_predict25_b200.models.dit import dit_tiny
from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
from cosmos_predict25_b200.trainer.callbacks import Callback
from cosmos_predict25_b200.trainer.optim import OptimizerConfig
from cosmos_predict25_b200.trainer.trainer import Trainer, TrainerConfig


def _batches(n, fail_at=None):
    g = torch.Generator().manual_seed(0)
    for i in range(n):
        if fail_at is not None and i == fail_at:
            raise OSError("storage backend went away")
        yield {"latents": torch.randn(1, 16, 4, 16, 16, generator=g), "t5_text_embeddings": torch.randn(1, 32, 256, generator=g),
               "fps": torch.tensor([16.0]), "padding_mask": torch.zeros(1, 1, 16, 16)}


def _trainer(tmp_path, callbacks=None, **kw):
    torch.manual_seed(0)
    model = Video2WorldModelRectifiedFlow(Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4), device=torch.device("cpu"))
    return Trainer(TrainerConfig(output_dir=str(tmp_path), logging_iter=1, **kw), model, OptimizerConfig(lr=1e-3), callbacks=callbacks)


class _Stall(Callback):
    def __init__(self, at, seconds):
        self.at, self.seconds = at, seconds

    def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0):
        if iteration == self.at:
            time.sleep(self.seconds)      # a rank that stops making progress (hung collective, dead storage, ...)


def test_watchdog_raises_on_a_hung_step_and_disarms(tmp_path):
    t = _trainer(tmp_path, callbacks=[_Stall(at=2, seconds=5.0)], max_iter=5, timeout_period=1)
    t0 = time.time()
    with pytest.raises(TimeoutError):
        t.train(list(_batches(5)))
    assert time.time() - t0 < 4.5 and t.iteration == 2
    assert signal.alarm(0) == 0           # nothing left armed


def test_dataloader_failure_surfaces_and_disarms(tmp_path):
    t = _trainer(tmp_path, max_iter=5, timeout_period=30)
    with pytest.raises(OSError, match="went away"):
        t.train(_batches(5, fail_at=2))
    assert t.iteration == 2 and signal.alarm(0) == 0


def test_loop_without_faults_runs_to_max_iter(tmp_path):
    t = _trainer(tmp_path, max_iter=3, timeout_period=30)
    t.train(list(_batches(2)))            # the loader is shorter than max_iter: it is restarted
    assert t.iteration == 3 and signal.alarm(0) == 0


def test_wandb_run_id_survives_a_restart(tmp_path, monkeypatch):
    import sys
    import types

    from cosmos_predict25_b200.trainer.callbacks import WandbCallback
    calls = []
    fake = types.ModuleType("wandb")

    class _Run:
        def log(self, rec, step=None):
            calls.append(("log", step))

        def finish(self):
            calls.append(("finish",))

    def init(**kw):
        calls.append(("init", kw["id"], kw["resume"]))
        return _Run()

    fake.init = init
    monkeypatch.setitem(sys.modules, "wandb", fake)
    ids = []
    for _ in range(2):                                   # the second trainer stands for the restarted job
        cb = WandbCallback(logging_iter=1, mode="online")
        t = _trainer(tmp_path, callbacks=[cb], max_iter=1)
        t.train(list(_batches(1)))
        ids.append([c for c in calls if c[0] == "init"][-1][1])
    assert ids[0] == ids[1] and len(ids[0]) == 8
    assert (tmp_path / "checkpoints" / "wandb_id.txt").read_text().strip() == ids[0]
    assert ("log", 1) in calls and ("finish",) in calls and (tmp_path / "metrics.jsonl").exists()


class _RecordingCheckpointer:
    callbacks = None

    def __init__(self):
        self.saved = []

    def load(self, *a, **k):
        return 0

    def save(self, model, optimizer, scheduler, iteration, trainer=None):
        self.saved.append(iteration)

    def finalize(self):
        pass


def test_kernel_error_word_stops_the_run_before_a_checkpoint(tmp_path):
    """A bounded device wait that gave up is reported through the engine's health check (here a fake of the error word that
    turns non-zero after step 2): the trainer raises at the next check and writes no checkpoint after the failure."""
    ck = _RecordingCheckpointer()
    torch.manual_seed(0)
    model = Video2WorldModelRectifiedFlow(Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4), device=torch.device("cpu"))
    t = Trainer(TrainerConfig(output_dir=str(tmp_path), logging_iter=0, max_iter=6, save_iter=2), model, OptimizerConfig(lr=1e-3),
                checkpointer=ck)
    assert ck.callbacks is t.callbacks            # checkpoint callbacks reach the trainer's callback bus
    state = {"code": 0}

    def check_health():
        if state["code"]:
            raise RuntimeError(f"a peer-memory kernel gave up waiting (error code {state['code']})")

    model.engine.check_health = check_health

    class _Break(Callback):
        def on_training_step_end(self, model, data_batch, output_batch, loss, iteration=0):
            if iteration == 3:
                state["code"] = 101

    t.callbacks.append(_Break())
    with pytest.raises(RuntimeError, match="gave up waiting"):
        t.train(list(_batches(6)))
    assert ck.saved == [2]                        # iteration 4's save was refused


def test_arena_guard_words_catch_an_overrun():
    """Guard words behind every allocation of the peer arena: untouched guards pass, a write one byte past the end of a buffer
    (what a kernel with a wrong bound would do to this rank's or a peer's memory) is reported with the allocation it follows."""
    import pytest
    import torch
    from cosmos_predict25_b200.parallel.symm import CANARY_BYTES, BumpArena
    arena = BumpArena(torch.zeros(1 << 16, dtype=torch.uint8), [0, 1 << 20], canary=True)
    a = arena.alloc(100, torch.float32)
    b = arena.alloc(64, torch.bfloat16, zero=False)
    assert a.ptrs == [0, 1 << 20] and b.ptrs[0] == 512 + CANARY_BYTES and b.tensor.numel() == 64
    a.tensor.fill_(1.0)
    b.tensor.fill_(2.0)
    arena.check_canaries()
    arena.buf[512 + 3] = 0                          # first guard = bytes [512, 768): a's 400 bytes round up to 512
    with pytest.raises(RuntimeError, match=r"allocation #0 \(400 bytes of torch.float32, guard at offset 512\).*guard byte 3"):
        arena.check_canaries()
    plain = BumpArena(torch.zeros(1024, dtype=torch.uint8), [0])
    assert plain.alloc(64, torch.float32).tensor.numel() == 64 and plain.offset == 256
    plain.check_canaries()
    with pytest.raises(MemoryError):
        plain.alloc(1024, torch.float32)


def test_sigma_loss_analysis_on_the_noise_level_model(tmp_path):
    """One process: the EDM-era model's training output feeds the per-frame analysis; statistics match a direct computation; the
    placeholder callbacks accept the real ones' arguments and do nothing."""
    import json
    import types
    from cosmos_predict25_b200.models import edm
    from cosmos_predict25_b200.models.dit import NET_PRESETS
    from cosmos_predict25_b200.trainer.analysis_callbacks import (DummyFrameLossLog, DummySigmaLossAnalysisPerFrame,
                                                                  SigmaLossAnalysisPerFrame, normal_quantile_bins)
    torch.manual_seed(0)
    m = edm.Video2WorldModel(edm.EDMConfig(net=NET_PRESETS["tiny"](), precision="float32"), device=torch.device("cpu"))
    net = NET_PRESETS["tiny"]()
    d = net.crossattn_proj_in_channels if net.use_crossattn_projection else net.crossattn_emb_channels
    batch = {"latents": torch.randn(2, 16, 3, 8, 8), "t5_text_embeddings": torch.randn(2, 8, d), "fps": torch.full((2,), 16.0),
             "padding_mask": torch.zeros(2, 1, 8, 8)}
    cb = SigmaLossAnalysisPerFrame()
    cb.config = types.SimpleNamespace(trainer=types.SimpleNamespace(logging_iter=1), output_dir=str(tmp_path))
    out, loss = m.training_step(batch, 1)
    assert out["edm_loss_per_frame"].shape == (2, 3) and out["weights_per_sigma"].shape == (2, 1)
    cb.on_training_step_end(m, batch, out, loss, 1)
    rec = json.loads(open(tmp_path / "sigma_loss_analysis.jsonl").read())
    lf = out["edm_loss_per_frame"].to(torch.bfloat16).float()
    assert rec["sigma_loss_video/total_samples"] == 2
    assert abs(rec["sigma_loss_video/frame_1/loss_mean"] - lf[:, 1].mean().item()) < 1e-6
    assert abs(rec["sigma_loss_video/frame_2/sigma_log_mean"] - out["sigma"].to(torch.bfloat16).float().log().mean().item()) < 1e-6
    edges = normal_quantile_bins()
    assert len(edges) == 11 and bool((edges[1:] > edges[:-1]).all()) and abs(edges[5].item() - 1.0) < 1e-6
    for dummy in (DummyFrameLossLog(2, 4, True), DummySigmaLossAnalysisPerFrame(2, 4, True)):
        assert dummy.on_training_step_end(m, batch, out, loss, 1) is None
