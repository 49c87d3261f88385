"""Host-side failure tests of the distributed checkpointer: a damaged shard, a failed background save, a stale pointer."""

import os

import pytest
import torch

from cosmos_predict25_b200.checkpoint.dcp import DistributedCheckpointer
from cosmos_predict25_b200.models.dit import dit_tiny
from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig


def _make():
    torch.manual_seed(0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"))
    o, s = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="constant"))
    return m, o, s


def test_truncated_shard_is_an_error_not_silent_garbage(tmp_path):
    m, o, s = _make()
    ck = DistributedCheckpointer({}, str(tmp_path))
    ck.save(m, o, s, iteration=1)
    shard_dir = tmp_path / "checkpoints" / "iter_000000001" / "model"
    shards = [f for f in os.listdir(shard_dir) if f.endswith(".distcp")]
    assert shards
    p = shard_dir / shards[0]
    data = p.read_bytes()
    p.write_bytes(data[: len(data) // 3])
    m2, o2, s2 = _make()
    with pytest.raises(RuntimeError, match="damaged or incomplete"):
        DistributedCheckpointer({}, str(tmp_path)).load(m2, o2, s2)


def test_failed_background_save_keeps_the_previous_pointer(tmp_path, monkeypatch):
    m, o, s = _make()
    ck = DistributedCheckpointer({"dcp_async_mode_enabled": True}, str(tmp_path))
    ck.save(m, o, s, iteration=1)
    ck.finalize()
    latest = tmp_path / "checkpoints" / "latest_checkpoint.txt"
    assert latest.read_text().strip() == "iter_000000001"

    def broken_write(self, sds, name, group=None):
        raise OSError("no space left on device")

    monkeypatch.setattr(DistributedCheckpointer, "_write", broken_write)
    ck.save(m, o, s, iteration=2)          # must not raise into the training loop
    ck.finalize()                          # the failure is reported here (logged) and cleared
    assert ck._bg_error is None and latest.read_text().strip() == "iter_000000001"
    monkeypatch.undo()
    m2, o2, s2 = _make()
    assert DistributedCheckpointer({}, str(tmp_path)).load(m2, o2, s2) == 1     # resume from the last good checkpoint


def test_pointer_to_a_missing_checkpoint(tmp_path):
    os.makedirs(tmp_path / "checkpoints")
    (tmp_path / "checkpoints" / "latest_checkpoint.txt").write_text("iter_000000099\n")
    m, o, s = _make()
    with pytest.raises(FileNotFoundError):
        DistributedCheckpointer({}, str(tmp_path)).load(m, o, s)
    lenient = DistributedCheckpointer({"strict_resume": False}, str(tmp_path))
    assert lenient.load(m, o, s) == 0      # non-strict: missing parts are skipped with a warning
