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
    ck = DistributedCheckpointer({"dcp_async_mode_enabled": True, "dcp_async_writer": "thread"}, str(tmp_path))
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


def test_writer_process_saves_reports_failure_and_recovers(tmp_path):
    """The child-process writer: a save lands and resumes bit-exactly; a save that cannot be written (its directory name is taken
    by a regular file) is reported at ``finalize`` without raising and leaves the pointer alone; a writer that was killed is
    replaced on the next save."""
    seen = []

    class _Callbacks:
        def on_save_checkpoint_start(self, model, iteration): pass
        def on_save_checkpoint_end(self, model, iteration): pass
        def on_save_checkpoint_success(self, iteration, elapsed_time): seen.append(iteration)

    m, o, s = _make()
    ck = DistributedCheckpointer({"dcp_async_mode_enabled": True}, str(tmp_path), callbacks=_Callbacks())
    assert ck.async_writer == "process"
    ck.save(m, o, s, iteration=1)
    ck.finalize()
    latest = tmp_path / "checkpoints" / "latest_checkpoint.txt"
    assert latest.read_text().strip() == "iter_000000001" and seen == [1]
    first_pid = ck._writer._proc.pid
    m2, o2, s2 = _make()
    with torch.no_grad():
        for p in m2.net.parameters():
            p.add_(1.0)
    m2.engine.sync_masters_from_params() if hasattr(m2.engine, "sync_masters_from_params") else None
    assert DistributedCheckpointer({}, str(tmp_path)).load(m2, o2, s2) == 1
    for (n1, p1), (_, p2) in zip(m.net.named_parameters(), m2.net.named_parameters()):
        assert torch.equal(p1, p2), n1

    (tmp_path / "checkpoints" / "iter_000000002").write_text("a file where the checkpoint directory should go")
    ck.save(m, o, s, iteration=2)          # must not raise into the training loop
    ck.finalize()                          # reported (logged) and cleared here
    assert ck._bg_error is None and latest.read_text().strip() == "iter_000000001" and seen == [1]

    ck.save(m, o, s, iteration=3)          # a fresh writer process serves the next save
    ck.finalize()
    assert latest.read_text().strip() == "iter_000000003" and seen == [1, 3]
    assert ck._writer._proc.pid != first_pid

    ck._writer._proc.terminate()           # host-side failure: the writer dies between saves
    ck._writer._proc.join(5)
    ck.save(m, o, s, iteration=4)
    ck.close()
    assert latest.read_text().strip() == "iter_000000004" and seen == [1, 3, 4]
    assert ck._writer is None
