"""Operand validation of the extension's operators, exercised on the host only: every call below must be rejected by the
binding before any kernel is launched (the tensors are CPU tensors or have the wrong dtype / shape, so a launch would be an
out-of-bounds access on a GPU)."""

import pytest
import torch

from cosmos_predict25_b200.ops import native

pytestmark = pytest.mark.skipif(not native.available(), reason="extension not built")


def _ops():
    return native.load()


def test_rmsnorm_rope_bwd_rejects_mismatched_operands():
    ops = _ops()
    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    w = torch.ones(128)
    with pytest.raises(RuntimeError):
        ops.rmsnorm_rope_bwd(x, x, w, torch.zeros(1, 4, 2), None, None)          # CPU tensors
    with pytest.raises(RuntimeError):
        ops.rmsnorm_rope_bwd(x.float(), x, w, torch.zeros(1, 4, 2), None, None)  # dtype


def test_peer_ops_reject_bad_operands_before_launch():
    ops = _ops()
    x = torch.zeros(1, 4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        ops.a2a_scatter_heads_peer(x, [0, 0], torch.ones(128), torch.zeros(4, 64), torch.zeros(4, 64), 0, 1e-6)
    segs = torch.zeros(1, 4, dtype=torch.int64)
    shard = torch.zeros(16)
    with pytest.raises(RuntimeError):
        ops.adamw_push_peer([0, 0], [0, 0], segs, shard, shard, shard, shard, None, 0, 1.0, 1e-3, 0.9, 0.99, 1e-8, 0.0, 1, -1.0, None)
    with pytest.raises(RuntimeError):
        ops.rs_cast_norm_peer([0, 0], segs, shard, torch.zeros(1), None, 0, 1.0)
    with pytest.raises(RuntimeError):
        ops.a2a_gather_seq_peer([0, 0], 1, 4, 2, 128, 0, x)


def test_segment_table_bounds_are_checked_on_the_host():
    from cosmos_predict25_b200.parallel.peer_fsdp import check_segment_table
    ok = torch.tensor([[0, 64, 0, 64], [128, 32, 64, 32]])
    check_segment_table(ok, world=2, full_numel=192, shard_numel=96)
    with pytest.raises(ValueError):
        check_segment_table(ok, world=2, full_numel=191, shard_numel=96)      # last chunk of the last peer runs past the buffer
    with pytest.raises(ValueError):
        check_segment_table(ok, world=2, full_numel=192, shard_numel=95)
    with pytest.raises(ValueError):
        check_segment_table(torch.tensor([[0, 32, 0, 64]]), world=2, full_numel=192, shard_numel=96)   # stride < chunk
