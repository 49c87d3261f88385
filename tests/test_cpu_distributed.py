"""world_size = 2 tests on CPU with the gloo backend: context-parallel plumbing, Ulysses attention
equivalence, the sharded engine against a single-rank run, and host-side failure detection."""

import os
import socket
import tempfile
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn_name, tmp, kwargs):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    torch.set_num_threads(2)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        globals()[fn_name](rank, world, tmp, **kwargs)
        dist.barrier()
        with open(os.path.join(tmp, f"ok{rank}"), "w") as f:
            f.write("ok")
    except Exception:
        with open(os.path.join(tmp, f"err{rank}"), "w") as f:
            f.write(traceback.format_exc())
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_distributed(fn_name: str, world: int = 2, **kwargs):
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker, args=(world, _free_port(), fn_name, tmp, kwargs), nprocs=world, join=True)
        errs = [open(os.path.join(tmp, f)).read() for f in sorted(os.listdir(tmp)) if f.startswith("err")]
        assert not errs, "\n".join(errs)
        assert all(os.path.exists(os.path.join(tmp, f"ok{r}")) for r in range(world))


# ------------------------------------------------------------------------------------------------
def _cp_utils_vs_reference(rank, world, tmp):
    """The sequence split / gather helpers and the Ulysses exchange against the reference's own files, on gloo ranks."""
    from reference_oracle import import_reference, reference_network_modules
    from cosmos_predict25_b200.parallel import context_parallel as cp, ulysses
    ref = import_reference("cosmos_predict2._src.predict2.utils.context_parallel")
    g = dist.group.WORLD
    torch.manual_seed(3)
    y = torch.randn(2, 8, 3, 5)
    for dim in (1, 2) if world == 3 else (1,):
        if y.shape[dim] % world:
            continue
        loc, loc_ref = cp.split_inputs_cp(y, dim, g), ref.split_inputs_cp(y, dim, g)
        assert torch.equal(loc, loc_ref)
        assert torch.equal(cp.cat_outputs_cp(loc, dim, g), ref.cat_outputs_cp(loc_ref, dim, g))
        z, z_ref = loc.clone().requires_grad_(True), loc_ref.clone().requires_grad_(True)
        w = torch.randn(y.shape, generator=torch.Generator().manual_seed(9))
        (cp.cat_outputs_cp_with_grad(z, dim, g) * w).sum().backward()
        (ref.cat_outputs_cp_with_grad(z_ref, dim, g) * w).sum().backward()
        assert torch.equal(z.grad, z_ref.grad)
    # Ulysses exchange: [B, S/P, H, D] -> [B, S, H/P, D] and back, forward and backward, against the reference's autograd functions
    reference_network_modules()
    a2a = import_reference("cosmos_predict2._src.predict2.networks.a2a_cp")

    class _Dist:                                                 # torch.distributed with an all-to-all that gloo can run
        def __getattr__(self, name):
            return getattr(dist, name)

        @staticmethod
        def all_to_all_single(output, input, group=None, async_op=False):
            output.copy_(ulysses._a2a(input, group))
    a2a.dist = _Dist()
    x = torch.randn(2, 6, 4, 8, generator=torch.Generator().manual_seed(20 + rank))
    x1, x2 = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    h = ulysses._SeqToHead.apply(x1, g)
    h_ref = a2a._SeqAllToAll.apply(g, x2, True)                  # local sequence -> local heads
    assert torch.equal(h, h_ref)
    back, back_ref = ulysses._HeadToSeq.apply(h, g), a2a._SeqAllToAll.apply(g, h_ref, False)
    assert torch.equal(back, back_ref) and torch.equal(back, x)
    wgt = torch.randn(back.shape, generator=torch.Generator().manual_seed(40 + rank))
    (back * wgt).sum().backward()
    (back_ref * wgt).sum().backward()
    assert torch.equal(x1.grad, x2.grad)


def test_context_parallel_helpers_match_the_reference():
    run_distributed("_cp_utils_vs_reference", 2)


def _cp_utils(rank, world, tmp):
    from cosmos_predict25_b200.parallel import context_parallel as cp
    g = dist.group.WORLD
    x = torch.arange(24, dtype=torch.float32).view(2, 6, 2) if rank == 0 else torch.zeros(1)
    y = cp.broadcast(x if rank == 0 else None, g)
    assert y.shape == (2, 6, 2) and y[1, 5, 1] == 23
    loc = cp.split_inputs_cp(y, 1, g)
    assert loc.shape == (2, 3, 2) and loc[0, 0, 0] == rank * 6
    full = cp.cat_outputs_cp(loc, 1, g)
    assert torch.equal(full, y)
    z = loc.clone().requires_grad_(True)
    out = cp.cat_outputs_cp_with_grad(z, 1, g)
    (out * torch.arange(24, dtype=torch.float32).view(2, 6, 2)).sum().backward()
    assert torch.equal(z.grad, cp.split_inputs_cp(torch.arange(24, dtype=torch.float32).view(2, 6, 2), 1, g))
    obj = cp.broadcast({"a": 1} if rank == 0 else None, g)
    assert obj == {"a": 1}


def test_context_parallel_tensor_utils():
    run_distributed("_cp_utils")


def _ulysses(rank, world, tmp):
    from cosmos_predict25_b200.ops import ref
    from cosmos_predict25_b200.parallel import context_parallel as cp
    from cosmos_predict25_b200.parallel import ulysses
    torch.manual_seed(0)
    g = dist.group.WORLD
    B, S, H, D = 2, 12, 4, 16
    q, k, v = (torch.randn(B, S, H, D) for _ in range(3))
    full, _ = ref.attention(q, k, v)
    ql, kl, vl = (cp.split_inputs_cp(t, 1, g).clone().requires_grad_(True) for t in (q, k, v))
    out = ulysses.ulysses_attention(ql, kl, vl, g)
    assert torch.allclose(out, cp.split_inputs_cp(full, 1, g), atol=1e-5)
    # round trip of the exchange and gradient = reverse exchange
    h = ulysses.seq_to_head(ql.detach(), g)
    assert h.shape == (B, S, H // world, D)
    assert torch.equal(ulysses.head_to_seq(h, g), ql.detach())
    w = torch.randn(B, S, H, D)
    (out * cp.split_inputs_cp(w, 1, g)).sum().backward()
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    (ref.attention(qf, kf, vf)[0] * w).sum().backward()
    assert torch.allclose(ql.grad, cp.split_inputs_cp(qf.grad, 1, g), atol=1e-5)
    assert torch.allclose(kl.grad, cp.split_inputs_cp(kf.grad, 1, g), atol=1e-5)
    assert torch.allclose(vl.grad, cp.split_inputs_cp(vf.grad, 1, g), atol=1e-5)


def test_ulysses_attention_matches_full_attention():
    run_distributed("_ulysses")


def _dit_cp(rank, world, tmp):
    """Tiny DiT: context-parallel forward/backward over T equals the single-rank result."""
    from cosmos_predict25_b200.models.dit import CosmosDiT, dit_tiny
    from cosmos_predict25_b200.parallel import context_parallel as cp
    torch.manual_seed(0)
    g = dist.group.WORLD
    net = CosmosDiT(dit_tiny())
    net.init_weights()
    for p in net.parameters():
        if p.abs().sum() == 0:
            torch.nn.init.normal_(p, std=0.05)
    x = torch.randn(1, 16, 4, 16, 16)
    mask = torch.zeros(1, 1, 4, 16, 16)
    mask[:, :, :1] = 1
    t = torch.tensor([[300.0, 700.0, 700.0, 700.0]])
    ctx = torch.randn(1, 32, 256)
    want = net(x, t, ctx, condition_video_input_mask_B_C_T_H_W=mask)
    want.pow(2).mean().backward()
    ref_grads = {n: p.grad.clone() for n, p in net.named_parameters() if p.grad is not None}
    net.zero_grad()
    net.enable_context_parallel(g)
    xl, ml = cp.split_inputs_cp(x, 2, g), cp.split_inputs_cp(mask, 2, g)
    tl = cp.split_inputs_cp(t, 1, g)
    out = net(xl, tl, ctx, condition_video_input_mask_B_C_T_H_W=ml)
    assert torch.allclose(out, cp.split_inputs_cp(want, 2, g), atol=2e-4), (out - cp.split_inputs_cp(want, 2, g)).abs().max()
    (out.pow(2).sum() / want.numel()).backward()
    for n, p in net.named_parameters():
        if p.grad is None:
            continue
        gsum = p.grad.clone()
        dist.all_reduce(gsum)
        assert torch.allclose(gsum, ref_grads[n], atol=2e-4, rtol=1e-3), n


def test_dit_context_parallel_equals_single_rank():
    run_distributed("_dit_cp")


def _engine(rank, world, tmp):
    """Two-rank sharded engine == single-process engine on the summed batch gradient."""
    from cosmos_predict25_b200.parallel.fsdp import ShardedEngine
    torch.manual_seed(0)

    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 7, bias=False))

    data = torch.randn(2, 5, 24)
    net1 = make()
    eng1 = ShardedEngine(net1, group=None, compute_dtype=torch.float32, use_ema=True, units=[net1[0]])
    netP = make()
    engP = ShardedEngine(netP, group=dist.group.WORLD, compute_dtype=torch.float32, use_ema=True, units=[netP[0]])
    assert engP.units[0].shard_numel < eng1.units[0].shard_numel
    for step in range(3):
        sum(net1(data[r]).pow(2).mean() for r in range(world)).div(world).backward()
        n1 = eng1.step(lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01, max_grad_norm=0.5, ema_beta=0.9)
        netP(data[rank]).pow(2).mean().backward()
        nP = engP.step(lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01, max_grad_norm=0.5, ema_beta=0.9)
        assert torch.allclose(n1, nP, atol=1e-5), (n1, nP)
        for p1, pP in zip(net1.parameters(), netP.parameters()):
            assert torch.allclose(p1, pP, atol=1e-6), step
    sd1, sdP = eng1.full_state_dict("ema"), engP.full_state_dict("ema")
    for k in sd1:
        assert torch.allclose(sd1[k], sdP[k], atol=1e-6)
    # consolidated load restores both shards and the full parameters
    engP.load_full_state_dict({k: torch.zeros_like(v) for k, v in sdP.items()}, "master")
    assert all(p.abs().sum() == 0 for p in netP.parameters())


def test_sharded_engine_two_ranks_equals_one():
    run_distributed("_engine")


def _pt_checkpoint_resume(rank, world, tmp):
    """Single-file checkpoint of a 2-rank sharded run: after save -> perturb -> load every rank has its OWN rows of the
    masters and moments back (not rank 0's), the parameters are bit-identical and the next step gives the same loss."""
    from cosmos_predict25_b200.checkpoint.simple import PtCheckpointer
    from cosmos_predict25_b200.parallel.fsdp import ShardedEngine
    from cosmos_predict25_b200.trainer.optim import ShardedAdamW
    job = [tmp]
    dist.broadcast_object_list(job, src=0)   # every rank uses rank 0's directory

    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 8, bias=False))

    torch.manual_seed(1)
    data = torch.randn(world, 5, 24)
    net = make()
    eng = ShardedEngine(net, group=dist.group.WORLD, compute_dtype=torch.float32, use_ema=False, units=[net[0]])
    opt = ShardedAdamW(eng, lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01)
    for _ in range(2):
        net(data[rank]).pow(2).mean().backward()
        opt.step()
    before = [p.detach().clone() for p in net.parameters()]
    shard_before = {w: [getattr(u, w).clone() for u in eng.units] for w in ("master", "exp_avg", "exp_avg_sq")}
    ck = PtCheckpointer({}, job[0])
    ck.save(net, opt, None, 2)
    ck.finalize()
    dist.barrier()
    net(data[rank]).pow(2).mean().backward()
    opt.step()
    loss_ref = net(data[rank]).pow(2).mean().item()
    # a fresh process would start from the initial weights: emulate it with a new engine
    net2 = make()
    eng2 = ShardedEngine(net2, group=dist.group.WORLD, compute_dtype=torch.float32, use_ema=False, units=[net2[0]])
    opt2 = ShardedAdamW(eng2, lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01)
    assert PtCheckpointer({}, job[0]).load(net2, opt2, None) == 2
    for a, b in zip(before, net2.parameters()):
        assert torch.equal(a, b)
    for w, bufs in shard_before.items():
        for u, ref_buf in zip(eng2.units, bufs):
            assert torch.equal(getattr(u, w), ref_buf), (w, rank)
    net2(data[rank]).pow(2).mean().backward()
    opt2.step()
    assert net2(data[rank]).pow(2).mean().item() == loss_ref


def test_pt_checkpointer_resume_two_ranks():
    run_distributed("_pt_checkpoint_resume")


def _dcp_writer_processes(rank, world, tmp):
    """Asynchronous DCP save of a 2-rank sharded model through the per-rank writer processes (own gloo group): the trainer ranks
    keep stepping while the files are written, a fresh pair of ranks resumes bit-exactly, and a save that cannot be written on
    rank 0 is reported on every rank and the next save works again."""
    from cosmos_predict25_b200.checkpoint.dcp import DistributedCheckpointer
    from cosmos_predict25_b200.models.dit import dit_tiny
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    job = [tmp]
    dist.broadcast_object_list(job, src=0)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)

    def make():
        torch.manual_seed(0)
        m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"), fsdp_group=dist.group.WORLD)
        o, s = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="constant"))
        return m, o, s

    torch.manual_seed(3 + rank)
    batch = {"latents": torch.randn(1, 16, 4, 16, 16), "t5_text_embeddings": torch.randn(1, 32, 256), "fps": torch.tensor([16.0]),
             "padding_mask": torch.zeros(1, 1, 16, 16)}
    m, o, s = make()
    _, loss = m.training_step(dict(batch), 0)
    loss.backward()
    o.step()
    ck = DistributedCheckpointer({"dcp_async_mode_enabled": True}, job[0])
    ck.save(m, o, s, iteration=1)
    masters = [u.master.clone() for u in m.engine.units]
    _, loss = m.training_step(dict(batch), 1)      # the trainer goes on while the children write
    loss.backward()
    o.step()
    ck.finalize()
    dist.barrier()
    latest = os.path.join(job[0], "checkpoints", "latest_checkpoint.txt")
    assert open(latest).read().strip() == "iter_000000001"
    m2, o2, s2 = make()
    assert DistributedCheckpointer({}, job[0]).load(m2, o2, s2) == 1
    for a, u in zip(masters, m2.engine.units):
        assert torch.equal(a, u.master), rank
    # rank 0 cannot create the directory of iteration 2: every rank learns of the failure, the pointer stays
    if rank == 0:
        with open(os.path.join(job[0], "checkpoints", "iter_000000002"), "w") as f:
            f.write("taken")
    dist.barrier()
    ck.save(m, o, s, iteration=2)
    ck.finalize()
    assert ck._bg_error is None and open(latest).read().strip() == "iter_000000001"
    ck.save(m, o, s, iteration=3)
    ck.close()
    dist.barrier()
    assert open(latest).read().strip() == "iter_000000003"


def test_dcp_async_save_through_writer_processes():
    run_distributed("_dcp_writer_processes", world=2)


def _dcp_hybrid_sharding(rank, world, tmp):
    """DCP save / load of a model whose state is sharded over 2 ranks and replicated over 2 groups (world 4): the tensors are
    written as [Replicate, Shard(0)] DTensors on the (replicate, shard) mesh, a fresh set of ranks resumes bit-exactly, and the
    asynchronous writer processes produce the same checkpoint."""
    from cosmos_predict25_b200.checkpoint.dcp import DistributedCheckpointer
    from cosmos_predict25_b200.models.dit import dit_tiny
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.parallel.mesh import build_groups
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    job = [tmp]
    dist.broadcast_object_list(job, src=0)
    groups = build_groups(world, cp_size=1, shard_size=2)
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)

    def make():
        torch.manual_seed(0)
        m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"), fsdp_group=groups.fsdp, replicate_group=groups.replicate)
        o, s = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="constant"))
        return m, o, s

    torch.manual_seed(3 + rank)
    batch = {"latents": torch.randn(1, 16, 4, 16, 16), "t5_text_embeddings": torch.randn(1, 32, 256), "fps": torch.tensor([16.0]),
             "padding_mask": torch.zeros(1, 1, 16, 16)}
    m, o, s = make()
    assert m.engine.P == 2 and m.engine.R == 2
    _, loss = m.training_step(dict(batch), 0)
    loss.backward()
    o.step()
    masters = [u.master.clone() for u in m.engine.units]
    for sub, cfg_ck in (("sync", {}), ("async", {"dcp_async_mode_enabled": True})):
        ck = DistributedCheckpointer(cfg_ck, os.path.join(job[0], sub))
        ck.save(m, o, s, iteration=1)
        getattr(ck, "close", ck.finalize)()
        dist.barrier()
        m2, o2, s2 = make()
        assert DistributedCheckpointer({}, os.path.join(job[0], sub)).load(m2, o2, s2) == 1
        for a, u in zip(masters, m2.engine.units):
            assert torch.equal(a, u.master), (sub, rank)
        for (n1, p1), (_, p2) in zip(m.net.named_parameters(), m2.net.named_parameters()):
            assert torch.equal(p1, p2), (sub, n1)


def test_dcp_under_hybrid_sharding_four_ranks():
    run_distributed("_dcp_hybrid_sharding", world=4)


def _hsdp(rank, world, tmp, shard_size):
    """Hybrid sharding (shard groups of ``shard_size`` ranks, replicated ``world / shard_size`` times) and plain data
    parallelism (``shard_size`` 1) give the same parameters as one process that sees the whole batch."""
    from cosmos_predict25_b200.parallel.fsdp import ShardedEngine
    from cosmos_predict25_b200.parallel.mesh import build_groups

    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Linear(24, 40), torch.nn.GELU(), torch.nn.Linear(40, 8, bias=False))

    torch.manual_seed(3)
    data = torch.randn(world, 5, 24)
    g = build_groups(cp_size=1, shard_size=shard_size)
    assert g.shard_size == shard_size and g.replicate_size == world // shard_size and g.replicate is not None
    net1 = make()
    eng1 = ShardedEngine(net1, group=None, compute_dtype=torch.float32, use_ema=False, units=[net1[0]])
    netP = make()
    engP = ShardedEngine(netP, group=g.fsdp, compute_dtype=torch.float32, use_ema=False, units=[netP[0]],
                         replicate_group=g.replicate)
    assert engP.P == shard_size and engP.R == world // shard_size
    for step in range(3):
        sum(net1(data[r]).pow(2).mean() for r in range(world)).div(world).backward()
        n1 = eng1.step(lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01, max_grad_norm=0.5)
        netP(data[rank]).pow(2).mean().backward()
        nP = engP.step(lr=1e-2, betas=(0.9, 0.99), weight_decay=0.01, max_grad_norm=0.5)
        assert torch.allclose(n1, nP, atol=1e-5), (n1, nP)
        for p1, pP in zip(net1.parameters(), netP.parameters()):
            assert torch.allclose(p1, pP, atol=1e-6), step


@pytest.mark.parametrize("shard_size", [2, 1])
def test_hybrid_sharding_and_data_parallel_four_ranks(shard_size):
    run_distributed("_hsdp", world=4, shard_size=shard_size)


def _model_fsdp_cp(rank, world, tmp):
    """Full model with parameter sharding + context parallelism over the same two ranks: both ranks see the
    same loss (one sample, sequence-sharded) and the step keeps parameters identical across ranks."""
    from cosmos_predict25_b200.models.dit import dit_tiny
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    torch.manual_seed(0)
    g = dist.group.WORLD
    cfg = Video2WorldRFConfig(net=dit_tiny(), precision="float32", state_t=4)
    m = Video2WorldModelRectifiedFlow(cfg, device=torch.device("cpu"), fsdp_group=g, cp_group=g)
    opt, sch = m.init_optimizer_scheduler(OptimizerConfig(lr=1e-3), SchedulerConfig(kind="constant"))
    torch.manual_seed(10 + rank)  # different local data: rank 0's sample must win
    batch = {"latents": torch.randn(1, 16, 4, 16, 16), "t5_text_embeddings": torch.randn(1, 32, 256),
             "fps": torch.tensor([16.0]), "padding_mask": torch.zeros(1, 1, 16, 16), "num_conditional_frames": 1}
    out, loss = m.training_step(batch, 0)
    assert out["x0"].shape[2] == 2  # T-sharded
    loss.backward()
    opt.step()
    flat = torch.cat([p.detach().reshape(-1) for p in m.net.parameters()])
    other = [torch.empty_like(flat) for _ in range(world)]
    dist.all_gather(other, flat)
    assert torch.equal(other[0], other[1])
    s = m.generate_samples_from_batch(dict(batch), guidance=2.0, seed=3, num_steps=2, solver="euler")
    assert s.shape == (1, 16, 4, 16, 16)


def test_model_with_fsdp_and_context_parallel():
    run_distributed("_model_fsdp_cp")


def _missing_rank(rank, world, tmp):
    """Failure detection on the host: a rank that never joins a collective ends it with an error on
    the others after a short process-group timeout (no GPU involved)."""
    import datetime
    g = dist.new_group([0, 1], timeout=datetime.timedelta(seconds=2), backend="gloo")
    if rank == 0:
        with pytest.raises(Exception):
            dist.all_reduce(torch.ones(1), group=g)
    else:
        import time
        time.sleep(4)  # never joins


def test_short_timeout_surfaces_a_missing_rank():
    with tempfile.TemporaryDirectory() as tmp:
        mp.spawn(_worker_nobarrier, args=(2, _free_port(), "_missing_rank", tmp), nprocs=2, join=True)
        errs = [open(os.path.join(tmp, f)).read() for f in sorted(os.listdir(tmp)) if f.startswith("err")]
        assert not errs, "\n".join(errs)


def _worker_nobarrier(rank, world, port, fn_name, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world)
        globals()[fn_name](rank, world, tmp)
    except Exception:
        with open(os.path.join(tmp, f"err{rank}"), "w") as f:
            f.write(traceback.format_exc())


# ------------------------------------------------------------------------------------------------
def _tp_qwen(rank, world, tmp, sequence_parallel):
    from cosmos_predict25_b200.models.text_encoder import QwenConfig, QwenLanguageModel
    from cosmos_predict25_b200.parallel.parallel_dims import ParallelDims
    from cosmos_predict25_b200.parallel.parallelize_qwen import parallelize_qwen
    torch.manual_seed(0)
    cfg = QwenConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2)
    ref = QwenLanguageModel(cfg)
    tp_model = QwenLanguageModel(cfg)
    tp_model.load_state_dict(ref.state_dict())
    dims = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, world_size=world)
    mesh = dims.build_mesh("cpu")
    parallelize_qwen(tp_model, mesh, dims, sequence_parallel=sequence_parallel)
    from torch.distributed.tensor import DTensor
    assert isinstance(tp_model.layers[0].self_attn.q_proj.weight, DTensor)
    assert tp_model.layers[0].self_attn.q_proj.weight.to_local().shape[0] == 32 // world
    ids = torch.randint(0, 64, (2, 8), generator=torch.Generator().manual_seed(1))
    want = ref(ids)[-1]
    got = tp_model(ids)[-1]
    if isinstance(got, DTensor):
        got = got.full_tensor()
    assert torch.allclose(got, want, atol=1e-4), (got - want).abs().max()


def _tp_qwen_float8(rank, world, tmp):
    """Float8 linears under the tensor-parallel plan: logits and every gradient stay within the 8-bit error of the fp32 model."""
    from cosmos_predict25_b200.models.text_encoder import QwenConfig
    from cosmos_predict25_b200.models.vlm_train import QwenForCausalLM
    from cosmos_predict25_b200.modules.float8 import Float8Linear
    from cosmos_predict25_b200.parallel.parallel_dims import ParallelDims
    from cosmos_predict25_b200.parallel.parallelize_qwen import parallelize_qwen
    from torch.distributed.tensor import DTensor
    torch.manual_seed(0)
    cfg = QwenConfig(vocab_size=64, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2)
    ref = QwenForCausalLM(cfg)
    tp_model = QwenForCausalLM(cfg)
    tp_model.load_state_dict(ref.state_dict())
    dims = ParallelDims(dp_replicate=1, dp_shard=1, cp=1, tp=world, pp=1, world_size=world)
    parallelize_qwen(tp_model.model, dims.build_mesh("cpu"), dims, enable_float8=True)
    q = tp_model.model.layers[0].self_attn.q_proj
    assert isinstance(q, Float8Linear) and isinstance(q.weight, DTensor) and q.weight.to_local().shape[0] == 64 // world
    assert type(tp_model.lm_head) is torch.nn.Linear
    ids = torch.randint(0, 64, (2, 16), generator=torch.Generator().manual_seed(1))
    want = ref(ids)
    got = tp_model(ids)
    got = got.full_tensor() if isinstance(got, DTensor) else got
    rel = lambda a, b: ((a - b).norm() / b.norm()).item()
    assert rel(got, want) < 0.1, rel(got, want)
    g = torch.randn(want.shape, generator=torch.Generator().manual_seed(2))
    (want * g).sum().backward()
    (got * g).sum().backward()
    checked = 0
    for (n, p), (_, pr) in zip(tp_model.named_parameters(), ref.named_parameters()):
        if pr.grad is None:
            continue
        assert p.grad is not None, n
        grad = p.grad.full_tensor() if isinstance(p.grad, DTensor) else p.grad
        assert rel(grad, pr.grad) < 0.25, (n, rel(grad, pr.grad))
        checked += 1
    assert checked >= 20


def test_tensor_parallel_float8_qwen():
    run_distributed("_tp_qwen_float8", 2)


@pytest.mark.parametrize("sequence_parallel", [False])
def test_tensor_parallel_qwen_matches_single_rank(sequence_parallel):
    run_distributed("_tp_qwen", 2, sequence_parallel=sequence_parallel)


def test_parallel_dims_layout():
    from cosmos_predict25_b200.parallel.parallel_dims import ParallelDims
    d = ParallelDims(dp_replicate=2, dp_shard=-1, cp=2, tp=2, pp=1, world_size=32)
    assert d.dp_shard == 4 and d.mesh_shape() == ([2, 4, 2, 2], ["dp_replicate", "dp_shard", "cp", "tp"])
    assert d.flattened_views() == {"dp": ["dp_replicate", "dp_shard"], "dp_shard_cp": ["dp_shard", "cp"], "dp_cp": ["dp_replicate", "dp_shard", "cp"]}
    assert d.coordinates(0) == {"tp": 0, "cp": 0, "dp_shard": 0, "dp_replicate": 0, "pp": 0}
    assert d.coordinates(7) == {"tp": 1, "cp": 1, "dp_shard": 1, "dp_replicate": 0, "pp": 0}
    assert d.non_data_parallel_size == 4 and d.dp_enabled and d.tp_enabled and not d.pp_enabled
    fixed = ParallelDims(dp_replicate=3, dp_shard=2, cp=1, tp=2, pp=1, world_size=8)     # 3*2*2 != 8 -> dp_replicate recomputed
    assert fixed.dp_replicate == 2
    with pytest.raises(AssertionError):
        ParallelDims(dp_replicate=1, dp_shard=3, cp=1, tp=1, pp=1, world_size=8)
    from cosmos_predict25_b200.utils.train_metrics import dit_flop_per_sample, get_num_flop_per_token, get_peak_flops, mfu
    assert get_peak_flops("NVIDIA B200") == 2.25e15 and get_peak_flops("NVIDIA H100 80GB HBM3") == 989e12
    f = dit_flop_per_sample(2048, 28, 84480, training=False)
    assert 1.7e15 < f < 2.2e15                                    # ~1.9 PFLOP per 2B forward at 84,480 tokens
    assert abs(mfu(f * 3, 8.0, 1, 2.25e15) - f * 3 / 8.0 / 2.25e15) < 1e-12
    assert get_num_flop_per_token(7_000_000_000, 28, 28, 128, 4096) == 6 * 7_000_000_000 + 12 * 28 * 28 * 128 * 4096


# ------------------------------------------------------------------------------------------------
def _vae_row_sharded(rank, world, tmp):
    """Row-sharded VAE decode with halo exchange equals the single-rank decode (attention block included)."""
    from cosmos_predict25_b200.models.vae_wan import Wan2pt1VAEInterface
    torch.manual_seed(0)
    tok = Wan2pt1VAEInterface(device="cpu", dtype=torch.float32, dim=8)
    for p in tok.model.parameters():            # the attention projection starts at zero: make it count
        if p.abs().sum() == 0:
            torch.nn.init.normal_(p, std=0.05)
    torch.manual_seed(1)
    lat = torch.randn(1, 16, 3, 2 * world, 6)
    full = tok.decode(lat)
    got = tok.decode_parallel(lat, dist.group.WORLD)
    assert got.shape == full.shape == (1, 3, 9, 16 * world, 48)
    assert (got - full).abs().max() < 1e-4 * max(1.0, full.abs().max().item())
    only0 = tok.decode_parallel(lat, dist.group.WORLD, dst=0)
    assert (only0 is None) == (rank != 0)
    if rank == 0:
        assert torch.equal(only0, got)
    # rows that do not divide over the group: plain decode on every rank
    odd = tok.decode_parallel(torch.randn(1, 16, 1, 3, 4), dist.group.WORLD)
    assert odd.shape == (1, 3, 1, 24, 32)
    # encoder: bands of 16 pixel rows (even through the three stride-2 stages), one row from the next rank per stage
    torch.manual_seed(2)
    vid = torch.rand(1, 3, 5, 16 * world, 24) * 2 - 1
    lat_full = tok.encode(vid)
    lat_par = tok.encode_parallel(vid, dist.group.WORLD)
    assert lat_par.shape == lat_full.shape == (1, 16, 2, 2 * world, 3)
    assert (lat_par - lat_full).abs().max() < 1e-4 * max(1.0, lat_full.abs().max().item())
    assert tok.encode_parallel(vid[:, :, :, :24], dist.group.WORLD).shape[3] == 3       # 24 rows: no even bands, plain encode


def test_vae_decode_row_sharded_matches_single_rank():
    run_distributed("_vae_row_sharded", world=2)


def test_vae_decode_row_sharded_three_ranks():
    run_distributed("_vae_row_sharded", world=3)


# ------------------------------------------------------------------------------------------------
def _ring_attention(rank, world, tmp):
    """Ring attention over a sequence-sharded q/k/v equals attention over the gathered sequence, forward and backward;
    a DiT running with comm_type="p2p" equals the same DiT with the all-to-all exchange."""
    from cosmos_predict25_b200.ops import ref
    from cosmos_predict25_b200.parallel.ring_attention import ring_attention
    g = dist.group.WORLD
    torch.manual_seed(0)
    B, S, H, D = 2, 6, 3, 8                      # 3 heads: not divisible by 2 ranks, which Ulysses could not shard
    full = [torch.randn(B, S * world, H, D, dtype=torch.float64) for _ in range(3)]
    go = torch.randn(B, S * world, H, D, dtype=torch.float64)
    loc = [t[:, rank * S:(rank + 1) * S].clone().requires_grad_(True) for t in full]
    out = ring_attention(loc[0], loc[1], loc[2], g)
    out.backward(go[:, rank * S:(rank + 1) * S])
    ref_in = [t.clone().requires_grad_(True) for t in full]
    want, _ = ref.attention(*ref_in, D ** -0.5)
    want.backward(go.to(want.dtype))
    sl = slice(rank * S, (rank + 1) * S)
    assert torch.allclose(out.double(), want[:, sl].double(), atol=1e-5)
    for a, b in zip(loc, ref_in):
        assert torch.allclose(a.grad.double(), b.grad[:, sl].double(), atol=1e-4), (a.grad - b.grad[:, sl]).abs().max()

    from cosmos_predict25_b200.models.dit import NET_PRESETS, CosmosDiT
    torch.manual_seed(1)
    cfg = NET_PRESETS["tiny"]()
    net = CosmosDiT(cfg).eval()
    net.init_weights()
    T = 2 * world
    x = torch.randn(1, cfg.in_channels, T, 8, 8)
    ctx_dim = cfg.crossattn_proj_in_channels if cfg.use_crossattn_projection else cfg.crossattn_emb_channels
    kw = dict(crossattn_emb=torch.randn(1, 8, ctx_dim), fps=torch.tensor([16.0]), padding_mask=torch.zeros(1, 1, 8, 8))
    ts = torch.full((1, T), 0.5)
    mask = torch.zeros(1, 1, T, 8, 8)
    tl = slice(rank * 2, rank * 2 + 2)
    outs = {}
    with torch.no_grad():
        kinds = ("a2a", "p2p") if cfg.num_heads % world == 0 else ("p2p",)   # the all-to-all needs heads % ranks == 0
        for kind in kinds:
            net.enable_context_parallel(g, kind)
            outs[kind] = net(x[:, :, tl], ts[:, tl], condition_video_input_mask_B_C_T_H_W=mask[:, :, tl], **kw)
        net.disable_context_parallel()
        whole = net(x, ts, condition_video_input_mask_B_C_T_H_W=mask, **kw)
    if "a2a" in outs:
        assert torch.allclose(outs["p2p"], outs["a2a"], atol=1e-4)
    assert torch.allclose(outs["p2p"], whole[:, :, tl], atol=1e-4)


@pytest.mark.parametrize("world", [2, 3])
def test_ring_attention_matches_gathered_attention(world):
    run_distributed("_ring_attention", world=world)


# ------------------------------------------------------------------------------------------------
def _qwen_allgather_kv_cp(rank, world, tmp):
    """The language tower with all-gather-KV context parallelism returns the single-rank hidden states."""
    from cosmos_predict25_b200.models.text_encoder import QwenConfig, QwenLanguageModel
    torch.manual_seed(0)
    cfg = QwenConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2)
    lm = QwenLanguageModel(cfg).eval()
    ids = torch.randint(0, 64, (2, 6 * world))
    att = torch.ones(2, 6 * world, dtype=torch.long)
    att[1, -4:] = 0                                        # right padding on one sample
    want = lm(ids, att)
    got = lm(ids, att, cp_group=dist.group.WORLD)
    assert len(got) == len(want) == 3
    valid = att.bool()[..., None]
    for a, b in zip(got, want):
        assert a.shape == b.shape
        assert torch.allclose(a * valid, b * valid, atol=1e-5)
    nomask = lm(ids, None, cp_group=dist.group.WORLD)
    assert torch.allclose(nomask[-1], lm(ids, None)[-1], atol=1e-5)


@pytest.mark.parametrize("world", [2, 3])
def test_text_tower_all_gather_kv_context_parallel(world):
    run_distributed("_qwen_allgather_kv_cp", world=world)


# ------------------------------------------------------------------------------------------------
def _sparse_attention_under_cp(rank, world, tmp):
    """Neighbourhood attention in a DiT under context parallelism (q/k/v exchanged to whole-sequence / local-heads, operator
    applied on the full T x H x W grid, output exchanged back) equals the single-rank sparse network."""
    from cosmos_predict25_b200.models.dit import NET_PRESETS, CosmosDiT, replace_selfattn_op_with_sparse_attn_op
    g = dist.group.WORLD
    torch.manual_seed(2)
    cfg = NET_PRESETS["tiny"]()
    net = CosmosDiT(cfg).eval()
    net.init_weights()
    replace_selfattn_op_with_sparse_attn_op(net, 0, {"window_size": (2, 3, 3), "stride": (1, 1, 2)})
    T = 2 * world
    x = torch.randn(1, cfg.in_channels, T, 8, 8)
    ctx_dim = cfg.crossattn_proj_in_channels if cfg.use_crossattn_projection else cfg.crossattn_emb_channels
    kw = dict(crossattn_emb=torch.randn(1, 8, ctx_dim), fps=torch.tensor([16.0]), padding_mask=torch.zeros(1, 1, 8, 8))
    ts = torch.full((1, T), 0.5)
    mask = torch.zeros(1, 1, T, 8, 8)
    tl = slice(rank * 2, rank * 2 + 2)
    with torch.no_grad():
        whole = net(x, ts, condition_video_input_mask_B_C_T_H_W=mask, **kw)
        net.enable_context_parallel(g)
        part = net(x[:, :, tl], ts[:, tl], condition_video_input_mask_B_C_T_H_W=mask[:, :, tl], **kw)
    assert torch.allclose(part, whole[:, :, tl], atol=1e-4), (part - whole[:, :, tl]).abs().max()


def test_sparse_attention_under_context_parallel():
    run_distributed("_sparse_attention_under_cp", world=2)


# ------------------------------------------------------------------------------------------------
def _network_jvp_under_cp(rank, world, tmp):
    """Forward-mode (JVP) network pass under context parallelism equals the T-slice of the single-rank pass."""
    from cosmos_predict25_b200.models.distill import network_jvp
    from cosmos_predict25_b200.models.dit import NET_PRESETS, CosmosDiT
    g = dist.group.WORLD
    torch.manual_seed(3)
    cfg = NET_PRESETS["tiny"]()
    net = CosmosDiT(cfg).eval()
    net.init_weights()
    for p in net.parameters():                   # AdaLN output layers start at zero: perturb so that every path carries signal
        if p.abs().sum() == 0:
            torch.nn.init.normal_(p, std=0.02)
    T = 2 * world
    x, tx = torch.randn(1, cfg.in_channels, T, 8, 8), torch.randn(1, cfg.in_channels, T, 8, 8)
    ts, tt = torch.full((1, T), 0.4), torch.ones(1, T)
    ctx_dim = cfg.crossattn_proj_in_channels if cfg.use_crossattn_projection else cfg.crossattn_emb_channels
    kw = dict(crossattn_emb=torch.randn(1, 8, ctx_dim), fps=torch.tensor([16.0]), padding_mask=torch.zeros(1, 1, 8, 8))
    mask = torch.zeros(1, 1, T, 8, 8)
    F_full, dF_full = network_jvp(net, x, ts, tx, tt, condition_video_input_mask_B_C_T_H_W=mask, **kw)
    tl = slice(rank * 2, rank * 2 + 2)
    net.enable_context_parallel(g)
    F_loc, dF_loc = network_jvp(net, x[:, :, tl], ts[:, tl], tx[:, :, tl], tt[:, tl], condition_video_input_mask_B_C_T_H_W=mask[:, :, tl], **kw)
    net.disable_context_parallel()
    assert dF_full.abs().max() > 1e-4
    assert torch.allclose(F_loc, F_full[:, :, tl], atol=1e-4)
    assert torch.allclose(dF_loc, dF_full[:, :, tl], atol=1e-4), (dF_loc - dF_full[:, :, tl]).abs().max()


def test_network_jvp_under_context_parallel():
    run_distributed("_network_jvp_under_cp", world=2)


# ------------------------------------------------------------------------------------------------
def _sigma_loss_analysis(rank, world, tmp):
    """Ranks hold different numbers of rows (rank 1 has image rows only on some steps): rank 0's record covers all of them."""
    import json
    import types
    from cosmos_predict25_b200.trainer.analysis_callbacks import SigmaLossAnalysisPerFrame
    out_dir = os.path.join(tmp, "run")
    cb = SigmaLossAnalysisPerFrame(logging_iter_multipler=1, logging_viz_iter_multipler=2, save_dir=os.path.join(tmp, "dump"))
    cb.config = types.SimpleNamespace(trainer=types.SimpleNamespace(logging_iter=2), output_dir=out_dir)
    model = types.SimpleNamespace(is_image_batch=lambda b: b["image"])
    g = torch.Generator().manual_seed(rank)
    rows = {0: 2, 1: 3}[rank]
    for it in (1, 2, 3, 4):
        image = rank == 1 and it == 3                      # only rank 1 ever sees an image batch
        T = 1 if image else 4
        out = {"sigma": torch.rand(rows, 1, generator=g) + 0.1, "edm_loss_per_frame": torch.rand(rows, T, generator=g)}
        cb.on_training_step_end(model, {"image": image}, out, None, it)
    if rank == 0:
        recs = [json.loads(l) for l in open(os.path.join(out_dir, "sigma_loss_analysis.jsonl"))]
        assert [r["iteration"] for r in recs] == [2, 4]
        assert recs[0]["sigma_loss_video/total_samples"] == 2 * (2 + 3)          # two steps x both ranks' rows
        assert recs[1]["sigma_loss_video/total_samples"] == 2 * 2 + 3 and recs[1]["sigma_loss_image/total_samples"] == 3
        assert "sigma_loss_video/frame_3/loss_q3" in recs[0] and "sigma_loss_video/frame_0/loss_by_sigma_bin" not in recs[0]
        bins = recs[1]["sigma_loss_video/frame_0/loss_by_sigma_bin"]
        assert sum(b["count"] for b in bins) == 7 and "sigma_loss_image/loss_mean" in recs[1]
        assert sorted(os.listdir(os.path.join(tmp, "dump"))) == ["sigma_loss_image_Iter000000004.pkl", "sigma_loss_video_Iter000000002.pkl",
                                                                 "sigma_loss_video_Iter000000004.pkl"]


def test_sigma_loss_analysis_gathers_uneven_ranks():
    run_distributed("_sigma_loss_analysis", world=2)
