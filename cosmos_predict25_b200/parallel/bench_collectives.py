"""Device timing and roofline fractions of the kernels that fuse a collective with compute, on N GPUs of one node.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 -m cosmos_predict25_b200.parallel.bench_collectives

Rows (every time is the maximum over ranks of a CUDA-event median, L2 flushed between iterations):

  * all-gather fused into the GEMM (``gemm_bf16_gather``) at the 2B / 14B projection shapes, next to the same GEMM on a resident
    weight and next to NCCL all-gather followed by that GEMM;
  * gradient reduce-scatter fused with cast / scale / scrub / norm (``rs_cast_norm_peer``) and AdamW + EMA + parameter push
    (``adamw_push_peer``) on one 2B block unit, next to their NCCL + torch twins.

Roofline of a fused kernel: the slower of FLOPs / measured bf16 peak, NVLink bytes per GPU and direction / 770 GB/s (measured peer
copy on this pool) and HBM bytes / measured copy bandwidth; ``frac`` = that time / measured time.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics

import torch
import torch.distributed as dist

NVLINK_GBS = 770.0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=84480)
    ap.add_argument("--json", default=None)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import native
    from ..ops.bench_kernels import flush_l2, peaks
    from .symm import PeerContext, SymmetricArena
    ops = native.load()
    pk = peaks()
    g = dist.group.WORLD
    rows_out = []

    def timed(fn, iters=5, warmup=2):
        for _ in range(warmup):
            fn()
        ts = []
        for _ in range(iters):
            flush_l2()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([statistics.median(ts)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def add(name, shape, ms, flops=0.0, nvlink_bytes=0.0, hbm_bytes=0.0, note=""):
        bound_ms = max(flops / (pk["tflops"] * 1e9), nvlink_bytes / (NVLINK_GBS * 1e6), hbm_bytes / (pk["hbm_gbs"] * 1e6))
        r = {"kernel": name, "shape": shape, "n_gpus": world, "ms": round(ms, 4), "roofline_ms": round(bound_ms, 4),
             "frac_of_roofline": round(bound_ms / ms, 3) if bound_ms > 0 else None, "note": note}
        rows_out.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)

    M = args.tokens
    arena = SymmetricArena(1 << 30, g, dev)
    # ---- all-gather -> GEMM ----------------------------------------------------------------------------------------------
    for rows, K, tag in ((2048, 2048, "2B q/k/v/out"), (8192, 2048, "2B mlp.layer1"), (5120, 5120, "14B q/k/v/out")):
        if rows % (8 * world):
            continue
        torch.manual_seed(0)
        W = (torch.randn(rows, K, device=dev) * 0.02).bfloat16()
        chunk = rows // world
        shard = arena.alloc(chunk * K, torch.bfloat16)
        shard.tensor.copy_(W[rank * chunk:(rank + 1) * chunk].reshape(-1))
        torch.cuda.synchronize()
        dist.barrier()
        ws = torch.zeros(rows, K, device=dev, dtype=torch.bfloat16)
        counters = torch.zeros((rows + 255) // 256, dtype=torch.int32, device=dev)
        x = torch.randn(M, K, device=dev).bfloat16()
        fl = 2.0 * M * rows * K
        nv = (world - 1) * chunk * K * 2.0                     # bytes this GPU receives
        shp = f"{M}x{rows}x{K} {tag}"
        t_fused = timed(lambda: ops.gemm_bf16_gather(x, ws, shard.ptrs, chunk, counters, None, 0, False, None))
        t_plain = timed(lambda: ops.gemm_bf16(x, W, None, 0, False, False))
        full = torch.empty(world * chunk * K, device=dev, dtype=torch.bfloat16)

        def nccl_then_gemm():
            dist.all_gather_into_tensor(full, shard.tensor, group=g)
            return ops.gemm_bf16(x, full.view(rows, K), None, 0, False, False)

        t_nccl = timed(nccl_then_gemm)
        add("gemm_bf16_gather (all-gather fused into the GEMM)", shp, t_fused, fl, nv, 0.0,
            note=f"resident-weight GEMM {t_plain:.3f} ms; NCCL all-gather + GEMM {t_nccl:.3f} ms")
        del W, ws, x, full
    # ---- reduce-scatter + AdamW on one 2B block unit ---------------------------------------------------------------------
    n_full = 69_206_016 // (8 * world) * (8 * world)       # elements of one 2B block (69 M parameters)
    chunk = n_full // world
    ctx = PeerContext(g, dev, arena=arena)
    grad = arena.alloc(n_full, torch.bfloat16)
    full = arena.alloc(n_full, torch.bfloat16)
    sumsq_slot = arena.alloc(64, torch.float32)
    grad.tensor.normal_()
    segs = torch.tensor([[0, chunk, 0, chunk]], dtype=torch.int64, device=dev)
    g32 = torch.zeros(chunk, device=dev)
    master, m_, v_, ema = (torch.zeros(chunk, device=dev) for _ in range(4))
    unit_ss = torch.zeros(1, device=dev)
    norm_out = torch.zeros(1, device=dev)
    torch.cuda.synchronize()
    dist.barrier()

    def rs():
        ctx.barrier()
        ops.rs_cast_norm_peer(grad.ptrs, segs, g32, unit_ss, sumsq_slot.tensor[:1], rank, 1.0 / world)

    def push():
        ctx.barrier()
        ops.adamw_push_peer(full.ptrs, sumsq_slot.ptrs, segs, master, g32, m_, v_, ema, rank, 1.0, 1e-4, 0.9, 0.999, 1e-8, 1e-3, 1,
                            0.99, norm_out)
        ctx.barrier()

    t_rs = timed(rs)
    t_push = timed(push)
    out16 = torch.empty(chunk, device=dev, dtype=torch.bfloat16)
    gathered = torch.empty(n_full, device=dev, dtype=torch.bfloat16)

    def rs_nccl():
        dist.reduce_scatter_tensor(out16, grad.tensor, group=g)
        red = torch.nan_to_num(out16.float() / world)
        g32.copy_(red)
        unit_ss.copy_(red.pow(2).sum().view(1))

    def push_nccl():
        ops.adamw_ema_shard(master, g32, m_, v_, ema, out16, torch.ones(1, device=dev), 1e-4, 0.9, 0.999, 1e-8, 1e-3, 1, 0.99)
        dist.all_gather_into_tensor(gathered, out16, group=g)

    t_rs_n = timed(rs_nccl)
    t_push_n = timed(push_nccl)
    shp = f"{n_full} params, {world} ranks"
    add("rs_cast_norm_peer (+ device barrier)", shp, t_rs, 0.0, (world - 1) * chunk * 2.0, world * chunk * 2.0 / 1 + chunk * 4.0,
        note=f"NCCL reduce-scatter + cast + nan_to_num + norm: {t_rs_n:.3f} ms")
    add("adamw_push_peer (+ 2 device barriers)", shp, t_push, 0.0, (world - 1) * chunk * 2.0, chunk * (4.0 * 9 + 2.0),
        note=f"adamw_ema_shard + NCCL all-gather: {t_push_n:.3f} ms")
    ctx.check()
    err = ops.kernel_error(local, True)
    if rank == 0:
        print(json.dumps({"kernel_error": int(err), "peaks": pk, "nvlink_gbs_per_direction": NVLINK_GBS}))
        if args.json:
            with open(args.json, "w") as f:
                json.dump({"rows": rows_out, "peaks": pk}, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
