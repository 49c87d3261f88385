"""Device-timed comparison of the Ulysses exchange inside the compute kernels against compute + stand-alone exchange.

Launch with one process per GPU, e.g.
``python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 -m cosmos_predict25_b200.parallel.bench_exchange``

Shapes are those of one 2B self-attention call during sampling (batch 2 = cond + uncond, 84,480 tokens split over the
ranks, 16 heads of 128, model width 2048). For each direction it prints one JSON line with the fused and the unfused
time (CUDA events on the launching stream, max over ranks, L2 flushed between iterations) and the roofline of the fused
kernel: max(FLOPs / measured GEMM peak, bytes that must cross NVLink per GPU / 770 GB/s).
"""

from __future__ import annotations

import argparse
import json
import math
import os

import torch
import torch.distributed as dist


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=84480)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--width", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--iters", type=int, default=5)
    args = ap.parse_args()
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    dist.init_process_group("nccl", device_id=dev)
    from ..ops import bench_kernels
    from ..ops import functional as F_ops
    from ..ops import native
    from .symm import PeerAllToAll, PeerContext

    g = dist.group.WORLD
    B, D, H = args.batch, args.width, args.heads
    S = args.tokens // world
    per_rank = B * S * H * 128
    ctx = PeerContext(g, dev, arena_bytes=8 * (per_rank * 2 + 4096) + (1 << 20))
    t = PeerAllToAll(ctx, max_elems=per_rank)
    torch.manual_seed(rank)
    x = torch.randn(B, S, D, device=dev).bfloat16()
    torch.manual_seed(99)
    wq, wk, wv = ((torch.randn(H * 128, D, device=dev) * D ** -0.5).bfloat16() for _ in range(3))
    nq, nk = (1 + 0.1 * torch.randn(128, device=dev) for _ in range(2))
    half = torch.rand(S, 64, device=dev) * 30
    rope = F_ops.RopeTable(torch.cat([half, half], -1))
    pk = bench_kernels.peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        times = []
        for i in range(args.iters + 2):
            flush.zero_()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            if i >= 2:
                times.append(e0.elapsed_time(e1))
        ms = torch.tensor([sum(times) / len(times)], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms)

    x2d = x.view(B * S, D)

    def unfused_qkv():
        q = F_ops.linear(x2d, wq).view(B, S, H, 128)
        k = F_ops.linear(x2d, wk).view(B, S, H, 128)
        v = F_ops.linear(x2d, wv).view(B, S, H, 128)
        return t.scatter_heads([q, k, v], [nq, nk, None], rope, 1e-6, copy_out=False)[0]

    def fused_qkv():
        return t.project_scatter_heads(x2d, [wq, wk, wv], [nq, nk, None], rope, B, S, 1e-6)

    with torch.no_grad():
        ms_u, ms_f = timed(unfused_qkv), timed(fused_qkv)
        flops = 3 * 2.0 * B * S * D * H * 128
        link_bytes = 3 * B * S * H * 128 * 2 * (world - 1) / world
        bound_ms = max(flops / (pk["tflops"] * 1e9), link_bytes / 770e6)
        if rank == 0:
            print(json.dumps({"path": "q/k/v projection + RMSNorm + RoPE + seq->head exchange", "n_gpus": world,
                              "unfused_ms (3 GEMM + 3 scatter kernels + barrier)": round(ms_u, 3),
                              "fused_ms (3 GEMMs with exchange epilogue + barrier)": round(ms_f, 3),
                              "roofline_ms": round(bound_ms, 3), "fused_fraction_of_roofline": round(bound_ms / ms_f, 3),
                              "peaks": pk["src"], "nvlink_GBs_assumed": 770}), flush=True)
        qh, kh, vh = fused_qkv()
        qh, kh, vh = qh.clone(), kh.clone(), vh.clone()
        scale = 1.0 / math.sqrt(128)

        def unfused_attn():
            return t.head_to_seq(F_ops.attention(qh, kh, vh, scale))

        def fused_attn():
            return t.attention_scatter_seq(qh, kh, vh, scale)

        ms_u, ms_f = timed(unfused_attn), timed(fused_attn)
        flops = 4.0 * B * (S * world) ** 2 * 128 * (H // world)
        link_bytes = B * S * H * 128 * 2 * (world - 1) / world
        bound_ms = max(flops / (pk["tflops"] * 1e9), link_bytes / 770e6)
        if rank == 0:
            print(json.dumps({"path": "attention + head->seq exchange", "n_gpus": world,
                              "unfused_ms (attention + stage copy + gather kernel + 2 barriers)": round(ms_u, 3),
                              "fused_ms (attention with exchange store + barrier)": round(ms_f, 3),
                              "roofline_ms": round(bound_ms, 3), "fused_fraction_of_roofline": round(bound_ms / ms_f, 3),
                              "peaks": pk["src"], "nvlink_GBs_assumed": 770}), flush=True)
        ctx.check()
    err = native.load().kernel_error(local, True)
    dist.barrier()
    dist.destroy_process_group()
    return int(err != 0)


if __name__ == "__main__":
    raise SystemExit(main())
