"""Video2World inference latency: seconds per 720p x 93-frame video, 35 UniPC steps, classifier-free guidance 7 with
batched cond/uncond rows, then the Wan2.1 VAE decode of the latent to 93 RGB frames.

    python bench_inference.py [--steps 35] [--model 2B]                       # one GPU
    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 bench_inference.py --gpus N   # context parallel N

Synthetic inputs (random conditioning video, random text embeddings [1,512,100352]) and random-init weights of the named
architecture. Times are CUDA events on the launching stream, max over ranks; rank 0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _conv_native() -> bool:
    from cosmos_predict25_b200.ops import functional as F_ops
    return F_ops.settings.conv == "native"


def run_inference(*, model_name="2B", frames=24, height=88, width=160, steps=35, guidance=7.0, decode=True, transport="peer",
                  cp_comm="a2a", sparse_window=None, sparse_stride=(1, 4, 8), dense_blocks=0, warmup_steps=2) -> dict:
    """Video2World sampling (+ VAE decode) through ``generate_samples_from_batch`` / ``decode`` on the current process group, the
    whole group being one context-parallel group. Returns the result record (every rank; times are max over ranks)."""
    from types import SimpleNamespace
    args = SimpleNamespace(model=model_name, frames=frames, height=height, width=width, steps=steps, guidance=guidance,
                           no_decode=not decode, transport=transport, cp_comm=cp_comm, sparse_window=sparse_window,
                           sparse_stride=sparse_stride, dense_blocks=dense_blocks)
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    dev = torch.device("cuda", torch.cuda.current_device())
    local_rank = dev.index
    from cosmos_predict25_b200.models.dit import NET_PRESETS
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.models.vae_wan import Wan2pt1VAEInterface
    from cosmos_predict25_b200.ops import native
    from cosmos_predict25_b200.parallel.mesh import build_groups

    groups = build_groups(world, cp_size=world)
    net_cfg = NET_PRESETS[args.model]()
    tok = None if args.no_decode else Wan2pt1VAEInterface(device=dev, dtype=torch.bfloat16)
    cfg = Video2WorldRFConfig(net=net_cfg, precision="bfloat16", state_t=args.frames, tokenizer=tok, cp_comm_type=args.cp_comm)
    torch.manual_seed(1234)
    model = Video2WorldModelRectifiedFlow(cfg, device=dev, cp_group=groups.cp if world > 1 else None)
    model.net.to(torch.bfloat16)
    model.eval()
    if args.sparse_window is not None:
        model.net.use_sparse_attention(args.dense_blocks, {"window_size": tuple(args.sparse_window), "stride": tuple(args.sparse_stride)})
    if world > 1:
        model.net.enable_context_parallel(groups.cp, args.cp_comm)
        if args.transport == "peer":
            from cosmos_predict25_b200.parallel import ulysses
            from cosmos_predict25_b200.parallel.symm import PeerAllToAll, PeerContext
            per_rank = 2 * (args.frames // world + 1) * (args.height // 2) * (args.width // 2) * net_cfg.model_channels
            ctx = PeerContext(groups.cp, dev, arena_bytes=8 * (per_rank * 2 + 4096) + (1 << 20))
            ulysses.attach_peer_transport(groups.cp, PeerAllToAll(ctx, max_elems=per_rank))
    g = torch.Generator().manual_seed(7)
    batch = {"latents": torch.randn(1, 16, args.frames, args.height, args.width, generator=g).to(dev),
             "t5_text_embeddings": torch.randn(1, 512, 100352, generator=g).to(dev, torch.bfloat16),
             "neg_t5_text_embeddings": torch.randn(1, 512, 100352, generator=g).to(dev, torch.bfloat16),
             "fps": torch.tensor([16.0], device=dev), "padding_mask": torch.zeros(1, 1, args.height, args.width, device=dev),
             "num_conditional_frames": 2}

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        out = fn()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms), out

    with torch.no_grad():
        model.generate_samples_from_batch(dict(batch), guidance=args.guidance, seed=0, is_negative_prompt=True,
                                          num_steps=warmup_steps)   # warm-up
        native.reset_launches()
        ms_sample, lat = timed(lambda: model.generate_samples_from_batch(dict(batch), guidance=args.guidance, seed=1,
                                                                         is_negative_prompt=True, num_steps=args.steps))
        launches = native.launches()
        ms_decode, frames = 0.0, None
        ms_encode, encode_frames = None, None
        if tok is not None:
            model.tokenizer = tok
            model.decode(lat[:, :, :2])                                                                                    # warm-up
            ms_decode, video = timed(lambda: model.decode(lat))   # row bands over the CP group; every rank gets the video
            frames = int(video.shape[2])
            if world == 1:
                # the encoder (conditioning clips at inference, every sample of online training): the decoded video back to latents
                clip = video[:, :, : 1 + 4 * (args.frames - 1)].to(torch.bfloat16).clamp(-1, 1)
                tok.encode(clip[:, :, :5])                                                                                  # warm-up
                ms_encode, z = timed(lambda: tok.encode(clip))
                encode_frames = int(clip.shape[2])
    err = native.load().kernel_error(local_rank, True)
    total = (ms_sample + ms_decode) / 1e3
    return {
        "metric": "Video2World inference latency (2B, 720p x 93 frames, device-timed, max over ranks)", "value": total, "unit": "s/video",
        "n_gpus": world, "higher_is_better": False, "dtype": "bf16", "data": "synthetic conditioning video + text embeddings, random-init weights",
        "sampling_s": ms_sample / 1e3, "s_per_denoising_step": ms_sample / 1e3 / args.steps, "vae_decode_s": ms_decode / 1e3,
        "s_per_video_35_steps": 35 * ms_sample / 1e3 / args.steps + ms_decode / 1e3,
        "decoded_frames": frames, "vae_encode_s": None if ms_encode is None else ms_encode / 1e3, "encoded_frames": encode_frames,
        "gpu_launches_sampling": launches, "kernel_error": int(err),
        "config": {"model": f"cosmos-predict2.5-{args.model}-video2world", "steps": args.steps, "guidance": args.guidance,
                   "cfg": "batched cond/uncond (one batch-2 forward per step)", "latent_shape": [1, 16, args.frames, args.height, args.width],
                   "parallelism": f"cp{world}" + (" (ring)" if world > 1 and args.cp_comm == "p2p" else ""),
                   "self_attention": "dense" if args.sparse_window is None else
                   f"neighbourhood window={tuple(args.sparse_window)} stride={tuple(args.sparse_stride)}, {args.dense_blocks} dense blocks", "transport": args.transport if world > 1 else "single",
                   "vae": ("Wan2.1 causal Conv3d decode (" + ("channels-last implicit-GEMM kernel" if _conv_native() else "cuDNN convolutions") + ")"
                           + (f", {world} row bands with halo exchange" if world > 1 else ""))
                   if tok is not None else "skipped"}}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=35)
    ap.add_argument("--model", default="2B", choices=["2B", "14B", "mini"])
    ap.add_argument("--frames", type=int, default=24)
    ap.add_argument("--height", type=int, default=88)
    ap.add_argument("--width", type=int, default=160)
    ap.add_argument("--guidance", type=float, default=7.0)
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--transport", default="peer", choices=["peer", "nccl"])
    ap.add_argument("--cp-comm", default="a2a", choices=["a2a", "p2p"], help="context-parallel exchange: Ulysses all-to-all or ring")
    ap.add_argument("--sparse-window", type=int, nargs=3, default=None, metavar=("T", "H", "W"),
                    help="switch self-attention to neighbourhood attention with this window (e.g. 24 12 24)")
    ap.add_argument("--sparse-stride", type=int, nargs=3, default=(1, 4, 8))
    ap.add_argument("--dense-blocks", type=int, default=0, help="blocks that keep dense self-attention in sparse mode")
    args = ap.parse_args()
    rank, world, local_rank = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    rec = run_inference(model_name=args.model, frames=args.frames, height=args.height, width=args.width, steps=args.steps,
                        guidance=args.guidance, decode=not args.no_decode, transport=args.transport, cp_comm=args.cp_comm,
                        sparse_window=args.sparse_window, sparse_stride=tuple(args.sparse_stride), dense_blocks=args.dense_blocks)
    if rank == 0:
        print(json.dumps(rec))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
