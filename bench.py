#!/usr/bin/env python
"""Headline benchmark: 2B Video2World DiT training throughput (latent tokens / s) on N B200s.

One rank per GPU (launch with torch.distributed.run for N > 1). Every rank trains on its own
720p x 93-frame sample (latent [1,16,24,88,160] = 84 480 tokens, text embedding [1,512,100352]):
rectified-flow loss, activation checkpointing that keeps attention outputs, gradients reduced over
the ranks, AdamW with fp32 masters + EMA on parameter shards. Weak scaling: per-GPU work is fixed.

Two timed regions of K steps each, both bracketed by barrier + synchronize and timed with CUDA events
(max over ranks):
  value      inputs already on the device
  e2e.value  through ``Trainer.train_step`` with the step's inputs copied from pinned host memory and the
             loss read back to the host every step
After them, in the same process and on the same model object:
  library_twin  3 warm-up + 3 timed steps with every contraction switched to the libraries the reference selects on this
                GPU (cuDNN SDPA, cuBLAS GEMMs); ``vs_baseline`` is value / twin value (the reference publishes no number)
  inference     the other half of the headline metric: Video2World sampling through ``generate_samples_from_batch`` with all
                N ranks as one context-parallel group (a few UniPC steps, classifier-free guidance 7, batched) + the full VAE
                decode; reports seconds per denoising step, decode seconds and the 35-step seconds per video they imply
`python bench.py --impl reference` reports why the unmodified reference cannot run offline.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="train", choices=["train", "distill"],
                    help="train: rectified-flow training step (the headline); distill: sCM / rCM consistency-distillation step "
                         "(teacher forward, student forward-mode JVP on the JVP attention kernel, student forward + backward, optimizer)")
    ap.add_argument("--model", default="2B", choices=["2B", "14B", "mini", "tiny"])
    ap.add_argument("--frames", type=int, default=24, help="latent frames per sample")
    ap.add_argument("--height", type=int, default=88)
    ap.add_argument("--width", type=int, default=160)
    ap.add_argument("--cp", type=int, default=1, help="context-parallel size (Ulysses)")
    ap.add_argument("--transport", default=os.environ.get("COSMOS_B200_TRANSPORT", "peer"), choices=["peer", "nccl", "peer_reshard"])
    ap.add_argument("--attention", default=None, choices=[None, "native", "cudnn"])
    ap.add_argument("--gemm", default=None, choices=[None, "native", "cublas"])
    ap.add_argument("--checkpoint", default="save_attention")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-twin", action="store_true", help="skip the cuDNN + cuBLAS twin of the training step")
    ap.add_argument("--no-inference", action="store_true", help="skip the Video2World sampling + decode block")
    ap.add_argument("--inference-steps", type=int, default=3, help="UniPC steps timed in the inference block")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.index)], stdout=subprocess.PIPE, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        sm, smax, reasons = [], [], set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                smax.append(float(p[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """The unmodified reference cannot be installed offline: its build backend (hatchling) is not in the
    wheelhouse and its runtime needs transformer_engine, megatron-core, hydra-core and omegaconf."""
    ref_dir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "baseline", "_ref", "cosmos_predict2")
    why = ("pip install of the reference fails offline: build backend 'hatchling' is not in /opt/wheelhouse, and its "
           "imports need transformer_engine, megatron-core, hydra-core, omegaconf, which are not installed")
    if os.path.isdir(ref_dir):
        why = "baseline/_ref exists but its dependencies (transformer_engine, megatron-core, hydra-core, omegaconf) are missing"
    print(json.dumps({"impl": "reference", "unavailable": why}))


def main():
    args = parse()
    if args.impl == "reference":
        reference_arm(args)
        return 0

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    from cosmos_predict25_b200.models.dit import NET_PRESETS
    from cosmos_predict25_b200.models.rectified_flow import Video2WorldModelRectifiedFlow, Video2WorldRFConfig
    from cosmos_predict25_b200.ops import functional as F_ops
    from cosmos_predict25_b200.ops import native
    from cosmos_predict25_b200.parallel.mesh import build_groups
    from cosmos_predict25_b200.trainer.optim import OptimizerConfig, SchedulerConfig
    from cosmos_predict25_b200.trainer.trainer import Trainer, TrainerConfig

    if args.attention:
        F_ops.settings.attention = args.attention
    if args.gemm:
        F_ops.settings.gemm = args.gemm

    groups = build_groups(world, cp_size=args.cp)
    ctx_dim = 256 if args.model == "tiny" else 100352
    net_cfg = NET_PRESETS[args.model](checkpoint_mode=args.checkpoint)
    model_kw = dict(net=net_cfg, precision="bfloat16", state_t=args.frames, conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25},
                    sharding_transport=args.transport if world > 1 else "nccl")
    torch.manual_seed(1234 + rank)
    if args.mode == "distill":
        from cosmos_predict25_b200.models.distill import ConsistencyDistillModel, DistillConfig
        model = ConsistencyDistillModel(DistillConfig(**model_kw), device=dev, fsdp_group=groups.fsdp, cp_group=groups.cp)
    else:
        model = Video2WorldModelRectifiedFlow(Video2WorldRFConfig(**model_kw), device=dev, fsdp_group=groups.fsdp, cp_group=groups.cp)
    model.train()
    if args.cp > 1 and args.transport == "peer":
        from cosmos_predict25_b200.parallel import ulysses
        from cosmos_predict25_b200.parallel.symm import PeerAllToAll, PeerContext
        per_rank = (args.frames // args.cp) * (args.height // 2) * (args.width // 2) * net_cfg.model_channels
        ctx = PeerContext(groups.cp, dev, arena_bytes=8 * (per_rank * 2 + 4096) + (1 << 20))
        ulysses.attach_peer_transport(groups.cp, PeerAllToAll(ctx, max_elems=per_rank))
    out_dir = os.path.join("/tmp", f"cosmos_b200_bench_{os.getpid()}")
    trainer = Trainer(TrainerConfig(max_iter=10 ** 9, output_dir=out_dir), model,
                      OptimizerConfig(lr=2 ** -14.5, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-3, max_grad_norm=1.0),
                      SchedulerConfig(kind="lambdalinear", warm_up_steps=(2000,), cycle_lengths=(10 ** 8,), f_start=(1e-6,),
                                      f_max=(1.0,), f_min=(1.0,)))

    g = torch.Generator().manual_seed(99 + rank)
    host = {
        "latents": torch.randn(1, 16, args.frames, args.height, args.width, generator=g).pin_memory(),
        "t5_text_embeddings": torch.randn(1, 512, ctx_dim, generator=g).to(torch.bfloat16).pin_memory(),
        "fps": torch.tensor([16.0]).pin_memory(),
        "padding_mask": torch.zeros(1, 1, args.height, args.width).pin_memory(),
    }
    h2d_bytes = sum(t.numel() * t.element_size() for t in host.values())
    tokens_per_sample = args.frames * (args.height // 2) * (args.width // 2)
    dp = world // args.cp
    global_batch = dp

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n, fn):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    device_batch = {k: v.to(dev) for k, v in host.items()}
    losses = []

    def step_device():
        losses.append(trainer.train_step(dict(device_batch), return_loss_tensor=True))

    def step_e2e():
        losses.append(trainer.train_step(dict(host)))  # H2D from pinned memory + D2H read of the loss

    for _ in range(max(args.warmup, 3)):
        step_device()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    native.reset_launches()
    ms = timed(args.steps, step_device)
    launches = native.launches()
    e2e_ms = None
    if not args.no_e2e:
        step_e2e()
        e2e_ms = timed(args.steps, step_e2e)
    clocks = sampler.stop() if rank == 0 else None
    err = native.load().kernel_error(local_rank, True)
    last_loss = float(losses[-1]) if losses else float("nan")

    resident_bytes = int(model.engine.resident_parameter_bytes()) if hasattr(model.engine, "resident_parameter_bytes") else \
        int(sum(u.full_numel for u in model.engine.units) * 2)

    # ---- library twin: the same model, optimizer and data with cuDNN attention and cuBLAS GEMMs (the reference's choice on sm_100)
    twin = None
    if args.mode == "train" and not args.no_twin and args.attention is None and args.gemm is None and args.model in ("2B", "14B"):
        saved = (F_ops.settings.attention, F_ops.settings.gemm)
        F_ops.settings.attention, F_ops.settings.gemm = "cudnn", "cublas"
        try:
            for _ in range(3):
                step_device()
            twin_ms = timed(3, step_device)
            twin = {"tokens_s": global_batch * tokens_per_sample * 3 / (twin_ms / 1e3), "ms_per_step": twin_ms / 3, "steps": 3,
                    "warmup": 3, "attention": "cudnn sdpa", "gemm": "cublas", "same_process": True}
        finally:
            F_ops.settings.attention, F_ops.settings.gemm = saved

    # ---- inference half of the metric: all ranks form one context-parallel group
    inference = None
    if args.mode == "train" and not args.no_inference and args.model == "2B" and args.cp == 1 and args.frames % world == 0:
        del trainer, model, device_batch
        losses.clear()
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        from bench_inference import run_inference
        rec = run_inference(model_name=args.model, frames=args.frames, height=args.height, width=args.width,
                            steps=args.inference_steps, transport="peer" if args.transport.startswith("peer") else args.transport)
        inference = {k: rec[k] for k in ("s_per_denoising_step", "vae_decode_s", "s_per_video_35_steps", "decoded_frames",
                                         "gpu_launches_sampling", "kernel_error")}
        inference.update(unit="s", timed_unipc_steps=args.inference_steps, guidance=7.0, parallelism=rec["config"]["parallelism"],
                         transport=rec["config"]["transport"], vae=rec["config"]["vae"])

    if rank == 0:
        tok = global_batch * tokens_per_sample * args.steps
        value = tok / (ms / 1e3)
        line = {
            "metric": (f"DiT training latent-tokens/s ({args.model} Video2World, 720p x 93 frames, device-timed, max over ranks)"
                       if args.mode == "train" else
                       f"sCM / rCM distillation step latent-tokens/s ({args.model} Video2World student and teacher, 720p x 93 frames, "
                       "teacher forward + student forward-mode JVP + student forward / backward + optimizer, device-timed, max over ranks)"),
            "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": (value / twin["tokens_s"]) if twin else None,
            "dtype": "bf16", "data": "synthetic latents + text embeddings, random-init weights", "impl": "ours",
            "config": {"model": f"cosmos-predict2.5-{args.model}-video2world", "global_batch": global_batch,
                       "seq_len": tokens_per_sample, "parallelism": (f"fsdp{world}" if args.cp == 1 else f"fsdp{world} (masters, moments, EMA, gradients sharded over all ranks) x cp{args.cp} x dp{dp}"),
                       "latent_shape": [1, 16, args.frames, args.height, args.width], "text_context": [1, 512, ctx_dim],
                       "activation_checkpointing": args.checkpoint, "optimizer": "AdamW fp32 masters + EMA",
                       "transport": args.transport if world > 1 else "single", "attention": F_ops.settings.attention,
                       "attention_bwd": F_ops.settings.attention_bwd if hasattr(native.load(), "fa_bwd") else "cudnn-recompute",
                       "gemm": F_ops.settings.gemm,
                       "l2": "per-step working set (>10 GB of activations) exceeds the 126 MB L2; no explicit flush"},
            "clocks": clocks, "gpu_launches": launches, "kernel_error": int(err), "final_loss": last_loss,
            "resident_parameter_bytes": resident_bytes, "max_memory_allocated_bytes": int(torch.cuda.max_memory_allocated(dev)),
        }
        if twin:
            line["library_twin"] = twin
        if inference:
            line["inference"] = inference
        if e2e_ms is not None:
            line["e2e"] = {"value": tok / (e2e_ms / 1e3), "unit": "tokens/s", "ms_per_step": e2e_ms / args.steps,
                           "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4}
        print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
