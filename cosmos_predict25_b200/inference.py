"""``Inference(setup_args).generate(inference_args, output_dir)``: the public generation API
(parity: cosmos_predict2/inference.py:29-120): model + optional guardrails on rank 0, one video per sample saved as
``<output_dir>/<sample>.mp4`` at 16 fps."""

from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

from .config import InferenceArguments, SetupArguments
from .guardrail import presets as guardrail_presets
from .pipeline.video2world import Video2WorldInference
from .utils import distributed, log
from .utils.lazy_config import LazyConfig
from .utils.video_io import save_img_or_video


class Inference:
    def __init__(self, args: SetupArguments, pipe: Video2WorldInference = None, **pipe_kwargs):
        torch.set_grad_enabled(False)
        self.rank0 = distributed.is_rank0()
        self.setup_args = args
        self.pipe = pipe or Video2WorldInference(experiment_name=args.experiment, ckpt_path=args.checkpoint_path, s3_credential_path="",
                                                 context_parallel_size=args.context_parallel_size, **pipe_kwargs)
        if self.rank0:
            args.output_dir.mkdir(parents=True, exist_ok=True)
            if self.pipe.config is not None:
                LazyConfig.save_yaml(self.pipe.config, str(args.output_dir / "config.yaml"))
        self.text_guardrail_runner = self.video_guardrail_runner = None
        if self.rank0 and args.enable_guardrails:
            self.text_guardrail_runner = guardrail_presets.create_text_guardrail_runner(offload_model_to_cpu=args.offload_guardrail_models)
            self.video_guardrail_runner = guardrail_presets.create_video_guardrail_runner(offload_model_to_cpu=args.offload_guardrail_models)

    def generate(self, args: InferenceArguments, output_dir: Path):
        output_dir = Path(output_dir)
        if self.rank0:
            log.info(f"Running {args.inference_type} generation")
            output_dir.mkdir(parents=True, exist_ok=True)
        paths = []
        for i, (name, sample) in enumerate(args.samples.items()):
            if self.rank0:
                log.info(f"[{i + 1}/{len(args.samples)}] Processing sample {name}")
                if self.text_guardrail_runner is not None:
                    if not guardrail_presets.run_text_guardrail(sample.prompt, self.text_guardrail_runner):
                        log.critical(f"Guardrail blocked generation. Prompt: {sample.prompt}")
                        sys.exit(1)
                else:
                    log.warning("Guardrail checks on prompt are disabled")
            video = self.pipe.generate_vid2world(prompt=sample.prompt, input_path=str(sample.input_path) if sample.input_path else "",
                                                 guidance=args.guidance, num_video_frames=args.num_output_frames,
                                                 num_latent_conditional_frames=args.num_input_frames, resolution=args.resolution,
                                                 seed=args.seed, negative_prompt=args.negative_prompt)
            if self.rank0:
                video = (1.0 + video[0].float()) / 2
                if self.video_guardrail_runner is not None:
                    frames = (video * 255.0).clamp(0, 255).to(torch.uint8).permute(1, 2, 3, 0).cpu().numpy().astype(np.uint8)
                    processed = guardrail_presets.run_video_guardrail(frames, self.video_guardrail_runner)
                    if processed is None:
                        log.critical("Guardrail blocked video generation.")
                        sys.exit(1)
                    video = torch.from_numpy(processed).float().permute(3, 0, 1, 2) / 255.0
                else:
                    log.warning("Guardrail checks on video are disabled")
                p = save_img_or_video(video, str(output_dir / name), fps=16)
                paths.append(p)
                log.info(f"Saved video for {name} to {p}")
        distributed.barrier()
        return paths

    def cleanup(self):
        self.pipe.cleanup()
