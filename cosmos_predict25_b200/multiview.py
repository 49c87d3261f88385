"""Public multiview entry point (parity: cosmos_predict2/multiview.py ``MultiviewInference``)."""

from __future__ import annotations

import os

import torch

from .data.multiview_dataset import (DrivingVideoDataloaderConfig, LocalMultiviewAugmentorConfig, LocalMultiviewDatasetBuilder,
                                     multiview_caption)
from .models.multiview import NUM_CONDITIONAL_FRAMES_KEY
from .multiview_config import MultiviewInferenceArguments, MultiviewSetupArguments
from .pipeline.multiview import Vid2VidInference
from .utils import log
from .utils.lazy_config import LazyConfig
from .utils.video_io import save_img_or_video

# frames per view the registered driving checkpoints were trained with, per resolution key
FRAMES_PER_VIEW = {"720p": 29, "480p": 61, "720": 93, "480": 93}


class MultiviewInference:
    def __init__(self, args: MultiviewSetupArguments, pipe: Vid2VidInference | None = None):
        self.experiment_name = args.experiment
        self.checkpoint_path = args.checkpoint_path
        self.context_parallel_size = args.context_parallel_size
        self.output_dir = str(args.output_dir)
        self.pipe = pipe

    def generate(self, inference_args: MultiviewInferenceArguments, decode_fn=None):
        torch.backends.cudnn.benchmark = False
        torch.backends.cudnn.deterministic = True
        torch.set_grad_enabled(False)
        pipe = self.pipe or Vid2VidInference(self.experiment_name, self.checkpoint_path, context_parallel_size=self.context_parallel_size)
        rank0 = (not torch.distributed.is_initialized()) or torch.distributed.get_rank() == 0
        if rank0:
            os.makedirs(self.output_dir, exist_ok=True)
            if pipe.config is not None:
                LazyConfig.save_yaml(pipe.config, os.path.join(self.output_dir, "config.yaml"))
        res = str(pipe.model.config.resolution)
        tok = pipe.model.tokenizer
        fpv = tok.get_pixel_num_frames(pipe.model.state_t) if tok is not None else FRAMES_PER_VIEW.get(res, 29)
        dl_cfg = DrivingVideoDataloaderConfig(n_views=inference_args.n_views, num_video_frames_per_view=fpv)
        aug = LocalMultiviewAugmentorConfig(resolution=res, driving_dataloader_config=dl_cfg, target_fps=float(inference_args.fps))
        builder = LocalMultiviewDatasetBuilder(inference_args.input_paths)
        dataset = builder.build_dataset(aug) if decode_fn is None else builder.build_dataset(aug, decode_fn)
        loader = torch.utils.data.DataLoader(dataset, batch_size=1, shuffle=False, num_workers=0)
        outputs = []
        for i, batch in enumerate(loader):
            cams = [c[0] if isinstance(c, (list, tuple)) else c for c in batch["camera_keys_selection"]]
            batch["ai_caption"] = [multiview_caption(inference_args.prompt or "", cams, dl_cfg.add_view_prefix_to_caption)]
            batch[NUM_CONDITIONAL_FRAMES_KEY] = inference_args.num_input_frames
            video = pipe.generate_from_batch(batch, guidance=inference_args.guidance, seed=inference_args.seed,
                                             stack_mode=inference_args.stack_mode, num_steps=inference_args.num_steps)
            if rank0:
                out = f"{self.output_dir}/output_{i}"
                outputs.append(save_img_or_video((1.0 + video[0].float().clamp(-1, 1)) / 2, out, fps=inference_args.fps))
                log.info(f"Saved video to {outputs[-1]}")
        pipe.cleanup()
        return outputs
