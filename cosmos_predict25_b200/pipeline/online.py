"""Folder-watching text-to-video service and text-to-image inference.

Parity targets: ``FolderMonitor`` / ``OnlineVideo2WorldInference`` (cosmos_predict2/_src/predict2/inference/video2world_online.py:117-400:
poll a prompt folder for new ``*.txt`` files, generate one video per file into ``<result>/<stem>/generated_video.mp4`` with the
prompt and a generation-info file beside it, skip prompts whose video already exists, keep the model resident; under context
parallelism rank 0 watches the folder and broadcasts each job) and ``Text2ImageInference``
(cosmos_predict2/_src/predict2/inference/text2image.py:85-150: a single latent frame sampled with the image data type).
"""

from __future__ import annotations

import argparse
import os
import time
from pathlib import Path
from typing import List, Optional

import torch
import torch.distributed as dist

from ..utils import log
from ..utils.video_io import save_img_or_video
from .video2world import Video2WorldInference

VIDEO_EXTS = (".mp4", ".avi", ".mov", ".mkv")


class FolderMonitor:
    def __init__(self, pipe: Video2WorldInference, prompt_folder: str, result_folder: str, guidance: float = 7.0, num_video_frames: int = 93,
                 resolution: str = "none", seed: int = 0, negative_prompt: Optional[str] = None, num_steps: int = 35,
                 poll_interval: float = 2.0, fps: int = 16):
        self.pipe = pipe
        self.prompt_folder, self.result_folder = Path(prompt_folder), Path(result_folder)
        self.guidance, self.num_video_frames, self.resolution = guidance, num_video_frames, resolution
        self.negative_prompt, self.num_steps, self.poll_interval, self.fps = negative_prompt, num_steps, poll_interval, fps
        self.seed_counter = seed
        self.processed_files = set()
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        if self.rank == 0:
            self.prompt_folder.mkdir(parents=True, exist_ok=True)
            self.result_folder.mkdir(parents=True, exist_ok=True)

    def get_new_prompt_files(self) -> List[Path]:
        cur = {p for p in self.prompt_folder.glob("*.txt") if p.is_file()} if self.prompt_folder.exists() else set()
        return sorted(cur - self.processed_files)

    def existing_video(self, stem: str) -> Optional[Path]:
        for ext in VIDEO_EXTS:
            p = self.result_folder / stem / f"generated_video{ext}"
            if p.exists():
                return p
        return None

    def _broadcast_job(self, job):
        """rank 0 decides; every rank of the context-parallel group must run the same generation."""
        if not dist.is_initialized() or dist.get_world_size() == 1:
            return job
        box = [job]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def process_prompt_file(self, file_path: Optional[Path]) -> Optional[str]:
        job = None
        if self.rank == 0 and file_path is not None:
            prompt = file_path.read_text(encoding="utf-8").strip()
            if not prompt:
                log.warning(f"empty prompt file: {file_path}")
            elif self.existing_video(file_path.stem) is not None:
                log.info(f"video already exists for {file_path.name}; skipping")
            else:
                job = {"prompt": prompt, "stem": file_path.stem, "seed": self.seed_counter, "source": file_path.name}
        job = self._broadcast_job(job)
        if job is None:
            return None
        t0 = time.time()
        video = self.pipe.generate_vid2world(prompt=job["prompt"], input_path=None, guidance=self.guidance,
                                             num_video_frames=self.num_video_frames, num_latent_conditional_frames=0,
                                             resolution=self.resolution, seed=job["seed"], negative_prompt=self.negative_prompt,
                                             num_steps=self.num_steps)
        out = None
        if self.rank == 0:
            folder = self.result_folder / job["stem"]
            folder.mkdir(parents=True, exist_ok=True)
            vid = video[0].float()
            if vid.shape[0] > 3:            # latent-space output (no tokenizer configured): keep three channels for the preview
                vid = vid[:3]
            out = save_img_or_video((1.0 + vid.clamp(-1, 1)) / 2, str(folder / "generated_video"), fps=self.fps)
            (folder / "prompt.txt").write_text(job["prompt"], encoding="utf-8")
            (folder / "generation_info.txt").write_text(
                f"Prompt: {job['prompt']}\nSeed: {job['seed']}\nGuidance: {self.guidance}\nFrames: {self.num_video_frames}\n"
                f"Resolution: {self.resolution}\nGeneration time: {time.time() - t0:.2f} seconds\nSource file: {job['source']}\n"
                f"Context parallel size: {self.pipe.context_parallel_size}\n", encoding="utf-8")
            log.info(f"video saved to {folder}")
        self.seed_counter += 1
        return out

    def run_once(self) -> int:
        files = self.get_new_prompt_files() if self.rank == 0 else []
        n = self._broadcast_job(len(files))
        for i in range(n):
            f = files[i] if self.rank == 0 else None
            self.process_prompt_file(f)
            if f is not None:
                self.processed_files.add(f)
        return n

    def run(self, max_idle_polls: Optional[int] = None):
        """Loop forever (or until ``max_idle_polls`` consecutive empty polls; a file named ``STOP`` in the prompt folder ends it)."""
        idle = 0
        while True:
            stop = self._broadcast_job((self.prompt_folder / "STOP").exists() if self.rank == 0 else None)
            if stop:
                break
            n = self.run_once()
            idle = 0 if n else idle + 1
            if max_idle_polls is not None and idle >= max_idle_polls:
                break
            if n == 0:
                time.sleep(self.poll_interval)


class Text2ImageInference:
    """Single-frame generation with the image data type (the conditioner sees ``images``; no video conditioning)."""

    def __init__(self, experiment_name: str, ckpt_path: Optional[str], s3_credential_path: str = "", pipe: Optional[Video2WorldInference] = None,
                 **pipe_kw):
        self.pipe = pipe or Video2WorldInference(experiment_name, ckpt_path, s3_credential_path, **pipe_kw)
        self.model = self.pipe.model

    @torch.no_grad()
    def generate_image(self, prompt: str, negative_prompt: Optional[str] = None, aspect_ratio: str = "16,9", guidance: float = 7.0,
                       seed: int = 0, num_steps: int = 35, resolution: str = "none") -> torch.Tensor:
        """Returns [1, 3, 1, H, W] in [-1, 1] (or the latent when no tokenizer is configured)."""
        H, W = self.pipe.resolve_resolution(resolution, aspect_ratio)
        dev = self.model.device_
        enc = self.pipe.text_encoder
        batch = {"dataset_name": "image_data", "images": torch.zeros(1, 3, H, W, dtype=torch.uint8, device=dev),
                 "t5_text_embeddings": enc.encode_prompts([prompt]).to(dev, self.model.precision),
                 "fps": torch.full((1,), 1.0, device=dev), "padding_mask": torch.zeros(1, 1, H, W, device=dev), "ai_caption": [prompt]}
        neg = negative_prompt is not None
        if neg:
            batch["neg_t5_text_embeddings"] = enc.encode_prompts([negative_prompt]).to(dev, self.model.precision)
        tok = self.model.tokenizer
        f = tok.spatial_compression_factor if tok is not None else 8
        shape = (self.model.config.state_ch, 1, H // f, W // f)
        lat = self.model.generate_samples_from_batch(batch, guidance=guidance, seed=seed, state_shape=shape, n_sample=1,
                                                     is_negative_prompt=neg, num_steps=num_steps)
        return self.model.decode(lat).float().clamp(-1, 1) if tok is not None else lat


def main(argv=None):
    ap = argparse.ArgumentParser(description="Watch a folder for prompt files and generate a video for each")
    ap.add_argument("--experiment", required=True)
    ap.add_argument("--ckpt_path", default="")
    ap.add_argument("--prompt_folder", default="prompts")
    ap.add_argument("--result_folder", default="results")
    ap.add_argument("--context_parallel_size", type=int, default=1)
    ap.add_argument("--guidance", type=float, default=7.0)
    ap.add_argument("--num_video_frames", type=int, default=93)
    ap.add_argument("--resolution", default="none")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--negative_prompt", default=None)
    ap.add_argument("--num_steps", type=int, default=35)
    a = ap.parse_args(argv)
    if a.context_parallel_size > 1:
        from ..utils import distributed
        distributed.init()
    pipe = Video2WorldInference(a.experiment, a.ckpt_path or None, context_parallel_size=a.context_parallel_size)
    FolderMonitor(pipe, a.prompt_folder, a.result_folder, a.guidance, a.num_video_frames, a.resolution, a.seed, a.negative_prompt,
                  a.num_steps).run()
    pipe.cleanup()


if __name__ == "__main__":
    main()
