"""Post-training from data to samples in one resumable script.

``python examples/posttraining/pipeline.py --preset nemo_assets [--max-iters 200] [--stages prompts,train,convert,infer]``

Parity: the reference's end-to-end post-training examples (examples/posttraining/nemo/post_training_nemo_assets.py,
examples/posttraining/groot/post_training_groot.py): prepare the dataset's captions, train the registered post-training
experiment, convert the distributed checkpoint to consolidated ``.pt`` files, run inference with the trained weights, and
remember in ``pipeline_state.json`` which stages are done so that a re-run continues where the last one stopped.
Stages run in-process on one GPU (or CPU for the tiny preset); multi-GPU training is the same command line under
``torchrun`` with ``--stages train``.
"""

import argparse
import json
import os
import sys
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

STAGES = ("prompts", "train", "convert", "infer")


@dataclass
class Preset:
    experiment: str
    dataset_dir: str
    prompt: str
    config: str = "cosmos_predict25_b200/configs/video2world.py"
    overrides: List[str] = field(default_factory=list)
    needs_prompts: bool = True


PRESETS: Dict[str, Preset] = {
    "nemo_assets": Preset("predict2_video2world_training_2b_cosmos_nemo_assets", "datasets/cosmos_nemo_assets",
                          "A video of sks teal robot."),
    "groot": Preset("predict2_video2world_training_2b_groot_gr1_480", "datasets/benchmark_train/gr1",
                    "A robot arm manipulating objects on a table.", needs_prompts=False),
    # offline smoke configuration: synthetic latents, two-block network, runs on a CPU in seconds
    "tiny": Preset("tiny_video2world_cpu", "", "", needs_prompts=False),
}


class PostTrainingPipeline:
    def __init__(self, preset: str, work_dir: str, max_iters: Optional[int] = None, save_iter: Optional[int] = None,
                 prompt: Optional[str] = None, extra_overrides: Optional[List[str]] = None):
        self.preset = PRESETS[preset]
        self.work_dir = Path(work_dir)
        self.work_dir.mkdir(parents=True, exist_ok=True)
        self.max_iters = int(os.environ.get("MAX_ITERS", max_iters or 200))
        self.save_iter = save_iter or self.max_iters
        self.prompt = prompt or self.preset.prompt
        self.extra = list(extra_overrides or [])
        self.state_file = self.work_dir / "pipeline_state.json"
        self.state = json.loads(self.state_file.read_text()) if self.state_file.exists() else {s: False for s in STAGES}
        self.job_dir: Optional[str] = self.state.get("job_dir")

    def _done(self, stage: str, **extra) -> None:
        self.state[stage] = True
        self.state.update(extra)
        self.state_file.write_text(json.dumps(self.state, indent=1))

    # ---- stages --------------------------------------------------------------------------------------------------
    def prompts(self) -> None:
        """One caption file per video (metas/<name>.txt) with the instance prompt."""
        if not self.preset.needs_prompts:
            return self._done("prompts")
        from scripts.create_prompts_for_dataset import main as make_prompts
        make_prompts(["--dataset_path", self.preset.dataset_dir, "--prompt", self.prompt])
        self._done("prompts")

    def _overrides(self) -> List[str]:
        return ["--", f"experiment={self.preset.experiment}", f"trainer.max_iter={self.max_iters}",
                f"checkpoint.save_iter={self.save_iter}", "job.wandb_mode=disabled"] + self.preset.overrides + self.extra

    def train(self) -> None:
        from cosmos_predict25_b200.cli import train as cli
        from cosmos_predict25_b200.utils.config import load_config_module, override
        config = override(load_config_module(self.preset.config).make_config(), self._overrides())
        self.job_dir = config.job_path_local
        cli.launch(config, None)
        self._done("train", job_dir=self.job_dir)

    def convert(self) -> None:
        """Distributed checkpoint of the last iteration -> model.pt / model_ema_fp32.pt / model_ema_bf16.pt."""
        from cosmos_predict25_b200.checkpoint.dcp import convert_distcp_to_pt
        ckpt_root = Path(self.job_dir) / "checkpoints"
        latest = (ckpt_root / "latest_checkpoint.txt").read_text().strip()
        out = self.work_dir / "converted" / latest
        out.mkdir(parents=True, exist_ok=True)
        paths = convert_distcp_to_pt(str(ckpt_root / latest / "model"), str(out))
        self._done("convert", converted={k: str(v) for k, v in paths.items()})

    def infer(self, num_steps: int = 35) -> None:
        """Sample one clip from the trained weights (EMA file when present) and save it under ``<work_dir>/samples``."""
        import torch
        from cosmos_predict25_b200.utils.model_loader import load_model_from_checkpoint
        from cosmos_predict25_b200.utils.video_io import save_img_or_video
        conv = self.state.get("converted", {})
        ckpt = conv.get("ema_bf16") or conv.get("ema_fp32") or conv.get("model")
        model, config = load_model_from_checkpoint(self.preset.experiment, ckpt, config_file=self.preset.config,
                                                   experiment_opts=self.preset.overrides + self.extra)
        from cosmos_predict25_b200.utils.lazy_config import instantiate
        from cosmos_predict25_b200.utils.config import load_config_module, override
        cfg = override(load_config_module(self.preset.config).make_config(), self._overrides())
        batch = next(iter(instantiate(cfg["dataloader_train"])))
        batch = {k: (v.to(model.device_) if isinstance(v, torch.Tensor) else v) for k, v in batch.items()}
        batch.setdefault("num_conditional_frames", 1)
        with torch.no_grad():
            latents = model.generate_samples_from_batch(batch, guidance=0.0, seed=0, num_steps=num_steps)
            video = model.decode(latents) if model.tokenizer is not None else latents[:, :3]
        out = self.work_dir / "samples"
        out.mkdir(exist_ok=True)
        path = save_img_or_video((1.0 + video[0].float().clamp(-1, 1)) / 2, str(out / "sample_0"), fps=16)
        self._done("infer", sample=path)

    def run(self, stages=STAGES, force: bool = False, **infer_kw) -> Dict:
        for s in stages:
            if self.state.get(s) and not force:
                print(f"[{s}] already done, skipping")
                continue
            print(f"[{s}] running")
            getattr(self, s)(**(infer_kw if s == "infer" else {}))
        return self.state


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--preset", default="nemo_assets", choices=sorted(PRESETS))
    ap.add_argument("--work-dir", default="outputs/posttraining")
    ap.add_argument("--max-iters", type=int, default=None)
    ap.add_argument("--save-iter", type=int, default=None)
    ap.add_argument("--prompt", default=None)
    ap.add_argument("--stages", default=",".join(STAGES))
    ap.add_argument("--force", action="store_true", help="re-run stages that are marked done")
    ap.add_argument("--num-steps", type=int, default=35)
    ap.add_argument("overrides", nargs="*", help="extra config overrides (key=value)")
    a = ap.parse_args(argv)
    pipe = PostTrainingPipeline(a.preset, os.path.join(a.work_dir, a.preset), a.max_iters, a.save_iter, a.prompt, a.overrides)
    state = pipe.run([s for s in a.stages.split(",") if s], a.force, num_steps=a.num_steps)
    print(json.dumps(state, indent=1))
    return state


if __name__ == "__main__":
    main()
