"""Callbacks that draw samples and measure validation loss during training.

Parity targets: ``EveryNDrawSample`` (cosmos_predict2/_src/predict2/callbacks/every_n_draw_sample.py:65-400: every n iterations,
optionally under EMA weights, denoise the current batch from several noise levels with one step ("x0 prediction", with the
mean-squared error per level) and run the full sampler at several guidance scales; tile [guidance rows x batch columns]
plus the ground truth into one grid written as mp4 / jpg), ``ValLossComputation``
(cosmos_predict2/_src/predict2/callbacks/val_loss_computation.py:45-330: loss on a held-out set at fixed noise levels) and
``EveryNDrawSampleMultiviewVideo`` (cosmos_predict2/_src/predict2_multiview/callbacks/every_n_draw_sample_multiviewvideo.py:
views laid out side by side). Outputs go under ``<job dir>/<callback name>/``; metrics go to wandb when a run is active.
"""

from __future__ import annotations

import contextlib
import json
import math
import os
from typing import Dict, Iterable, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from ..utils import log
from ..utils.video_io import save_img_or_video
from .callbacks import EveryN, _rank, _world


def is_primitive(v) -> bool:
    return isinstance(v, (int, float, str, bool, type(None)))


def convert_to_primitive(v):
    if isinstance(v, (list, tuple)):
        return [convert_to_primitive(x) for x in v if is_primitive(x) or isinstance(x, (list, dict))]
    if isinstance(v, dict):
        return {k: convert_to_primitive(x) for k, x in v.items() if is_primitive(x) or isinstance(x, (list, dict))}
    return v if is_primitive(v) else "non-primitive"


def resize_image(image: torch.Tensor, size: int = 1024) -> torch.Tensor:
    """[C,H,W]: shrink so that the longer side is at most ``size``."""
    _, h, w = image.shape
    r = size / max(h, w)
    if r >= 1:
        return image
    return torch.nn.functional.interpolate(image[None], size=(max(1, int(h * r)), max(1, int(w * r))), mode="bilinear",
                                           align_corners=False, antialias=True)[0]


class EveryNDrawSample(EveryN):
    def __init__(self, every_n: int, step_size: int = 1, n_viz_sample: int = 3, n_sample_to_save: int = 128, num_sampling_step: int = 35,
                 guidance: Iterable[float] = (0.0, 3.0, 7.0), do_x0_prediction: bool = True, n_sigmas_for_x0_prediction: int = 4,
                 save_s3: bool = False, is_ema: bool = False, use_negative_prompt: bool = False, fps: int = 16, run_at_start: bool = False):
        super().__init__(every_n, step_size, run_at_start=run_at_start)
        self.n_viz_sample, self.n_sample_to_save = n_viz_sample, n_sample_to_save
        self.num_sampling_step, self.guidance = num_sampling_step, list(guidance)
        self.do_x0_prediction, self.n_sigmas = do_x0_prediction, n_sigmas_for_x0_prediction
        self.save_s3, self.is_ema, self.use_negative_prompt, self.fps = save_s3, is_ema, use_negative_prompt, fps
        self.name = type(self).__name__
        self.local_dir = None
        self.negative_prompt_data: Optional[Dict] = None
        self.data_parallel_id = 0

    def on_train_start(self, model, iteration: int = 0) -> None:
        out = getattr(self.config, "output_dir", None) or "."
        self.local_dir = os.path.join(out, self.name)
        if _rank() == 0:
            os.makedirs(self.local_dir, exist_ok=True)
        cp = getattr(model, "cp_group", None)
        cp_size = dist.get_world_size(cp) if (cp is not None and dist.is_initialized()) else 1
        self.data_parallel_id = _rank() // max(cp_size, 1)
        self._saver_rank = cp is None or dist.get_rank(cp) == 0          # one writer per context-parallel group

    # ---- pieces -------------------------------------------------------------------------------------------------
    def _x0_levels(self, model) -> np.ndarray:
        """Noise levels as rectified-flow times in (0, 1), log-spaced in sigma = t / (1 - t)."""
        lo, hi = math.log(0.02), math.log(80.0)
        s = np.exp(np.linspace(lo, hi, self.n_sigmas + 1)[1:])
        return s / (1 + s)

    @torch.no_grad()
    def x0_pred(self, trainer, model, data_batch, iteration):
        raw, x0, condition = model.get_data_and_condition(dict(data_batch))
        x0, condition, _, _ = model.broadcast_split_for_model_parallelsim(x0, condition, None, None)
        B = x0.shape[0]
        g = torch.Generator(device=x0.device).manual_seed(0)
        eps = torch.randn(x0.shape, generator=g, device=x0.device, dtype=x0.dtype)
        ts = self._x0_levels(model)
        shows, mses = [], []
        for t in ts:
            xt = (1 - t) * x0 + t * eps
            tt = torch.full((B, 1), float(t) * 1000.0, device=x0.device, dtype=torch.float32)
            v = model.denoise(eps, xt.to(**model.tensor_kwargs), tt, condition)
            pred = xt - t * v                               # x0 = x_t - t * v  for  x_t = (1 - t) x0 + t eps,  v = eps - x0
            mse = torch.nn.functional.mse_loss(pred.float(), x0.float())
            if dist.is_initialized() and _world() > 1:
                dist.all_reduce(mse, op=dist.ReduceOp.SUM)
                mse = mse / _world()
            mses.append(float(mse))
            shows.append(self._to_pixels(model, pred))
        shows.append(self._gt_pixels(model, raw, x0))
        path = self.run_save(shows, B, f"{self._tag()}_ReplicateID{self.data_parallel_id:04d}_x0_Iter{iteration:09d}")
        return path, mses, ts

    def _tag(self) -> str:
        return "ema" if self.is_ema else "reg"

    def _to_pixels(self, model, latent):
        cpn = getattr(model, "cp_group", None)
        if cpn is not None and model.net.is_context_parallel_enabled:
            from ..parallel import context_parallel as cpm
            latent = cpm.cat_outputs_cp(latent, 2, cpn)
        if getattr(model, "tokenizer", None) is not None:
            latent = model.decode(latent)
        return latent.float().cpu()

    def _gt_pixels(self, model, raw, x0):
        if raw is not None:
            return raw.float().cpu()
        return self._to_pixels(model, x0)

    @torch.no_grad()
    def sample(self, trainer, model, data_batch, iteration):
        batch = dict(data_batch)
        raw, x0, _ = model.get_data_and_condition(dict(batch))
        if self.use_negative_prompt and self.negative_prompt_data is not None:
            neg = self.negative_prompt_data["t5_text_embeddings"].to(**model.tensor_kwargs)
            batch["neg_t5_text_embeddings"] = neg.expand(x0.shape[0], *neg.shape[-2:]) if neg.ndim == 2 or neg.shape[0] == 1 else neg
        shows = []
        for g in self.guidance:
            s = model.generate_samples_from_batch(dict(batch), guidance=g, state_shape=tuple(x0.shape[1:]), n_sample=x0.shape[0],
                                                  num_steps=self.num_sampling_step, is_negative_prompt=self.use_negative_prompt)
            shows.append(model.decode(s).float().cpu() if getattr(model, "tokenizer", None) is not None else s.float().cpu())
        shows.append(raw.float().cpu() if raw is not None else (model.decode(x0) if getattr(model, "tokenizer", None) is not None else x0).float().cpu())
        return self.run_save(shows, x0.shape[0], f"{self._tag()}_ReplicateID{self.data_parallel_id:04d}_Sample_Iter{iteration:09d}")

    def layout(self, to_show: torch.Tensor) -> torch.Tensor:
        """[n, b, c, t, h, w] -> [c, t, n*h, b*w]."""
        n, b, c, t, h, w = to_show.shape
        return to_show.permute(2, 3, 0, 4, 1, 5).reshape(c, t, n * h, b * w)

    def run_save(self, to_show: List[torch.Tensor], batch_size: int, base: str) -> Optional[str]:
        if not getattr(self, "_saver_rank", True) or self.data_parallel_id >= self.n_sample_to_save:
            return None
        grid = (1.0 + torch.stack([t[: self.n_viz_sample] for t in to_show], 0).clamp(-1, 1)) / 2.0
        grid = self.layout(grid)
        if grid.shape[0] > 3:                     # latent-space samples (no tokenizer): show the first three channels
            grid = grid[:3]
        os.makedirs(self.local_dir, exist_ok=True)
        return save_img_or_video(grid, os.path.join(self.local_dir, base), fps=self.fps)

    # ---- driver -------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def every_n_impl(self, trainer, model, data_batch, output_batch, loss, iteration):
        if self.is_ema and not model.config.ema.enabled:
            return
        ctx = model.ema_scope("every_n_sampling") if self.is_ema else contextlib.nullcontext()
        was_training = model.training
        model.eval()
        info = {"iteration": iteration, "data": {k: convert_to_primitive(v) for k, v in data_batch.items()
                                                 if is_primitive(v) or isinstance(v, (list, dict))}}
        metrics: Dict[str, float] = {}
        with ctx:
            if self.do_x0_prediction:
                path, mses, ts = self.x0_pred(trainer, model, data_batch, iteration)
                info["x0"] = {"path": path, "mse_loss": mses, "t": [float(t) for t in ts]}
                metrics.update({f"x0_pred_mse_{self._tag()}/T{t:0.5f}": m for t, m in zip(ts, mses)})
            info["sample_path"] = self.sample(trainer, model, data_batch, iteration)
        if was_training:
            model.train()
        if _rank() == 0 and self.local_dir:
            with open(os.path.join(self.local_dir, f"{self._tag()}_Info_Iter{iteration:09d}.json"), "w") as f:
                json.dump(info, f, indent=1, default=str)
            try:
                import wandb
                if wandb.run:
                    wandb.log(dict(metrics, **{"trainer/global_step": iteration}), step=iteration)
            except ImportError:
                pass
        self.last_info = info
        if torch.cuda.is_available():
            torch.cuda.empty_cache()


class EveryNDrawSampleMultiviewVideo(EveryNDrawSample):
    """Views are unfolded from the time axis and placed side by side: [c, t, n*h, (b v) * w]."""

    def __init__(self, *args, sample_n_views: int = 7, **kw):
        super().__init__(*args, **kw)
        self.sample_n_views = sample_n_views

    def layout(self, to_show: torch.Tensor) -> torch.Tensor:
        n, b, c, vt, h, w = to_show.shape
        v = self.sample_n_views if vt % self.sample_n_views == 0 else 1
        x = to_show.view(n, b, c, v, vt // v, h, w).permute(2, 4, 0, 5, 1, 3, 6)
        return x.reshape(c, vt // v, n * h, b * v * w)


class ValLossComputation(EveryN):
    """Mean training-objective loss over a validation loader at fixed times, under EMA weights when enabled."""

    def __init__(self, every_n: int, dataloader=None, max_batches: int = 8, times: Iterable[float] = (0.2, 0.5, 0.8), is_ema: bool = False,
                 run_at_start: bool = False):
        super().__init__(every_n, run_at_start=run_at_start)
        self.dataloader, self.max_batches, self.times, self.is_ema = dataloader, max_batches, list(times), is_ema
        self.name = type(self).__name__
        self.history: List[Dict] = []

    @torch.no_grad()
    def every_n_impl(self, trainer, model, data_batch, output_batch, loss, iteration):
        loader = self.dataloader if self.dataloader is not None else [data_batch]
        ctx = model.ema_scope("val_loss") if (self.is_ema and model.config.ema.enabled) else contextlib.nullcontext()
        sums = {t: 0.0 for t in self.times}
        n = 0
        was_training = model.training
        model.eval()
        with ctx:
            for i, batch in enumerate(loader):
                if i >= self.max_batches:
                    break
                batch = trainer.to_device(batch) if trainer is not None else batch
                raw, x0, condition = model.get_data_and_condition(dict(batch))
                g = torch.Generator(device=x0.device).manual_seed(1234 + i)
                eps = torch.randn(x0.shape, generator=g, device=x0.device, dtype=x0.dtype)
                x0s, cond, epss, _ = model.broadcast_split_for_model_parallelsim(x0, condition, eps, None)
                for t in self.times:
                    xt = (1 - t) * x0s + t * epss
                    tt = torch.full((x0s.shape[0], 1), t * 1000.0, device=x0.device, dtype=torch.float32)
                    v = model.denoise(epss, xt.to(**model.tensor_kwargs), tt, cond)
                    sums[t] += float(torch.mean((v.float() - (epss - x0s).float()) ** 2))
                n += 1
        if was_training:
            model.train()
        res = {f"val_loss/t{t:.2f}": s / max(n, 1) for t, s in sums.items()}
        if dist.is_initialized() and _world() > 1:
            vals = torch.tensor(list(res.values()), device=model.device_ if model.device_.type == "cuda" else "cpu")
            dist.all_reduce(vals)
            res = {k: float(v) / _world() for k, v in zip(res, vals)}
        res["val_loss/mean"] = float(np.mean(list(res.values())))
        res["iteration"] = iteration
        self.history.append(res)
        log.info(f"validation loss at iteration {iteration}: {res['val_loss/mean']:.4f}")
        try:
            import wandb
            if wandb.run and _rank() == 0:
                wandb.log(res, step=iteration)
        except ImportError:
            pass
