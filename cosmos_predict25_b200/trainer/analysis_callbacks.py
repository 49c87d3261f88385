"""Per-frame analysis of the training loss against the noise level.

Parity targets: ``SigmaLossAnalysisPerFrame`` / ``DummySigmaLossAnalysisPerFrame``
(cosmos_predict2/_src/predict2_multiview/callbacks/sigma_loss_analysis_per_frame.py:32-338) and ``DummyFrameLossLog``
(cosmos_predict2/_src/predict2_multiview/callbacks/frame_loss_log.py:26-43). The two ``Dummy*`` classes take the arguments of the
real callbacks and do nothing: multi-camera runs with view dropout swap them in, because their batches do not all have the
same number of frames.

Every training step the callback keeps the step's ``sigma`` ``[B, T]`` (or ``[B, 1]``) and ``edm_loss_per_frame`` ``[B, T]`` on the
host in bf16, separately for image and video batches. Every ``logging_iter * logging_iter_multipler`` iterations the ranks' caches
are gathered (padded to the longest one), rank 0 computes per-frame statistics (log-sigma mean / std, loss mean / std / min / max /
median / quartiles), appends them to ``<output_dir>/sigma_loss_analysis.jsonl``, logs them to wandb when a run is active and, on
the coarser ``logging_viz_iter_multipler`` cadence, adds a table of the mean loss inside ten noise-level bins whose edges are the
deciles of exp(N(0, 1)) (the figure of the reference, as numbers). With ``save_dir`` set the gathered arrays are written there
with easy_io (any backend it knows, object stores included).
"""

from __future__ import annotations

import json
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..utils import log
from .callbacks import Callback, _rank, _world


class DummyFrameLossLog(Callback):
    def __init__(self, logging_iter_multipler: int = 1, save_logging_iter_multipler: int = 1, save_s3: bool = False) -> None:
        pass


class DummySigmaLossAnalysisPerFrame(Callback):
    def __init__(self, logging_iter_multipler: int = 1, logging_viz_iter_multipler: int = 1, save_s3: bool = False) -> None:
        pass


def normal_quantile_bins() -> torch.Tensor:
    """Eleven edges of ten bins: the deciles of exp(N(0, 1)); the two infinite ends are replaced by a geometric extrapolation of
    their neighbours."""
    pts = torch.exp(torch.special.ndtri(torch.linspace(0.0, 1.0, 11)))
    pts[0] = pts[1] / (pts[2] / pts[1])
    pts[-1] = pts[-2] * (pts[-2] / pts[-3])
    return pts


class _SigmaLossCache:
    def __init__(self):
        self.reset()

    def reset(self):
        self.sigma_list: List[torch.Tensor] = []
        self.loss_list: List[torch.Tensor] = []

    def add(self, sigma: torch.Tensor, loss: torch.Tensor):
        self.sigma_list.append(sigma.detach().to("cpu", torch.bfloat16).reshape(sigma.shape[0], -1))
        self.loss_list.append(loss.detach().to("cpu", torch.bfloat16).reshape(loss.shape[0], -1))

    def get_arrays(self) -> Tuple[torch.Tensor, torch.Tensor, Optional[int]]:
        if not self.sigma_list:
            empty = torch.zeros(0, dtype=torch.bfloat16)
            return empty, empty, None
        sigma, loss = torch.cat(self.sigma_list, 0), torch.cat(self.loss_list, 0)
        if sigma.shape[-1] == 1 and loss.shape[-1] > 1:
            sigma = sigma.expand(-1, loss.shape[-1])
        assert sigma.shape == loss.shape, (sigma.shape, loss.shape)
        return sigma, loss, loss.shape[-1]


def frame_stats(sigma: torch.Tensor, loss: torch.Tensor) -> Dict[str, float]:
    sigma, loss = sigma.float(), loss.float()
    std = lambda x: float(x.std()) if x.numel() > 1 else 0.0
    return {"sigma_log_mean": float(sigma.log().mean()), "sigma_log_std": std(sigma.log()), "loss_mean": float(loss.mean()),
            "loss_std": std(loss), "loss_min": float(loss.min()), "loss_max": float(loss.max()), "loss_median": float(loss.median()),
            "loss_q1": float(torch.quantile(loss, 0.25)), "loss_q3": float(torch.quantile(loss, 0.75))}


def binned_loss(sigma: torch.Tensor, loss: torch.Tensor) -> List[Dict[str, float]]:
    """Mean loss and count inside each noise-level bin (empty bins are left out)."""
    edges = normal_quantile_bins()
    idx = torch.bucketize(sigma.float().contiguous(), edges) - 1
    rows = []
    for b in range(len(edges) - 1):
        pick = idx == b
        if pick.any():
            rows.append({"sigma_lo": float(edges[b]), "sigma_hi": float(edges[b + 1]), "count": int(pick.sum()),
                         "loss_mean": float(loss.float()[pick].mean())})
    return rows


class SigmaLossAnalysisPerFrame(Callback):
    def __init__(self, logging_iter_multipler: int = 1, logging_viz_iter_multipler: int = 1, save_s3: bool = False,
                 save_dir: Optional[str] = None) -> None:
        assert logging_viz_iter_multipler % logging_iter_multipler == 0
        self.logging_iter_multipler = logging_iter_multipler
        self.logging_viz_iter_multipler = logging_viz_iter_multipler
        self.save_s3, self.save_dir = save_s3, save_dir
        self.name = type(self).__name__
        self.image_cache, self.video_cache = _SigmaLossCache(), _SigmaLossCache()

    # ---- gather -----------------------------------------------------------------------------------------------------------
    @staticmethod
    def _gather(sigma: torch.Tensor, loss: torch.Tensor, n_frames: Optional[int]) -> Tuple[torch.Tensor, torch.Tensor, Optional[int]]:
        """All ranks' rows on every rank. Ranks may hold different numbers of rows (and a rank may hold none)."""
        world = _world()
        if world == 1:
            return sigma, loss, n_frames
        dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
        meta = torch.tensor([sigma.shape[0], n_frames or 0], dtype=torch.long, device=dev)
        metas = [torch.zeros_like(meta) for _ in range(world)]
        dist.all_gather(metas, meta)
        sizes = [int(m[0]) for m in metas]
        T = max(int(m[1]) for m in metas)
        if max(sizes) == 0:
            return sigma, loss, n_frames
        pad = torch.zeros(2, max(sizes), T, dtype=torch.bfloat16, device=dev)
        if sigma.shape[0]:
            pad[0, : sigma.shape[0]], pad[1, : loss.shape[0]] = sigma.to(dev), loss.to(dev)
        gathered = [torch.zeros_like(pad) for _ in range(world)]
        dist.all_gather(gathered, pad)
        rows = torch.cat([g[:, :n] for g, n in zip(gathered, sizes) if n], dim=1).cpu()
        return rows[0], rows[1], T

    def _gather_and_save(self, cache: _SigmaLossCache, iteration: int, prefix: str, log_viz: bool = True) -> Dict:
        sigma, loss, T = self._gather(*cache.get_arrays())
        cache.reset()
        info: Dict = {}
        if _rank() != 0 or sigma.shape[0] == 0:
            return info
        info[f"{prefix}/total_samples"] = int(sigma.shape[0])
        if T and T > 1:
            for t in range(T):
                info.update({f"{prefix}/frame_{t}/{k}": v for k, v in frame_stats(sigma[:, t], loss[:, t]).items()})
                if log_viz:
                    info[f"{prefix}/frame_{t}/loss_by_sigma_bin"] = binned_loss(sigma[:, t], loss[:, t])
        else:
            info.update({f"{prefix}/{k}": v for k, v in frame_stats(sigma.reshape(-1), loss.reshape(-1)).items()})
            if log_viz:
                info[f"{prefix}/loss_by_sigma_bin"] = binned_loss(sigma.reshape(-1), loss.reshape(-1))
        if self.save_s3 or self.save_dir:
            from ..utils.easy_io import easy_io
            root = self.save_dir or os.path.join(self.config.output_dir if self.config else ".", self.name)
            easy_io.dump({"sigma": sigma, "loss": loss, "stats": info}, f"{root.rstrip('/')}/{prefix}_Iter{iteration:09d}.pkl")
        return info

    # ---- hook -------------------------------------------------------------------------------------------------------------
    def on_training_step_end(self, model, data, output, loss, iteration: int = 0):
        if "edm_loss_per_frame" not in output:
            return
        cache = self.image_cache if model.is_image_batch(data) else self.video_cache
        cache.add(output["sigma"], output["edm_loss_per_frame"])
        every = (self.config.trainer.logging_iter if self.config else 1)
        if iteration % (every * self.logging_iter_multipler):
            return
        log_viz = iteration % (every * self.logging_viz_iter_multipler) == 0
        info: Dict = {}
        # every rank takes part in the gathers of both caches: whether a cache is empty differs between ranks
        for cache, prefix in ((self.image_cache, "sigma_loss_image"), (self.video_cache, "sigma_loss_video")):
            info.update(self._gather_and_save(cache, iteration, prefix, log_viz))
        if _rank() == 0 and info:
            out_dir = self.config.output_dir if self.config else "."
            os.makedirs(out_dir, exist_ok=True)
            with open(os.path.join(out_dir, "sigma_loss_analysis.jsonl"), "a") as f:
                f.write(json.dumps({"iteration": iteration, **info}) + "\n")
            try:
                import wandb
                if wandb.run:
                    wandb.log({k: v for k, v in info.items() if not isinstance(v, list)}, step=iteration)
            except Exception as e:       # not installed / offline: the JSONL record is the sink
                log.debug(f"wandb not used for the sigma-loss analysis: {e}")
