"""Multiview datasets: a local one-sample dataset built from per-camera video files, and a synthetic latent dataset.

Parity targets: ``LocalMultiviewDataset`` / ``LocalMultiviewDatasetBuilder`` / ``LocalMultiviewAugmentorConfig``
(cosmos_predict2/_src/predict2_multiview/datasets/local_dataset.py:18-200) and the per-sample keys the multiview model
consumes (``MultiviewInput`` :18-41): the views are concatenated on the time axis in camera order, ``view_indices`` gives
the camera id of every frame, ``sample_n_views`` / ``num_video_frames_per_view`` describe the layout.

The reference decodes through its webdataset augmentor chain; here the same steps (pick a frame window at the target
fps, resize-and-pad to the training resolution, build the padding mask and bookkeeping keys) are ordinary functions
applied in sequence, and an augmentor may be a generator (skip / replicate samples) exactly as there.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

from ..utils import log

VIEW_INDEX_DICT = {"front_wide": 0, "cross_right": 1, "rear_right": 2, "rear": 3, "rear_left": 4, "cross_left": 5, "front_tele": 6}
CAMERA_TO_CAPTION_PREFIX = {
    "front_wide": "The video is captured from a camera mounted on a car. The camera is facing forward.",
    "cross_right": "The video is captured from a camera mounted on a car. The camera is facing to the right.",
    "rear_right": "The video is captured from a camera mounted on a car. The camera is facing the rear right side.",
    "rear": "The video is captured from a camera mounted on a car. The camera is facing backwards.",
    "rear_left": "The video is captured from a camera mounted on a car. The camera is facing the rear left side.",
    "cross_left": "The video is captured from a camera mounted on a car. The camera is facing to the left.",
    "front_tele": "The video is captured from a telephoto camera mounted on a car. The camera is facing forward.",
}
RESOLUTION_HW = {"720p": (720, 1280), "720": (704, 1280), "480p": (480, 832), "480": (432, 768), "tiny": (64, 64)}


@dataclass
class DrivingVideoDataloaderConfig:
    """Which cameras are sampled, in which order, and how many frames per view."""
    camera_keys: Sequence[str] = ("front_wide", "cross_right", "rear_right", "rear", "rear_left", "cross_left", "front_tele")
    n_views: int = 7
    num_video_frames_per_view: int = 29
    ref_cam_view_idx: int = -1
    single_caption_camera_name: str = "front_wide"
    add_view_prefix_to_caption: bool = True


@dataclass
class LocalMultiviewAugmentorConfig:
    resolution: str
    driving_dataloader_config: DrivingVideoDataloaderConfig = field(default_factory=DrivingVideoDataloaderConfig)
    caption_type: str = "t2w_qwen2p5_7b"
    min_fps_thres: int = 10
    max_fps_thres: int = 60
    num_video_frames: int = 121
    use_native_fps: bool = False
    use_original_fps: bool = False
    target_fps: float = 30.0


def wrap_augmentor_func_as_generator(func: Callable, data: Iterable):
    for d in data:
        out = func(d)
        if out is not None:   # None marks an unhealthy sample: skip it
            yield out


def _decode_video_bytes(raw: bytes) -> Tuple[np.ndarray, float]:
    """mp4 bytes -> (uint8 [T,H,W,3], fps)."""
    import os
    import tempfile

    import cv2
    with tempfile.NamedTemporaryFile(suffix=".mp4", delete=False) as f:
        f.write(raw)
        path = f.name
    try:
        cap = cv2.VideoCapture(path)
        fps = cap.get(cv2.CAP_PROP_FPS) or 30.0
        frames = []
        while True:
            ok, fr = cap.read()
            if not ok:
                break
            frames.append(cv2.cvtColor(fr, cv2.COLOR_BGR2RGB))
        cap.release()
    finally:
        os.unlink(path)
    if not frames:
        raise ValueError("no frames decoded")
    return np.stack(frames), float(fps)


def resize_and_pad(frames_T_H_W_C: np.ndarray, size_hw: Tuple[int, int]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Aspect-preserving resize, reflect-free zero padding to ``size_hw``. Returns (uint8 [3,T,H,W], padding mask [1,H,W])."""
    T, h, w, _ = frames_T_H_W_C.shape
    H, W = size_hw
    s = min(H / h, W / w)
    nh, nw = max(1, round(h * s)), max(1, round(w * s))
    x = torch.from_numpy(frames_T_H_W_C).permute(0, 3, 1, 2).float()
    x = torch.nn.functional.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False, antialias=True)
    out = torch.zeros(T, 3, H, W)
    out[:, :, :nh, :nw] = x
    mask = torch.ones(1, H, W)
    mask[:, :nh, :nw] = 0
    return out.round().clamp(0, 255).to(torch.uint8).permute(1, 0, 2, 3).contiguous(), mask


class MultiviewVideoParsing:
    """bytes of ``video_<camera index>`` entries -> the multiview sample dict."""

    def __init__(self, cfg: LocalMultiviewAugmentorConfig, decode: Callable = _decode_video_bytes):
        self.cfg, self.decode = cfg, decode

    def __call__(self, d: Dict[str, Any]) -> Optional[Dict[str, Any]]:
        dl = self.cfg.driving_dataloader_config
        cams = list(dl.camera_keys)[: dl.n_views]
        size = RESOLUTION_HW[str(self.cfg.resolution)]
        n = dl.num_video_frames_per_view
        videos, view_idx, mask, fps_out, n_orig, sel = [], [], None, None, [], []
        for cam in cams:
            key = f"video_{VIEW_INDEX_DICT[cam]}"
            if key not in d:
                log.warning(f"camera {cam} missing from sample {d.get('__key__')}")
                return None
            frames, fps = self.decode(d[key])
            if not (self.cfg.min_fps_thres <= fps <= self.cfg.max_fps_thres):
                return None
            stride = 1 if (self.cfg.use_native_fps or self.cfg.use_original_fps) else max(1, round(fps / self.cfg.target_fps))
            idx = np.arange(n) * stride
            if idx[-1] >= len(frames):
                idx = np.clip(idx, 0, len(frames) - 1)     # short clip: repeat the last frame
            v, m = resize_and_pad(frames[idx], size)
            videos.append(v)
            view_idx.append(torch.full((n,), VIEW_INDEX_DICT[cam], dtype=torch.int64))
            sel.append(torch.from_numpy(idx.astype(np.int64)))
            n_orig.append(torch.tensor(len(frames)))
            mask, fps_out = m, fps / stride
        H, W = size
        ref = dl.ref_cam_view_idx
        return {
            "__key__": d.get("__key__", "local_dataset"), "aspect_ratio": d.get("aspect_ratio", "16,9"),
            "video": torch.cat(videos, dim=1), "view_indices": torch.cat(view_idx), "frame_indices": sel,
            "view_indices_selection": [torch.tensor(VIEW_INDEX_DICT[c]) for c in cams], "camera_keys_selection": cams,
            "sample_n_views": torch.tensor(len(cams)), "num_video_frames_per_view": torch.tensor(n),
            "n_orig_video_frames_per_view": n_orig, "fps": torch.tensor(float(fps_out)), "padding_mask": mask,
            "image_size": torch.tensor([H, W, H, W], dtype=torch.float32), "num_frames": torch.tensor(n * len(cams)),
            "ref_cam_view_idx_sample_position": torch.tensor(cams.index(_cam_of(ref)) if ref >= 0 and _cam_of(ref) in cams else -1),
            "front_cam_view_idx_sample_position": torch.tensor(cams.index("front_wide") if "front_wide" in cams else -1),
            "ai_caption": d.get("ai_caption", ""),
        }


def _cam_of(index: int) -> str:
    for k, v in VIEW_INDEX_DICT.items():
        if v == index:
            return k
    return ""


def multiview_caption(caption: str, cameras: Sequence[str], add_prefix: bool = True) -> str:
    """One caption per view joined by `` -- `` (the separator the model's view sub-sampling splits on)."""
    parts = []
    for cam in cameras:
        parts.append(f"{CAMERA_TO_CAPTION_PREFIX[cam]} {caption}".strip() if add_prefix else caption)
    return " -- ".join(parts)


class LocalMultiviewDataset(Dataset):
    """One sample assembled from ``{camera name: path}``; files are read as bytes and passed through the augmentors."""

    def __init__(self, video_file_dict: Dict[str, str], augmentor_fn: Optional[Callable]):
        self.video_file_dict = {k: str(v) for k, v in video_file_dict.items() if v is not None}
        self.augmentor_fn = augmentor_fn
        self.total_images = len(self.video_file_dict)

    def __len__(self):
        return 1

    def __getitem__(self, idx):
        d: Dict[str, Any] = {"__key__": "local_dataset", "aspect_ratio": "16,9"}
        for view, path in self.video_file_dict.items():
            with open(path, "rb") as f:
                d[f"video_{VIEW_INDEX_DICT[view]}"] = f.read()
        if self.augmentor_fn is None:
            return d
        for sample in self.augmentor_fn([d]):
            return sample
        raise RuntimeError(f"every augmentor rejected the sample built from {self.video_file_dict}")


class LocalMultiviewDatasetBuilder:
    def __init__(self, video_file_dict: Dict[str, str]):
        self.video_file_dict = video_file_dict

    @staticmethod
    def augmentor_fn(data, augmentations: List[Callable]):
        for aug in augmentations:
            data = aug(data) if getattr(aug, "is_generator", False) else wrap_augmentor_func_as_generator(aug, data)
        yield from data

    def build_data_augmentor(self, augmentors: Sequence[Callable]) -> Callable:
        from functools import partial
        return partial(LocalMultiviewDatasetBuilder.augmentor_fn, augmentations=list(augmentors))

    def build_dataset(self, cfg: LocalMultiviewAugmentorConfig, decode: Callable = _decode_video_bytes) -> LocalMultiviewDataset:
        files = {k: v for k, v in self.video_file_dict.items() if v is not None}
        assert len(files) > 0, "Did not find any video files."
        return LocalMultiviewDataset(files, self.build_data_augmentor([MultiviewVideoParsing(cfg, decode)]))


class MockMultiviewLatentDataset(Dataset):
    """Synthetic pre-encoded multiview sample: latents [16, V*T, H, W], one 512-token caption embedding per view."""

    def __init__(self, n_views=7, state_t=8, height=90, width=160, text_dim=100352, text_len=512, length=1 << 30, channels=16, seed=0):
        self.V, self.T, self.shape = n_views, state_t, (channels, n_views * state_t, height, width)
        self.text = (n_views * text_len, text_dim)
        self.length, self.seed = length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 15485863 + int(i))
        return {"latents": torch.randn(self.shape, generator=g),
                "t5_text_embeddings": torch.randn(self.text, generator=g).to(torch.bfloat16), "fps": torch.tensor(10.0),
                "padding_mask": torch.zeros(1, self.shape[2], self.shape[3]),
                "latent_view_indices_B_T": torch.arange(self.V).repeat_interleave(self.T),
                "ref_cam_view_idx_sample_position": torch.tensor(0), "sample_n_views": torch.tensor(self.V),
                "ai_caption": " -- ".join(f"synthetic view {v} of sample {i}" for v in range(self.V)), "dataset_name": "mock_multiview"}
