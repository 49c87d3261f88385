"""Local folder video dataset for post-training: ``<root>/videos/*.mp4`` with captions in ``<root>/metas/*.txt``
(and optional pre-computed text embeddings in ``<root>/t5_xxl/*.pickle`` or ``<root>/embeddings/*.pt``).

Parity target: ``VideoDataset`` (cosmos_predict2/_src/predict2/datasets/local_datasets/dataset_video.py:34-183): a random
contiguous window of ``num_frames`` frames, resize to ``video_size`` WITHOUT preserving aspect, uint8 [3,T,H,W]; on
a decode failure another random sample is drawn (bounded retries). Decoding uses OpenCV.
"""

from __future__ import annotations

import os
import pickle
import random
import traceback
from typing import Any, Dict, Optional, Tuple

import numpy as np
import torch
from torch.utils.data import Dataset

from ..utils import log


class VideoDataset(Dataset):
    def __init__(self, dataset_dir: str, num_frames: int = 93, video_size: Tuple[int, int] = (704, 1280), caption_dir: str = "metas",
                 video_dir: str = "videos", embedding_dir: Optional[str] = None, max_retries: int = 10, text_len: int = 512):
        self.dataset_dir = dataset_dir
        self.num_frames = num_frames
        self.video_size = tuple(video_size)
        self.caption_dir = os.path.join(dataset_dir, caption_dir)
        self.video_dir = os.path.join(dataset_dir, video_dir)
        self.embedding_dir = os.path.join(dataset_dir, embedding_dir) if embedding_dir else None
        self.max_retries = max_retries
        self.text_len = text_len
        self.video_paths = sorted(os.path.join(self.video_dir, f) for f in os.listdir(self.video_dir) if f.endswith(".mp4")) \
            if os.path.isdir(self.video_dir) else []
        log.info(f"{len(self.video_paths)} videos in {self.video_dir}")

    def __len__(self):
        return len(self.video_paths)

    def _load_video(self, path: str):
        import cv2
        cap = cv2.VideoCapture(path)
        total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
        fps = cap.get(cv2.CAP_PROP_FPS) or 24.0
        if total < self.num_frames:
            cap.release()
            raise ValueError(f"video {path} has only {total} frames, at least {self.num_frames} are required")
        start = random.randint(0, total - self.num_frames)
        cap.set(cv2.CAP_PROP_POS_FRAMES, start)
        H, W = self.video_size
        frames = []
        for _ in range(self.num_frames):
            ok, f = cap.read()
            if not ok:
                break
            f = cv2.cvtColor(f, cv2.COLOR_BGR2RGB)
            frames.append(cv2.resize(f, (W, H), interpolation=cv2.INTER_AREA))
        cap.release()
        if len(frames) != self.num_frames:
            raise ValueError(f"decoded {len(frames)} of {self.num_frames} frames from {path}")
        return np.stack(frames), float(fps), list(range(start, start + self.num_frames))

    def _caption(self, video_path: str) -> str:
        stem = os.path.splitext(os.path.basename(video_path))[0]
        p = os.path.join(self.caption_dir, stem + ".txt")
        return open(p).read().strip() if os.path.exists(p) else ""

    def _embedding(self, video_path: str) -> Optional[torch.Tensor]:
        if self.embedding_dir is None:
            return None
        stem = os.path.splitext(os.path.basename(video_path))[0]
        for ext in (".pt", ".pickle", ".pkl"):
            p = os.path.join(self.embedding_dir, stem + ext)
            if os.path.exists(p):
                e = torch.load(p, map_location="cpu") if ext == ".pt" else pickle.load(open(p, "rb"))
                e = torch.as_tensor(np.asarray(e[0] if isinstance(e, (list, tuple)) else e))
                out = torch.zeros(self.text_len, e.shape[-1], dtype=e.dtype)
                n = min(self.text_len, e.shape[0])
                out[:n] = e[:n]
                return out
        return None

    def __getitem__(self, index) -> Dict[str, Any]:
        for attempt in range(self.max_retries):
            path = self.video_paths[index]
            try:
                frames, fps, ids = self._load_video(path)
                video = torch.from_numpy(frames).permute(3, 0, 1, 2).contiguous()  # [3,T,H,W] uint8
                H, W = self.video_size
                data = {"video": video, "ai_caption": self._caption(path), "fps": torch.tensor(fps), "num_frames": self.num_frames,
                        "image_size": torch.tensor([H, W, H, W], dtype=torch.float32), "padding_mask": torch.zeros(1, H, W),
                        "frame_start": ids[0], "frame_end": ids[-1] + 1, "video_name": os.path.basename(path), "dataset_name": "video_data"}
                emb = self._embedding(path)
                if emb is not None:
                    data["t5_text_embeddings"] = emb
                    data["t5_text_mask"] = torch.ones(self.text_len, dtype=torch.int64)
                return data
            except Exception:
                log.warning(f"failed to load {path} (attempt {attempt + 1}): {traceback.format_exc(limit=1)}", rank0_only=False)
                index = random.randrange(len(self.video_paths))
        raise RuntimeError(f"could not load any video after {self.max_retries} attempts")
