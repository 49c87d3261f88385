"""Item datasets for validation sampling: prompt only, prompt + image, prompt + video; rank-wise index split.

Parity target: ``PromptOnlyItemDataset`` / ``ItemDatasetConfig`` (cosmos_predict2/_src/predict2/datasets/item_dataset.py:30-150): a
directory (local or object store) holding ``meta_info.json`` (``{"length": N}``) and one pickle per item
(``{idx:06d}.pkl`` with ``prompt`` and ``t5_xxl_fp8`` / ``t5_text_embeddings``); items carry a blank video of the target
size so that the regular sampling path can be used unchanged.
"""

from __future__ import annotations

import dataclasses
import os

import numpy as np
import torch

from ..utils.easy_io import easy_io


@dataclasses.dataclass
class ItemDatasetConfig:
    path: str
    length: int


class PromptOnlyItemDataset(torch.utils.data.Dataset):
    def __init__(self, path: str, start_index: int = 0, end_index: int = 32, max_t5_length: int = 512, height: int = 704, width: int = 1280,
                 num_video_frames: int = 93, backend_args=None):
        self.path, self.start_index, self.end_index = path, start_index, end_index
        self.max_t5_length, self.height, self.width, self.num_video_frames = max_t5_length, height, width, num_video_frames
        self.backend_args = backend_args
        n = easy_io.load(os.path.join(path, "meta_info.json"), backend_args=backend_args)["length"]
        assert n >= end_index, f"dataset {path} has {n} items, end_index is {end_index}"

    def __len__(self):
        return self.end_index - self.start_index

    def __getitem__(self, idx):
        i = self.start_index + idx
        item = easy_io.load(os.path.join(self.path, f"{i:06d}.pkl"), backend_args=self.backend_args)
        emb = item.get("t5_text_embeddings", item.get("t5_xxl_fp8"))
        emb = torch.as_tensor(np.asarray(emb[0] if isinstance(emb, (list, tuple)) else emb)).float()
        n = min(emb.shape[0], self.max_t5_length)
        out = torch.zeros(self.max_t5_length, emb.shape[-1])
        out[:n] = emb[:n]
        mask = torch.zeros(self.max_t5_length, dtype=torch.int64)
        mask[:n] = 1
        return {"video": torch.zeros(3, self.num_video_frames, self.height, self.width, dtype=torch.uint8), "t5_text_embeddings": out,
                "t5_text_mask": mask, "ai_caption": item.get("prompt", ""), "fps": torch.tensor(16.0),
                "image_size": torch.tensor([self.height, self.width, self.height, self.width], dtype=torch.float32),
                "num_frames": self.num_video_frames, "padding_mask": torch.zeros(1, self.height, self.width), "__key__": f"{i:06d}"}


def calculate_indices(dataset_length: int, world_size: int, rank: int):
    """Contiguous [start, end) of ``rank`` when ``dataset_length`` items are spread over ``world_size`` ranks (the first
    ``length % world`` ranks get one more). A rank that would get nothing takes item 0 and reports ``overflow=True`` so that it
    can still join collectives (item_dataset.py:413-439 of the reference)."""
    per, rem = divmod(dataset_length, world_size)
    start = rank * per + min(rank, rem)
    end = start + per + (1 if rank < rem else 0)
    if start >= dataset_length:
        return 0, 1, True
    return start, end, False


def _padded_embedding(item: dict, max_len: int):
    emb = item.get("t5_text_embeddings", item.get("t5_xxl_fp8"))
    if isinstance(emb, dict):                       # several encoders: stack along a new last axis
        emb = np.concatenate([np.asarray(e)[:, :, None] for e in emb.values()], axis=2)
    emb = torch.as_tensor(np.asarray(emb[0] if isinstance(emb, (list, tuple)) else emb)).float()
    n = min(emb.shape[0], max_len)
    out = torch.zeros(max_len, *emb.shape[1:])
    out[:n] = emb[:n]
    mask = torch.zeros(max_len, dtype=torch.int64)
    mask[:n] = 1
    return out, mask


class _PairedItemDataset(torch.utils.data.Dataset):
    """Items are pairs ``<stem>.pkl`` (``prompt`` and optionally text embeddings) + ``<stem><media_ext>`` in one directory; the
    stems are listed once and sorted, so indices are stable across ranks."""

    media_ext = ""

    def __init__(self, path: str, start_index: int = 0, end_index: int = None, max_t5_length: int = 512, height: int = 704,
                 width: int = 1280):
        self.path, self.max_t5_length, self.height, self.width = path, max_t5_length, height, width
        self.stems = sorted(f[: -len(self.media_ext)] for f in os.listdir(path)
                            if f.endswith(self.media_ext) and os.path.exists(os.path.join(path, f[: -len(self.media_ext)] + ".pkl")))
        self.start_index = start_index
        self.end_index = len(self.stems) if end_index is None else min(end_index, len(self.stems))

    def __len__(self):
        return max(0, self.end_index - self.start_index)

    def _base(self, idx: int) -> dict:
        if idx < 0 or idx >= len(self):
            raise IndexError(idx)
        stem = self.stems[self.start_index + idx]
        item = dict(easy_io.load(os.path.join(self.path, stem + ".pkl")))
        out = {"ai_caption": item.get("prompt", ""), "prompt": item.get("prompt", ""), "__idx__": self.start_index + idx, "__file__": stem,
               "image_size": torch.tensor([self.height, self.width, self.height, self.width], dtype=torch.float32),
               "padding_mask": torch.zeros(1, self.height, self.width)}
        if "t5_text_embeddings" in item or "t5_xxl_fp8" in item:
            out["t5_text_embeddings"], out["t5_text_mask"] = _padded_embedding(item, self.max_t5_length)
        return out, stem


class PromptImageItemDataset(_PairedItemDataset):
    """Prompt + conditioning image: the image is area-resized to (height, width) and becomes frame 0 of an otherwise blank
    clip of ``num_video_frames`` frames (item_dataset.py:127-227 of the reference)."""

    media_ext = ".jpg"

    def __init__(self, path: str, num_video_frames: int = 93, **kw):
        super().__init__(path, **kw)
        self.num_video_frames = num_video_frames

    def __getitem__(self, idx):
        import cv2
        from PIL import Image
        out, stem = self._base(idx)
        img = np.asarray(Image.open(os.path.join(self.path, stem + self.media_ext)).convert("RGB"))
        img = cv2.resize(img, (self.width, self.height), interpolation=cv2.INTER_AREA)
        video = torch.zeros(3, self.num_video_frames, self.height, self.width, dtype=torch.uint8)
        video[:, 0] = torch.from_numpy(img).permute(2, 0, 1)
        out.update(video=video, fps=torch.tensor(16.0), num_frames=self.num_video_frames, num_conditional_frames=1)
        return out


class PromptVideoItemDataset(_PairedItemDataset):
    """Prompt + conditioning video: up to ``num_video_frames`` frames, each area-resized to (height, width); shorter clips are
    zero-padded at the end and ``num_frames`` reports how many are real (item_dataset.py:229-335 of the reference)."""

    media_ext = ".mp4"

    def __init__(self, path: str, num_video_frames: int = 93, **kw):
        super().__init__(path, **kw)
        self.num_video_frames = num_video_frames

    def __getitem__(self, idx):
        import cv2
        from ..utils.video_io import _read_video
        out, stem = self._base(idx)
        frames, fps = _read_video(os.path.join(self.path, stem + self.media_ext), max_frames=self.num_video_frames)
        clip = np.zeros((self.num_video_frames, self.height, self.width, 3), dtype=np.uint8)
        for i in range(frames.shape[0]):
            clip[i] = cv2.resize(frames[i], (self.width, self.height), interpolation=cv2.INTER_AREA)
        video = torch.from_numpy(clip).permute(3, 0, 1, 2).contiguous()
        out.update(video=video, raw_video=video.clone(), fps=torch.tensor(float(fps or 30.0)), num_frames=int(frames.shape[0]))
        return out
