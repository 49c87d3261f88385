"""Prompt-only item dataset for validation sampling.

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
