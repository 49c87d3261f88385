"""Synthetic datasets with the shapes of the real pipelines, and the dataloader builder.

Parity targets: mock datasets (cosmos_predict2/_src/predict2/datasets/data_sources/mock_data.py:28-115,
cosmos_predict2/_src/imaginaire/datasets/mock_dataset.py) and the sampler rule of
``get_sampler`` (cosmos_predict2/_src/predict2/datasets/local_datasets/dataset_video.py:186-194): samples are
sharded by *data-parallel* rank so that all ranks of one context-parallel group read the same sample.
"""

from __future__ import annotations

from typing import Any, Callable, Dict, Optional

import torch
from torch.utils.data import DataLoader, Dataset, DistributedSampler


class MockVideoLatentDataset(Dataset):
    """Pre-encoded latents + text embeddings: {latents [16,T,H,W] fp32, t5_text_embeddings [L,C] bf16, fps, padding_mask}."""

    def __init__(self, num_frames=24, height=88, width=160, text_dim=100352, text_len=512, length=1 << 30, channels=16, seed=0):
        self.shape = (channels, num_frames, height, width)
        self.text = (text_len, text_dim)
        self.length, self.seed = length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i) -> Dict[str, Any]:
        g = torch.Generator().manual_seed(self.seed * 1000003 + int(i))
        return {"latents": torch.randn(self.shape, generator=g),
                "t5_text_embeddings": torch.randn(self.text, generator=g).to(torch.bfloat16),
                "fps": torch.tensor(16.0), "padding_mask": torch.zeros(1, self.shape[2], self.shape[3]),
                "ai_caption": f"synthetic sample {i}", "dataset_name": "mock_video"}


class MockVideoPixelDataset(Dataset):
    """uint8 video [3,T,H,W] + text embeddings + the keys of the reference's video batches."""

    def __init__(self, num_frames=93, height=704, width=1280, text_dim=1024, text_len=512, length=1 << 30, seed=0):
        self.shape = (3, num_frames, height, width)
        self.text = (text_len, text_dim)
        self.length, self.seed = length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 7919 + int(i))
        H, W = self.shape[2:]
        return {"video": torch.randint(0, 256, self.shape, dtype=torch.uint8, generator=g),
                "t5_text_embeddings": torch.randn(self.text, generator=g).to(torch.bfloat16),
                "t5_text_mask": torch.ones(self.text[0], dtype=torch.int64), "fps": torch.tensor(24.0),
                "image_size": torch.tensor([H, W, H, W], dtype=torch.float32), "num_frames": self.shape[1],
                "padding_mask": torch.zeros(1, H, W), "ai_caption": f"synthetic sample {i}", "dataset_name": "mock_video"}


class MockImageDataset(Dataset):
    def __init__(self, height=704, width=1280, text_dim=1024, text_len=512, length=1 << 30, seed=0):
        self.h, self.w, self.text, self.length, self.seed = height, width, (text_len, text_dim), length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        g = torch.Generator().manual_seed(self.seed * 104729 + int(i))
        return {"images": torch.randint(0, 256, (3, self.h, self.w), dtype=torch.uint8, generator=g),
                "t5_text_embeddings": torch.randn(self.text, generator=g).to(torch.bfloat16), "fps": torch.tensor(1.0),
                "padding_mask": torch.zeros(1, self.h, self.w), "ai_caption": f"synthetic image {i}", "dataset_name": "mock_image"}


MAX_LENGTH = 1 << 15


class LambdaDataset(Dataset):
    """Items are whatever ``fn()`` returns (imaginaire/datasets/mock_dataset.py:29-84 of the reference)."""

    def __init__(self, fn, length: int = MAX_LENGTH):
        self.fn, self.length = fn, length

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        return self.fn()


class RepeatDataset(Dataset):
    """Cycles over the first ``num_item`` items of ``dataset`` (one fixed sample by default) for ``length`` indices."""

    def __init__(self, dataset, length: int = MAX_LENGTH, num_item: int = 1):
        self.length = length
        self.items = [dataset[i] for i in range(num_item)]

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        return self.items[index % len(self.items)]


class CombinedDictDataset(Dataset):
    """{key: dataset} -> items {key: dataset[i]}; the length is the shortest member's."""

    def __init__(self, **datasets):
        self.datasets = datasets
        self.length = min(len(d) for d in datasets.values())

    def __len__(self):
        return self.length

    def __getitem__(self, index):
        return {k: d[index] for k, d in self.datasets.items()}


def get_sampler(dataset, dp_size: int = 1, dp_rank: int = 0, shuffle: bool = True, seed: int = 0):
    """Shard by data-parallel rank (all ranks of a context-parallel group share ``dp_rank``)."""
    return DistributedSampler(dataset, num_replicas=dp_size, rank=dp_rank, shuffle=shuffle, seed=seed)


def build_dataloader(dataset, batch_size: int = 1, num_workers: int = 0, dp_size: Optional[int] = None, dp_rank: Optional[int] = None,
                     shuffle: bool = False, pin_memory: bool = True, drop_last: bool = True, collate_fn: Optional[Callable] = None,
                     seed: int = 0) -> DataLoader:
    if dp_size is None:
        import torch.distributed as dist
        dp_size = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
        dp_rank = dist.get_rank() if dp_size > 1 else 0
    sampler = get_sampler(dataset, dp_size, dp_rank or 0, shuffle, seed) if dp_size > 1 else None
    return DataLoader(dataset, batch_size=batch_size, num_workers=num_workers, sampler=sampler, shuffle=shuffle and sampler is None,
                      pin_memory=pin_memory and torch.cuda.is_available(), drop_last=drop_last, collate_fn=collate_fn,
                      persistent_workers=num_workers > 0)
