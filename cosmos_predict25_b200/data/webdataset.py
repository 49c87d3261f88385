"""Sharded tar datasets ("webdataset" layout) without external dependencies.

Parity targets: the reference's webdataset stack — ``Dataset`` / ``build_dataset`` (cosmos_predict2/_src/imaginaire/datasets/webdataset/webdataset.py,
cosmos_predict2/_src/predict2/datasets/webdataset.py), shard distributors ``ShardlistBasic`` / ``ShardlistMultiAspectRatio``
(.../webdataset/distributors/{basic,multi_aspect_ratio}.py) and ``ShardlistMultiAspectRatioParallelSync``
(cosmos_predict2/_src/predict2/datasets/distributor/parallel_sync_multi_aspect_ratio.py:38), decoders and the augmentor
chain (.../webdataset/{decoders,augmentors}), ``dataset_provider`` style config objects.

Layout: a dataset is a list of ``DatasetInfo`` (root, wdinfo json listing shard paths per data key, per-key sub-directories);
a sample is the set of tar members sharing a key (``<key>.<ext>``), possibly spread over parallel shards of several data keys
(``video/part_000.tar`` + ``metas/part_000.tar`` + ``t5_xxl/part_000.tar``). Shards are read through the unified file API, so
``s3://`` and local paths both work. Distributors decide which shards a (rank, worker) pair reads:

* basic: shards are dealt round-robin over ``dp_world * workers`` readers;
* multi aspect ratio: shards are grouped by the aspect-ratio directory in their path and a reader sticks to one group so
  that a batch has one shape;
* parallel sync: the reader id is the *data-parallel* rank, so all ranks of one context-parallel group read identical data.
"""

from __future__ import annotations

import io
import json
import os
import pickle
import random
import re
import tarfile
from dataclasses import dataclass, field
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence

import torch
import torch.distributed as dist
from torch.utils.data import IterableDataset, get_worker_info

from ..utils import log
from ..utils.easy_io import easy_io


@dataclass
class DatasetInfo:
    """One source: ``wdinfo`` json files (``{"root": ..., "data_list": ["aspect_ratio_16_9/part_000.tar", ...], "data_keys": [...]}``)."""
    wdinfo: Sequence[str]
    object_store_config: Optional[dict] = None
    opts: dict = field(default_factory=dict)
    per_dataset_keys: Sequence[str] = ()
    source: str = ""


@dataclass
class DatasetConfig:
    keys: Sequence[str]
    buffer_size: int
    dataset_info: Sequence[DatasetInfo]
    distributor: Any
    decoders: Sequence[Callable] = ()
    augmentation: Dict[str, Callable] = field(default_factory=dict)
    streaming_download: bool = True
    remove_extension_from_keys: bool = True
    sample_keys_full_list_path: Optional[str] = None


@dataclass
class TarSample:
    root: str
    path: str                      # relative shard path, with ``{key}`` replaced per data key
    keys: Sequence[str]
    dset_id: Any = 0
    sample_keys_full_list: Optional[str] = None
    meta: Any = None               # the DatasetInfo this shard came from (its ``opts`` carry e.g. the aspect ratio)


def _aspect_of(path: str) -> str:
    m = re.search(r"aspect_ratio_(\d+)_(\d+)", path)
    return f"{m.group(1)},{m.group(2)}" if m else "none"


# ---- distributors ----------------------------------------------------------------------------------------------------
class ShardlistBasic:
    def __init__(self, shuffle: bool = True, split_by_node: bool = True, split_by_worker: bool = True, resume_flag: bool = True,
                 verbose: bool = False, is_infinite_loader: bool = True, seed: int = 0):
        self.shuffle, self.split_by_node, self.split_by_worker, self.infinite, self.seed = shuffle, split_by_node, split_by_worker, is_infinite_loader, seed
        self.epoch = 0
        self.urls: List[TarSample] = []

    def set_urls(self, urls: List[TarSample]):
        self.urls = list(urls)

    def reader_id(self):
        rank = dist.get_rank() if (dist.is_available() and dist.is_initialized()) else 0
        world = dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1
        return rank, world

    def _reader(self):
        rank, world = self.reader_id() if self.split_by_node else (0, 1)
        wi = get_worker_info()
        wid, nw = (wi.id, wi.num_workers) if (wi is not None and self.split_by_worker) else (0, 1)
        return rank * nw + wid, world * nw

    def select(self, urls: List[TarSample], rid: int, n: int) -> List[TarSample]:
        return urls[rid::n] if len(urls) >= n else [urls[rid % len(urls)]]

    def __iter__(self) -> Iterator[TarSample]:
        rid, n = self._reader()
        while True:
            urls = list(self.urls)
            if self.shuffle:
                random.Random(self.seed + self.epoch).shuffle(urls)      # same permutation on every reader, then strided
            for u in self.select(urls, rid, n):
                yield u
            self.epoch += 1
            if not self.infinite:
                return


class ShardlistMultiAspectRatio(ShardlistBasic):
    """A reader draws all its shards from one aspect-ratio group (chosen round-robin by reader id, re-drawn every epoch)."""

    def select(self, urls, rid, n):
        groups: Dict[str, List[TarSample]] = {}
        for u in urls:
            groups.setdefault(_aspect_of(u.path), []).append(u)
        names = sorted(groups)
        g = groups[names[(rid + self.epoch) % len(names)]]
        same = [r for r in range(n) if (r + self.epoch) % len(names) == (rid + self.epoch) % len(names)]
        return super().select(g, same.index(rid), len(same))


class ShardlistMultiAspectRatioParallelSync(ShardlistMultiAspectRatio):
    """Readers are data-parallel ranks: every rank of a context- (or tensor-) parallel group iterates the same shards."""

    def __init__(self, *a, model_parallel_size: int = 1, **kw):
        super().__init__(*a, **kw)
        self.model_parallel_size = max(1, model_parallel_size)

    def reader_id(self):
        rank, world = super().reader_id()
        return rank // self.model_parallel_size, max(1, world // self.model_parallel_size)


class ShardlistMultiAspectRatioInfinite(IterableDataset):
    """Endless shard stream in which every reader (rank x loader worker) stays inside ONE aspect-ratio group, so that a batch never
    mixes frame shapes. Readers are dealt to the groups in proportion to the groups' shard counts (at least one each); inside a
    group the readers take interleaved slices. The group of a shard is ``shard.meta.opts["aspect_ratio"]``. Reader identity comes
    from RANK / WORLD_SIZE / WORKER / NUM_WORKERS when set (tests, external launchers), else from torch.distributed and the loader's
    worker info. Yields ``{"url": shard}`` (imaginaire/datasets/webdataset/distributors/multi_aspect_ratio_v2.py:30-252 of the
    reference)."""

    def __init__(self, shuffle: bool = True, split_by_node: bool = True, split_by_worker: bool = True, chunk_size: int = 1,
                 resume_flag: bool = True, verbose: bool = False, is_infinite_loader: bool = True, seed: int = 0):
        super().__init__()
        assert is_infinite_loader, "this distributor only runs as an endless stream"
        self.shuffle, self.split_by_node, self.split_by_worker, self.verbose, self.seed = shuffle, split_by_node, split_by_worker, verbose, seed
        self.chunk_size, self.resume_flag = chunk_size, resume_flag            # accepted for compatibility, unused
        self.groups: Dict[str, List[TarSample]] = {}

    def set_urls(self, urls: List[TarSample]):
        groups: Dict[str, List[TarSample]] = {}
        for u in urls:
            opts = getattr(u.meta, "opts", None) or {}
            if "aspect_ratio" not in opts:
                raise ValueError("aspect_ratio should be specified in dataset_info when using multi aspect distributor")
            groups.setdefault(opts["aspect_ratio"], []).append(u)
        self.groups = {k: sorted(v, key=lambda t: (t.path, t.root)) for k, v in sorted(groups.items())}

    def set_chunk_size(self, chunk_size: int):
        self.chunk_size = chunk_size

    def set_epoch(self, epoch: int, start_index: int = 0):
        self.epoch, self.start_index = epoch, start_index

    def _reader(self):
        env = os.environ
        if self.split_by_node:
            rank = int(env["RANK"]) if "RANK" in env else (dist.get_rank() if dist.is_available() and dist.is_initialized() else 0)
            world = int(env["WORLD_SIZE"]) if "WORLD_SIZE" in env else (dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1)
        else:
            rank, world = 0, 1
        wi = get_worker_info()
        if not self.split_by_worker:
            wid, nw = 0, 1
        elif "WORKER" in env and "NUM_WORKERS" in env:
            wid, nw = int(env["WORKER"]), int(env["NUM_WORKERS"])
        else:
            wid, nw = (wi.id, wi.num_workers) if wi is not None else (0, 1)
        return rank * nw + wid, world * nw

    def allocate_readers(self, n_readers: int) -> List[str]:
        """Group name of every reader: one reader per group first, the rest by largest remainder of the shard shares."""
        names = list(self.groups)
        if n_readers < len(names):
            return [names[r % len(names)] for r in range(n_readers)]          # fewer readers than groups: each reader rotates
        total = sum(len(v) for v in self.groups.values())
        extra = n_readers - len(names)
        share = {k: extra * len(self.groups[k]) / total for k in names}
        counts = {k: 1 + int(share[k]) for k in names}
        for k in sorted(names, key=lambda k: share[k] - int(share[k]), reverse=True)[: n_readers - sum(counts.values())]:
            counts[k] += 1
        return [k for k in names for _ in range(counts[k])]

    def __iter__(self):
        rid, n = self._reader()
        alloc = self.allocate_readers(n)
        names = list(self.groups)
        rotate = n < len(names)
        group = alloc[rid]
        peers = [r for r in range(n) if alloc[r] == group]
        j, k = peers.index(rid), len(peers)
        if self.verbose:
            log.info(f"reader {rid}/{n}: aspect ratio {group}, slice {j} of {k}, {len(self.groups[group])} shards")
        rng = random.Random(self.seed + 7919 * rid)
        epoch = 0
        while True:
            if rotate:
                group = names[(rid + epoch * n) % len(names)]
                j, k = 0, 1
            urls = self.groups[group]
            mine = urls[j::k] if len(urls) >= k else [urls[j % len(urls)]]
            if self.shuffle:
                mine = list(mine)
                rng.shuffle(mine)
            for u in mine:
                yield {"url": u}
            epoch += 1


# ---- decoders -----------------------------------------------------------------------------------------------------------
def basic_decoder(key: str, data: bytes):
    ext = key.rsplit(".", 1)[-1].lower()
    if ext in ("txt", "text"):
        return data.decode("utf-8")
    if ext == "json":
        return json.loads(data)
    if ext in ("pkl", "pickle"):
        return pickle.loads(data)
    if ext in ("pt", "pth"):
        return torch.load(io.BytesIO(data), map_location="cpu", weights_only=False)
    if ext == "npy":
        import numpy as np
        return np.load(io.BytesIO(data), allow_pickle=True)
    return None


def image_decoder(key: str, data: bytes):
    if key.rsplit(".", 1)[-1].lower() not in ("jpg", "jpeg", "png", "webp"):
        return None
    from PIL import Image
    img = Image.open(io.BytesIO(data))
    img.load()
    return img.convert("RGB")


def video_bytes_passthrough(key: str, data: bytes):
    """Videos stay as bytes; a video-parsing augmentor decodes the window it needs."""
    return data if key.rsplit(".", 1)[-1].lower() in ("mp4", "mov", "avi", "webm") else None


# ---- dataset -------------------------------------------------------------------------------------------------------------
class Dataset(IterableDataset):
    def __init__(self, config: DatasetConfig, handler: Callable = None, world_size: Optional[int] = None):
        super().__init__()
        self.config = config
        self.handler = handler or (lambda e, ctx: log.warning(f"skipping {ctx}: {e}"))
        self.wdinfo: List[TarSample] = []
        self.parse_dataset_info(config.dataset_info, config.keys)
        config.distributor.set_urls(self.wdinfo)
        self.decoders = list(config.decoders) or [basic_decoder, image_decoder, video_bytes_passthrough]

    def parse_dataset_info(self, infos: Sequence[DatasetInfo], use_keys: Sequence[str]):
        for dset_id, info in enumerate(infos):
            backend = info.object_store_config
            keys = list(info.per_dataset_keys) or list(use_keys)
            for wd in info.wdinfo:
                meta = easy_io.load(wd, backend_args=backend) if isinstance(wd, str) else wd
                root = meta["root"]
                for rel in meta["data_list"]:
                    self.wdinfo.append(TarSample(root=root, path=rel, keys=keys, dset_id=dset_id))
        log.info(f"webdataset: {len(self.wdinfo)} shards from {len(infos)} sources")

    @staticmethod
    def _members(raw: bytes) -> Iterator:
        with tarfile.open(fileobj=io.BytesIO(raw), mode="r:*") as tf:
            for m in tf:
                if m.isfile():
                    yield m.name, tf.extractfile(m).read()

    def _open(self, url: TarSample, key: str, backend) -> bytes:
        return easy_io.get(os.path.join(url.root, key, url.path), backend_args=backend)

    def samples_of_shard(self, url: TarSample) -> Iterator[Dict[str, Any]]:
        backend = self.config.dataset_info[url.dset_id].object_store_config
        grouped: Dict[str, Dict[str, Any]] = {}
        order: List[str] = []
        for dkey in url.keys:
            for name, data in self._members(self._open(url, dkey, backend)):
                base = os.path.basename(name)
                sample_key, _, ext = base.partition(".")
                if sample_key not in grouped:
                    grouped[sample_key] = {"__key__": sample_key, "__url__": os.path.join(url.root, url.path), "__dset_id__": url.dset_id}
                    order.append(sample_key)
                field_name = dkey if self.config.remove_extension_from_keys else f"{dkey}.{ext}"
                val = None
                for dec in self.decoders:
                    val = dec(base, data)
                    if val is not None:
                        break
                grouped[sample_key][field_name] = data if val is None else val
        for k in order:
            s = grouped[k]
            if all((dk if self.config.remove_extension_from_keys else None) in s or not self.config.remove_extension_from_keys for dk in url.keys):
                yield s

    def _augment(self, samples: Iterable[Dict]) -> Iterator[Dict]:
        def mapped(fn, it):          # a function per stage: generator expressions would capture the loop variable late
            for d in it:
                o = fn(d)
                if o is not None:
                    yield o

        data = samples
        for name, aug in self.config.augmentation.items():
            data = aug(data) if getattr(aug, "is_generator", False) else mapped(aug, data)
        yield from data

    def _shuffled(self, it: Iterator[Dict]) -> Iterator[Dict]:
        n = self.config.buffer_size
        if n <= 1:
            yield from it
            return
        buf: List[Dict] = []
        rng = random.Random(1234)
        for s in it:
            if len(buf) < n:
                buf.append(s)
                continue
            i = rng.randrange(n)
            buf[i], s = s, buf[i]
            yield s
        rng.shuffle(buf)
        yield from buf

    def __iter__(self) -> Iterator[Dict[str, Any]]:
        def raw():
            for url in self.config.distributor:
                try:
                    yield from self.samples_of_shard(url)
                except Exception as e:       # a broken shard must not end an infinite training stream
                    self.handler(e, url.path)
        yield from self._augment(self._shuffled(raw()))

    def build_dataset(self, **_):
        return self


def write_shard(path: str, samples: Sequence[Dict[str, bytes]]):
    """Test / tooling helper: ``samples`` = [{"__key__": k, "<ext>": bytes, ...}] -> one tar shard."""
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    with tarfile.open(path, "w") as tf:
        for s in samples:
            for ext, data in s.items():
                if ext == "__key__":
                    continue
                ti = tarfile.TarInfo(f"{s['__key__']}.{ext}")
                ti.size = len(data)
                tf.addfile(ti, io.BytesIO(data))
