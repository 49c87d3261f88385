"""Tar-shard datasets, distributors, item dataset, resolution tables (CPU)."""
import json
import pickle

import torch

from cosmos_predict25_b200.data import webdataset as wd
from cosmos_predict25_b200.data.item_dataset import PromptOnlyItemDataset
from cosmos_predict25_b200.data.utils import VIDEO_RES_SIZE_INFO, closest_aspect_ratio


def _make(tmp_path, n_shards=4, per=3):
    root = tmp_path / "ds"
    rels = []
    for s in range(n_shards):
        ar = "aspect_ratio_16_9" if s % 2 == 0 else "aspect_ratio_1_1"
        rel = f"{ar}/part_{s:03d}.tar"
        rels.append(rel)
        keys = [f"s{s}_{i}" for i in range(per)]
        wd.write_shard(str(root / "video" / rel), [{"__key__": k, "mp4": f"video-{k}".encode()} for k in keys])
        wd.write_shard(str(root / "metas" / rel), [{"__key__": k, "json": json.dumps({"caption": k, "fps": 24}).encode()} for k in keys])
    info = tmp_path / "wdinfo.json"
    info.write_text(json.dumps({"root": str(root), "data_list": rels, "data_keys": ["video", "metas"]}))
    return str(info)


def _cfg(info, dist_cls=wd.ShardlistBasic, **kw):
    return wd.DatasetConfig(keys=["video", "metas"], buffer_size=1, dataset_info=[wd.DatasetInfo(wdinfo=[info])],
                            distributor=dist_cls(shuffle=False, is_infinite_loader=False, **kw))


def test_samples_are_joined_across_data_keys(tmp_path):
    ds = wd.Dataset(_cfg(_make(tmp_path)))
    items = list(ds)
    assert len(items) == 12
    s = items[0]
    assert s["__key__"] == "s0_0" and s["video"] == b"video-s0_0" and s["metas"] == {"caption": "s0_0", "fps": 24}


def test_augmentors_filter_and_generate(tmp_path):
    cfg = _cfg(_make(tmp_path))

    def drop_odd(d):
        return None if d["__key__"].endswith("1") else d

    def twice(data):
        for d in data:
            yield d
            yield dict(d, replica=True)
    twice.is_generator = True
    cfg.augmentation = {"drop": drop_odd, "dup": twice}
    items = list(wd.Dataset(cfg))
    assert len(items) == 16 and sum(1 for i in items if i.get("replica")) == 8


def test_distributors_partition_shards(tmp_path):
    info = _make(tmp_path, n_shards=8, per=1)
    urls = wd.Dataset(_cfg(info)).wdinfo
    d = wd.ShardlistBasic(shuffle=False, is_infinite_loader=False)
    seen = [u.path for r in range(4) for u in d.select(urls, r, 4)]
    assert sorted(seen) == sorted(u.path for u in urls)                   # disjoint cover
    m = wd.ShardlistMultiAspectRatio(shuffle=False, is_infinite_loader=False)
    for r in range(4):
        ars = {wd._aspect_of(u.path) for u in m.select(urls, r, 4)}
        assert len(ars) == 1                                              # one shape per reader
    ps = wd.ShardlistMultiAspectRatioParallelSync(shuffle=False, is_infinite_loader=False, model_parallel_size=2)
    assert ps.model_parallel_size == 2 and ps.reader_id() == (0, 1)


def test_item_dataset_and_tables(tmp_path):
    (tmp_path / "meta_info.json").write_text(json.dumps({"length": 3}))
    for i in range(3):
        with open(tmp_path / f"{i:06d}.pkl", "wb") as f:
            pickle.dump({"prompt": f"p{i}", "t5_text_embeddings": torch.randn(5, 16).numpy()}, f)
    ds = PromptOnlyItemDataset(str(tmp_path), 1, 3, max_t5_length=8, height=16, width=32, num_video_frames=5)
    assert len(ds) == 2
    it = ds[0]
    assert it["ai_caption"] == "p1" and it["t5_text_embeddings"].shape == (8, 16) and it["t5_text_mask"].sum() == 5 and it["video"].shape == (3, 5, 16, 32)
    assert VIDEO_RES_SIZE_INFO["720"]["16,9"] == (1280, 704) and closest_aspect_ratio(1920, 1080) == "16,9" and closest_aspect_ratio(500, 510) == "1,1"
