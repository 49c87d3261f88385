"""Data and I/O helpers: mock datasets, local video dataset, video read / write / resize, composite loaders, small utilities."""

import os
import time

import pytest
import torch

from cosmos_predict25_b200.data import loaders as L
from cosmos_predict25_b200.data import mock
from cosmos_predict25_b200.utils import misc, video_io


def test_mock_datasets_are_deterministic_and_shaped():
    ds = mock.MockVideoLatentDataset(num_frames=3, height=8, width=6, text_dim=16, text_len=5, length=10)
    a, b = ds[3], ds[3]
    assert a["latents"].shape == (16, 3, 8, 6) and torch.equal(a["latents"], b["latents"]) and not torch.equal(a["latents"], ds[4]["latents"])
    assert a["t5_text_embeddings"].dtype == torch.bfloat16 and a["padding_mask"].shape == (1, 8, 6)
    px = mock.MockVideoPixelDataset(num_frames=5, height=16, width=24, text_dim=8, text_len=4, length=4)[0]
    assert px["video"].dtype == torch.uint8 and px["video"].shape == (3, 5, 16, 24) and px["image_size"].tolist() == [16, 24, 16, 24]
    im = mock.MockImageDataset(height=8, width=8, text_dim=8, text_len=4, length=4)[1]
    assert im["images"].shape == (3, 8, 8) and im["dataset_name"] == "mock_image"
    dl = mock.build_dataloader(ds, batch_size=2, dp_size=2, dp_rank=1, shuffle=False)
    batch = next(iter(dl))
    assert batch["latents"].shape == (2, 16, 3, 8, 6)
    assert torch.equal(batch["latents"][0], ds[1]["latents"])          # rank 1 of 2 starts at sample 1


def test_resize_cover_and_center_crop():
    x = torch.zeros(1, 3, 40, 100, dtype=torch.uint8)
    x[..., :, 40:60] = 255                                             # a vertical bar in the middle
    y = video_io.resize_input(x, (20, 20))
    assert y.shape == (1, 3, 20, 20) and y.dtype == torch.uint8
    assert y[0, 0, 10, 10] > 200 and y[0, 0, 10, 0] < 50               # scaled by 0.5, cropped around the centre: bar survives
    f = video_io.resize_input(torch.rand(2, 3, 10, 10), (20, 30))
    assert f.shape == (2, 3, 20, 30) and f.dtype == torch.float32


def test_video_and_image_write_read_roundtrip(tmp_path):
    t = torch.linspace(0, 1, 9).view(1, 9, 1, 1).expand(3, 9, 32, 48).contiguous()
    path = video_io.save_img_or_video(t, str(tmp_path / "clip"), fps=12)
    assert path.endswith(".mp4") and os.path.getsize(path) > 0
    frames, fps = video_io._read_video(path)
    assert frames.shape == (9, 32, 48, 3) and abs(fps - 12) < 0.5
    assert abs(float(frames[-1].mean()) - 255.0) < 12 and float(frames[0].mean()) < 12
    clip = video_io.read_and_process_video(path, (16, 24), num_video_frames=13, num_latent_conditional_frames=2)
    assert clip.shape == (1, 3, 13, 16, 24) and clip.dtype == torch.uint8
    assert torch.equal(clip[0, :, 5:], clip[0, :, 4:5].expand(-1, 8, -1, -1))   # padded with the last conditioning frame
    with pytest.raises(ValueError):
        video_io.read_and_process_video(path, (16, 24), 13, num_latent_conditional_frames=4)   # needs 13 frames, clip has 9
    img = video_io.save_img_or_video(t[:, :1] * 0 + 0.5, str(tmp_path / "still"))
    assert img.endswith(".jpg")
    vid = video_io.read_and_process_image(img, (16, 24), num_video_frames=5)
    assert vid.shape == (1, 3, 5, 16, 24) and abs(int(vid[0, 0, 0, 8, 8]) - 128) <= 3 and int(vid[0, :, 1:].max()) == 0


def test_local_video_dataset(tmp_path):
    from cosmos_predict25_b200.data.video_dataset import VideoDataset
    root = tmp_path / "ds"
    os.makedirs(root / "videos")
    os.makedirs(root / "metas")
    os.makedirs(root / "t5_xxl")
    clip = torch.rand(3, 12, 32, 48)
    video_io.save_img_or_video(clip, str(root / "videos" / "a"), fps=10)
    (root / "metas" / "a.txt").write_text("a red cube\n")
    torch.save(torch.randn(7, 16), root / "t5_xxl" / "a.pt")
    ds = VideoDataset(str(root), num_frames=8, video_size=(16, 24), embedding_dir="t5_xxl", text_len=10)
    assert len(ds) == 1
    s = ds[0]
    assert s["video"].shape == (3, 8, 16, 24) and s["video"].dtype == torch.uint8 and s["ai_caption"] == "a red cube"
    assert s["t5_text_embeddings"].shape == (10, 16) and float(s["t5_text_embeddings"][7:].abs().sum()) == 0.0
    assert 0 <= s["frame_start"] <= 4 and s["frame_end"] - s["frame_start"] == 8
    too_long = VideoDataset(str(root), num_frames=50, video_size=(16, 24), max_retries=2)
    with pytest.raises(RuntimeError):
        too_long[0]


def test_joint_loader_ratios_and_tags():
    img = [{"images": i} for i in range(3)]
    vid = [{"video": i} for i in range(100)]
    joint = L.IterativeJointDataLoader({"image": {"dataloader": img, "ratio": 1}, "video": {"dataloader": vid, "ratio": 2},
                                        "off": {"dataloader": [], "ratio": 0}})
    it = iter(joint)
    names = [next(it)["dataset_name"] for _ in range(9)]
    assert names == ["image", "video", "video"] * 3
    assert next(it)["dataset_name"] == "image"                       # the exhausted image loader restarts


def test_cached_replay_loader_replays_augments_and_reports_errors():
    base = [{"x": i} for i in range(4)]
    aug = lambda b: [b, {"x": b["x"] + 100}]
    dl = L.CachedReplayDataLoader(base, cache_size=3, cache_replay_n=2, cache_augmentation_fn=aug)
    got = [b["x"] for b in dl]
    assert got == [0, 0, 100, 100, 1, 1, 101, 101, 2, 2, 102, 102, 3, 3, 103, 103] and len(dl) == 8
    shuffled = sorted(b["x"] for b in L.CachedReplayDataLoader(base, cache_size=2, shuffle_cache=True))
    assert shuffled == [0, 1, 2, 3]

    def broken():
        yield {"x": 0}
        raise OSError("disk went away")

    with pytest.raises(OSError):
        list(L.CachedReplayDataLoader(broken(), cache_size=2))


def test_operation_watchdog_warns_only_when_slow():
    with L.OperationWatchdog("fast", warning_threshold=5.0, interval=0.05) as w:
        time.sleep(0.1)
    assert w.warnings == 0
    with L.OperationWatchdog("slow", warning_threshold=0.1, interval=0.05) as w:
        time.sleep(0.35)
    assert w.warnings >= 1


def test_misc_helpers():
    a = misc.arch_invariant_rand((2, 3), torch.float32, "cpu", seed=5)
    assert torch.equal(a, misc.arch_invariant_rand((2, 3), torch.float32, "cpu", seed=5)) and a.shape == (2, 3)
    moved = misc.to({"a": torch.ones(2), "b": [torch.zeros(1), "s"], "c": 3}, dtype=torch.float64)
    assert moved["a"].dtype == torch.float64 and moved["b"][1] == "s" and moved["c"] == 3
    assert misc.get_data_batch_size({"k": "v", "t": torch.zeros(5, 2)}) == 5
    timer = misc.TrainingTimer()
    with timer("forward"):
        time.sleep(0.01)
    with timer("forward"):
        time.sleep(0.01)
    avg = timer.compute_average_results()
    assert 0.005 < avg["forward"] < 0.2
    assert misc.count_params(torch.nn.Linear(3, 2)) == 8


def test_item_datasets_with_media_and_rank_split(tmp_path):
    import pickle

    from PIL import Image

    from cosmos_predict25_b200.data.item_dataset import PromptImageItemDataset, PromptVideoItemDataset, calculate_indices
    assert calculate_indices(10, 4, 0) == (0, 3, False) and calculate_indices(10, 4, 1) == (3, 6, False)
    assert calculate_indices(10, 4, 3) == (8, 10, False) and calculate_indices(2, 4, 3) == (0, 1, True)
    covered = [i for r in range(4) for i in range(*calculate_indices(10, 4, r)[:2])]
    assert covered == list(range(10))
    for i, name in enumerate(["b", "a"]):
        with open(tmp_path / f"{name}.pkl", "wb") as f:
            pickle.dump({"prompt": f"prompt {name}", "t5_text_embeddings": torch.randn(3 + i, 8).numpy()}, f)
        Image.fromarray((torch.rand(20, 30, 3) * 255).byte().numpy()).save(tmp_path / f"{name}.jpg")
        video_io.save_img_or_video(torch.rand(3, 4 + i, 20, 30), str(tmp_path / name), fps=8)
    (tmp_path / "orphan.jpg").write_bytes((tmp_path / "a.jpg").read_bytes())          # no pickle: ignored
    img = PromptImageItemDataset(str(tmp_path), num_video_frames=5, height=16, width=24, max_t5_length=6)
    assert len(img) == 2 and img.stems == ["a", "b"]
    it = img[0]
    assert it["prompt"] == "prompt a" and it["video"].shape == (3, 5, 16, 24) and int(it["video"][:, 1:].max()) == 0
    assert int(it["video"][:, 0].max()) > 0 and it["t5_text_embeddings"].shape == (6, 8) and int(it["t5_text_mask"].sum()) == 4
    vid = PromptVideoItemDataset(str(tmp_path), num_video_frames=6, height=16, width=24, start_index=1)
    assert len(vid) == 1
    iv = vid[0]
    assert iv["__file__"] == "b" and iv["video"].shape == (3, 6, 16, 24) and iv["num_frames"] == 4
    assert int(iv["video"][:, 4:].max()) == 0 and abs(float(iv["fps"]) - 8) < 0.5
    with pytest.raises(IndexError):
        vid[1]


def test_video_decoders_sample_windows_from_an_encoded_clip(tmp_path):
    """Both shard decoders on a real encoded clip whose frame k has brightness 40 + 6 (k mod 30) (inside the
    codec's video range, so no level is clipped), with one caption chunk per 30 frames:
    consecutive window inside one chunk, strided window with the lowered frame rate, clips outside the frame-rate bounds dropped,
    non-video members ignored."""
    cv2 = pytest.importorskip("cv2")
    import numpy as np
    from cosmos_predict25_b200.data.video_decoder import construct_video_decoder
    path = str(tmp_path / "clip.mp4")
    w = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), 24.0, (32, 32))
    for k in range(60):
        w.write(np.full((32, 32, 3), 40 + 6 * (k % 30), np.uint8))
    w.release()
    data = open(path, "rb").read()
    dec = construct_video_decoder("chunked_video_decoder", chunk_size=30, sequence_length=8, min_fps_thres=10, max_fps_thres=60)
    for _ in range(4):
        out = dec("a/clip.mp4", data)
        assert out["video"].shape == (3, 8, 32, 32) and out["video"].dtype == torch.uint8 and out["fps"] == 24 and out["n_orig_video_frames"] == 60
        level = out["video"].float().mean((0, 2, 3))
        assert torch.allclose(level[1:] - level[:-1], torch.full((7,), 6.0), atol=2.5)              # consecutive frames, one chunk
        assert abs(level[0].item() - 40 - 6 * (out["frame_start"] % 30)) < 4 and out["frame_start"] // 30 == out["chunk_index"]
    low = construct_video_decoder("chunked_video_decoder_w_lower_fps", chunk_size=30, sequence_length=5, min_fps_thres=4,
                                  max_fps_thres=12)("clip.mp4", data)
    stride = low["frame_indices"][1] - low["frame_indices"][0]
    assert stride in (5, 6) and low["fps"] == 24 / stride and low["frame_indices"][0] // 30 == low["frame_indices"][-1] // 30
    lv = low["video"].float().mean((0, 2, 3))
    assert torch.allclose(lv[1:] - lv[:-1], torch.full((4,), 6.0 * stride), atol=4.0)
    assert construct_video_decoder("chunked_video_decoder", sequence_length=8, min_fps_thres=30, max_fps_thres=60)("clip.mp4", data) is None
    assert dec("a/clip.txt", b"caption") is None
    assert construct_video_decoder("video_naive_bytes")("clip.mp4", data) is data


def test_infinite_multi_aspect_distributor_deals_readers_by_shard_share(monkeypatch):
    from cosmos_predict25_b200.data.webdataset import DatasetInfo, ShardlistMultiAspectRatioInfinite, TarSample
    urls = []
    for aspect, count in (("16:9", 60), ("1:1", 30), ("9:16", 10)):
        info = DatasetInfo(wdinfo=[], opts={"aspect_ratio": aspect})
        urls += [TarSample(root="r/", path=f"{aspect}/part_{i:04d}.tar", keys=[], meta=info) for i in range(count)]
    d = ShardlistMultiAspectRatioInfinite(shuffle=False)
    d.set_urls(urls)
    alloc = d.allocate_readers(10)
    assert len(alloc) == 10 and {a: alloc.count(a) for a in set(alloc)} == {"16:9": 5, "1:1": 3, "9:16": 2}
    assert sorted(set(d.allocate_readers(2))) == ["16:9", "1:1"] or len(set(d.allocate_readers(2))) == 2      # fewer readers than groups
    seen = {}
    for worker in range(10):                                    # every reader stays in its group and the slices of a group are disjoint
        for k, v in (("RANK", "0"), ("WORLD_SIZE", "1"), ("WORKER", str(worker)), ("NUM_WORKERS", "10")):
            monkeypatch.setenv(k, v)
        it = iter(d)
        got = [next(it)["url"] for _ in range(4)]
        assert len({u.meta.opts["aspect_ratio"] for u in got}) == 1
        seen.setdefault(got[0].meta.opts["aspect_ratio"], []).append({u.path for u in got})
    for group in seen.values():
        assert all(a.isdisjoint(b) for i, a in enumerate(group) for b in group[i + 1:])
    with pytest.raises(ValueError):
        d.set_urls([TarSample(root="r/", path="x.tar", keys=[], meta=DatasetInfo(wdinfo=[]))])
