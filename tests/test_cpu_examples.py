"""The end-to-end post-training example on the offline tiny preset: train, convert, sample, resume skips finished stages."""

import importlib.util
import os
import sys


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def test_posttraining_pipeline_tiny(tmp_path, monkeypatch):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    monkeypatch.setenv("IMAGINAIRE_OUTPUT_ROOT", str(tmp_path / "jobs"))
    monkeypatch.delenv("MAX_ITERS", raising=False)
    mod = _load(os.path.join(root, "examples", "posttraining", "pipeline.py"), "posttraining_pipeline_example")
    pipe = mod.PostTrainingPipeline("tiny", str(tmp_path / "work"), max_iters=2, save_iter=2)
    state = pipe.run(num_steps=2)
    assert all(state[s] for s in mod.STAGES)
    assert os.path.exists(state["converted"]["model"]) and os.path.exists(state["sample"])
    again = mod.PostTrainingPipeline("tiny", str(tmp_path / "work"), max_iters=2, save_iter=2)
    assert again.state["train"] and again.job_dir == state["job_dir"]
    ran = []
    for s in mod.STAGES:
        setattr(again, s, lambda s=s, **k: ran.append(s))
    again.run()
    assert ran == []                                     # everything was marked done: nothing runs again


def test_multiview_example_parses_arguments(tmp_path):
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    mod = _load(os.path.join(root, "examples", "multiview.py"), "multiview_example")
    assert callable(mod.main)


def test_robot_dataset_preparation(tmp_path):
    import json
    import tarfile

    import torch

    from cosmos_predict25_b200.utils import video_io
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    mod = _load(os.path.join(root, "scripts", "prepare_robot_video_dataset.py"), "prepare_robot_video_dataset")
    # window planning follows the 5 s / 7.5 s rule
    assert [(round(a), round(b)) for _, a, b in mod.plan_windows(27.0)] == [(0, 5), (5, 10), (10, 15), (15, 20), (20, 27)]
    assert [(round(a), round(b)) for _, a, b in mod.plan_windows(28.0)][-2:] == [(20, 25), (25, 28)]
    assert len(mod.plan_windows(32.0)) == 6 and mod.plan_windows(3.0) == [(0, 0.0, 3.0)]   # 32 s: ..., [20, 25], [25, 32]
    # raw layout: observations/<task>/<episode>/videos/<camera>.mp4 (+ clutter), one episode packed in a tar
    raw = tmp_path / "raw"
    for ep in ("100", "101"):
        d = raw / "observations" / "327" / ep / "videos"
        d.mkdir(parents=True)
        video_io.save_img_or_video(torch.rand(3, 30, 16, 24), str(d / "head"), fps=10)          # 3 s at 10 fps
        video_io.save_img_or_video(torch.rand(3, 4, 16, 24), str(d / "hand_left"), fps=10)
        (raw / "observations" / "327" / ep / "depth").mkdir()
    packed = raw / "observations" / "327" / "101"
    with tarfile.open(raw / "observations" / "327" / "101.tar", "w") as tf:
        tf.add(packed, arcname="101")
    import shutil
    shutil.rmtree(packed)
    out = tmp_path / "prepared"
    (tmp_path / "prepared.jsonl").write_text("\n".join(json.dumps(r) for r in [
        {"video_clip": "task_327_episode_100_window_0_frame_0-9", "caption": "pick the cup", "episode_id": "100"},
        {"video_clip": "task_327_episode_101_window_0_frame_0-9", "caption": "place the cup", "episode_id": "101"},
        {"video_clip": "missing_clip", "caption": "nothing", "episode_id": "100"}]))
    summary = mod.main(["--data-dir", str(raw), "--camera", "head", "--out", str(out), "--val-episode-ids", "101",
                        "--window", "1.0", "--min-last", "1.5"])
    assert summary["archives_extracted"] == 1 and summary["kept_removed"][0] == 2
    assert not (raw / "observations" / "327" / "100" / "depth").exists()
    assert summary["windows"] == {"train": 3, "val": 3}          # 3 s -> [0,1], [1,2], [2,3]
    names = sorted(p.name for p in (out / "train" / "videos").iterdir())
    assert names[0] == "task_327_episode_100_window_0_frame_0-9.mp4" and names[2].endswith("frame_20-29.mp4")
    frames, fps = video_io._read_video(str(out / "train" / "videos" / names[0]))
    assert frames.shape[0] == 10 and abs(fps - 10) < 0.5
    assert summary["captions"] == {"train": 2, "val": 1}
    v = summary["validation"]
    assert v["train"]["matched"] == 1 and v["train"]["videos_without_caption"] == 2 and v["train"]["captions_without_video"] == 1
    assert v["val"]["matched"] == 1
