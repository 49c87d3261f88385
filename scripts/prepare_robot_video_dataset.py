"""Turn raw robot-episode recordings into the ``videos/`` + ``metas/`` layout that ``VideoDataset`` reads.

Offline counterpart of the reference's AgiBotWorld preparation script (scripts/prepare_agibot_fisheye_data.py:116-711;
the download step needs the Hugging Face hub and is left to the user). Stages, each selectable on its own:

  extract   unpack every ``*.tar`` under ``--data-dir`` next to itself (optionally deleting the archive);
  clean     under ``observations/<task>/<episode>/videos/`` keep only ``<camera>.mp4`` and drop everything else;
  split     cut each kept video into windows of ``--window`` seconds: the tail is one longer window when it is at most
            ``--min-last`` seconds long, two windows otherwise (27 s with 5 s windows: ..., [20, 27]; 28 s: ..., [20, 25],
            [25, 28]); files are named ``task_T_episode_E_window_W_frame_A-B.mp4`` and go to ``<out>/train|val/videos``;
  captions  read ``<out>.jsonl`` (one JSON object per line with ``video_clip``, ``caption``, ``episode_id``) and write
            ``<out>/train|val/metas/<video_clip>.txt``;
  validate  report videos without caption and captions without video per split.

Videos are cut with OpenCV (no ffmpeg binary needed).
"""

import argparse
import json
import os
import shutil
import sys
import tarfile
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def extract_tar_files(data_dir: Path, remove_tar: bool = True) -> int:
    n = 0
    for tar_path in sorted(data_dir.rglob("*.tar")):
        with tarfile.open(tar_path) as tf:
            tf.extractall(tar_path.parent, filter="data")
        if remove_tar:
            tar_path.unlink()
        n += 1
    return n


def clean_observations(data_dir: Path, camera: str, task_ids: Sequence[int] = ()) -> Tuple[int, int]:
    """Returns (kept videos, removed entries)."""
    obs = data_dir / "observations"
    kept = removed = 0
    if not obs.is_dir():
        return kept, removed
    for task in sorted(p for p in obs.iterdir() if p.is_dir()):
        if task_ids and int(task.name) not in set(task_ids):
            continue
        for episode in sorted(p for p in task.iterdir() if p.is_dir()):
            for entry in sorted(episode.iterdir()):
                if entry.name != "videos":
                    shutil.rmtree(entry) if entry.is_dir() else entry.unlink()
                    removed += 1
                    continue
                for f in sorted(entry.iterdir()):
                    if f.name == f"{camera}.mp4":
                        kept += 1
                    else:
                        shutil.rmtree(f) if f.is_dir() else f.unlink()
                        removed += 1
    return kept, removed


def plan_windows(duration: float, window: float = 5.0, min_last: float = 7.5) -> List[Tuple[int, float, float]]:
    """(window id, start, end) in seconds."""
    out, t, wid = [], 0.0, 0
    while t < duration:
        rest = duration - t
        if rest <= window + min_last:
            if rest <= min_last:
                out.append((wid, t, duration))
            else:
                out.append((wid, t, t + window))
                out.append((wid + 1, t + window, duration))
            break
        out.append((wid, t, t + window))
        t += window
        wid += 1
    return out


def split_video_into_windows(video_path: Path, out_dir: Path, task_id, episode_id, window: float = 5.0,
                             min_last: float = 7.5) -> List[Path]:
    import cv2
    cap = cv2.VideoCapture(str(video_path))
    if not cap.isOpened():
        return []
    fps = cap.get(cv2.CAP_PROP_FPS) or 0.0
    total = int(cap.get(cv2.CAP_PROP_FRAME_COUNT))
    if fps <= 0 or total <= 0:
        cap.release()
        return []
    W, H = int(cap.get(cv2.CAP_PROP_FRAME_WIDTH)), int(cap.get(cv2.CAP_PROP_FRAME_HEIGHT))
    out_dir.mkdir(parents=True, exist_ok=True)
    files: List[Path] = []
    frame_idx = 0
    for wid, t0, t1 in plan_windows(total / fps, window, min_last):
        a, b = int(t0 * fps), min(total, int(t1 * fps)) - 1
        path = out_dir / f"task_{task_id}_episode_{episode_id}_window_{wid}_frame_{a}-{b}.mp4"
        wr = cv2.VideoWriter(str(path), cv2.VideoWriter_fourcc(*"mp4v"), fps, (W, H))
        while frame_idx <= b:
            ok, frame = cap.read()
            if not ok:
                break
            if frame_idx >= a:
                wr.write(frame)
            frame_idx += 1
        wr.release()
        files.append(path)
    cap.release()
    return files


def split_videos(data_dir: Path, out_root: Path, camera: str, val_episode_ids: Sequence[str] = (), window: float = 5.0,
                 min_last: float = 7.5) -> Dict[str, int]:
    counts = {"train": 0, "val": 0}
    obs = data_dir / "observations"
    if not obs.is_dir():
        return counts
    val = {str(v) for v in val_episode_ids}
    for task in sorted(p for p in obs.iterdir() if p.is_dir()):
        for episode in sorted(p for p in task.iterdir() if p.is_dir()):
            src = episode / "videos" / f"{camera}.mp4"
            if not src.exists():
                continue
            split = "val" if episode.name in val else "train"
            counts[split] += len(split_video_into_windows(src, out_root / split / "videos", task.name, episode.name, window, min_last))
    return counts


def extract_captions_from_jsonl(jsonl_path: Path, out_root: Path, val_episode_ids: Sequence[str] = ()) -> Dict[str, int]:
    counts = {"train": 0, "val": 0}
    val = {str(v) for v in val_episode_ids}
    for line in jsonl_path.read_text().splitlines():
        if not line.strip():
            continue
        rec = json.loads(line)
        clip, caption = rec.get("video_clip", ""), rec.get("caption", "")
        if not clip or not caption:
            continue
        split = "val" if str(rec.get("episode_id", "")) in val else "train"
        d = out_root / split / "metas"
        d.mkdir(parents=True, exist_ok=True)
        (d / f"{clip}.txt").write_text(caption)
        counts[split] += 1
    return counts


def validate_video_caption_correspondence(out_root: Path) -> Dict[str, Dict[str, List[str]]]:
    report = {}
    for split in ("train", "val"):
        vids = {p.stem for p in (out_root / split / "videos").glob("*.mp4")} if (out_root / split / "videos").is_dir() else set()
        caps = {p.stem for p in (out_root / split / "metas").glob("*.txt")} if (out_root / split / "metas").is_dir() else set()
        report[split] = {"videos_without_caption": sorted(vids - caps), "captions_without_video": sorted(caps - vids),
                         "matched": sorted(vids & caps)}
    return report


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--data-dir", type=Path, default=Path("datasets/agibot/raw"))
    ap.add_argument("--camera", default="head_center_fisheye_color")
    ap.add_argument("--out", type=Path, default=None, help="output root (default: <data-dir>/../agibot_<camera>)")
    ap.add_argument("--task-ids", nargs="*", type=int, default=[])
    ap.add_argument("--val-episode-ids", nargs="*", default=[])
    ap.add_argument("--window", type=float, default=5.0)
    ap.add_argument("--min-last", type=float, default=7.5)
    ap.add_argument("--stages", default="extract,clean,split,captions,validate")
    ap.add_argument("--keep-tar", action="store_true")
    a = ap.parse_args(argv)
    out = a.out or a.data_dir.parent / f"agibot_{a.camera}"
    summary = {}
    stages = [s for s in a.stages.split(",") if s]
    if "extract" in stages:
        summary["archives_extracted"] = extract_tar_files(a.data_dir, remove_tar=not a.keep_tar)
    if "clean" in stages:
        summary["kept_removed"] = clean_observations(a.data_dir, a.camera, a.task_ids)
    if "split" in stages:
        summary["windows"] = split_videos(a.data_dir, out, a.camera, a.val_episode_ids, a.window, a.min_last)
    if "captions" in stages:
        jsonl = Path(str(out) + ".jsonl")
        summary["captions"] = extract_captions_from_jsonl(jsonl, out, a.val_episode_ids) if jsonl.exists() else "no caption file"
    if "validate" in stages:
        rep = validate_video_caption_correspondence(out)
        summary["validation"] = {s: {k: len(v) for k, v in r.items()} for s, r in rep.items()}
    print(json.dumps(summary, indent=1, default=str))
    return summary


if __name__ == "__main__":
    main()
