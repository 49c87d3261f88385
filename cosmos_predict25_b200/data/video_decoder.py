"""Video decoders of the tar-shard dataset stack: which frames of a stored clip become a training sample.

Sampling rules of the reference's decoders (cosmos_predict2/_src/predict2/datasets/decoders/video_decoder.py:40-530):

* clips are stored whole with one caption per ``chunk_size`` frames; a trailing piece of at least half a chunk is a chunk of its
  own (when it still holds the requested number of frames), a shorter one belongs to the last chunk;
* ``chunked_video_decoder``: a random chunk, a random window of ``sequence_length`` consecutive frames inside it; clips whose
  frame rate is outside [min, max] are skipped (the decoder returns None, the pipeline drops the sample);
* ``chunked_video_decoder_w_lower_fps``: frames taken with a stride so that the resulting frame rate stays inside [min, max];
  among the valid strides the largest is taken 99 % of the time, the second largest otherwise.

Decoding itself uses OpenCV (``utils/video_io``) on a temporary file; every decoder returns a dict with the frames as
``uint8 [C, T, H, W]`` plus ``fps``, ``orig_fps``, ``num_frames``, ``chunk_index``, ``frame_start``, ``frame_end``,
``n_orig_video_frames``.
"""

from __future__ import annotations

import os
import re
import tempfile
from random import randint
from typing import Callable, Dict, List, Optional, Tuple

import numpy as np
import torch

VIDEO_EXTENSIONS = ("mp4", "avi", "mov", "mkv", "webm")
VIDEO_DECODER_OPTIONS: Dict[str, Callable] = {}


def video_decoder_register(key: str):
    def deco(fn):
        VIDEO_DECODER_OPTIONS[key] = fn
        return fn
    return deco


def basic_check_on_inputs(n_video_frames: int, n_target_frames: int, video_fps: float, min_fps_thres: int, max_fps_thres: int) -> str:
    """"success" or the reason why the clip cannot give the requested sample."""
    if n_video_frames <= 0:
        return "n_video_frames must be positive"
    if min_fps_thres <= 0:
        return "min_fps_thres must be positive"
    if video_fps < 1:
        return "Video fps lower than 1, skipping"
    if max_fps_thres < min_fps_thres:
        return "max_fps_thres must be greater than or equal to min_fps_thres"
    if n_target_frames <= 1:
        return "sequence_length must be greater than 1"
    if n_target_frames > n_video_frames:
        return f"Specified sequence_length {n_target_frames} exceeds num frames in video {n_video_frames}."
    return "success"


def sample_chunk_index_from_chunked_video(n_video_frames: int, n_target_frames: int, chunk_size: int) -> Tuple[int, int, str]:
    """(chunk index, frames in that chunk, "success") or (-1, 0, reason)."""
    n_chunks = max(n_video_frames // chunk_size, 1)
    tail = n_video_frames - n_chunks * chunk_size
    if tail >= int(0.5 * chunk_size) and tail > n_target_frames:
        n_chunks += 1
    idx = randint(0, n_chunks - 1)
    n_in_chunk = n_video_frames - idx * chunk_size if idx == n_chunks - 1 else chunk_size
    if n_target_frames > n_in_chunk:
        return -1, 0, (f"Requested sequence_length {n_target_frames} exceeds curr_chunk_size {n_in_chunk}, "
                       f"n_video_frames={n_video_frames}, chunk_size={chunk_size}, sampled_chunk_index={idx}.")
    return idx, n_in_chunk, "success"


def get_frame_indices_w_lowered_fps(n_video_frames: int, video_fps: int, min_fps_thres: int, max_fps_thres: int,
                                    n_target_frames: int) -> Tuple[List[int], float]:
    """Evenly strided frame indices whose frame rate ``video_fps / stride`` lies in [min, max]; prefers the largest stride."""
    max_stride = (n_video_frames - 1) // (n_target_frames - 1)
    valid = [s for s in range(1, max_stride + 1)
             if n_video_frames - s * (n_target_frames - 1) > 0 and min_fps_thres <= video_fps / s <= max_fps_thres]
    if not valid:
        raise ValueError(f"No valid stride options available for the given constraints. stride range = [1, {max_stride}]; "
                         f"original FPS = {video_fps}; n_target_frames = {n_target_frames}; min_fps_thres = {min_fps_thres}; "
                         f"max_fps_thres = {max_fps_thres}; original num_frames = {n_video_frames}")
    stride = int(np.random.choice(valid[-2:], p=[0.01, 0.99])) if len(valid) >= 2 else valid[0]
    start = int(np.random.randint(0, n_video_frames - (n_target_frames - 1) * stride))
    return [start + i * stride for i in range(n_target_frames)], video_fps / stride


def _is_video(key: str) -> bool:
    return re.sub(r".*[.]", "", key).lower() in VIDEO_EXTENSIONS


def _open(data: bytes):
    """(cv2 capture, temp path, frame count, rounded fps)."""
    import cv2
    f = tempfile.NamedTemporaryFile(suffix=".mp4", delete=False)
    f.write(data)
    f.close()
    cap = cv2.VideoCapture(f.name)
    return cap, f.name, int(cap.get(cv2.CAP_PROP_FRAME_COUNT)), int(np.round(cap.get(cv2.CAP_PROP_FPS) or 0))


def _read(cap, indices: List[int]) -> Optional[torch.Tensor]:
    import cv2
    want, frames, pos = set(indices), {}, 0
    cap.set(cv2.CAP_PROP_POS_FRAMES, indices[0])
    pos = indices[0]
    while pos <= indices[-1]:
        ok, fr = cap.read()
        if not ok:
            return None
        if pos in want:
            frames[pos] = cv2.cvtColor(fr, cv2.COLOR_BGR2RGB)
        pos += 1
    return torch.from_numpy(np.stack([frames[i] for i in indices])).permute(3, 0, 1, 2).contiguous()      # [C, T, H, W]


def _finish(cap, path):
    cap.release()
    try:
        os.unlink(path)
    except OSError:
        pass


@video_decoder_register("video_naive_bytes")
def video_naive_bytes(*_args, **_kwargs):
    """Leave the bytes alone (a later augmentor decodes)."""
    return lambda key, data: data if _is_video(key) else None


@video_decoder_register("chunked_video_decoder")
def chunked_video_decoder(chunk_size: int = 0, sequence_length: int = 34, min_fps_thres: int = 1, max_fps_thres: int = 9999,
                          num_threads: int = 4):
    def decode(key: str, data: bytes):
        if not _is_video(key):
            return None
        cap, path, n, fps = _open(data)
        try:
            target = sequence_length if sequence_length > 0 else n
            if basic_check_on_inputs(n, target, fps, min_fps_thres, max_fps_thres) != "success" or not min_fps_thres <= fps <= max_fps_thres:
                return None
            cs = n if chunk_size == 0 else chunk_size
            chunk, n_in_chunk, msg = sample_chunk_index_from_chunked_video(n, target, cs)
            if msg != "success":
                return None
            start = chunk * cs + randint(0, n_in_chunk - target)
            frames = _read(cap, list(range(start, start + target)))
            if frames is None:
                return None
            return {"video": frames, "fps": fps, "orig_fps": fps, "num_frames": target, "chunk_index": chunk, "frame_start": start,
                    "frame_end": start + target, "n_orig_video_frames": n}
        finally:
            _finish(cap, path)
    return decode


@video_decoder_register("chunked_video_decoder_w_lower_fps")
def chunked_video_decoder_w_lower_fps(chunk_size: int = 0, sequence_length: int = 34, min_fps_thres: int = 1, max_fps_thres: int = 9999,
                                      num_threads: int = 4):
    def decode(key: str, data: bytes):
        if not _is_video(key):
            return None
        cap, path, n, fps = _open(data)
        try:
            target = sequence_length if sequence_length > 0 else n
            if basic_check_on_inputs(n, target, fps, min_fps_thres, max_fps_thres) != "success":
                return None
            cs = n if chunk_size == 0 else chunk_size
            chunk, n_in_chunk, msg = sample_chunk_index_from_chunked_video(n, target, cs)
            if msg != "success":
                return None
            try:
                rel, new_fps = get_frame_indices_w_lowered_fps(n_in_chunk, fps, min_fps_thres, max_fps_thres, target)
            except ValueError:
                return None
            idx = [chunk * cs + i for i in rel]
            frames = _read(cap, idx)
            if frames is None:
                return None
            return {"video": frames, "fps": new_fps, "orig_fps": fps, "num_frames": target, "chunk_index": chunk,
                    "frame_start": idx[0], "frame_end": idx[-1] + 1, "n_orig_video_frames": n, "frame_indices": idx}
        finally:
            _finish(cap, path)
    return decode


def construct_video_decoder(video_decoder_name: str = "chunked_video_decoder", **kwargs) -> Callable:
    if video_decoder_name not in VIDEO_DECODER_OPTIONS:
        raise ValueError(f"unknown video decoder {video_decoder_name!r}; options: {sorted(VIDEO_DECODER_OPTIONS)}")
    return VIDEO_DECODER_OPTIONS[video_decoder_name](**kwargs)
