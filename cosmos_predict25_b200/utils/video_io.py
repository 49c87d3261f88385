"""Reading conditioning images / videos and writing generated ones.

Parity targets: ``read_and_process_image`` / ``read_and_process_video`` / ``resize_input``
(cosmos_predict2/_src/predict2/inference/video2world.py:121-279) and ``save_img_or_video``
(cosmos_predict2/_src/imaginaire/visualize/video.py:45-97). Decoding/encoding goes through OpenCV (the only
video library on the image); a GPU never touches these paths.
"""

from __future__ import annotations

import os
from typing import Optional, Tuple

import numpy as np
import torch

IMAGE_EXT = (".png", ".jpg", ".jpeg", ".webp", ".bmp")
VIDEO_EXT = (".mp4", ".mov", ".avi", ".mkv", ".webm")


def resize_input(video: torch.Tensor, resolution: Tuple[int, int]) -> torch.Tensor:
    """Aspect-preserving resize (cover) then center crop. video [..., H, W] float or uint8."""
    import torch.nn.functional as F
    H, W = video.shape[-2:]
    th, tw = resolution
    scale = max(th / H, tw / W)
    nh, nw = int(np.ceil(scale * H)), int(np.ceil(scale * W))
    lead = video.shape[:-2]
    x = video.reshape(-1, 1, H, W).float()
    x = F.interpolate(x, size=(nh, nw), mode="bilinear", align_corners=False, antialias=True)
    # offsets rounded half-to-even like torchvision's center_crop, which the reference calls (an odd margin puts the extra pixel first)
    top, left = int(round((nh - th) / 2.0)), int(round((nw - tw) / 2.0))
    x = x[..., top:top + th, left:left + tw]
    x = x.reshape(*lead, th, tw)
    return x.round().clamp(0, 255).to(torch.uint8) if video.dtype == torch.uint8 else x


def _read_image(path: str) -> np.ndarray:
    from PIL import Image
    return np.asarray(Image.open(path).convert("RGB"))


def _read_video(path: str, max_frames: Optional[int] = None) -> Tuple[np.ndarray, float]:
    import cv2
    cap = cv2.VideoCapture(path)
    if not cap.isOpened():
        raise FileNotFoundError(f"cannot open video {path}")
    fps = cap.get(cv2.CAP_PROP_FPS) or 0.0
    frames = []
    while True:
        ok, f = cap.read()
        if not ok:
            break
        frames.append(cv2.cvtColor(f, cv2.COLOR_BGR2RGB))
        if max_frames is not None and len(frames) >= max_frames:
            break
    cap.release()
    if not frames:
        raise ValueError(f"video {path} has no decodable frames")
    return np.stack(frames), float(fps)


def read_and_process_image(img_path: str, resolution: Tuple[int, int], num_video_frames: int, resize: bool = True) -> torch.Tensor:
    """Image -> uint8 [1, 3, T, H, W]: the image is frame 0, the rest of the clip is zero (to be generated)."""
    ext = os.path.splitext(img_path)[1].lower()
    if ext not in IMAGE_EXT:
        raise ValueError(f"unsupported image extension {ext}")
    img = torch.from_numpy(_read_image(img_path)).permute(2, 0, 1).unsqueeze(0)  # [1,3,H,W] uint8
    if resize:
        img = resize_input(img, resolution)
    H, W = img.shape[-2:]
    vid = torch.zeros(1, 3, num_video_frames, H, W, dtype=torch.uint8)
    vid[:, :, 0] = img
    return vid


def read_and_process_video(video_path: str, resolution: Tuple[int, int], num_video_frames: int,
                           num_latent_conditional_frames: int = 2, resize: bool = True) -> torch.Tensor:
    """Video -> uint8 [1, 3, T, H, W]: the LAST 4(n-1)+1 frames of the clip become the first frames of the
    output, the remainder is padded with the last of those frames."""
    ext = os.path.splitext(video_path)[1].lower()
    if ext not in VIDEO_EXT:
        raise ValueError(f"unsupported video extension {ext}")
    frames, _ = _read_video(video_path)
    frames = torch.from_numpy(frames).permute(3, 0, 1, 2)  # [3, T, H, W]
    need = 4 * (num_latent_conditional_frames - 1) + 1
    if frames.shape[1] < need:
        raise ValueError(f"video has {frames.shape[1]} frames; {need} are needed for {num_latent_conditional_frames} latent frames")
    cond = frames[:, -need:]
    if resize:
        cond = resize_input(cond, resolution)
    C, _, H, W = cond.shape
    out = torch.zeros(1, C, num_video_frames, H, W, dtype=torch.uint8)
    out[0, :, :need] = cond
    out[0, :, need:] = cond[:, -1:].expand(-1, num_video_frames - need, -1, -1)
    return out


def save_img_or_video(sample_C_T_H_W_in01: torch.Tensor, save_fp_wo_ext: str, fps: int = 24, quality: Optional[int] = None) -> str:
    """[C,T,H,W] in [0,1]: T == 1 -> ``.jpg``; otherwise ``.mp4`` (mp4v through OpenCV). Returns the path."""
    x = sample_C_T_H_W_in01.detach().float().clamp(0, 1).cpu()
    assert x.ndim == 4 and x.shape[0] in (1, 3), f"expected [C,T,H,W], got {tuple(x.shape)}"
    os.makedirs(os.path.dirname(os.path.abspath(save_fp_wo_ext)) or ".", exist_ok=True)
    arr = (x * 255.0 + 0.5).to(torch.uint8).permute(1, 2, 3, 0).numpy()  # T,H,W,C
    if arr.shape[-1] == 1:
        arr = np.repeat(arr, 3, axis=-1)
    if arr.shape[0] == 1:
        from PIL import Image
        path = save_fp_wo_ext + ".jpg"
        Image.fromarray(arr[0]).save(path, quality=quality or 85)
        return path
    import cv2
    path = save_fp_wo_ext + ".mp4"
    H, W = arr.shape[1:3]
    wr = cv2.VideoWriter(path, cv2.VideoWriter_fourcc(*"mp4v"), float(fps), (W, H))
    if not wr.isOpened():
        raise RuntimeError(f"cannot open video writer for {path}")
    for f in arr:
        wr.write(cv2.cvtColor(f, cv2.COLOR_RGB2BGR))
    wr.release()
    return path
