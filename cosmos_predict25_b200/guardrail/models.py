"""Model-based guardrails as optional plug-ins: each loads its weights from the checkpoint registry when they are present
locally and otherwise declares itself unavailable (the runner then skips it with a warning instead of failing).

  * ``Qwen3Guard`` / ``LlamaGuard3``: LLM prompt classifiers (transformers causal LM + chat template, "unsafe" in the
    generated verdict blocks the prompt).
  * ``VideoContentSafetyFilter``: SigLIP image embeddings of sampled frames -> small MLP classifier; any unsafe frame
    blocks the video.
  * ``RetinaFaceFilter``: face detector; detected faces below a size threshold are pixelated (post-processor).

Parity targets: presets and model wrappers under cosmos_predict2/_src/imaginaire/auxiliary/guardrail/ (qwen3guard, llamaGuard3,
video_content_safety_filter, face_blur_filter)."""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch

from ..utils import log
from ..utils.checkpoint_db import get_checkpoint_path
from .core import ContentSafetyGuardrail, PostprocessingGuardrail


class _LLMGuard(ContentSafetyGuardrail):
    checkpoint = ""

    def __init__(self, offload_model_to_cpu: bool = True, device: str = "cuda"):
        self.available = False
        self.offload = offload_model_to_cpu
        self.device = device if torch.cuda.is_available() else "cpu"
        try:
            from transformers import AutoModelForCausalLM, AutoTokenizer
            path = get_checkpoint_path(self.checkpoint)
            self.tok = AutoTokenizer.from_pretrained(path)
            self.model = AutoModelForCausalLM.from_pretrained(path, torch_dtype=torch.bfloat16).eval()
            self.model.to("cpu" if offload_model_to_cpu else self.device)
            self.available = True
        except Exception as e:
            log.warning(f"{type(self).__name__} unavailable ({type(e).__name__}); prompt classifier skipped")

    @torch.no_grad()
    def is_safe(self, prompt: str) -> Tuple[bool, str]:
        if not self.available:
            return True, "classifier unavailable"
        if self.offload:
            self.model.to(self.device)
        ids = self.tok.apply_chat_template([{"role": "user", "content": prompt}], return_tensors="pt", add_generation_prompt=True)
        out = self.model.generate(ids.to(self.device), max_new_tokens=32, do_sample=False)
        verdict = self.tok.decode(out[0, ids.shape[1]:], skip_special_tokens=True).lower()
        if self.offload:
            self.model.to("cpu")
        return ("unsafe" not in verdict), verdict.strip()


class Qwen3Guard(_LLMGuard):
    checkpoint = "Qwen/Qwen3Guard-Gen-0.6B"


class LlamaGuard3(_LLMGuard):
    checkpoint = "meta-llama/Llama-Guard-3-8B"


class VideoContentSafetyFilter(ContentSafetyGuardrail):
    def __init__(self, offload_model_to_cpu: bool = True, device: str = "cuda", frames_per_video: int = 8):
        self.available = False
        self.n = frames_per_video
        self.device = device if torch.cuda.is_available() else "cpu"
        try:
            import os
            from transformers import SiglipModel, SiglipProcessor
            root = get_checkpoint_path("nvidia/Cosmos-Guardrail1")
            self.proc = SiglipProcessor.from_pretrained(os.path.join(root, "video_content_safety_filter", "siglip"))
            self.enc = SiglipModel.from_pretrained(os.path.join(root, "video_content_safety_filter", "siglip")).eval()
            sd = torch.load(os.path.join(root, "video_content_safety_filter", "safety_filter.pt"), map_location="cpu", weights_only=False)
            dims = [1152, 512, 256, 7]
            self.head = torch.nn.Sequential(*[m for i in range(3) for m in ([torch.nn.Linear(dims[i], dims[i + 1])] + ([torch.nn.ReLU()] if i < 2 else []))])
            self.head.load_state_dict(sd.get("model", sd), strict=False)
            self.available = True
        except Exception as e:
            log.warning(f"VideoContentSafetyFilter unavailable ({type(e).__name__}); video classifier skipped")

    @torch.no_grad()
    def is_safe(self, frames: np.ndarray) -> Tuple[bool, str]:
        if not self.available:
            return True, "classifier unavailable"
        idx = np.linspace(0, len(frames) - 1, min(self.n, len(frames))).astype(int)
        px = self.proc(images=[frames[i] for i in idx], return_tensors="pt")
        emb = self.enc.get_image_features(**px)
        emb = emb / emb.norm(dim=-1, keepdim=True)
        cls = self.head(emb).argmax(-1)
        unsafe = int((cls != 0).sum())
        return unsafe == 0, f"{unsafe} of {len(idx)} sampled frames classified unsafe"


class RetinaFaceFilter(PostprocessingGuardrail):
    """Pixelates detected faces. Uses OpenCV's bundled Haar cascade when the RetinaFace weights are not available."""

    def __init__(self, offload_model_to_cpu: bool = True, pixelation_scale: int = 16, max_face_fraction: float = 0.25):
        self.scale = pixelation_scale
        self.max_frac = max_face_fraction
        self.detector = None
        try:
            import cv2
            self.detector = cv2.CascadeClassifier(cv2.data.haarcascades + "haarcascade_frontalface_default.xml")
            if self.detector.empty():
                self.detector = None
        except Exception:
            self.detector = None
        if self.detector is None:
            log.warning("no face detector available; face blur skipped")

    def postprocess(self, frames: np.ndarray) -> np.ndarray:
        if self.detector is None:
            return frames
        import cv2
        out = frames.copy()
        for t in range(len(out)):
            gray = cv2.cvtColor(out[t], cv2.COLOR_RGB2GRAY)
            for (x, y, w, h) in self.detector.detectMultiScale(gray, 1.1, 5):
                if w * h > self.max_frac * gray.size:
                    continue
                roi = out[t, y:y + h, x:x + w]
                small = cv2.resize(roi, (max(1, w // self.scale), max(1, h // self.scale)), interpolation=cv2.INTER_LINEAR)
                out[t, y:y + h, x:x + w] = cv2.resize(small, (w, h), interpolation=cv2.INTER_NEAREST)
        return out
