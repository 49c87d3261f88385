"""Stock guardrail line-ups (parity: cosmos_predict2/_src/imaginaire/auxiliary/guardrail/common/presets.py:28-75):
text = blocklist + Qwen3Guard; video = SigLIP content-safety classifier + face blur."""

from __future__ import annotations

from typing import Optional

import numpy as np

from ..utils import log
from .blocklist import Blocklist
from .core import GuardrailRunner


def create_text_guardrail_runner(offload_model_to_cpu: bool = False, with_llm: bool = True) -> GuardrailRunner:
    models = [Blocklist()]
    if with_llm:
        from .models import Qwen3Guard
        g = Qwen3Guard(offload_model_to_cpu=offload_model_to_cpu)
        if g.available:
            models.append(g)
    return GuardrailRunner(safety_models=models, generic_block_msg="")


def create_video_guardrail_runner(offload_model_to_cpu: bool = False) -> GuardrailRunner:
    from .models import RetinaFaceFilter, VideoContentSafetyFilter
    v = VideoContentSafetyFilter(offload_model_to_cpu=offload_model_to_cpu)
    return GuardrailRunner(safety_models=[v] if v.available else [], postprocessors=[RetinaFaceFilter(offload_model_to_cpu)])


def run_text_guardrail(prompt: str, runner: GuardrailRunner) -> bool:
    safe, msg = runner.run_safety_check(prompt)
    if not safe:
        log.critical(f"GUARDRAIL BLOCKED: {msg}")
    return safe


def run_video_guardrail(frames: np.ndarray, runner: GuardrailRunner) -> Optional[np.ndarray]:
    """frames uint8 [T,H,W,3]; None when blocked, otherwise the post-processed frames."""
    safe, msg = runner.run_safety_check(frames)
    if not safe:
        log.critical(f"GUARDRAIL BLOCKED: {msg}")
        return None
    return runner.postprocess(frames)
