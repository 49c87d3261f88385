"""Guardrail runner: an ordered set of content-safety checks (block or pass) followed by post-processors (modify).

Parity target: ``GuardrailRunner`` / ``ContentSafetyGuardrail`` / ``PostprocessingGuardrail``
(cosmos_predict2/_src/imaginaire/auxiliary/guardrail/common/core.py:37). Guardrails run on rank 0 only and may keep their
models on the CPU between calls (``offload_model_to_cpu``).
"""

from __future__ import annotations

from typing import Any, List, Optional, Tuple

import numpy as np

from ..utils import log


class ContentSafetyGuardrail:
    def is_safe(self, **kwargs) -> Tuple[bool, str]:
        raise NotImplementedError


class PostprocessingGuardrail:
    def postprocess(self, frames: np.ndarray) -> np.ndarray:
        raise NotImplementedError


class GuardrailRunner:
    def __init__(self, safety_models: Optional[List[ContentSafetyGuardrail]] = None, generic_block_msg: str = "",
                 generic_safe_msg: str = "", postprocessors: Optional[List[PostprocessingGuardrail]] = None):
        self.safety_models = safety_models or []
        self.generic_block_msg = generic_block_msg
        self.generic_safe_msg = generic_safe_msg or "Prompt is safe"
        self.postprocessors = postprocessors or []

    def run_safety_check(self, input: Any) -> Tuple[bool, str]:
        """(True, message) when every model accepts; the first rejection stops the chain."""
        for g in self.safety_models:
            name = type(g).__name__
            safe, msg = g.is_safe(input)
            if not safe:
                reason = self.generic_block_msg or f"{name}: {msg}"
                log.critical(f"guardrail {name} blocked the input: {msg}", rank0_only=False)
                return False, reason
        return True, self.generic_safe_msg

    def postprocess(self, frames: np.ndarray) -> np.ndarray:
        for p in self.postprocessors:
            frames = p.postprocess(frames)
        return frames
