"""Registry of released models: which (size, variant, training stage) maps to which checkpoint.

The names are the public ones (``2B/post-trained``, ``14B/pre-trained``, ``2B/auto/multiview`` ...) and the checkpoint ids are
those of the released files, so that parameter files written for the reference select the same weights here
(cosmos_predict2/config.py:69-125). Kept apart from the argument schemas in ``config.py``: this is data, those are schemas.
"""

from __future__ import annotations

import enum
from dataclasses import dataclass
from functools import cached_property
from typing import Dict, Literal

from .utils.checkpoint_db import CheckpointConfig, get_checkpoint_by_uuid


class ModelSize(str, enum.Enum):
    _2B = "2B"
    _14B = "14B"

    def __str__(self):
        return self.value


class ModelVariant(str, enum.Enum):
    BASE = "base"
    AUTO_MULTIVIEW = "auto/multiview"
    ROBOT_MULTIVIEW = "robot/multiview"
    ROBOT_MULTIVIEW_AGIBOT = "robot/multiview-agibot"

    def __str__(self):
        return self.value


@dataclass(frozen=True, kw_only=True)
class ModelKey:
    post_trained: bool = True
    size: ModelSize = ModelSize._2B
    variant: ModelVariant = ModelVariant.BASE

    @cached_property
    def name(self) -> str:
        parts = [str(self.size)]
        parts.append(("post-trained" if self.post_trained else "pre-trained") if self.variant == ModelVariant.BASE else str(self.variant))
        return "/".join(parts)

    def __str__(self):
        return self.name


MODEL_CHECKPOINTS: Dict[ModelKey, CheckpointConfig] = {
    ModelKey(post_trained=False): get_checkpoint_by_uuid("d20b7120-df3e-4911-919d-db6e08bad31c"),
    ModelKey(): get_checkpoint_by_uuid("81edfebe-bd6a-4039-8c1d-737df1a790bf"),
    ModelKey(post_trained=False, size=ModelSize._14B): get_checkpoint_by_uuid("54937b8c-29de-4f04-862c-e67b04ec41e8"),
    ModelKey(variant=ModelVariant.AUTO_MULTIVIEW): get_checkpoint_by_uuid("6b9d7548-33bb-4517-b5e8-60caf47edba7"),
    ModelKey(variant=ModelVariant.ROBOT_MULTIVIEW): get_checkpoint_by_uuid("0e8177cc-0db5-4cfd-a8a4-b820c772f4fc"),
    ModelKey(variant=ModelVariant.ROBOT_MULTIVIEW_AGIBOT): get_checkpoint_by_uuid("7f6b99b7-7fac-4e74-8dbe-a394cb56ef99"),
}
MODEL_KEYS = {k.name: k for k in MODEL_CHECKPOINTS}


def get_model_literal(variant: ModelVariant = ModelVariant.BASE):
    return Literal[tuple(k.name for k in MODEL_CHECKPOINTS if k.variant == variant)]


DEFAULT_MODEL_KEY = ModelKey()
DEFAULT_CHECKPOINT = MODEL_CHECKPOINTS[DEFAULT_MODEL_KEY]
