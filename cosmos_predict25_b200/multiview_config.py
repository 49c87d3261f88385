"""Public arguments of the multiview inference entry point.

Parity target: cosmos_predict2/multiview_config.py (``MultiviewSetupArguments``, ``ViewConfig``,
``MultiviewInferenceArguments``, ``VIEW_INDEX_DICT``).
"""

from __future__ import annotations

from pathlib import Path
from typing import Annotated, Dict, Literal, Optional

import pydantic

from .config import MODEL_CHECKPOINTS, Arguments, ModelKey, ModelVariant, SetupArguments, get_model_literal
from .data.multiview_dataset import VIEW_INDEX_DICT  # noqa: F401  (re-exported)

DEFAULT_MODEL_KEY = ModelKey(variant=ModelVariant.AUTO_MULTIVIEW)
DEFAULT_CHECKPOINT = MODEL_CHECKPOINTS[DEFAULT_MODEL_KEY]
StackMode = Literal["time", "height"]


class MultiviewSetupArguments(SetupArguments):
    model_config = pydantic.ConfigDict(extra="forbid", protected_namespaces=())
    model: get_model_literal(ModelVariant.AUTO_MULTIVIEW) = DEFAULT_MODEL_KEY.name


class ViewConfig(pydantic.BaseModel):
    model_config = pydantic.ConfigDict(extra="forbid")
    video_path: Optional[Path] = None


class MultiviewInferenceArguments(Arguments):
    model_config = pydantic.ConfigDict(extra="forbid")
    prompt: Optional[str] = None
    prompt_path: Optional[Path] = None
    guidance: Annotated[int, pydantic.Field(ge=0, le=7)] = 3
    seed: int = 0
    n_views: int = 7
    num_input_frames: Annotated[int, pydantic.Field(ge=0, le=2)] = 2
    control_weight: Annotated[float, pydantic.Field(ge=0.0, le=1.0)] = 1.0
    stack_mode: StackMode = "time"
    front_wide: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    rear: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    rear_left: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    rear_right: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    cross_left: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    cross_right: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    front_tele: ViewConfig = pydantic.Field(default_factory=ViewConfig)
    fps: pydantic.PositiveInt = 30
    num_steps: pydantic.PositiveInt = 35

    @pydantic.model_validator(mode="after")
    def _load_prompt(self):
        if self.prompt_path is not None:
            self.prompt = Path(self.prompt_path).read_text().strip()
        return self

    @property
    def input_paths(self) -> Dict[str, Optional[Path]]:
        return {name: getattr(self, name).video_path for name in
                ("front_wide", "rear", "rear_left", "rear_right", "cross_left", "cross_right", "front_tele")}
