"""Public argument classes of the inference API (same field names, defaults and JSON/YAML format as the reference's
``cosmos_predict2/config.py:15-243``): ``SetupArguments``, ``InferenceArguments``, ``InferenceSample``, ``ModelKey``,
``MODEL_CHECKPOINTS``, ``init_script``."""

from __future__ import annotations

import enum
import json
import os
from dataclasses import dataclass
from functools import cached_property
from pathlib import Path
from typing import Annotated, Dict, Literal, Optional

import pydantic
import yaml

from .utils.checkpoint_db import CheckpointConfig, get_checkpoint_by_uuid


def init_script():
    """Initialise the script environment: tokenizer threads off, process group from the torchrun environment."""
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    if "RANK" in os.environ:
        from .utils import distributed
        distributed.init()


def _resolve_path(v: Path) -> Path:
    return v.expanduser().resolve()


ResolvedFilePath = Annotated[pydantic.FilePath, pydantic.AfterValidator(_resolve_path)]


class Arguments(pydantic.BaseModel):
    @classmethod
    def from_file(cls, path: Path):
        """Load from a json / yaml file; relative input paths are resolved against the file's directory."""
        path = Path(path)
        if path.suffix == ".json":
            data = json.loads(path.read_text())
        elif path.suffix in (".yaml", ".yml"):
            data = yaml.safe_load(path.read_text())
        else:
            raise ValueError(f"Unsupported file extension: {path.suffix}")
        cwd = os.getcwd()
        os.chdir(path.parent or ".")
        try:
            return cls.model_validate(data)
        finally:
            os.chdir(cwd)


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
DEFAULT_NEGATIVE_PROMPT = ("The video captures a series of frames showing ugly scenes, static with no motion, motion blur, "
                           "over-saturation, shaky footage, low resolution, grainy texture, pixelated images, poorly lit areas, "
                           "underexposed and overexposed scenes, poor color balance, washed out colors, choppy sequences, jerky "
                           "movements, low frame rate, artifacting, color banding, unnatural transitions, outdated special effects, "
                           "fake elements, unconvincing visuals, poorly edited content, jump cuts, visual noise, and flickering. "
                           "Overall, the video is of poor quality.")


class SetupArguments(Arguments):
    """Common arguments for model setup."""

    model_config = pydantic.ConfigDict(extra="forbid", protected_namespaces=())
    output_dir: Path
    model: get_model_literal() = DEFAULT_MODEL_KEY.name
    checkpoint_path: Optional[str] = None
    experiment: Optional[str] = None
    context_parallel_size: Optional[pydantic.PositiveInt] = None
    disable_guardrails: bool = False
    offload_guardrail_models: bool = False

    @property
    def enable_guardrails(self) -> bool:
        return not self.disable_guardrails

    @property
    def model_key(self) -> ModelKey:
        return MODEL_KEYS[self.model]

    @pydantic.model_validator(mode="after")
    def _fill_from_model_key(self):
        ck = MODEL_CHECKPOINTS[self.model_key]
        if self.checkpoint_path is None:
            self.checkpoint_path = ck.s3_uri or ck.uuid
        if self.experiment is None:
            if ck.experiment is None:
                raise ValueError(f"Experiment name is not set for {ck.name}")
            self.experiment = ck.experiment
        if self.context_parallel_size is None:
            self.context_parallel_size = int(os.environ.get("WORLD_SIZE", "1"))
        return self


class InferenceType(str, enum.Enum):
    TEXT2WORLD = "text2world"
    IMAGE2WORLD = "image2world"
    VIDEO2WORLD = "video2world"

    def __str__(self):
        return self.value


class InferenceSample(pydantic.BaseModel):
    model_config = pydantic.ConfigDict(extra="forbid")
    prompt: Optional[str] = None
    prompt_path: Optional[ResolvedFilePath] = None
    input_path: Optional[ResolvedFilePath] = None

    @pydantic.model_validator(mode="after")
    def _read_prompt(self):
        if self.prompt_path is not None:
            self.prompt = self.prompt_path.read_text().strip()
        return self


class InferenceArguments(Arguments):
    """Arguments for base model inference."""

    model_config = pydantic.ConfigDict(extra="forbid")
    inference_type: InferenceType
    samples: Dict[str, InferenceSample]
    negative_prompt: str = DEFAULT_NEGATIVE_PROMPT
    seed: int = 1
    guidance: Annotated[int, pydantic.Field(ge=0, le=7)] = 7
    resolution: str = "none"
    num_output_frames: pydantic.PositiveInt = 77

    @pydantic.model_validator(mode="after")
    def _check_inputs(self):
        if self.inference_type != InferenceType.TEXT2WORLD:
            for s in self.samples.values():
                if s.input_path is None:
                    raise ValueError("Input file is required")
        return self

    @property
    def num_input_frames(self) -> int:
        return {InferenceType.TEXT2WORLD: 0, InferenceType.IMAGE2WORLD: 1, InferenceType.VIDEO2WORLD: 2}[self.inference_type]
