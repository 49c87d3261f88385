"""Public argument classes of the inference API (same field names, defaults and JSON/YAML format as the reference's
``cosmos_predict2/config.py:15-243``): ``SetupArguments``, ``InferenceArguments``, ``InferenceSample``, ``init_script``. The model registry (``ModelKey``,
``MODEL_CHECKPOINTS`` ...) lives in ``model_registry.py`` and is re-exported here."""

from __future__ import annotations

import enum
import json
import os
from pathlib import Path
from typing import Annotated, Dict, Literal, Optional

import pydantic
import yaml



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


from .model_registry import (DEFAULT_CHECKPOINT, DEFAULT_MODEL_KEY, MODEL_CHECKPOINTS, MODEL_KEYS, ModelKey, ModelSize,  # noqa: E402,F401
                             ModelVariant, get_model_literal)

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
