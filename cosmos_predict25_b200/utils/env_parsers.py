"""Environment-variable parsers built from validators.

Parity target: ``EnvParser`` (cosmos_predict2/_src/imaginaire/utils/env_parsers/env_parser.py:38-140) and its subclasses
``CredentialEnvParser`` / ``InferenceEnvParser`` / ``CustomizationEnvParser`` (.../env_parsers/*.py): a class whose validator
attributes are filled from upper-cased environment variables, a json file or a base64 json blob, with a mandatory-value
check and round-trips to json / base64 / a string dict.
"""

from __future__ import annotations

import base64
import json
import os
from typing import Dict

from . import log
from .validator import Bool, Int, JsonDict, String, Validator


class EnvParser:
    def __init__(self, b64_str: str | None = None):
        if b64_str:
            self.from_b64(b64_str)
        else:
            self.from_env()

    @classmethod
    def get_val_dict(cls) -> Dict[str, Validator]:
        out: Dict[str, Validator] = {}
        for klass in reversed(cls.__mro__):
            out.update({k: v for k, v in klass.__dict__.items() if isinstance(v, Validator)})
        return out

    def from_env(self):
        for key in self.get_val_dict():
            val = os.getenv(key.upper())
            if val:
                setattr(self, key, val)
        self.check_mandatory_values()

    def _from_dict(self, d: dict):
        known = {k.upper(): k for k in self.get_val_dict()}
        for key, value in d.items():
            if key.upper() in known:
                setattr(self, known[key.upper()], value)
        self.check_mandatory_values()

    def from_json(self, file_name: str):
        with open(file_name) as f:
            self._from_dict(json.load(f))

    def from_b64(self, b64_str: str):
        self._from_dict(json.loads(base64.b64decode(b64_str).decode()))

    def check_mandatory_values(self):
        for key, validator in self.get_val_dict().items():
            try:
                val = getattr(self, key)
            except ValueError as e:
                raise ValueError(f"Missing mandatory env var: {key}") from e
            if val is None and validator.default is None:
                raise ValueError(f"Missing mandatory env var: {key}")

    def to_dict(self) -> dict:
        return {key.upper(): getattr(self, key) for key in self.get_val_dict()}

    def to_json(self, file_name: str | None = None) -> str:
        s = json.dumps(self.to_dict(), indent=4)
        if file_name:
            with open(file_name, "w") as f:
                f.write(s)
            log.info(f"wrote env params to {file_name}")
        return s

    def to_b64(self) -> str:
        return base64.b64encode(self.to_json().encode()).decode()

    def to_string_dict(self) -> Dict[str, str]:
        out = {}
        for key, validator in self.get_val_dict().items():
            value = getattr(self, key)
            out[key] = json.dumps(value) if isinstance(validator, JsonDict) else str(value)
        return out

    def __str__(self):
        return ", ".join(f"{k}={v}" for k, v in self.to_dict().items())


class CredentialEnvParser(EnvParser):
    APP_ENV = String(default="")
    PROD_FT_AWS_CREDS_ACCESS_KEY_ID = String(default="")
    PROD_FT_AWS_CREDS_SECRET_ACCESS_KEY = String(default="")
    PROD_FT_AWS_CREDS_ENDPOINT_URL = String(default="https://s3.us-west-2.amazonaws.com")
    PROD_FT_AWS_CREDS_REGION_NAME = String(default="us-west-2")
    PROD_S3_CHECKPOINT_ACCESS_KEY_ID = String(default="")
    PROD_S3_CHECKPOINT_SECRET_ACCESS_KEY = String(default="")
    PROD_S3_CHECKPOINT_ENDPOINT_URL = String(default="")
    PROD_S3_CHECKPOINT_REGION_NAME = String(default="")
    PROD_TEAM_DIR_ACCESS_KEY_ID = String(default="")
    PROD_TEAM_DIR_SECRET_ACCESS_KEY = String(default="")
    PROD_TEAM_DIR_ENDPOINT_URL = String(default="")
    PROD_TEAM_DIR_REGION_NAME = String(default="")

    def credentials(self, prefix: str) -> Dict[str, str]:
        """boto3 keyword arguments of one credential family (``PROD_FT_AWS_CREDS`` / ``PROD_S3_CHECKPOINT`` / ``PROD_TEAM_DIR``)."""
        return {"aws_access_key_id": getattr(self, f"{prefix}_ACCESS_KEY_ID"), "aws_secret_access_key": getattr(self, f"{prefix}_SECRET_ACCESS_KEY"),
                "endpoint_url": getattr(self, f"{prefix}_ENDPOINT_URL"), "region_name": getattr(self, f"{prefix}_REGION_NAME")}


class InferenceEnvParser(EnvParser):
    MODEL_NAME = String(default="")
    CHECKPOINT_PATH = String(default="")
    NUM_GPUS = Int(default=1, min=1, max=8)
    OUTPUT_DIR = String(default="outputs")
    DISABLE_GUARDRAILS = Bool(default=False)
    OFFLOAD_GUARDRAIL_MODELS = Bool(default=False)


class CustomizationEnvParser(EnvParser):
    EXPERIMENT = String(default="")
    DATASET_DIR = String(default="")
    MAX_ITER = Int(default=1000, min=1)
    NUM_GPUS = Int(default=8, min=1)
    OVERRIDES = JsonDict(default={})
