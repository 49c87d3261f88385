"""Parameter records built from validator descriptors (``utils/validator.py``).

A subclass lists its parameters as class attributes (``prompt = String()``, ``guidance = Float(7.5, min=5, max=10)``); an
instance is filled from a dict or from a legacy ``--key=value`` command line, every assignment is validated, unknown keys are
rejected and a mandatory parameter (no default) that was not given raises. Subclasses can override a parameter (for example hide
it from the user interface). API of the reference's class of the same name
(cosmos_predict2/_src/imaginaire/utils/validator_params.py:35-183): ``create``, ``createFromCmd``, ``from_kwargs``, ``to_kwargs``,
``validate_kwargs``, ``parse``, ``probe`` / ``probe_ex``, ``get_exposed_params``, ``exposed_params_dict``, ``get_val_dict``,
``debug_print``.
"""

from __future__ import annotations

import shlex
from typing import Any, Dict, List

from .validator import Validator


class ValidatorParams:
    @classmethod
    def get_val_dict(cls) -> Dict[str, Validator]:
        """{name: descriptor} over the class and its bases; a subclass's descriptor replaces the base's of the same name."""
        out: Dict[str, Validator] = {}
        for klass in reversed(cls.__mro__):
            for name, attr in vars(klass).items():
                if isinstance(attr, Validator):
                    out[name] = attr
        return out

    # ---- construction ------------------------------------------------------------------------------------------------------------
    @classmethod
    def create(cls, kwargs: Dict[str, Any]) -> "ValidatorParams":
        """A validated instance; raises ``ValueError`` for unknown keys, bad values and missing mandatory parameters."""
        self = cls()
        self.from_kwargs(kwargs)
        for name in cls.get_val_dict():
            getattr(self, name)                       # a mandatory parameter that is still unset raises here
        return self

    @classmethod
    def createFromCmd(cls, cmd: str) -> "ValidatorParams":
        return cls.create(cls.parse(cmd))

    def from_kwargs(self, kwargs: Dict[str, Any]) -> None:
        known = type(self).get_val_dict()
        for key, value in kwargs.items():
            if key not in known:
                raise ValueError(f"unknown parameter '{key}' for {type(self).__name__}; known: {sorted(known)}")
            try:
                setattr(self, key, value)
            except TypeError as e:                    # one error type for callers, whatever the validator raised
                raise ValueError(str(e)) from e

    def to_kwargs(self) -> Dict[str, Any]:
        return {name: getattr(self, name) for name in type(self).get_val_dict()}

    @classmethod
    def validate_kwargs(cls, kwargs: Dict[str, Any]) -> Dict[str, Any]:
        """The dict after validation and conversion, defaults filled in."""
        return cls.create(kwargs).to_kwargs()

    @staticmethod
    def parse(cmd: str) -> Dict[str, str]:
        """``--prompt='a cat' --num_samples=2`` -> {"prompt": "a cat", "num_samples": "2"} (values stay strings: the validators
        convert them)."""
        out: Dict[str, str] = {}
        for token in shlex.split(cmd):
            if not token.startswith("--"):
                raise ValueError(f"expected --key=value, got {token!r}")
            key, sep, value = token[2:].partition("=")
            out[key] = value if sep else "True"
        return out

    # ---- description (for user interfaces) -----------------------------------------------------------------------------------------
    @classmethod
    def probe(cls) -> List[str]:
        return [f"{name}: {desc!r}" for name, desc in cls.get_val_dict().items()]

    @classmethod
    def probe_ex(cls) -> Dict[str, Any]:
        return {name: desc.json() for name, desc in cls.get_val_dict().items()}

    @classmethod
    def get_exposed_params(cls) -> List[str]:
        return [name for name, desc in cls.get_val_dict().items() if not desc.hidden]

    def exposed_params_dict(self) -> Dict[str, Any]:
        return {name: getattr(self, name) for name in type(self).get_exposed_params()}

    @classmethod
    def debug_print(cls) -> None:
        for line in cls.probe():
            print(line)

    def __str__(self) -> str:
        vals = []
        for name in type(self).get_val_dict():
            try:
                vals.append(f"{name}={getattr(self, name)!r}")
            except ValueError:
                vals.append(f"{name}=<unset>")
        return f"{type(self).__name__}({', '.join(vals)})"

    __repr__ = __str__
