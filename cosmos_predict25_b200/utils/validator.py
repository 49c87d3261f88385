"""Typed, range-checked parameter descriptors for request / environment classes.

Parity target: cosmos_predict2/_src/imaginaire/utils/validator.py:35-520 (``Validator`` descriptor protocol and the
``Bool`` / ``Int`` / ``Float`` / ``String`` / ``Path`` / ``InputImage`` / ``JsonDict`` / ``Dict`` / ``OneOf`` / ``MultipleOf`` /
``HumanAttributes`` / ``BytesIOType`` kinds). A validator is a class attribute: assignment validates and converts, reading
returns the value or the default, reading an unset mandatory parameter raises; ``json()`` describes the parameter (for UI
generation) and ``get_range_iterator()`` enumerates representative values (for sweep tests).
"""

from __future__ import annotations

import base64
import io
import itertools
import json as _json
import os
from abc import ABC, abstractmethod

_UNSET = object()


class Validator(ABC):
    def __init__(self, default=_UNSET, hidden=False, tooltip=None):
        self.default, self.hidden, self.tooltip = default, hidden, tooltip

    def __set_name__(self, owner, name):
        self.private_name = "_" + name

    def __get__(self, obj, objtype=None):
        if obj is None:
            return self
        value = getattr(obj, self.private_name, self.default)
        if value is _UNSET:
            raise ValueError(f"Parameter '{self.private_name.lstrip('_')}' is mandatory but has not been set. "
                             "No default value was provided and no value was assigned.")
        return value

    def __set__(self, obj, value):
        setattr(obj, self.private_name, self.validate(value))

    @abstractmethod
    def validate(self, value): ...

    def get_range_iterator(self):
        return iter([self.default])

    def _base_json(self, type_name):
        return {"type": type_name, "default": None if self.default is _UNSET else self.default, "tooltip": self.tooltip}

    def json(self):
        return self._base_json(type(self).__name__)


class Bool(Validator):
    def validate(self, value):
        if isinstance(value, int):
            value = value != 0
        elif isinstance(value, str):
            v = value.lower()
            if v in ("true", "1"):
                value = True
            elif v in ("false", "0"):
                value = False
            else:
                raise ValueError(f"Expected {value!r} to be one of ['True', 'False', '1', '0']")
        elif not isinstance(value, bool):
            raise TypeError(f"Expected {value!r} to be an bool")
        return value

    def get_range_iterator(self):
        return iter([True, False])

    def __repr__(self):
        return f"Bool({self.private_name=!s} {self.default=} {self.hidden=})"

    def json(self):
        return self._base_json(bool.__name__)


class _Number(Validator):
    cast, type_name = int, "int"

    def __init__(self, default=_UNSET, min=None, max=None, step=1, hidden=False, tooltip=None):
        super().__init__(default, hidden, tooltip)
        self.min, self.max, self.step = min, max, step

    def validate(self, value):
        if isinstance(value, str) or (self.cast is float and isinstance(value, int)):
            value = self.cast(value)
        if not isinstance(value, self.cast) or isinstance(value, bool):
            raise TypeError(f"Expected {value!r} to be an {self.type_name}")
        if self.min is not None and value < self.min:
            raise ValueError(f"Expected {value!r} to be at least {self.min!r}")
        if self.max is not None and value > self.max:
            raise ValueError(f"Expected {value!r} to be no more than {self.max!r}")
        return value

    def get_range_iterator(self):
        lo = self.min if self.min is not None else self.default
        hi = self.max if self.max is not None else self.default
        if lo is _UNSET or hi is _UNSET:
            return iter([])
        n = int((hi - lo) / self.step) + 1
        return iter(self.cast(lo + i * self.step) for i in range(n))

    def __repr__(self):
        return f"{type(self).__name__}({self.private_name=!s} {self.default=}, {self.min=}, {self.max=} {self.hidden=})"

    def json(self):
        return dict(self._base_json(self.type_name), min=self.min, max=self.max, step=self.step)


class Int(_Number):
    cast, type_name = int, "int"


class Float(_Number):
    cast, type_name = float, "float"

    def __init__(self, default=_UNSET, min=None, max=None, step=0.5, hidden=False, tooltip=None):
        super().__init__(default, min, max, step, hidden, tooltip)


class String(Validator):
    def __init__(self, default=_UNSET, min=None, max=None, predicate=None, hidden=False, tooltip=None):
        super().__init__(default, hidden, tooltip)
        self.min, self.max, self.predicate = min, max, predicate

    def validate(self, value):
        if value is None:
            return value
        if not isinstance(value, str):
            raise TypeError(f"Expected {value!r} to be an str")
        if self.min is not None and len(value) < self.min:
            raise ValueError(f"Expected {value!r} to be no smaller than {self.min!r}")
        if self.max is not None and len(value) > self.max:
            raise ValueError(f"Expected {value!r} to be no bigger than {self.max!r}")
        if self.predicate is not None and not self.predicate(value):
            raise ValueError(f"Expected {self.predicate} to be true for {value!r}")
        return value

    def __repr__(self):
        return f"String({self.private_name=!s} {self.default=}, {self.min=}, {self.max=} {self.hidden=})"

    def json(self):
        return self._base_json(str.__name__)


class Path(Validator):
    def validate(self, value):
        if not isinstance(value, str):
            raise TypeError(f"Expected {value!r} to be an str")
        if not os.path.exists(value):
            raise ValueError(f"Expected {value!r} to be a valid path")
        return value

    def __repr__(self):
        return f"Path({self.private_name=!s} {self.default=} {self.hidden=})"


class InputImage(Validator):
    def __init__(self, default=_UNSET, hidden=False, tooltip=None, formats=("jpg", "jpeg", "png", "webp")):
        super().__init__(default, hidden, tooltip)
        self.formats = tuple(formats)

    def validate(self, value):
        if not isinstance(value, str):
            raise TypeError(f"Expected {value!r} to be an str")
        if not value.lower().endswith(tuple("." + f for f in self.formats)):
            raise ValueError(f"Expected {value!r} to be an image of one of {self.formats}")
        return value

    def json(self):
        return dict(self._base_json("image"), values=list(self.formats))


class JsonDict(Validator):
    """A dict, given as a dict or as its json text."""

    def validate(self, value):
        if isinstance(value, str):
            value = _json.loads(value)
        if not isinstance(value, dict):
            raise TypeError(f"Expected {value!r} to be a dict or a json string of one")
        return value

    def __repr__(self):
        return f"JsonDict({self.private_name=!s} {self.default=} {self.hidden=})"


class Dict(Validator):
    def validate(self, value):
        if not isinstance(value, dict):
            raise TypeError(f"Expected {value!r} to be a dict")
        return value


class OneOf(Validator):
    def __init__(self, default=_UNSET, options=None, type_cast=None, hidden=False, tooltip=None):
        super().__init__(default, hidden, tooltip)
        self.options, self.type_cast = set(options or []), type_cast

    def validate(self, value):
        if self.type_cast:
            value = self.type_cast(value)
        if value not in self.options:
            raise ValueError(f"Expected {value!r} to be one of {self.options!r}")
        return value

    def get_range_iterator(self):
        return iter(self.options)

    def json(self):
        return dict(self._base_json("OneOf"), values=sorted(self.options, key=str))


class MultipleOf(Validator):
    def __init__(self, default=_UNSET, multiple_of: int = 1, type_cast=None, hidden=False, tooltip=None):
        super().__init__(default, hidden, tooltip)
        if type(multiple_of) is not int:
            raise ValueError(f"Expected {multiple_of!r} to be an int")
        self.multiple_of, self.type_cast = multiple_of, type_cast

    def validate(self, value):
        if self.type_cast:
            value = self.type_cast(value)
        if value % self.multiple_of != 0:
            raise ValueError(f"Expected {value!r} to be a multiple of {self.multiple_of!r}")
        return value

    def get_range_iterator(self):
        return iter([self.multiple_of, self.multiple_of * 2])

    def json(self):
        return dict(self._base_json("MultipleOf"), multiple_of=self.multiple_of)


class HumanAttributes(Validator):
    """A comma-separated ``key:value`` string over a fixed vocabulary of attributes."""

    VOCAB = {"emotion": ["angry", "contemptful", "disgusted", "fearful", "happy", "neutral", "sad", "surprised"],
             "race": ["asian", "indian", "black", "white", "middle eastern", "latino hispanic"],
             "gender": ["male", "female"], "age group": ["young", "teen", "adult early twenties", "adult late twenties",
                                                          "adult early thirties", "adult late thirties", "adult middle aged", "older adult"]}

    def get_range_iterator(self):
        keys = list(self.VOCAB)
        return iter(",".join(f"{k}:{v}" for k, v in zip(keys, combo)) for combo in itertools.product(*[self.VOCAB[k] for k in keys]))

    def validate(self, value):
        for pair in str(value).split(","):
            k, _, v = pair.partition(":")
            k, v = k.strip(), v.strip()
            if k not in self.VOCAB or v not in self.VOCAB[k]:
                raise ValueError(f"Expected attribute {k!r}={v!r} to be in {self.VOCAB}")
        return value


class BytesIOType(Validator):
    """Binary payload: ``bytes``, a ``BytesIO`` or base64 text -> ``BytesIO``."""

    def validate(self, value):
        if isinstance(value, str):
            value = base64.b64decode(value)
        if isinstance(value, (bytes, bytearray)):
            value = io.BytesIO(value)
        if not isinstance(value, io.BytesIO):
            raise TypeError(f"Expected {value!r} to be bytes, BytesIO or a base64 string")
        return value
