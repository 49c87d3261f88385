"""Deferred construction: ``L(cls)(**kwargs)`` records a call as a plain nested dict (``_target_`` + kwargs)
that can be printed, overridden from the command line, serialised to YAML and instantiated later.

Parity targets: ``LazyCall`` / ``LazyConfig`` (cosmos_predict2/_src/imaginaire/lazy_config/lazy.py:87-230) and
``instantiate`` (cosmos_predict2/_src/imaginaire/lazy_config/instantiate.py:56-120, including the
``_recursive_=False`` switch). Self-contained: no omegaconf / hydra.
"""

from __future__ import annotations

import copy
import importlib
import inspect
from collections.abc import Mapping
from typing import Any, Callable, Dict

import yaml


class LazyDict(dict):
    """A dict with attribute access; nested dicts are promoted on read."""

    def __getattr__(self, k):
        try:
            v = self[k]
        except KeyError as e:
            raise AttributeError(k) from e
        if isinstance(v, dict) and not isinstance(v, LazyDict):
            v = LazyDict(v)
            self[k] = v
        return v

    def __setattr__(self, k, v):
        self[k] = v

    def __delattr__(self, k):
        del self[k]

    def __deepcopy__(self, memo):
        return LazyDict({k: copy.deepcopy(v, memo) for k, v in self.items()})


def _locate(path: str) -> Any:
    """Import ``pkg.mod.attr`` (tries progressively shorter module prefixes)."""
    parts = path.split(".")
    for i in range(len(parts), 0, -1):
        try:
            obj = importlib.import_module(".".join(parts[:i]))
        except ImportError:
            continue
        for p in parts[i:]:
            obj = getattr(obj, p)
        return obj
    raise ImportError(f"cannot locate {path!r}")


def _to_path(target: Any) -> str:
    if isinstance(target, str):
        return target
    return f"{target.__module__}.{target.__qualname__}"


class LazyCall:
    """``LazyCall(Foo)(a=1, b=LazyCall(Bar)())`` -> LazyDict(_target_=Foo, a=1, b={...})."""

    def __init__(self, target: Callable | str):
        if not (callable(target) or isinstance(target, (str, Mapping))):
            raise TypeError(f"target of LazyCall must be callable or a dotted path, got {target!r}")
        self._target = target

    def __call__(self, **kwargs) -> LazyDict:
        d = LazyDict(_target_=self._target)
        # fill defaults of the signature so that every tunable shows up in dumps and can be overridden
        try:
            sig = inspect.signature(self._target if callable(self._target) else _locate(self._target))
            for name, p in sig.parameters.items():
                if p.default is not inspect.Parameter.empty and name not in kwargs and p.kind in (
                        p.POSITIONAL_OR_KEYWORD, p.KEYWORD_ONLY) and isinstance(p.default, (int, float, str, bool, type(None))):
                    d[name] = p.default
        except (TypeError, ValueError):
            pass
        d.update(kwargs)
        return d


L = LazyCall


def is_lazy(x: Any) -> bool:
    return isinstance(x, Mapping) and "_target_" in x


def instantiate(cfg: Any, *args, **kwargs) -> Any:
    """Recursively build the object a LazyDict describes. Extra kwargs override recorded ones.
    ``_recursive_: False`` passes nested LazyDicts through un-instantiated. Lists/tuples/dicts are walked."""
    if cfg is None:
        return None
    if isinstance(cfg, (list, tuple)):
        return type(cfg)(instantiate(x) for x in cfg)
    if isinstance(cfg, Mapping) and not is_lazy(cfg):
        return type(cfg)((k, instantiate(v)) for k, v in cfg.items()) if not isinstance(cfg, LazyDict) \
            else LazyDict({k: instantiate(v) for k, v in cfg.items()})
    if not is_lazy(cfg):
        return cfg
    params = {k: v for k, v in cfg.items() if k not in ("_target_", "_recursive_", "_partial_")}
    params.update(kwargs)
    target = cfg["_target_"]
    if isinstance(target, str):
        target = _locate(target)
    recursive = cfg.get("_recursive_", True)
    if recursive:
        params = {k: instantiate(v) for k, v in params.items()}
    if cfg.get("_partial_", False):
        import functools
        return functools.partial(target, *args, **params)
    try:
        return target(*args, **params)
    except Exception as e:
        raise type(e)(f"while instantiating {_to_path(target)}: {e}") from e


def _plain(x: Any) -> Any:
    """YAML-friendly form: classes/functions become dotted paths, dtypes/enums tagged strings."""
    import enum

    import torch
    if isinstance(x, Mapping):
        return {str(k): _plain(v) for k, v in x.items()}
    if isinstance(x, (list, tuple)):
        return [_plain(v) for v in x]
    if isinstance(x, torch.dtype):
        return {"__type__": "torch.dtype", "__value__": str(x)}
    if isinstance(x, enum.Enum):
        return {"__type__": _to_path(type(x)), "__value__": x.name}
    if inspect.isclass(x) or inspect.isfunction(x) or inspect.isbuiltin(x):
        return _to_path(x)
    if isinstance(x, (int, float, str, bool, type(None))):
        return x
    if hasattr(x, "__dataclass_fields__"):
        import dataclasses
        return {"__type__": _to_path(type(x)), **{f.name: _plain(getattr(x, f.name)) for f in dataclasses.fields(x)}}
    return repr(x)


class LazyConfig:
    @staticmethod
    def to_yaml(cfg: Any) -> str:
        return yaml.safe_dump(_plain(cfg), sort_keys=False, default_flow_style=False)

    @staticmethod
    def save_yaml(cfg: Any, path: str) -> None:
        with open(path, "w") as f:
            f.write(LazyConfig.to_yaml(cfg))

    @staticmethod
    def load_yaml(path: str) -> Any:
        def revive(x):
            if isinstance(x, dict):
                if x.get("__type__") == "torch.dtype":
                    import torch
                    return getattr(torch, x["__value__"].split(".")[-1])
                if "__type__" in x and "__value__" in x:
                    return getattr(_locate(x["__type__"]), x["__value__"])
                d = LazyDict({k: revive(v) for k, v in x.items() if k != "__type__"})
                if "__type__" in x:
                    cls = _locate(x["__type__"])
                    return cls(**d)
                return d
            if isinstance(x, list):
                return [revive(v) for v in x]
            return x
        with open(path) as f:
            return revive(yaml.safe_load(f))
