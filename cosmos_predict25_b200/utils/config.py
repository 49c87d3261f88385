"""Experiment configuration: a nested, freezable config tree, a config store with groups, and the
command-line override grammar ``experiment=<name> a.b.c=value ~key +new.key=value``.

Parity targets: the attrs ``Config`` tree with ``make_freezable`` (cosmos_predict2/_src/imaginaire/config.py:57-449),
Hydra ``ConfigStore`` groups with ``defaults`` lists and ``_global_`` experiment nodes
(cosmos_predict2/_src/predict2/configs/video2world/config.py:37-102), and ``override``
(cosmos_predict2/_src/imaginaire/utils/config_helper.py:69-143). Implemented without attrs/hydra/omegaconf:
the tree is made of ``LazyDict`` nodes; ``${a.b}`` interpolations are resolved on ``resolve()``.
"""

from __future__ import annotations

import dataclasses
import copy
import os
import re
import time
from collections.abc import Mapping
from typing import Any, Dict, List, Optional, Tuple

import yaml

from .lazy_config import LazyConfig, LazyDict, instantiate, is_lazy

# where each config group lands in the tree
@dataclasses.dataclass
class ObjectStoreConfig:
    """Where a dataset or a checkpoint lives when it is not on the local disk (imaginaire/config.py:170-176 of the reference)."""
    enabled: bool = False
    credentials: str = ""
    bucket: str = ""


class JobConfig(LazyDict):
    """Where a run writes: ``<project>/<group>/<name>`` under the output root (imaginaire/config.py:104-166 of the reference)."""

    def __init__(self, project: str = "", group: str = "", name: str = "", wandb_mode: str = "offline", **extra):
        super().__init__(project=project, group=group, name=name, wandb_mode=wandb_mode, **extra)

    @property
    def path(self) -> str:
        return os.path.join(self["project"], self["group"], self["name"])

    @property
    def path_local(self) -> str:
        return os.path.join(os.environ.get("IMAGINAIRE_OUTPUT_ROOT", "/tmp/imaginaire4-output"), self.path)


class CheckpointConfig(LazyDict):
    """Settings of the trainer's checkpointer (imaginaire/config.py:284-330 of the reference); the registry of released
    checkpoints has its own ``CheckpointConfig`` in ``utils/checkpoint_db.py``."""

    def __init__(self, **kw):
        base = dict(type=None, dcp_async_mode_enabled=False, save_to_object_store=ObjectStoreConfig(),
                    load_from_object_store=ObjectStoreConfig(), save_iter=999999999, load_path="", load_training_state=False,
                    only_load_scheduler_state=False, strict_resume=True, keys_not_to_resume=[], load_ema_to_reg=False,
                    dcp_allow_mismatched_size=False, broadcast_via_filesystem=False, verbose=True)
        base.update(kw)
        super().__init__(**base)


GROUP_PATHS = {
    "model": "model", "net": "model.config.net", "conditioner": "model.config.conditioner",
    "tokenizer": "model.config.tokenizer", "ema": "model.config.ema", "optimizer": "optimizer", "scheduler": "scheduler",
    "data_train": "dataloader_train", "data_val": "dataloader_val", "callbacks": "trainer.callbacks",
    "checkpoint": "checkpoint", "ckpt_type": "checkpoint.type",
}


def _wrap(x: Any) -> Any:
    if isinstance(x, Mapping) and not isinstance(x, LazyDict):
        return LazyDict({k: _wrap(v) for k, v in x.items()})
    if isinstance(x, LazyDict):
        for k, v in list(x.items()):
            x[k] = _wrap(v)
        return x
    if isinstance(x, list):
        return [_wrap(v) for v in x]
    return x


def deep_merge(dst: LazyDict, src: Mapping) -> LazyDict:
    """Recursive update; a node carrying a different ``_target_`` replaces the old node wholesale."""
    for k, v in src.items():
        if isinstance(v, Mapping) and isinstance(dst.get(k), Mapping):
            if "_target_" in v and dst[k].get("_target_") is not None and v["_target_"] != dst[k].get("_target_"):
                dst[k] = _wrap(copy.deepcopy(v))
            else:
                deep_merge(dst[k], v)
        else:
            dst[k] = _wrap(copy.deepcopy(v))
    return dst


def get_path(tree: Mapping, path: str, default=KeyError):
    cur = tree
    for p in path.split("."):
        if isinstance(cur, Mapping) and p in cur:
            cur = cur[p]
        elif isinstance(cur, list) and p.isdigit() and int(p) < len(cur):
            cur = cur[int(p)]
        elif hasattr(cur, p) and not isinstance(cur, Mapping):
            cur = getattr(cur, p)
        else:
            if default is KeyError:
                raise KeyError(f"config has no key {path!r} (failed at {p!r})")
            return default
    return cur


def set_path(tree: LazyDict, path: str, value: Any, create: bool = False) -> None:
    parts = path.split(".")
    cur = tree
    for p in parts[:-1]:
        if isinstance(cur, Mapping):
            if p not in cur:
                if not create:
                    raise KeyError(f"config has no key {path!r} (failed at {p!r}); prefix with + to add")
                cur[p] = LazyDict()
            cur = cur[p]
        elif isinstance(cur, list):
            cur = cur[int(p)]
        else:
            cur = getattr(cur, p)
    last = parts[-1]
    if isinstance(cur, Mapping):
        if last not in cur and not create:
            raise KeyError(f"config has no key {path!r}; prefix with + to add")
        cur[last] = _wrap(value)
    elif isinstance(cur, list):
        cur[int(last)] = value
    else:
        setattr(cur, last, value)


def del_path(tree: LazyDict, path: str) -> None:
    parts = path.split(".")
    cur = get_path(tree, ".".join(parts[:-1])) if len(parts) > 1 else tree
    if isinstance(cur, Mapping):
        cur.pop(parts[-1], None)
    else:
        setattr(cur, parts[-1], None)


class ConfigStore:
    """Registry of named config nodes per group (singleton via ``ConfigStore.instance()``)."""

    _inst: Optional["ConfigStore"] = None

    def __init__(self):
        self.repo: Dict[str, Dict[str, Any]] = {}

    @classmethod
    def instance(cls) -> "ConfigStore":
        if cls._inst is None:
            cls._inst = ConfigStore()
        return cls._inst

    def store(self, name: str, node: Any, group: str = "", package: Optional[str] = None) -> None:
        self.repo.setdefault(group, {})[name] = {"node": node, "package": package}

    def get(self, group: str, name: str) -> Any:
        try:
            return self.repo[group][name]["node"]
        except KeyError:
            known = sorted(self.repo.get(group, {}))
            raise KeyError(f"no {group!r} config named {name!r}; known: {known[:20]}") from None

    def names(self, group: str) -> List[str]:
        return sorted(self.repo.get(group, {}))


class Config(LazyDict):
    """Top-level tree: model / optimizer / scheduler / dataloader_train / dataloader_val / job / trainer /
    model_parallel / checkpoint (+ ``defaults``)."""

    _frozen = False

    def __init__(self, *args, **kw):
        """``Config()`` is an empty tree (``Config.default()`` fills it); ``Config(model=..., optimizer=..., ...)`` - the
        reference's constructor call - is the default tree with those entries set."""
        super().__init__(*args)
        if kw:
            self.update(Config.default())
            for k, v in kw.items():
                self[k] = _wrap(v)

    @staticmethod
    def default() -> "Config":
        c = Config()
        c.update(_wrap(dict(
            defaults=["_self_"],
            job=dict(project="cosmos_b200", group="default", name="run_${now:%Y-%m-%d_%H-%M-%S}", wandb_mode="disabled"),
            trainer=dict(max_iter=1000, grad_accum_iter=1, logging_iter=20, validation_iter=100, max_val_iter=None, save_iter=200,
                         seed=0, timeout_period=999999999, run_validation=False, distributed_parallelism="fsdp",
                         cudnn=dict(deterministic=False, benchmark=True), memory_format="preserve_format", callbacks=dict(),
                         profiling=dict(enable_profiling=False, enable_memory_snapshot=False, profile_freq=1000, target_ranks=[0],
                                        record_shape=False, profile_memory=False, with_stack=False, with_modules=False),
                         straggler_detection=dict(enabled=False, report_freq=100, profile_freq=1, max_diff=1.5, raise_error=True,
                                                  analyze_forward=True, analyze_backward=True, analyze_optimizer=True,
                                                  analyze_dataloading=True),
                         grad_scaler_args=dict(enabled=False)),
            model_parallel=dict(context_parallel_size=1, tensor_model_parallel_size=1, pipeline_model_parallel_size=1,
                                sequence_parallel=False),
            checkpoint=dict(type=None, dcp_async_mode_enabled=False, save_iter=200, load_path="", load_training_state=False,
                            only_load_scheduler_state=False, strict_resume=True, keys_not_to_resume=[], load_ema_to_reg=False,
                            dcp_allow_mismatched_size=False, broadcast_via_filesystem=False, verbose=True,
                            jit=dict(enabled=False, input_shape=None, device="cuda", dtype="bfloat16", strict=True)),
            model=None, optimizer=None, scheduler=None, dataloader_train=None, dataloader_val=None,
            upload_reproducible_setup=False,
        )))
        return c

    # ---- freezing ----------------------------------------------------------------------------------
    def freeze(self):
        object.__setattr__(self, "_frozen", True)

    def unfreeze(self):
        object.__setattr__(self, "_frozen", False)

    def __setitem__(self, k, v):
        if getattr(self, "_frozen", False):
            raise AttributeError(f"config is frozen; cannot set {k!r}")
        super().__setitem__(k, v)

    # ---- derived values ------------------------------------------------------------------------------
    @property
    def job_path(self) -> str:
        j = self["job"]
        return os.path.join(j["project"], j["group"], j["name"])

    @property
    def job_path_local(self) -> str:
        root = os.environ.get("IMAGINAIRE_OUTPUT_ROOT", "/tmp/imaginaire4-output")
        return os.path.join(root, self.job_path)

    def resolve(self) -> "Config":
        """Resolve ``${a.b.c}`` and ``${now:<strftime>}`` interpolations in place."""
        pat = re.compile(r"\$\{([^}]+)\}")

        def res(v, depth=0):
            if isinstance(v, str) and depth < 8:
                full = pat.fullmatch(v)
                if full and not full.group(1).startswith("now:"):
                    return res(get_path(self, full.group(1)), depth + 1)

                def sub(m):
                    key = m.group(1)
                    if key.startswith("now:"):
                        return time.strftime(key[4:])
                    return str(res(get_path(self, key), depth + 1))
                return pat.sub(sub, v)
            if isinstance(v, Mapping):
                for k in list(v.keys()):
                    v[k] = res(v[k], depth)
                return v
            if isinstance(v, list):
                return [res(x, depth) for x in v]
            return v

        frozen = getattr(self, "_frozen", False)
        self.unfreeze()
        res(self)
        if frozen:
            self.freeze()
        return self

    def validate(self) -> None:
        assert self.get("job") is not None, "job config missing"
        mp = self["model_parallel"]
        assert mp["context_parallel_size"] >= 1 and mp["tensor_model_parallel_size"] >= 1
        t = self["trainer"]
        assert t["distributed_parallelism"] in ("ddp", "fsdp"), t["distributed_parallelism"]
        assert t["grad_accum_iter"] >= 1 and t["max_iter"] >= 0

    def to_yaml(self) -> str:
        return LazyConfig.to_yaml(self)

    def save(self, out_dir: str) -> None:
        """Reproducibility dump: ``config.yaml`` and ``config.pkl`` beside the checkpoints."""
        import pickle
        os.makedirs(out_dir, exist_ok=True)
        LazyConfig.save_yaml(self, os.path.join(out_dir, "config.yaml"))
        try:
            with open(os.path.join(out_dir, "config.pkl"), "wb") as f:
                pickle.dump(copy.deepcopy(dict(self)), f)
        except Exception:
            pass


def _parse_value(text: str) -> Any:
    try:
        return yaml.safe_load(text)
    except yaml.YAMLError:
        return text


def _apply_defaults(cfg: Config, node: Mapping, cs: ConfigStore, seen: Tuple[str, ...] = ()) -> None:
    """Apply an experiment node: first its ``defaults`` (parents, group overrides), then itself at ``_self_``."""
    defaults = list(node.get("defaults", ["_self_"]))
    if "_self_" not in defaults:
        defaults.append("_self_")
    body = {k: v for k, v in node.items() if k != "defaults"}
    for d in defaults:
        if d == "_self_":
            deep_merge(cfg, body)
        elif isinstance(d, str):
            grp, _, name = d.strip("/").partition("/")
            if grp == "experiment":
                if name in seen:
                    raise ValueError(f"experiment inheritance cycle at {name}")
                _apply_defaults(cfg, cs.get("experiment", name), cs, seen + (name,))
            else:
                _select_group(cfg, grp, name, cs)
        elif isinstance(d, Mapping):
            for k, name in d.items():
                grp = k.replace("override", "").strip().strip("/")
                if name is not None:
                    _select_group(cfg, grp, name, cs)


def _select_group(cfg: Config, group: str, name: str, cs: ConfigStore) -> None:
    node = copy.deepcopy(cs.get(group, name))
    if cs.repo[group][name].get("package") == "_global_":
        # a whole-tree node (e.g. the ``model`` group of the Text2World project sets ``trainer`` and ``model`` together)
        deep_merge(cfg, node)
        return
    path = GROUP_PATHS.get(group)
    if path is None:
        raise KeyError(f"unknown config group {group!r}")
    set_path(cfg, path, node, create=True)


def override(config: Config, overrides: Optional[List[str]] = None, cs: Optional[ConfigStore] = None) -> Config:
    """Apply ``["--", "experiment=foo", "trainer.max_iter=10", "~dataloader_val", "+job.tag=x"]`` to ``config``.
    Group selections (``net=...``, ``experiment=...``) are applied before dotted-key assignments, in the
    order: config defaults list, experiment, remaining groups, key assignments."""
    cs = cs or ConfigStore.instance()
    overrides = [o for o in (overrides or []) if o != "--"]
    groups, assigns, deletes = [], [], []
    for o in overrides:
        if o.startswith("~"):
            deletes.append(o[1:].split("=")[0])
            continue
        if "=" not in o:
            raise ValueError(f"override {o!r} must be key=value or ~key")
        k, v = o.split("=", 1)
        add = k.startswith("+")
        k = k.lstrip("+")
        if "." not in k and (k in GROUP_PATHS or k == "experiment") and not add and k in cs.repo:
            groups.append((k, v))
        else:
            assigns.append((k, _parse_value(v), add))
    # the config's own defaults list: [{"net": "x"}, "_self_", ...]
    for d in config.get("defaults", []):
        if isinstance(d, Mapping):
            for g, name in d.items():
                g = g.replace("override", "").strip().strip("/")
                if name is not None and g != "experiment" and not any(gg == g for gg, _ in groups):
                    _select_group(config, g, name, cs)
    for g, name in groups:
        if g == "experiment":
            _apply_defaults(config, cs.get("experiment", name), cs, (name,))
    for g, name in groups:
        if g != "experiment":
            _select_group(config, g, name, cs)
    for k, v, add in assigns:
        set_path(config, k, v, create=add)
    for k in deletes:
        del_path(config, k)
    config.resolve()
    return config


def load_config_module(path: str):
    """Import a config file (``a/b/config.py`` or dotted module) and return the module; it must expose
    ``make_config()``."""
    import importlib
    import importlib.util
    if path.endswith(".py") and os.path.exists(path):
        # a file inside an importable package is imported under its package name (relative imports work)
        rel = os.path.relpath(os.path.abspath(path), os.getcwd())
        if not rel.startswith(".."):
            try:
                return importlib.import_module(rel[:-3].replace(os.sep, "."))
            except ImportError:
                pass
        spec = importlib.util.spec_from_file_location("_cosmos_b200_config_" + str(abs(hash(path))), path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        return mod
    return importlib.import_module(path.replace("/", ".").removesuffix(".py"))


def import_all_modules_from_package(package: str, reload: bool = False) -> None:
    """Import every sub-module of ``package`` so that their ``ConfigStore`` registrations run."""
    import importlib
    import pkgutil
    pkg = importlib.import_module(package)
    for m in pkgutil.walk_packages(pkg.__path__, package + "."):
        mod = importlib.import_module(m.name)
        if reload:
            importlib.reload(mod)
