"""Import modules of the reference implementation as test oracles.

The reference tree is looked up in ``$COSMOS_REFERENCE_DIR`` and then in ``baseline/_ref`` under the repository root; tests that
need it are skipped when neither exists. Packages that the reference imports at module level but that the compared code paths
never touch (object-store clients, video writers) are replaced by inert stand-ins, so that its unmodified files load in an image
without them. Nothing here is used by the framework itself.
"""

import importlib
import os
import sys
import types
from unittest.mock import MagicMock

import pytest

_ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class _Inert(types.ModuleType):
    __path__ = []

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        return MagicMock(name=f"{self.__name__}.{name}")


def reference_dir():
    for cand in (os.environ.get("COSMOS_REFERENCE_DIR"), os.path.join(_ROOT, "baseline", "_ref")):
        if cand and os.path.isdir(os.path.join(cand, "cosmos_predict2")):
            return cand
    return None


def import_reference(module: str, max_stubs: int = 64):
    """Import ``module`` (dotted name under ``cosmos_predict2``) from the reference tree; skip the test if that is impossible."""
    root = reference_dir()
    if root is None:
        pytest.skip("no copy of the reference implementation here")
    if root not in sys.path:
        sys.path.insert(0, root)
    for _ in range(max_stubs):
        try:
            return importlib.import_module(module)
        except ModuleNotFoundError as e:
            if e.name is None or e.name.startswith("cosmos_predict2"):
                pytest.skip(f"the reference module {module} does not import here: {e}")
            sys.modules[e.name] = _Inert(e.name)      # and try again: modules that did import stay as they are
        except Exception as e:          # anything else (a missing compiled extension, a version clash): no oracle
            pytest.skip(f"the reference module {module} does not import here: {type(e).__name__}: {e}")
    pytest.skip(f"the reference module {module} needs more than {max_stubs} absent packages")


def install_transformer_engine_standins() -> None:
    """The three TransformerEngine entry points that the reference network calls, restated in plain torch from their documented
    semantics, so that the reference's network file imports and runs without the package: ``pytorch.RMSNorm`` (fp32 statistics,
    learnable weight), ``pytorch.attention.apply_rotary_pos_emb`` (non-interleaved rotation by the given angles) and
    ``pytorch.attention.DotProductAttention`` (plain softmax attention, used by the multi-camera cross-attention)."""
    import torch
    import torch.nn as nn
    if "transformer_engine" in sys.modules and not isinstance(sys.modules["transformer_engine"], _Inert):
        return

    class RMSNorm(nn.Module):
        def __init__(self, dim, eps=1e-6):
            super().__init__()
            self.weight, self.eps = nn.Parameter(torch.ones(dim)), eps

        def reset_parameters(self):
            nn.init.ones_(self.weight)

        def forward(self, x):
            h = x.float()
            return (h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)

    def apply_rotary_pos_emb(t, freqs, tensor_format="sbhd", fused=False, **_):
        f = freqs.transpose(0, 1) if tensor_format == "bshd" else freqs
        a, b = t[..., : t.shape[-1] // 2], t[..., t.shape[-1] // 2:]
        return t * f.cos().to(t.dtype) + torch.cat([-b, a], -1) * f.sin().to(t.dtype)

    class DotProductAttention(nn.Module):
        """softmax(q k^T / sqrt(d)) v for [batch, sequence, heads, d] operands, heads folded into the last output dimension."""

        def __init__(self, num_heads, head_dim, qkv_format="sbhd", **_):
            super().__init__()
            assert qkv_format == "bshd"

        def forward(self, q, k, v, **_):
            o = torch.nn.functional.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
            return o.transpose(1, 2).flatten(2)

        def set_context_parallel_group(self, *a, **k):
            pass

    te, tep, tea = (types.ModuleType(n) for n in ("transformer_engine", "transformer_engine.pytorch", "transformer_engine.pytorch.attention"))
    te.__path__, tep.__path__ = [], []
    tep.RMSNorm, tea.apply_rotary_pos_emb, tea.DotProductAttention = RMSNorm, apply_rotary_pos_emb, DotProductAttention
    te.pytorch, tep.attention = tep, tea
    sys.modules.update({"transformer_engine": te, "transformer_engine.pytorch": tep, "transformer_engine.pytorch.attention": tea})


def reference_network_modules():
    """(lvg network module, attention module) of the reference, prepared for a CPU run in fp32: its attention dispatcher only
    enables GPU back ends and casts to bf16, so here the math back end is added and the compute dtype is fp32. Nothing else of
    the reference is touched."""
    import torch
    from torch.nn.attention import SDPBackend, sdpa_kernel
    install_transformer_engine_standins()
    lvg = import_reference("cosmos_predict2._src.predict2.networks.minimal_v1_lvg_dit")
    att = import_reference("cosmos_predict2._src.predict2.networks.attention")
    a2a = import_reference("cosmos_predict2._src.predict2.networks.a2a_cp")
    att.sdpa_kernel = lambda backends, **kw: sdpa_kernel(list(backends) + [SDPBackend.MATH])
    a2a.attention = lambda q, k, v, *a, **kw: att.attention(q, k, v, *a, **{**kw, "dtype": torch.float32})
    return lvg, att


def install_diffusers_standins() -> None:
    """What the reference's multistep solver takes from diffusers is bookkeeping, not arithmetic: a mixin that records the
    constructor arguments as ``self.config``, two marker base classes, an enum of scheduler names and an output record. These
    stand-ins provide exactly that, so that the solver's own file runs unmodified."""
    import dataclasses
    import enum
    import functools
    import inspect
    if "diffusers" in sys.modules and not isinstance(sys.modules["diffusers"], _Inert):
        return

    class _Config(dict):
        __getattr__ = dict.__getitem__

    class ConfigMixin:
        def register_to_config(self, **kw):
            if not hasattr(self, "config"):
                self.config = _Config()
            self.config.update(kw)

    def register_to_config(init):
        @functools.wraps(init)
        def wrapper(self, *args, **kwargs):
            sig = inspect.signature(init)
            bound = sig.bind(self, *args, **kwargs)
            bound.apply_defaults()
            ConfigMixin.register_to_config(self, **{k: v for k, v in list(bound.arguments.items())[1:]})
            init(self, *args, **kwargs)
        return wrapper

    class SchedulerMixin:
        pass

    @dataclasses.dataclass
    class SchedulerOutput:
        prev_sample: object

    KarrasDiffusionSchedulers = enum.Enum("KarrasDiffusionSchedulers", ["DDIMScheduler", "UniPCMultistepScheduler"])
    mods = {n: types.ModuleType(n) for n in ("diffusers", "diffusers.configuration_utils", "diffusers.schedulers",
                                             "diffusers.schedulers.scheduling_utils", "diffusers.utils")}
    for m in mods.values():
        m.__path__ = []
    mods["diffusers.configuration_utils"].ConfigMixin = ConfigMixin
    mods["diffusers.configuration_utils"].register_to_config = register_to_config
    su = mods["diffusers.schedulers.scheduling_utils"]
    su.KarrasDiffusionSchedulers, su.SchedulerMixin, su.SchedulerOutput = KarrasDiffusionSchedulers, SchedulerMixin, SchedulerOutput
    mods["diffusers.utils"].deprecate = lambda *a, **k: None

    class FlowMatchEulerDiscreteScheduler:
        """Only what the reference's training schedule reads from this diffusers class: the table of the 1000 training noise
        levels sigma = shift * s / (1 + (shift - 1) s), s = 1 ... 1/1000, and the matching timesteps 1000 sigma."""

        def __init__(self, num_train_timesteps=1000, shift=1.0, use_dynamic_shifting=False, **_):
            import numpy as np
            import torch
            self.config = _Config(num_train_timesteps=num_train_timesteps, shift=shift, use_dynamic_shifting=use_dynamic_shifting)
            s = torch.from_numpy(np.linspace(1, num_train_timesteps, num_train_timesteps, dtype=np.float32)[::-1].copy()) / num_train_timesteps
            if not use_dynamic_shifting:
                s = shift * s / (1 + (shift - 1) * s)
            self.sigmas, self.timesteps = s, s * num_train_timesteps
    mods["diffusers"].FlowMatchEulerDiscreteScheduler = FlowMatchEulerDiscreteScheduler
    sys.modules.update(mods)


def install_omegaconf_standins() -> None:
    """``omegaconf`` as two empty container classes: the compared code only asks ``isinstance(x, DictConfig / ListConfig)`` of
    objects that are neither."""
    if "omegaconf" in sys.modules and not isinstance(sys.modules["omegaconf"], _Inert):
        return

    class DictConfig(dict):
        pass

    class ListConfig(list):
        pass

    class _OmegaConf(_Inert):
        pass
    om = _OmegaConf("omegaconf")
    om.DictConfig, om.ListConfig = DictConfig, ListConfig
    for sub, cls in (("dictconfig", DictConfig), ("listconfig", ListConfig), ("base", None)):
        m = _OmegaConf(f"omegaconf.{sub}")
        if cls is not None:
            setattr(m, cls.__name__, cls)
        setattr(om, sub, m)
        sys.modules[f"omegaconf.{sub}"] = m
    sys.modules["omegaconf"] = om


def install_import_time_patches() -> None:
    """Things some reference modules evaluate while they are being imported, and that only exist on a GPU box or with an older
    transformers: a default argument ``torch.cuda.current_device()``, ``is_flash_attn_2_available()``, a cache class name."""
    import torch
    import transformers.cache_utils as cache_utils
    import transformers.utils
    if not hasattr(cache_utils, "SlidingWindowCache"):
        cache_utils.SlidingWindowCache = type("SlidingWindowCache", (), {})
    transformers.utils.is_flash_attn_2_available = lambda: True
    if not torch.cuda.is_available():
        torch.cuda.current_device = lambda: 0
    if "diffusers" in sys.modules and not hasattr(sys.modules["diffusers"], "FlowMatchEulerDiscreteScheduler"):
        sys.modules["diffusers"].FlowMatchEulerDiscreteScheduler = type("FlowMatchEulerDiscreteScheduler", (), {})
