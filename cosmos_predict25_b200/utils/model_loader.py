"""Build a model from an experiment name and load a checkpoint into it.

Parity target: ``load_model_from_checkpoint`` / ``create_model_from_consolidated_checkpoint_with_fsdp``
(cosmos_predict2/_src/predict2/utils/model_loader.py:33-224): compose the experiment config, drop the training
dataloader (``~dataloader_train``), instantiate the model, load a consolidated ``.pt`` (``net.*`` / ``net_ema.*`` keys;
EMA weights can be loaded as the regular ones) or a DCP directory; for sharded training the consolidated file is
loaded first and the sharded engine built afterwards.
"""

from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

from . import log
from .checkpoint_db import get_checkpoint_path
from .config import Config, load_config_module, override
from .lazy_config import instantiate


def load_model_from_checkpoint(experiment_name: str, checkpoint_path: Optional[str] = None,
                               config_file: str = "cosmos_predict25_b200.configs.video2world", enable_fsdp: bool = False,
                               load_ema_to_reg: bool = False, experiment_opts: Optional[List[str]] = None, device=None,
                               fsdp_group=None, cp_group=None, strict: bool = False) -> Tuple[torch.nn.Module, Config]:
    mod = load_config_module(config_file)
    config = mod.make_config()
    opts = ["--", f"experiment={experiment_name}"] + list(experiment_opts or [])
    config = override(config, opts)
    config["dataloader_train"] = None
    if not enable_fsdp:
        config["model"]["config"]["fsdp_shard_size"] = 1
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    model = instantiate(config["model"], device=dev, fsdp_group=fsdp_group if enable_fsdp else None, cp_group=cp_group)
    if checkpoint_path:
        load_model_state_dict_from_checkpoint(model, checkpoint_path, load_ema_to_reg=load_ema_to_reg, strict=strict)
    model.eval()
    return model, config


def load_model_state_dict_from_checkpoint(model, checkpoint_path: str, load_ema_to_reg: bool = False, strict: bool = False) -> None:
    path = get_checkpoint_path(checkpoint_path)
    if os.path.isdir(path):
        from ..checkpoint.dcp import DistributedCheckpointer
        ck = DistributedCheckpointer({"load_path": path, "load_ema_to_reg": load_ema_to_reg, "strict_resume": strict}, job_dir=os.devnull)
        if model.engine is None:
            model.on_train_start()
        ck.load(model)
        return
    log.info(f"loading consolidated checkpoint {path}")
    sd = torch.load(path, map_location="cpu", weights_only=False)
    if "model" in sd and isinstance(sd["model"], dict):
        sd = sd["model"]
    missing, unexpected = model.load_state_dict(sd, strict=strict, load_ema_to_reg=load_ema_to_reg)
    if missing or unexpected:
        log.warning(f"checkpoint load: {len(missing)} missing and {len(unexpected)} unexpected keys")


def create_model_from_consolidated_checkpoint_with_fsdp(config: Config, device=None, fsdp_group=None, cp_group=None):
    """Training start from a released ``.pt``: instantiate unsharded, load, then build the sharded engine."""
    load_path = config["checkpoint"]["load_path"]
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu"))
    model = instantiate(config["model"], device=dev, fsdp_group=fsdp_group, cp_group=cp_group)
    load_model_state_dict_from_checkpoint(model, load_path, load_ema_to_reg=config["checkpoint"].get("load_ema_to_reg", False))
    model.on_train_start()
    return model
