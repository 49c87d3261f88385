"""Training entry point: ``torchrun --nproc_per_node=N -m cosmos_predict25_b200.cli.train --config=<config.py> -- experiment=<name> k=v ~key``.

Same grammar as the reference's launcher (scripts/train.py:34-110): ``--config`` names a config module exposing
``make_config()``; everything after ``--`` is an override list; ``--dryrun`` prints and saves the resolved config
without training; ``--smoke`` runs one iteration with logging side effects off and a checkpoint after it.
"""

from __future__ import annotations

import argparse
import importlib
import os
import sys

from ..parallel.mesh import build_groups
from ..utils import distributed, log
from ..utils.config import Config, load_config_module, override
from ..utils.lazy_config import instantiate, is_lazy, _locate


def launch(config: Config, args) -> None:
    import torch
    from ..trainer.trainer import Trainer, TrainerConfig

    local_rank = distributed.init()
    config.validate()
    config.freeze()
    out_dir = config.job_path_local
    if distributed.is_rank0():
        config.save(out_dir)
        log.init_loguru_file(os.path.join(out_dir, "stdout.log"))
    dev = torch.device("cuda", local_rank) if torch.cuda.is_available() else torch.device("cpu")
    t = config["trainer"]
    cp_size = config["model_parallel"]["context_parallel_size"]
    world = distributed.get_world_size()
    if t["distributed_parallelism"] == "ddp":
        shard_size = cp_size                     # nothing sharded beyond the ranks that share a sample
    else:
        mcfg = config["model"].get("config") if hasattr(config["model"], "get") else None
        shard_size = int((mcfg or {}).get("fsdp_shard_size", 0) or 0)
        if shard_size <= 1 or shard_size > world or world % shard_size != 0 or shard_size % cp_size != 0:
            shard_size = world                   # unset (or not a divisor of this job): shard over all ranks
    groups = build_groups(cp_size=cp_size, shard_size=shard_size)
    model = instantiate(config["model"], device=dev, fsdp_group=groups.fsdp, cp_group=groups.cp,
                        replicate_group=groups.replicate)
    callbacks = [instantiate(v) for v in (t.get("callbacks") or {}).values() if v is not None]
    ckpt_cls = config["checkpoint"].get("type")
    checkpointer = None
    if ckpt_cls:
        cls = _locate(ckpt_cls) if isinstance(ckpt_cls, str) else ckpt_cls
        checkpointer = cls(config["checkpoint"], out_dir) if cls.__name__ != "DummyCheckpointer" else cls()
    tcfg = TrainerConfig(max_iter=t["max_iter"], grad_accum_iter=t["grad_accum_iter"], logging_iter=t["logging_iter"],
                         validation_iter=t["validation_iter"], max_val_iter=t["max_val_iter"],
                         save_iter=config["checkpoint"]["save_iter"], seed=t["seed"],
                         timeout_period=t["timeout_period"] if t["timeout_period"] < 10 ** 8 else 0,
                         run_validation=t["run_validation"], distributed_parallelism=t["distributed_parallelism"],
                         cudnn_deterministic=t["cudnn"]["deterministic"], output_dir=out_dir)
    trainer = Trainer(tcfg, model, instantiate(config["optimizer"]), instantiate(config["scheduler"]), callbacks, checkpointer)
    dl_train = instantiate(config["dataloader_train"])
    dl_val = instantiate(config["dataloader_val"]) if config.get("dataloader_val") is not None else None
    model.train()
    trainer.train(dl_train, dl_val)
    distributed.destroy()


def main(argv=None):
    ap = argparse.ArgumentParser(description="training")
    ap.add_argument("--config", default="cosmos_predict25_b200/configs/video2world.py", help="config module or file with make_config()")
    ap.add_argument("opts", nargs=argparse.REMAINDER, default=None, help="overrides: -- experiment=name key=value ~key")
    ap.add_argument("--dryrun", action="store_true")
    ap.add_argument("--smoke", action="store_true", help="one iteration, no external logging")
    args = ap.parse_args(argv)
    mod = load_config_module(args.config)
    config = mod.make_config()
    opts = list(args.opts or [])
    if args.smoke:
        opts += ["job.wandb_mode=disabled", "trainer.max_iter=1", "trainer.logging_iter=1", "checkpoint.save_iter=1"]
    config = override(config, opts)
    if args.dryrun:
        os.makedirs(config.job_path_local, exist_ok=True)
        print(config.to_yaml())
        config.save(config.job_path_local)
        print(f"config saved to {config.job_path_local}/config.yaml")
        return 0
    launch(config, args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
