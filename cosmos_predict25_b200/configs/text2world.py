"""Text2World project config: the noise-level (EDM) parameterised model family that preceded the rectified-flow models, plus the
rectified-flow Text2World model and the Wan2.1 fine-tuning model.

``make_config()`` returns the default tree; the config groups (data, optimizer, scheduler, callbacks, net, conditioner, ema,
tokenizer, ckpt_type) are the ones ``configs/video2world.py`` registers; this module adds the ``model`` group
(``ddp`` / ``fsdp`` / ``fsdp_rectified_flow`` / ``fsdp_wan2pt1``, each a whole-tree node like the reference's
configs/text2world/defaults/model.py:26-63) and the smoke experiments that the reference's tests name
(configs/text2world/config_test.py, models/model_fsdp2_test.py: ``error-free_fsdp_mock-data_base-cb``).
"""

from __future__ import annotations

import copy

from ..data.mock import MockVideoLatentDataset, build_dataloader
from ..models.edm import DiffusionModel, EDMConfig
from ..models.rectified_flow import EMAConfig, Text2WorldModelRectifiedFlow, Text2WorldRFConfig
from ..models.wan2pt1 import WANDiffusionModel, WanRFConfig
from ..utils.config import Config, ConfigStore
from ..utils.lazy_config import L
from . import video2world as _groups  # noqa: F401  (registers the shared config groups)

cs = ConfigStore.instance()


def _parts(net: str, **kw):
    d = dict(net=copy.deepcopy(cs.get("net", net)), conditioner=copy.deepcopy(cs.get("conditioner", "add_fps_padding_mask")),
             tokenizer=copy.deepcopy(cs.get("tokenizer", "wan2pt1_tokenizer")), ema=L(EMAConfig)(enabled=True, rate=0.1),
             precision="bfloat16", state_ch=16, state_t=24)
    d.update(kw)
    return d


def _edm(shard: int, **kw):
    return L(DiffusionModel)(config=L(EDMConfig)(**_parts("cosmos_v1_2B", fsdp_shard_size=shard, **kw)))


cs.store(group="model", package="_global_", name="ddp", node=dict(trainer=dict(distributed_parallelism="ddp"), model=_edm(1)))
cs.store(group="model", package="_global_", name="fsdp", node=dict(trainer=dict(distributed_parallelism="fsdp"), model=_edm(8)))
cs.store(group="model", package="_global_", name="fsdp_rectified_flow", node=dict(
    trainer=dict(distributed_parallelism="fsdp"),
    model=L(Text2WorldModelRectifiedFlow)(config=L(Text2WorldRFConfig)(**_parts("cosmos_v1_2B", fsdp_shard_size=8)))))
cs.store(group="model", package="_global_", name="fsdp_wan2pt1", node=dict(
    trainer=dict(distributed_parallelism="fsdp"),
    model=L(WANDiffusionModel)(config=L(WanRFConfig)(fsdp_shard_size=8, precision="bfloat16", state_ch=16, state_t=21,
                                                      tokenizer=copy.deepcopy(cs.get("tokenizer", "wan2pt1_tokenizer")),
                                                      ema=L(EMAConfig)(enabled=True, rate=0.1)))))


def make_config() -> Config:
    c = Config.default()
    c["defaults"] = ["_self_", {"data_train": "mock"}, {"data_val": "mock"}, {"optimizer": "fusedadamw"}, {"scheduler": "lambdalinear"},
                     {"model": "ddp"}, {"callbacks": "basic"}, {"ckpt_type": "dummy"}, {"experiment": None}]
    c["job"]["project"] = "cosmos_diffusion_v2"
    c["job"]["group"] = "debug"
    c["job"]["name"] = "delete_${now:%Y-%m-%d}_${now:%H-%M-%S}"
    c["trainer"].update(max_iter=400_000, logging_iter=10, validation_iter=100, run_validation=False)
    return c


# ---- smoke experiments: must run without data, weights or a tokenizer ---------------------------------------------------------------
def _mock_loader(length):
    return L(build_dataloader)(dataset=L(MockVideoLatentDataset)(num_frames=4, height=32, width=32, text_dim=100352, text_len=64,
                                                                 length=length), batch_size=1, num_workers=0)


for _name, _group in (("error-free_fsdp_mock-data_base-cb", "fsdp"), ("error-free_ddp_mock-data_base-cb", "ddp")):
    cs.store(group="experiment", package="_global_", name=_name, node=dict(
        defaults=[{"override /model": _group}, {"override /callbacks": "basic"}, "_self_"],
        job=dict(group="tests", name=_name),
        model=dict(config=dict(net=copy.deepcopy(cs.get("net", "mini_net")), tokenizer=None, state_t=4)),
        dataloader_train=_mock_loader(64), dataloader_val=_mock_loader(4),
        trainer=dict(max_iter=4, logging_iter=2),
    ))
