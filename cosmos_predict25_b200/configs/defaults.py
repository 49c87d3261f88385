"""The reference's named default config objects, importable by name.

The reference's own code and tests build model configs from module-level constants:
``Video2WorldConfig(tokenizer=DummyJointImageVideoConfig, conditioner=VideoPredictionConditioner, net=mini_net, ema=PowerEMAConfig)``
(cosmos_predict2/_src/predict2/models/video2world_model_test.py:33-43; the constants live in
cosmos_predict2/_src/predict2/configs/common/defaults/{ema,tokenizer}.py and .../video2world/defaults/{conditioner,net}.py).
Here the same objects are the nodes registered in the config store; this module gives them those names. They are lazy calls: a
model constructor builds them (``models/rectified_flow.py: materialise_config``).
"""

from __future__ import annotations

import copy

from ..utils.config import ConfigStore
from . import video2world as _v2w  # noqa: F401  (registers the groups)

_cs = ConfigStore.instance()


def _node(group: str, name: str):
    return copy.deepcopy(_cs.get(group, name))


# networks
mini_net = _node("net", "mini_net")
tiny_net = _node("net", "tiny_net")
COSMOS_V1_2B_NET_MININET = _node("net", "cosmos_v1_2B")
COSMOS_V1_7B_NET_MININET = _node("net", "cosmos_v1_7B")
COSMOS_V1_14B_NET_MININET = _node("net", "cosmos_v1_14B")
# conditioners
VideoPredictionConditioner = _node("conditioner", "video_prediction_conditioner")
VideoConditionerFpsPaddingConfig = _node("conditioner", "add_fps_padding_mask")
# tokenizers
DummyJointImageVideoConfig = _node("tokenizer", "dummy_tokenizer")
Wan2pt1VAEConfig = _node("tokenizer", "wan2pt1_tokenizer")
# EMA
PowerEMAConfig = _node("ema", "power")
EMAOffConfig = _node("ema", "off")
