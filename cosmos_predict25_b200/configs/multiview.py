"""Project config for the multiview (N-camera) video-to-video model.

Registers the multiview network / conditioner groups and the experiment names of the reference
(cosmos_predict2/_src/predict2_multiview/configs/vid2vid/config.py,
.../experiment/buttercup/buttercup2p5_rectified_flow.py:29-580, .../buttercup2p5_rectified_flow_14b.py, and the noise-level
(predict2.1-era) ones of .../buttercup_predict2_frombase2p1.py:29-225) so that the checkpoint registry's ``experiment`` strings
resolve, plus the model groups ``ddp_multiview`` / ``fsdp_multiview`` / ``fsdp_rectified_flow_multiview``
(.../defaults/model.py:29-67). The training data groups of the reference (joint Alpamayo / MADS
webdataset shards) are replaced by the mock multiview dataset; point ``dataloader_train`` at your own data.
"""

from __future__ import annotations

import copy

from ..data.mock import build_dataloader
from ..data.multiview_dataset import MockMultiviewLatentDataset
from ..models.conditioner import BooleanFlag, ReMapkey, TextAttr
from ..models.multiview import (MultiViewConditioner, MultiviewRFConfig, MultiviewVid2VidModel, MultiviewVid2VidModelConfig,
                                MultiviewVid2VidModelRectifiedFlow)
from ..models.multiview_dit import MultiViewDiTConfig
from ..models.rectified_flow import EMAConfig
from ..utils.config import Config, ConfigStore
from ..utils.lazy_config import L
from . import video2world as _base  # registers the shared groups (tokenizer, optimizer, scheduler, callbacks, ...)

cs = ConfigStore.instance()

_MV_NET = dict(timestep_scale=0.001, use_wan_fp32_strategy=True, use_crossattn_projection=True, crossattn_proj_in_channels=100352,
               crossattn_emb_channels=1024, concat_view_embedding=True, view_condition_dim=7, n_cameras_emb=7, state_t=8,
               rope_enable_fps_modulation=True, rope_h_extrapolation_ratio=3.0, rope_w_extrapolation_ratio=3.0,
               rope_t_extrapolation_ratio=8.0 / 24.0, checkpoint_mode="predict2_2b_720")
cs.store(group="net", name="cosmos_v1_2B_multiview", node=L(MultiViewDiTConfig)(model_channels=2048, num_heads=16, num_blocks=28, **_MV_NET))
cs.store(group="net", name="cosmos_v1_14B_multiview", node=L(MultiViewDiTConfig)(model_channels=5120, num_heads=40, num_blocks=36, **_MV_NET))
cs.store(group="net", name="tiny_multiview", node=L(MultiViewDiTConfig)(
    model_channels=256, num_heads=4, num_blocks=2, crossattn_emb_channels=256, use_crossattn_projection=False, max_img_h=64,
    max_img_w=64, max_frames=32, adaln_lora_dim=64, state_t=2, n_cameras_emb=4, view_condition_dim=4, context_tokens_per_view=8))

cs.store(group="conditioner", name="video_prediction_multiview_conditioner", node=L(MultiViewConditioner)(
    fps=L(ReMapkey)(input_key="fps", output_key="fps"),
    padding_mask=L(ReMapkey)(input_key="padding_mask", output_key="padding_mask"),
    text=L(TextAttr)(input_key="t5_text_embeddings", dropout_rate=0.2),
    use_video_condition=L(BooleanFlag)(input_key="fps", output_key="use_video_condition", dropout_rate=0.0),
    view_indices_B_T=L(ReMapkey)(input_key="latent_view_indices_B_T", output_key="view_indices_B_T"),
    ref_cam_view_idx_sample_position=L(ReMapkey)(input_key="ref_cam_view_idx_sample_position",
                                                 output_key="ref_cam_view_idx_sample_position")))

cs.store(group="data_train", name="mock_multiview", node=L(build_dataloader)(
    dataset=L(MockMultiviewLatentDataset)(n_views=7, state_t=8, height=90, width=160, text_dim=100352, length=16),
    batch_size=1, num_workers=0))


def _mv_model(net="cosmos_v1_2B_multiview", tokenizer="wan2pt1_tokenizer", **cfg_kw):
    kw = dict(net=copy.deepcopy(cs.get("net", net)),
              conditioner=copy.deepcopy(cs.get("conditioner", "video_prediction_multiview_conditioner")),
              tokenizer=copy.deepcopy(cs.get("tokenizer", tokenizer)), ema=L(EMAConfig)(enabled=True, rate=0.1),
              precision="bfloat16", state_ch=16, state_t=8, resolution="720p", shift=5.0, train_time_distribution="logitnormal",
              min_num_conditional_frames_per_view=0, max_num_conditional_frames_per_view=2,
              condition_locations=["first_random_n"], conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25},
              text_dropout=0.2, sharding_transport="peer")
    kw.update(cfg_kw)
    return L(MultiviewVid2VidModelRectifiedFlow)(config=L(MultiviewRFConfig)(**kw))


def _mv_edm_model(net="cosmos_v1_2B_multiview", tokenizer="wan2pt1_tokenizer", **cfg_kw):
    """The noise-level twin with the settings of the base run those experiments start from: rectified-flow preconditioning at
    sigma_data 1, non-uniform loss weights, noise levels in (0.01, 200), 5 % of the video samples re-drawn log-uniformly in
    (200, 100000)."""
    kw = dict(net=copy.deepcopy(cs.get("net", net)),
              conditioner=copy.deepcopy(cs.get("conditioner", "video_prediction_multiview_conditioner")),
              tokenizer=copy.deepcopy(cs.get("tokenizer", tokenizer)), ema=L(EMAConfig)(enabled=True, rate=0.1),
              precision="bfloat16", state_ch=16, state_t=8, resolution="720p", scaling="rectified_flow", sigma_data=1.0,
              rectified_flow_loss_weight_uniform=False, sigma_max=200.0, sigma_min=0.01, high_sigma_strategy="LOGUNIFORM200_100000",
              high_sigma_ratio=0.05, min_num_conditional_frames_per_view=0, max_num_conditional_frames_per_view=2,
              condition_locations=["first_random_n"], conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25},
              online_text_embeddings_as_dict=False, text_dropout=0.2, sharding_transport="peer")
    kw.update(cfg_kw)
    kw["net"].update(timestep_scale=1.0)                       # the noise conditioning is c_noise(sigma), not a 0..1000 time
    return L(MultiviewVid2VidModel)(config=L(MultiviewVid2VidModelConfig)(**kw))


cs.store(group="model", package="_global_", name="ddp_multiview",
         node=dict(trainer=dict(distributed_parallelism="ddp"), model=_mv_edm_model()))
cs.store(group="model", package="_global_", name="fsdp_multiview",
         node=dict(trainer=dict(distributed_parallelism="fsdp"), model=_mv_edm_model(fsdp_shard_size=8)))
cs.store(group="model", package="_global_", name="fsdp_rectified_flow_multiview",
         node=dict(trainer=dict(distributed_parallelism="fsdp"), model=_mv_model()))


def make_config() -> Config:
    c = Config.default()
    c["defaults"] = ["_self_", {"data_train": "mock_multiview"}, {"data_val": "mock"}, {"optimizer": "adamw"},
                     {"scheduler": "lambdalinear"}, {"callbacks": "basic"}, {"ckpt_type": "dcp"}, {"experiment": None}]
    c["job"]["project"] = "cosmos_predict2_multiview"
    c["job"]["group"] = "debug"
    c["job"]["name"] = "multiview_${now:%Y-%m-%d_%H-%M-%S}"
    c["model"] = _mv_model()
    return c


def _exp(name, net="cosmos_v1_2B_multiview", state_t=8, resolution="720p", probs=None, fps_mod=True, cp=8, **model_kw):
    net_over = dict(state_t=state_t, rope_enable_fps_modulation=fps_mod,
                    rope_t_extrapolation_ratio=float(state_t) / 24.0)
    node = dict(
        defaults=[{"override /optimizer": "adamw"}, {"override /scheduler": "lambdalinear"}, {"override /callbacks": "basic"}, "_self_"],
        job=dict(project="cosmos_predict2_multiview", group="cosmos2_mv", name=name),
        model=_mv_model(net, state_t=state_t, resolution=resolution,
                        conditional_frames_probs=probs or {0: 0.5, 1: 0.25, 2: 0.25}, **model_kw),
        model_parallel=dict(context_parallel_size=cp),
        optimizer=dict(lr=2 ** -14.5, weight_decay=1e-3, betas=(0.9, 0.999)),
        scheduler=dict(f_max=(0.99,), f_min=(0.4,), warm_up_steps=(100,), cycle_lengths=(400_000,)),
        trainer=dict(max_iter=150_000, logging_iter=200, callbacks=dict(grad_clip=dict(clip_norm=0.1))),
        checkpoint=dict(save_iter=500),
    )
    node["model"]["config"]["net"].update(net_over)
    cs.store(group="experiment", package="_global_", name=name, node=node)


_P = "buttercup_predict2p5_2b_mv_7views_"
_exp(_P + "res720p_fps10_t8_frompred2p1multicaps8k_jointalpamayov2mads720pmulticaps")
_exp(_P + "res720p_fps15_t8_from16kfps10mv_jointalpamayov2mads720pmulticaps57framesto29")
_exp(_P + "res720p_fps30_t8_from16kfps10mv_jointalpamayov2mads720pmulticaps29frames")
_exp(_P + "res720p_fps30_t8_from16kfps10mv_jointalpamayov2mads720pmulticaps29frames_nofps", fps_mod=False)
_exp(_P + "res480p_fps30_t16_from16kfps10mv_jointalpamayov2mads480pmulticaps61frames", state_t=16, resolution="480p")
_exp(_P + "res720p_fps15_t8_frombase2p5_jointalpamayov2mads720pmulticaps57framesto29")
_exp(_P + "res720p_fps30_t8_frombase2p5_jointalpamayov2mads720pmulticaps29frames")
_exp(_P + "res720p_fps30_t8_frombase2p5_alpamayov2_720p_allviewcapswithprefix_29frames")
_exp(_P + "res720p_fps30_t8_from28kfps30mv_alpamayov2_720p_allviewcapswithprefix_29frames")
_Q = "buttercup_predict2p5_2b_7views_"
_C0442 = {0: 0.4, 1: 0.4, 2: 0.2}
_exp(_Q + "res720p_fps30_t8_from48kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames", probs=_C0442)
_exp(_Q + "res720p_fps30_t8_from48kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames_nofps",
     probs=_C0442, fps_mod=False)
_exp(_Q + "res480p_fps30_t16_from41kfps30mv_condprobs0442_joint_alpamayo1capnoviewprefix_allcapsviewprefix_61frames_nofps",
     probs=_C0442, fps_mod=False, state_t=16, resolution="480p")
_exp("buttercup_predict2p5_14b_7views_res720p_fps30_t8_joint_alpamayo1capnoviewprefix_allcapsviewprefix_29frames_nofps",
     net="cosmos_v1_14B_multiview", probs=_C0442, fps_mod=False, text_dropout=0.1, fsdp_shard_size=32)
# robot multi-camera checkpoints of the public registry
_exp("multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_multicam_syncam", state_t=24, resolution="720", fps_mod=False,
     condition_locations=["ref_cam", "first_random_n"])
_exp("multicamera_video2video_rectified_flow_2b_res_720_fps16_s3_agibot", state_t=24, resolution="720", fps_mod=False,
     condition_locations=["ref_cam", "first_random_n"])



def _exp_edm(name, lr=2 ** -14.5, **model_kw):
    node = dict(
        defaults=[{"override /optimizer": "adamw"}, {"override /scheduler": "lambdalinear"}, {"override /callbacks": "basic"}, "_self_"],
        job=dict(project="cosmos_predict2_multiview", group="cosmos2_mv", name=name),
        model=_mv_edm_model(**model_kw),
        model_parallel=dict(context_parallel_size=8),
        optimizer=dict(lr=lr, weight_decay=1e-3, betas=(0.9, 0.999)),
        checkpoint=dict(save_iter=500),
    )
    cs.store(group="experiment", package="_global_", name=name, node=node)


_R = "buttercup_predict2p1_2b_mv_7views_res720p_fps10_t8_"
_exp_edm(_R + "frombase2p1iter45k_alpamayo85to29res720p")
_exp_edm(_R + "frombase2p1iter45k_mads720p")
_exp_edm(_R + "frombase2p1iter45k_jointalpamayov2mads720p")
_exp_edm(_R + "from23klr1x_jointalpamayov2mads720p_lr2x", lr=2 ** -13.5)
_exp_edm(_R + "from42p5k_jointalpamayov2mads720p_multiwindow_multicaptions")

cs.store(group="experiment", package="_global_", name="tiny_multiview_edm_cpu", node=dict(
    defaults=["_self_"],
    job=dict(group="tests", name="tiny_multiview_edm_cpu"),
    model=_mv_edm_model("tiny_multiview", tokenizer="dummy_tokenizer", precision="float32", state_t=2, tokens_per_view=8,
                        resolution="tiny", sharding_transport="nccl"),
    dataloader_train=L(build_dataloader)(dataset=L(MockMultiviewLatentDataset)(n_views=3, state_t=2, height=8, width=8, text_dim=256,
                                                                               text_len=8, length=16), batch_size=1, num_workers=0),
    optimizer=dict(lr=1e-3),
    scheduler=dict(warm_up_steps=(0,), f_start=(1.0,)),
    trainer=dict(max_iter=2, logging_iter=1, callbacks=dict()),
    checkpoint=dict(save_iter=0),
))

cs.store(group="experiment", package="_global_", name="tiny_multiview_cpu", node=dict(
    defaults=["_self_"],
    job=dict(group="tests", name="tiny_multiview_cpu"),
    model=_mv_model("tiny_multiview", tokenizer="dummy_tokenizer", precision="float32", state_t=2, tokens_per_view=8,
                    resolution="tiny", sharding_transport="nccl"),
    dataloader_train=L(build_dataloader)(dataset=L(MockMultiviewLatentDataset)(n_views=3, state_t=2, height=8, width=8, text_dim=256,
                                                                               text_len=8, length=16), batch_size=1, num_workers=0),
    optimizer=dict(lr=1e-3),
    scheduler=dict(warm_up_steps=(0,), f_start=(1.0,)),
    trainer=dict(max_iter=2, logging_iter=1, callbacks=dict()),
    checkpoint=dict(save_iter=0),
))
