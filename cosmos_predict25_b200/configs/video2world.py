"""Project config for Video2World / Text2World rectified-flow training and inference.

``make_config()`` returns the default tree; importing this module registers the config groups
(net, conditioner, tokenizer, ema, optimizer, scheduler, callbacks, checkpoint, data_train, data_val) and the
experiments in the config store. Experiment names are the reference's, so ``experiment=<name>`` strings from its
docs and checkpoint registry resolve here (cosmos_predict2/_src/predict2/configs/video2world/config.py:37-102,
.../experiment/reason_embeddings/model_2B_reason_1p1_rectified_flow.py:262-457,
.../model_14b_reason_1p1_rectified_flow.py:78-509, cosmos_predict2/experiments/base/cosmos_nemo_assets.py:31-117,
cosmos_predict2/experiments/base/groot.py:49).
"""

from __future__ import annotations

from ..data.mock import MockVideoLatentDataset, MockVideoPixelDataset, build_dataloader
from ..data.video_dataset import VideoDataset
from ..models.conditioner import (BooleanFlag, ReMapkey, TextAttr, Video2WorldConditioner, VideoConditioner)
from ..models.dit import DiTConfig
from ..models.rectified_flow import (EMAConfig, Text2WorldModelRectifiedFlow, Text2WorldRFConfig, Video2WorldModelRectifiedFlow,
                                     Video2WorldRFConfig)
from ..models.vae_wan import DummyTokenizer, Wan2pt1VAEInterface
from ..trainer import callbacks as cb
from ..trainer.optim import OptimizerConfig, SchedulerConfig
from ..utils.config import Config, ConfigStore
from ..utils.lazy_config import L

cs = ConfigStore.instance()

# ---- networks (cosmos_predict2/_src/predict2/configs/video2world/defaults/net.py:26-110) -------------------------------
_RF_NET = dict(timestep_scale=0.001, use_wan_fp32_strategy=True, use_crossattn_projection=True, crossattn_proj_in_channels=100352,
               crossattn_emb_channels=1024, rope_enable_fps_modulation=False, rope_h_extrapolation_ratio=3.0,
               rope_w_extrapolation_ratio=3.0, rope_t_extrapolation_ratio=1.0)
cs.store(group="net", name="cosmos_v1_2B", node=L(DiTConfig)(model_channels=2048, num_heads=16, num_blocks=28,
                                                             checkpoint_mode="predict2_2b_720_aggressive", **_RF_NET))
cs.store(group="net", name="cosmos_v1_14B", node=L(DiTConfig)(model_channels=5120, num_heads=40, num_blocks=36,
                                                              checkpoint_mode="predict2_14b_720_aggressive", **_RF_NET))
cs.store(group="net", name="cosmos_v1_7B", node=L(DiTConfig)(model_channels=4096, num_heads=32, num_blocks=28,
                                                             extra_per_block_abs_pos_emb=True, **_RF_NET))
cs.store(group="net", name="mini_net", node=L(DiTConfig)(model_channels=1024, num_heads=8, num_blocks=2, **_RF_NET))
cs.store(group="net", name="tiny_net", node=L(DiTConfig)(model_channels=256, num_heads=4, num_blocks=2, crossattn_emb_channels=256,
                                                         use_crossattn_projection=False, adaln_lora_dim=64, max_img_h=64,
                                                         max_img_w=64, max_frames=32))

# ---- conditioners ----------------------------------------------------------------------------------------------------
def _v2w_conditioner(text_dropout):
    return L(Video2WorldConditioner)(
        fps=L(ReMapkey)(input_key="fps", output_key="fps", dropout_rate=0.0),
        padding_mask=L(ReMapkey)(input_key="padding_mask", output_key="padding_mask", dropout_rate=0.0),
        text=L(TextAttr)(input_key="t5_text_embeddings", dropout_rate=text_dropout),
        use_video_condition=L(BooleanFlag)(input_key="fps", output_key="use_video_condition", dropout_rate=0.0))


cs.store(group="conditioner", name="video_prediction_conditioner", node=_v2w_conditioner(0.2))
cs.store(group="conditioner", name="video_prediction_conditioner_14b", node=_v2w_conditioner(0.1))
cs.store(group="conditioner", name="add_fps_padding_mask", node=L(VideoConditioner)(
    fps=L(ReMapkey)(input_key="fps", output_key="fps"), padding_mask=L(ReMapkey)(input_key="padding_mask", output_key="padding_mask"),
    text=L(TextAttr)(input_key="t5_text_embeddings", dropout_rate=0.2)))

# ---- tokenizers, EMA --------------------------------------------------------------------------------------------------------
cs.store(group="tokenizer", name="wan2pt1_tokenizer", node=L(Wan2pt1VAEInterface)(chunk_duration=81, vae_pth="Wan2.1/vae"))
cs.store(group="tokenizer", name="dummy_tokenizer", node=L(DummyTokenizer)())
cs.store(group="tokenizer", name="none", node=None)
cs.store(group="ema", name="power", node=L(EMAConfig)(enabled=True, rate=0.1))
cs.store(group="ema", name="off", node=L(EMAConfig)(enabled=False))

# ---- optimizer / scheduler (defaults/optimizer.py:23-42, common/functional/lr_scheduler.py:157-178) ----------------------------------
cs.store(group="optimizer", name="adamw", node=L(OptimizerConfig)(lr=2 ** -14.5, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-3,
                                                                  max_grad_norm=1.0))
cs.store(group="optimizer", name="fusedadamw", node=L(OptimizerConfig)(lr=2 ** -14.5, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1,
                                                                       max_grad_norm=1.0))
cs.store(group="scheduler", name="lambdalinear", node=L(SchedulerConfig)(kind="lambdalinear", warm_up_steps=(1000,),
                                                                         cycle_lengths=(10_000_000_000,), f_start=(1e-6,),
                                                                         f_max=(1.0,), f_min=(1.0,)))
cs.store(group="scheduler", name="constant", node=L(SchedulerConfig)(kind="constant"))

# ---- callbacks (configs/common/defaults/callbacks.py:32-44) -----------------------------------------------------------------------
BASIC_CALLBACKS = dict(
    grad_clip=L(cb.GradClip)(clip_norm=1.0),
    iter_speed=L(cb.IterSpeed)(every_n="${trainer.logging_iter}", hit_thres=5),
    heart_beat=L(cb.HeartBeat)(every_n=10, update_interval_in_minutes=20),
    device_monitor=L(cb.DeviceMonitor)(every_n="${trainer.logging_iter}"),
    manual_gc=L(cb.ManualGarbageCollection)(every_n=5),
    low_prec=L(cb.LowPrecisionCallback)(update_iter=1),
    wandb=L(cb.WandbCallback)(logging_iter="${trainer.logging_iter}", mode="${job.wandb_mode}"),
    dataloader_speed=L(cb.DetailedDataLoadingSpeedMonitor)(every_n=100),
)
cs.store(group="callbacks", name="basic", node=BASIC_CALLBACKS)
cs.store(group="callbacks", name="none", node=dict())

# ---- checkpoint types ------------------------------------------------------------------------------------------------------------------
cs.store(group="ckpt_type", name="dcp", node="cosmos_predict25_b200.checkpoint.dcp.DistributedCheckpointer")
cs.store(group="ckpt_type", name="dummy", node="cosmos_predict25_b200.checkpoint.simple.DummyCheckpointer")
cs.store(group="ckpt_type", name="pt", node="cosmos_predict25_b200.checkpoint.simple.PtCheckpointer")

# ---- data (configs/common/defaults/dataloader.py:128-133) ----------------------------------------------------------------------------------
cs.store(group="data_train", name="mock", node=L(build_dataloader)(
    dataset=L(MockVideoLatentDataset)(num_frames=24, height=88, width=160, text_dim=100352, length=1 << 30), batch_size=1, num_workers=0))
cs.store(group="data_train", name="mock_video", node=L(build_dataloader)(
    dataset=L(MockVideoPixelDataset)(num_frames=93, height=704, width=1280, text_dim=100352, length=1 << 30), batch_size=1, num_workers=2))
cs.store(group="data_val", name="mock", node=L(build_dataloader)(
    dataset=L(MockVideoLatentDataset)(num_frames=24, height=88, width=160, text_dim=100352, length=16), batch_size=1, num_workers=0))


def _model(net="cosmos_v1_2B", conditioner="video_prediction_conditioner", tokenizer="wan2pt1_tokenizer", **cfg_kw):
    import copy
    kw = dict(net=copy.deepcopy(cs.get("net", net)), conditioner=copy.deepcopy(cs.get("conditioner", conditioner)),
              tokenizer=copy.deepcopy(cs.get("tokenizer", tokenizer)), ema=L(EMAConfig)(enabled=True, rate=0.1), precision="bfloat16",
              state_ch=16, state_t=24, resolution="720", shift=5.0, train_time_distribution="logitnormal",
              min_num_conditional_frames=0, max_num_conditional_frames=2, conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25},
              text_dropout=0.2, sharding_transport="peer")
    kw.update(cfg_kw)
    return L(Video2WorldModelRectifiedFlow)(config=L(Video2WorldRFConfig)(**kw))


def make_config() -> Config:
    c = Config.default()
    c["defaults"] = ["_self_", {"data_train": "mock"}, {"data_val": "mock"}, {"optimizer": "adamw"}, {"scheduler": "lambdalinear"},
                     {"callbacks": "basic"}, {"ckpt_type": "dcp"}, {"experiment": None}]
    c["job"]["project"] = "cosmos_predict_v2p5"
    c["job"]["group"] = "debug"
    c["job"]["name"] = "video2world_${now:%Y-%m-%d_%H-%M-%S}"
    c["model"] = _model()
    return c


# ---- experiments ---------------------------------------------------------------------------------------------------------------------------------
BASE_2B = "Stage-c_pt_4-reason_embeddings-v1p1-Index-26-Size-2B-Res-720-Fps-16-Note-T2V_high_sigma_loss_reweighted_1_1_rectified_flow_only"
BASE_14B = "Stage-c_pt_4-reason_embeddings-v1p1-Index-43-Size-14B-Res-720-Fps-16_resume_from_reason1p1_rectified_flow_shift5_high_sigma"
POST_2B = "Stage-c_pt_4-Index-2-Size-2B-Res-720-Fps-16-Note-rf_with_edm_ckpt"

cs.store(group="experiment", package="_global_", name=BASE_2B, node=dict(
    defaults=[{"override /optimizer": "adamw"}, {"override /scheduler": "lambdalinear"}, {"override /callbacks": "basic"}, "_self_"],
    job=dict(group="official_runs_vid2vid", name=BASE_2B),
    model=_model("cosmos_v1_2B", use_high_sigma_strategy=True, fsdp_shard_size=8),
    model_parallel=dict(context_parallel_size=2),
    optimizer=dict(lr=2 ** -14.5, weight_decay=1e-3, betas=(0.9, 0.999)),
    scheduler=dict(f_max=(0.99,), f_min=(0.4,), warm_up_steps=(100,), cycle_lengths=(400_000,)),
    trainer=dict(max_iter=150_000, logging_iter=200, callbacks=dict(grad_clip=dict(clip_norm=0.1))),
    checkpoint=dict(save_iter=2500),
))
cs.store(group="experiment", package="_global_", name=BASE_2B + "_resume2", node=dict(defaults=[f"/experiment/{BASE_2B}", "_self_"],
                                                                                      job=dict(name=BASE_2B + "_resume2")))
cs.store(group="experiment", package="_global_", name=BASE_14B, node=dict(
    defaults=[f"/experiment/{BASE_2B}", "_self_"],
    job=dict(name=BASE_14B),
    model=_model("cosmos_v1_14B", conditioner="video_prediction_conditioner_14b", use_high_sigma_strategy=True, fsdp_shard_size=32,
                 text_dropout=0.1),
    optimizer=dict(weight_decay=0.2),
))
cs.store(group="experiment", package="_global_", name=POST_2B, node=dict(
    defaults=[f"/experiment/{BASE_2B}", "_self_"],
    job=dict(name=POST_2B),
    model=dict(config=dict(use_kerras_sigma_at_inference=True, conditional_frame_timestep=0.1, use_high_sigma_strategy=False)),
))
# public post-training examples
cs.store(group="experiment", package="_global_", name="predict2_video2world_training_2b_cosmos_nemo_assets", node=dict(
    defaults=[f"/experiment/{BASE_2B}", "_self_"],
    job=dict(project="cosmos_predict_v2p5", group="video2world", name="2b_cosmos_nemo_assets"),
    dataloader_train=L(build_dataloader)(dataset=L(VideoDataset)(dataset_dir="datasets/cosmos_nemo_assets", num_frames=93,
                                                                 video_size=(704, 1280)), batch_size=1, num_workers=4),
    model=dict(config=dict(fsdp_shard_size=8, min_num_conditional_frames=0, max_num_conditional_frames=2,
                           conditional_frames_probs={0: 0.5, 1: 0.25, 2: 0.25})),
    model_parallel=dict(context_parallel_size=1),
    optimizer=dict(lr=2 ** -14.5, weight_decay=0.001),
    scheduler=dict(f_max=(0.5,), f_min=(0.2,), warm_up_steps=(2_000,), cycle_lengths=(100000,)),
    trainer=dict(max_iter=1000, logging_iter=100, callbacks=dict(heart_beat=dict(every_n=200), iter_speed=dict(hit_thres=200))),
    checkpoint=dict(save_iter=200),
))
cs.store(group="experiment", package="_global_", name="predict2_video2world_training_2b_groot_gr1_480", node=dict(
    defaults=["/experiment/predict2_video2world_training_2b_cosmos_nemo_assets", "_self_"],
    job=dict(name="2b_groot_gr1_480"),
    dataloader_train=L(build_dataloader)(dataset=L(VideoDataset)(dataset_dir="datasets/benchmark_train/gr1", num_frames=93,
                                                                 video_size=(432, 768)), batch_size=1, num_workers=4),
    model=dict(config=dict(resolution="480")),
))
# small configurations used by tests and smoke runs
cs.store(group="experiment", package="_global_", name="tiny_video2world_cpu", node=dict(
    defaults=["_self_"],
    job=dict(group="tests", name="tiny_video2world_cpu"),
    model=_model("tiny_net", tokenizer="dummy_tokenizer", precision="float32", state_t=4, sharding_transport="nccl"),
    dataloader_train=L(build_dataloader)(dataset=L(MockVideoLatentDataset)(num_frames=4, height=16, width=16, text_dim=256, text_len=32,
                                                                           length=64), batch_size=1, num_workers=0),
    dataloader_val=L(build_dataloader)(dataset=L(MockVideoLatentDataset)(num_frames=4, height=16, width=16, text_dim=256, text_len=32,
                                                                         length=4), batch_size=1, num_workers=0),
    optimizer=dict(lr=1e-3),
    scheduler=dict(warm_up_steps=(0,), f_start=(1.0,)),
    trainer=dict(max_iter=4, logging_iter=2, callbacks=dict()),
    checkpoint=dict(save_iter=2),
))
cs.store(group="experiment", package="_global_", name="error-free_fsdp_mock-data_mini", node=dict(
    defaults=["_self_"],
    job=dict(group="tests", name="error-free_fsdp_mock-data_mini"),
    model=_model("mini_net", tokenizer="none", state_t=4),
    dataloader_train=L(build_dataloader)(dataset=L(MockVideoLatentDataset)(num_frames=4, height=32, width=32, text_dim=100352,
                                                                           text_len=64, length=64), batch_size=1, num_workers=0),
    trainer=dict(max_iter=4, logging_iter=2),
))

from . import sparse as _sparse_experiments  # noqa: E402,F401  (registers the sparse-attention experiments; needs the names above)
