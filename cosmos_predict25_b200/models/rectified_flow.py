"""Rectified-flow world models: Text2World and Video2World (Image2World = 1 conditioning frame).

The algorithm object the trainer and the inference pipeline talk to. Parity targets:
``Text2WorldModelRectifiedFlow`` (cosmos_predict2/_src/predict2/models/text2world_model_rectified_flow.py:106-919)
and ``Video2WorldModelRectifiedFlow`` (cosmos_predict2/_src/predict2/models/video2world_model_rectified_flow.py:44-211).

Contract (the reference's ``ImaginaireModel``, cosmos_predict2/_src/imaginaire/model.py:23-129):
``training_step(batch, iteration) -> (outputs, loss)``, ``generate_samples_from_batch``, ``encode`` / ``decode``,
``init_optimizer_scheduler``, ``on_train_start``, ``on_before_zero_grad``, ``state_dict`` /
``load_state_dict`` with ``net.`` / ``net_ema.`` prefixes, ``ema_scope``, ``clip_grad_norm_``.

Differences by design:
  * parameters, fp32 masters, Adam moments and the EMA live in the flat sharded buffers of
    ``parallel.fsdp.ShardedEngine`` (world size 1 is the same code path);
  * classifier-free guidance runs cond and uncond as ONE batch-2 forward, and the projected text
    context and cross-attention K/V are computed once per prompt instead of once per call;
  * a batch may carry pre-encoded ``latents`` instead of pixels.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass, field, replace
from typing import Any, Callable, Dict, Optional, Tuple

import numpy as np
import torch
import torch.nn as nn

from ..ops import functional as ops
from ..parallel import context_parallel as cp
from ..parallel.fsdp import ShardedEngine
from .conditioner import (DataType, GeneralConditioner, Text2WorldCondition, Video2WorldCondition,
                          default_text2world_conditioner, default_video2world_conditioner)
from .dit import NET_PRESETS, CosmosDiT, DiTConfig
from .schedulers import FlowEulerSolver, FlowUniPCSolver, RectifiedFlowSchedule

NUM_CONDITIONAL_FRAMES_KEY = "num_conditional_frames"
IS_PREPROCESSED_KEY = "is_preprocessed"


@dataclass
class EMAConfig:
    enabled: bool = True
    rate: float = 0.1
    iteration_shift: int = 0


@dataclass
class Text2WorldRFConfig:
    net: DiTConfig = field(default_factory=DiTConfig)
    tokenizer: Any = None            # object with the VideoTokenizer interface (or None -> latents only)
    conditioner: Any = None
    ema: EMAConfig = field(default_factory=EMAConfig)
    fsdp_shard_size: int = 1
    precision: str = "bfloat16"
    input_data_key: str = "video"
    input_image_key: str = "images"
    input_latent_key: str = "latents"
    input_caption_key: str = "ai_caption"
    state_ch: int = 16
    state_t: int = 24
    resolution: str = "720"
    text_encoder: Any = None          # optional online text encoder (compute_text_embeddings_online)
    use_lora: bool = False
    lora_rank: int = 32
    lora_alpha: int = 32
    lora_target_modules: str = "q_proj,k_proj,v_proj,output_proj,mlp.layer1,mlp.layer2"
    shift: float = 5.0
    train_time_distribution: str = "logitnormal"
    train_time_weight: str = "uniform"
    use_high_sigma_strategy: bool = False
    high_sigma_ratio: float = 0.05
    high_sigma_timesteps_min: int = 980
    high_sigma_timesteps_max: int = 1000
    use_kerras_sigma_at_inference: bool = False
    text_dropout: float = 0.2
    sharding_transport: str = "nccl"   # nccl | peer | peer_reshard
    cp_comm_type: str = "a2a"          # context-parallel exchange in self-attention: a2a (Ulysses) | p2p (ring)


@dataclass
class Video2WorldRFConfig(Text2WorldRFConfig):
    min_num_conditional_frames: int = 1
    max_num_conditional_frames: int = 2
    conditional_frame_timestep: float = -1.0
    denoise_replace_gt_frames: bool = True
    conditional_frames_probs: Optional[Dict[int, float]] = None


_PRECISION = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}


def ema_exp_coefficient(rate: float) -> float:
    """gamma of the power-function EMA: largest real root of x^3 + 7x^2 + (16 - s^-2)x + (12 - s^-2)."""
    s = rate
    return float(np.roots([1, 7, 16 - s ** -2, 12 - s ** -2]).real.max())


def materialise_config(config):
    """Build the fields of a model config that were given as lazy calls (network, tokenizer, conditioner, EMA, text encoder): the
    reference's way of writing ``Config(net=mini_net, tokenizer=DummyJointImageVideoConfig, ...)`` with registry constants."""
    from ..utils.lazy_config import instantiate, is_lazy
    for name in ("net", "tokenizer", "conditioner", "ema", "text_encoder"):
        v = getattr(config, name, None)
        if is_lazy(v):
            setattr(config, name, instantiate(v))
    return config


class Text2WorldModelRectifiedFlow(nn.Module):
    condition_is_video2world = False

    def __init__(self, config: Text2WorldRFConfig, device: Optional[torch.device] = None, fsdp_group=None, cp_group=None,
                 replicate_group=None):
        super().__init__()
        config = materialise_config(config)
        self.config = config
        self.replicate_group = replicate_group
        self.precision = _PRECISION[config.precision]
        self.device_ = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                                  else torch.device("cpu"))
        self.tensor_kwargs = {"device": self.device_, "dtype": self.precision}
        self.tensor_kwargs_fp32 = {"device": self.device_, "dtype": torch.float32}
        self.fsdp_group = fsdp_group
        self.cp_group = cp_group
        self.tokenizer = config.tokenizer
        self.text_encoder = config.text_encoder
        self.conditioner: GeneralConditioner = config.conditioner or (
            default_video2world_conditioner(config.text_dropout) if self.condition_is_video2world
            else default_text2world_conditioner(config.text_dropout))
        self.rectified_flow = RectifiedFlowSchedule(config.shift, 1000, config.train_time_distribution,
                                                    config.train_time_weight)
        self.sample_scheduler = FlowUniPCSolver(num_train_timesteps=1000, shift=1.0)
        self.net = self.build_net()
        self.engine: Optional[ShardedEngine] = None
        self.ema_exp_coefficient = ema_exp_coefficient(config.ema.rate) if config.ema.enabled else None
        self._ema_active = False

    # ---- construction ----------------------------------------------------------------------
    def build_net(self) -> CosmosDiT:
        net = CosmosDiT(self.config.net).to(self.device_)
        net.init_weights()
        if self.config.use_lora:
            from .lora import add_lora
            add_lora(net, self.config.lora_rank, self.config.lora_alpha, self.config.lora_target_modules)
        return net

    def on_train_start(self):
        """Move parameters into the flat sharded buffers (bf16 compute copies + fp32 masters + EMA)."""
        if self.engine is None:
            if self.config.use_lora:  # frozen base weights take the compute dtype; adapters get fp32 masters in the engine
                for p in self.net.parameters():
                    if not p.requires_grad and p.is_floating_point():
                        p.data = p.data.to(self.precision)
            make = ShardedEngine
            import torch.distributed as dist
            n_shard = dist.get_world_size(self.fsdp_group) if (self.fsdp_group is not None and dist.is_initialized()) else 1
            # peer kernels address one NVSwitch domain (2..8 ranks); anything else goes through NCCL
            if self.config.sharding_transport == "peer_reshard" and self.device_.type == "cuda" and 2 <= n_shard <= 8:
                # block parameters are not kept resident: their all-gather is fused into the consuming GEMMs
                from ..parallel.reshard_fsdp import ReshardEngine as make
            elif self.config.sharding_transport in ("peer", "peer_reshard") and self.device_.type == "cuda" and 2 <= n_shard <= 8:
                from ..parallel.peer_fsdp import PeerShardedEngine as make
            self.engine = make(self.net, group=self.fsdp_group, compute_dtype=self.precision,
                               use_ema=self.config.ema.enabled, replicate_group=self.replicate_group,
                               transport="nccl" if make is ShardedEngine else "peer")
        if self.tokenizer is not None and hasattr(self.tokenizer, "reset_dtype"):
            self.tokenizer.reset_dtype()

    def init_optimizer_scheduler(self, optimizer_config, scheduler_config):
        from ..trainer.optim import build_optimizer, build_scheduler
        if self.engine is None:
            self.on_train_start()
        opt = build_optimizer(optimizer_config, self.engine)
        return opt, build_scheduler(scheduler_config, opt)

    # ---- EMA -----------------------------------------------------------------------------------
    def ema_beta(self, iteration: int) -> float:
        """beta_i = (1 - 1/(i+1))^(gamma+1), 0 before the first update."""
        it = iteration + self.config.ema.iteration_shift
        if it < 1:
            return 0.0
        return (1 - 1 / (it + 1)) ** (self.ema_exp_coefficient + 1)

    def on_before_zero_grad(self, optimizer, scheduler, iteration: int):
        """EMA is folded into the optimizer kernel; nothing left to do here."""

    @contextlib.contextmanager
    def ema_scope(self, context: Optional[str] = None, is_cpu: bool = False):
        """Temporarily run the network with EMA weights."""
        if self.config.ema.enabled and self.engine is not None:
            self.engine.load_ema_into_params()
            self._ema_active = True
            try:
                yield
            finally:
                self.engine.restore_params()
                self._ema_active = False
        else:
            yield

    # ---- data ----------------------------------------------------------------------------------
    def is_image_batch(self, batch: Dict) -> bool:
        has_img = self.config.input_image_key in batch
        has_vid = self.config.input_data_key in batch or self.config.input_latent_key in batch
        assert has_img != has_vid, "a batch must carry exactly one of images / video"
        return has_img

    def _normalize_video_databatch_inplace(self, batch: Dict):
        key = self.config.input_data_key
        if key in batch and not batch.get(IS_PREPROCESSED_KEY, False):
            v = batch[key]
            if v.dtype == torch.uint8:
                batch[key] = v.to(**self.tensor_kwargs_fp32) / 127.5 - 1.0
            batch[IS_PREPROCESSED_KEY] = True

    def _augment_image_dim_inplace(self, batch: Dict):
        key = self.config.input_image_key
        if key in batch and batch[key].ndim == 4:
            x = batch[key]
            if x.dtype == torch.uint8:
                x = x.to(**self.tensor_kwargs_fp32) / 127.5 - 1.0
            batch[key] = x.unsqueeze(2)

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        """Pixels -> latent. With ``shard_vae_encode`` set (the inference pipeline sets it: there every rank of the
        context-parallel group holds the same conditioning clip) the ranks encode one horizontal band each."""
        if getattr(self, "shard_vae_encode", False) and self.cp_group is not None and cp._size_rank(self.cp_group)[0] > 1 \
                and hasattr(self.tokenizer, "encode_parallel"):
            return self.tokenizer.encode_parallel(state, self.cp_group)
        return self.tokenizer.encode(state)

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        """Latent -> pixels. Under context parallelism every rank holds the gathered latent after sampling; the ranks
        of the group then decode one horizontal band of the frame each (exact, neighbours exchange boundary rows)
        and all of them return the whole video."""
        if self.cp_group is not None and cp._size_rank(self.cp_group)[0] > 1 and hasattr(self.tokenizer, "decode_parallel"):
            return self.tokenizer.decode_parallel(latent, self.cp_group)
        return self.tokenizer.decode(latent)

    def get_data_and_condition(self, batch: Dict) -> Tuple[Optional[torch.Tensor], torch.Tensor, Text2WorldCondition]:
        self._normalize_video_databatch_inplace(batch)
        self._augment_image_dim_inplace(batch)
        is_image = self.is_image_batch(batch)
        if self.config.input_latent_key in batch and not is_image:
            raw, latent = None, batch[self.config.input_latent_key].to(**self.tensor_kwargs_fp32)
        else:
            raw = batch[self.config.input_image_key if is_image else self.config.input_data_key]
            latent = self.encode(raw.to(**self.tensor_kwargs)).contiguous().float()
        condition = self.conditioner(batch)
        condition = replace(condition, data_type=DataType.IMAGE if is_image else DataType.VIDEO)
        return raw, latent, condition

    # ---- context parallel ------------------------------------------------------------------------
    def broadcast_split_for_model_parallelsim(self, x0, condition, eps, t):
        """Make the CP group agree on rank-0's sample, then keep the local T-slice. CP is enabled for
        video batches and disabled for images."""
        group = self.cp_group
        size = cp._size_rank(group)[0]
        is_video = condition.data_type == DataType.VIDEO
        if size > 1 and is_video:
            if x0 is not None:
                x0 = cp.broadcast_split_tensor(x0, 2, group)
            if eps is not None:
                eps = cp.broadcast_split_tensor(eps, 2, group)
            if t is not None:
                t = cp.broadcast(t, group)
            condition = condition.broadcast(group)
            self.net.enable_context_parallel(group, getattr(self.config, "cp_comm_type", "a2a"))
        else:
            self.net.disable_context_parallel()
        return x0, condition, eps, t

    # ---- training --------------------------------------------------------------------------------
    def training_step(self, data_batch: Dict, iteration: int):
        cfg = self.config
        if self.text_encoder is not None and "t5_text_embeddings" not in data_batch:
            emb = self.text_encoder.compute_text_embeddings_online(data_batch, cfg.input_caption_key)
            data_batch["t5_text_embeddings"] = emb
        _, x0, condition = self.get_data_and_condition(data_batch)
        eps = torch.randn(x0.shape, **self.tensor_kwargs_fp32)
        B = x0.shape[0]
        u = self.rectified_flow.sample_train_time(B).to(**self.tensor_kwargs_fp32).view(B, 1)
        x0, condition, eps, u = self.broadcast_split_for_model_parallelsim(x0, condition, eps, u)
        # the time tables live on the device, so the index never comes back to the host (no synchronisation per step)
        table_t, table_s = self._rf_tables()
        idx = self.rectified_flow.indices(u)
        if cfg.use_high_sigma_strategy:
            cand = torch.nonzero((table_t >= cfg.high_sigma_timesteps_min) & (table_t <= cfg.high_sigma_timesteps_max)).view(-1)
            if len(cand) == 0:
                raise ValueError("no candidate timesteps for the high-sigma strategy")
            pick = torch.rand(idx.shape, device=idx.device) < cfg.high_sigma_ratio
            idx = torch.where(pick, cand[torch.randint(0, len(cand), idx.shape, device=idx.device)], idx)
            if cp._size_rank(self.cp_group)[0] > 1:
                idx = cp.broadcast(idx, self.cp_group)
        timesteps = table_t[idx].view(B, 1)
        sigmas = table_s[idx].view(B, 1)
        xt, vt = self.rectified_flow.interpolate(eps, x0, sigmas)
        v_pred = self.denoise(eps, xt.to(**self.tensor_kwargs), timesteps, condition)
        w = self.rectified_flow.loss_weight(timesteps.view(-1))
        per_instance = torch.mean((v_pred - vt) ** 2, dim=list(range(1, v_pred.ndim)))
        loss = torch.mean(w * per_instance)
        out = {"x0": x0, "xt": xt, "sigma": sigmas, "condition": condition, "model_pred": v_pred, "edm_loss": loss}
        return out, loss

    def _rf_tables(self):
        """(timesteps, sigmas) of the training schedule as fp32 tensors on the model's device (copied once)."""
        if getattr(self, "_rf_tables_dev", None) is None:
            self._rf_tables_dev = (self.rectified_flow.timesteps.to(**self.tensor_kwargs_fp32),
                                   self.rectified_flow.sigmas.to(**self.tensor_kwargs_fp32))
        return self._rf_tables_dev

    def _net_kwargs(self, condition: Text2WorldCondition) -> Dict[str, Any]:
        return {"crossattn_emb": condition.crossattn_emb.to(self.precision) if condition.crossattn_emb is not None else None,
                "fps": condition.fps, "padding_mask": condition.padding_mask}

    def denoise(self, noise: torch.Tensor, xt_B_C_T_H_W: torch.Tensor, timesteps_B_T: torch.Tensor,
                condition: Text2WorldCondition, context_cache=None) -> torch.Tensor:
        """Velocity prediction (fp32 out)."""
        return self.net(xt_B_C_T_H_W.to(**self.tensor_kwargs), timesteps_B_T, context_cache=context_cache,
                        **self._net_kwargs(condition)).float()

    # ---- sampling ----------------------------------------------------------------------------------
    def _conditions_for_sampling(self, batch: Dict, is_negative_prompt: bool):
        if is_negative_prompt:
            c, u = self.conditioner.get_condition_with_negative_prompt(batch)
        else:
            c, u = self.conditioner.get_condition_uncondition(batch)
        dt = DataType.IMAGE if self.is_image_batch(batch) else DataType.VIDEO
        return replace(c, data_type=dt), replace(u, data_type=dt)

    def get_velocity_fn_from_batch(self, data_batch: Dict, guidance: float = 1.5, is_negative_prompt: bool = False) -> Callable:
        condition, uncondition = self._conditions_for_sampling(data_batch, is_negative_prompt)
        _, condition, _, _ = self.broadcast_split_for_model_parallelsim(None, condition, None, None)
        _, uncondition, _, _ = self.broadcast_split_for_model_parallelsim(None, uncondition, None, None)
        return self._batched_cfg_fn(condition, uncondition, guidance, t2w_formula=True)

    def _batched_cfg_fn(self, condition, uncondition, guidance: float, t2w_formula: bool) -> Callable:
        """One batch-2 forward per step: rows [cond; uncond]. Text2World combines as
        uncond + g*(cond - uncond), Video2World as cond + g*(cond - uncond)."""
        both = _stack_conditions(condition, uncondition)
        with torch.no_grad():
            cache = self.net.build_context_cache(both.crossattn_emb.to(self.precision))

        def velocity_fn(noise: torch.Tensor, noise_x: torch.Tensor, timestep: torch.Tensor) -> torch.Tensor:
            B = noise_x.shape[0]
            x2 = torch.cat([noise_x, noise_x], 0)
            n2 = torch.cat([noise, noise], 0)
            t2 = torch.cat([timestep, timestep], 0)
            v = self.denoise(n2, x2, t2, both, context_cache=cache)
            cond_v, uncond_v = v[:B], v[B:]
            if t2w_formula:
                return uncond_v + guidance * (cond_v - uncond_v)
            return ops.cfg_combine(cond_v, uncond_v, guidance)

        return velocity_fn

    @torch.no_grad()
    def generate_samples_from_batch(self, data_batch: Dict, guidance: float = 1.5, seed: int = 1,
                                    state_shape: Optional[Tuple] = None, n_sample: Optional[int] = None,
                                    is_negative_prompt: bool = False, num_steps: int = 35, shift: float = 5.0,
                                    solver: str = "unipc", **kwargs) -> torch.Tensor:
        """Sample latents [n, C, T, H, W] with the multistep flow solver and classifier-free guidance."""
        self._normalize_video_databatch_inplace(data_batch)
        self._augment_image_dim_inplace(data_batch)
        is_image = self.is_image_batch(data_batch)
        key = self.config.input_image_key if is_image else (
            self.config.input_data_key if self.config.input_data_key in data_batch else self.config.input_latent_key)
        if n_sample is None:
            n_sample = data_batch[key].shape[0]
        if state_shape is None:
            if key == self.config.input_latent_key:
                state_shape = tuple(data_batch[key].shape[1:])
            else:
                _T, _H, _W = data_batch[key].shape[-3:]
                tk = self.tokenizer
                state_shape = (self.config.state_ch, tk.get_latent_num_frames(_T),
                               _H // tk.spatial_compression_factor, _W // tk.spatial_compression_factor)
        from ..utils.misc import arch_invariant_rand
        noise = arch_invariant_rand((n_sample,) + tuple(state_shape), torch.float32, self.device_, seed)
        velocity_fn = self.get_velocity_fn_from_batch(data_batch, guidance, is_negative_prompt)
        cp_size = cp._size_rank(self.cp_group)[0]
        if self.net.is_context_parallel_enabled and cp_size > 1:
            noise = cp.broadcast_split_tensor(noise, 2, self.cp_group)
        sched = FlowUniPCSolver(1000, shift=1.0) if solver == "unipc" else FlowEulerSolver(1000, shift=1.0)
        sched.set_timesteps(num_steps, device="cpu", shift=shift, use_kerras_sigma=self.config.use_kerras_sigma_at_inference)
        latents = noise
        ones = torch.ones(n_sample, 1, **self.tensor_kwargs_fp32)
        for t in sched.timesteps.tolist():
            v = velocity_fn(noise, latents, ones * float(t))      # the fp32 state: denoise casts where it replaces the frames
            latents = sched.step(v, t, latents)
        if self.net.is_context_parallel_enabled and cp_size > 1:
            latents = cp.cat_outputs_cp(latents, 2, self.cp_group)
        return latents

    # ---- gradient clipping (global norm over shards) -------------------------------------------------
    def clip_grad_norm_(self, max_norm: float, **_):
        """Clipping is applied inside ``ShardedEngine.step``; this returns the current global norm."""
        self.engine.finish_backward()
        return self.engine.grad_norm()

    # ---- checkpoints -------------------------------------------------------------------------------------
    def state_dict(self, *args, **kwargs) -> Dict[str, torch.Tensor]:
        """Consolidated state: ``net.*`` (compute dtype) and ``net_ema.*`` (fp32), plus buffers."""
        out = {}
        if self.engine is not None:
            for k, v in self.engine.full_state_dict("master", self.precision).items():
                out["net." + k] = v
            if self.config.ema.enabled:
                for k, v in self.engine.full_state_dict("ema", torch.float32).items():
                    out["net_ema." + k] = v
            pnames = {n for n, _ in self.net.named_parameters()}
            for k, v in self.net.state_dict().items():
                if k not in pnames:
                    out["net." + k] = v
                    if self.config.ema.enabled:
                        out["net_ema." + k] = v
        else:
            for k, v in self.net.state_dict().items():
                out["net." + k] = v
        return out

    def load_state_dict(self, state_dict: Dict[str, torch.Tensor], strict: bool = True, assign: bool = False,
                        load_ema_to_reg: bool = False):
        """Accepts ``net.*`` / ``net_ema.*`` keys; skips ``_extra_state`` entries and (when not strict)
        shape-mismatched tensors. ``load_ema_to_reg`` loads the EMA weights as the regular ones."""
        reg = {k[len("net."):]: v for k, v in state_dict.items() if k.startswith("net.") and not k.endswith("_extra_state")}
        ema = {k[len("net_ema."):]: v for k, v in state_dict.items() if k.startswith("net_ema.") and not k.endswith("_extra_state")}
        if not reg and not ema:  # a bare network state dict
            reg = {k: v for k, v in state_dict.items() if not k.endswith("_extra_state")}
        if load_ema_to_reg and ema:
            reg = ema
        reg = {k.replace(".base_layer.", "."): v for k, v in reg.items()}
        own = self.net.state_dict()
        bad = [k for k, v in reg.items() if k in own and tuple(own[k].shape) != tuple(v.shape)]
        if bad and strict:
            raise RuntimeError(f"shape mismatch for {bad[:4]}")
        for k in bad:
            reg.pop(k)
        if self.engine is not None:
            pnames = {n for n, _ in self.net.named_parameters()}
            missing = self.engine.load_full_state_dict({k: v for k, v in reg.items() if k in pnames}, "master", strict=False)
            if ema and self.config.ema.enabled:
                self.engine.load_full_state_dict({k: v for k, v in ema.items() if k in pnames}, "ema", strict=False)
            elif self.config.ema.enabled:
                for u in self.engine.units:
                    u.ema.copy_(u.master)
            bufs = {k: v for k, v in reg.items() if k not in pnames}
            res = self.net.load_state_dict(bufs, strict=False)
            unexpected = list(res.unexpected_keys)
        else:
            res = self.net.load_state_dict(reg, strict=False)
            missing, unexpected = list(res.missing_keys), list(res.unexpected_keys)
        if strict and (missing or unexpected):
            raise RuntimeError(f"missing {missing[:4]} unexpected {unexpected[:4]}")
        return missing, unexpected


def _stack_conditions(a, b):
    """Concatenate two condition records along the batch dim."""
    kw = {}
    for k, va in a.to_dict(skip_underscore=False).items():
        vb = getattr(b, k)
        if isinstance(va, torch.Tensor) and va.ndim > 0 and isinstance(vb, torch.Tensor):
            kw[k] = torch.cat([va, vb], 0)
        elif k == "use_video_condition":
            kw[k] = (va, vb)
        else:
            kw[k] = va
    return type(a)(**kw)


class Video2WorldModelRectifiedFlow(Text2WorldModelRectifiedFlow):
    """Adds clean-frame conditioning: frame replacement on the input, the mask as a network input,
    optional fixed timestep on conditioning frames, exact velocity on conditioning frames."""

    condition_is_video2world = True

    def get_data_and_condition(self, batch: Dict):
        raw, latent, condition = super().get_data_and_condition(batch)
        cfg = self.config
        condition = condition.set_video_condition(
            gt_frames=latent.to(**self.tensor_kwargs), random_min_num_conditional_frames=cfg.min_num_conditional_frames,
            random_max_num_conditional_frames=cfg.max_num_conditional_frames,
            num_conditional_frames=batch.get(NUM_CONDITIONAL_FRAMES_KEY), conditional_frames_probs=cfg.conditional_frames_probs)
        return raw, latent, condition

    @staticmethod
    def _use_flags(condition, B: int, like: torch.Tensor) -> torch.Tensor:
        u = condition.use_video_condition
        if isinstance(u, tuple):  # stacked cond/uncond halves
            parts = [torch.full((B // 2,), float(bool(x)), device=like.device) for x in u]
            return torch.cat(parts).view(B, 1, 1, 1, 1).to(like.dtype)
        return torch.full((B, 1, 1, 1, 1), float(bool(u)), device=like.device, dtype=like.dtype)

    def denoise(self, noise, xt_B_C_T_H_W, timesteps_B_T, condition: Video2WorldCondition, context_cache=None):
        cfg = self.config
        is_video = condition.data_type == DataType.VIDEO
        mask = None
        if is_video:
            B, C = xt_B_C_T_H_W.shape[:2]
            mask = condition.condition_video_input_mask_B_C_T_H_W.type_as(xt_B_C_T_H_W)
            # conditioning frames replace the noisy ones; on a GPU one kernel that writes the network's input dtype directly
            xt_B_C_T_H_W = ops.frame_blend(xt_B_C_T_H_W, condition.gt_frames.type_as(xt_B_C_T_H_W), None, mask,
                                           self._use_flags(condition, B, xt_B_C_T_H_W), out_dtype=self.tensor_kwargs.get("dtype"))
            if cfg.conditional_frame_timestep >= 0:
                m_B_T = mask.mean(dim=[1, 3, 4]).float()
                timesteps_B_T = cfg.conditional_frame_timestep * m_B_T + timesteps_B_T.float().view(B, -1) * (1 - m_B_T)
        out = self.net(xt_B_C_T_H_W.to(**self.tensor_kwargs), timesteps_B_T,
                       condition_video_input_mask_B_C_T_H_W=mask, context_cache=context_cache,
                       **self._net_kwargs(condition)).float()
        if is_video and cfg.denoise_replace_gt_frames:
            out = ops.frame_blend(out, condition.gt_frames.type_as(out), noise.type_as(out), mask)
        return out

    def get_velocity_fn_from_batch(self, data_batch: Dict, guidance: float = 1.5, is_negative_prompt: bool = False):
        n_cond = data_batch.get(NUM_CONDITIONAL_FRAMES_KEY, 1)
        condition, uncondition = self._conditions_for_sampling(data_batch, is_negative_prompt)
        _, x0, _ = Text2WorldModelRectifiedFlow.get_data_and_condition(self, data_batch)
        x0 = x0.to(**self.tensor_kwargs)
        condition = condition.set_video_condition(x0, 0, 0, num_conditional_frames=n_cond)
        uncondition = uncondition.set_video_condition(x0, 0, 0, num_conditional_frames=n_cond)
        condition = condition.edit_for_inference(True, n_cond)
        uncondition = uncondition.edit_for_inference(False, n_cond)
        _, condition, _, _ = self.broadcast_split_for_model_parallelsim(None, condition, None, None)
        _, uncondition, _, _ = self.broadcast_split_for_model_parallelsim(None, uncondition, None, None)
        return self._batched_cfg_fn(condition, uncondition, guidance, t2w_formula=False)
