"""Multiview (N-camera) video-to-video world model on rectified flow.

Parity targets: ``MultiViewCondition`` / ``ConditionLocation`` / ``MultiViewConditioner``
(cosmos_predict2/_src/predict2_multiview/configs/vid2vid/defaults/conditioner.py:40-420),
``MultiviewVid2VidModelRectifiedFlow`` (cosmos_predict2/_src/predict2_multiview/models/multiview_vid2vid_model_rectified_flow.py:59-400:
per-view VAE encode/decode, view-distributed ``encode_cp``/``decode_cp``, per-view context-parallel split, latent view
indices, training-time view sub-sampling, prompt embeddings computed online per view), its noise-level (EDM-era) twin
``MultiviewVid2VidModel`` (cosmos_predict2/_src/predict2_multiview/models/multiview_vid2vid_model.py:64-430) and adaptive projected
guidance (cosmos_predict2/_src/predict2_multiview/models/cfg.py:17-80).

Layout convention everywhere: the V views of a sample are concatenated on the time axis, ``[B, C, V*T, H, W]``.
"""

from __future__ import annotations

import random
from dataclasses import dataclass, field, replace
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from ..parallel import context_parallel as cp
from . import edm
from .conditioner import (BooleanFlag, DataType, GeneralConditioner, ReMapkey, Text2WorldCondition, TextAttr,
                          Video2WorldCondition)
from .multiview_dit import MultiViewDiT
from .rectified_flow import (IS_PREPROCESSED_KEY, NUM_CONDITIONAL_FRAMES_KEY, Text2WorldModelRectifiedFlow,
                             Video2WorldModelRectifiedFlow, Video2WorldRFConfig)

TRAIN_SAMPLE_N_VIEWS_KEY = "train_sample_n_views"
TRAIN_SAMPLING_APPLIED_KEY = "train_sampling_applied"


class ConditionLocation(Enum):
    NO_CAM = "no_cam"                  # text2world
    REF_CAM = "ref_cam"                # all frames of a reference camera are clean
    ANY_CAM = "any_cam"                # all frames of one (random or chosen) camera are clean
    FIRST_RANDOM_N = "first_random_n"  # the first n frames of every camera are clean


def validate_condition_locations(locs: Sequence) -> List[ConditionLocation]:
    out = [l if isinstance(l, ConditionLocation) else ConditionLocation(l) for l in locs]
    if ConditionLocation.NO_CAM in out and len(out) > 1:
        raise ValueError("NO_CAM cannot be combined with another condition location")
    if ConditionLocation.REF_CAM in out and ConditionLocation.ANY_CAM in out:
        raise ValueError("REF_CAM and ANY_CAM cannot be set together")
    return out


def _views(x: torch.Tensor, V: int, dim: int = 2) -> torch.Tensor:
    """[..., V*T, ...] -> [..., V, T, ...] on ``dim``."""
    s = list(x.shape)
    return x.reshape(s[:dim] + [V, s[dim] // V] + s[dim + 1:])


def _unviews(x: torch.Tensor, dim: int = 2) -> torch.Tensor:
    s = list(x.shape)
    return x.reshape(s[:dim] + [s[dim] * s[dim + 1]] + s[dim + 2:])


def views_to_batch(x: torch.Tensor, V: int) -> torch.Tensor:
    """``B C (V T) H W -> (B V) C T H W``."""
    B, C, VT, H, W = x.shape
    return x.view(B, C, V, VT // V, H, W).permute(0, 2, 1, 3, 4, 5).reshape(B * V, C, VT // V, H, W)


def batch_to_views(x: torch.Tensor, V: int) -> torch.Tensor:
    """``(B V) C T H W -> B C (V T) H W``."""
    BV, C, T, H, W = x.shape
    return x.view(BV // V, V, C, T, H, W).permute(0, 2, 1, 3, 4, 5).reshape(BV // V, C, V * T, H, W)


@dataclass(frozen=True)
class MultiViewCondition(Video2WorldCondition):
    state_t: Optional[int] = None
    view_indices_B_T: Optional[torch.Tensor] = None
    ref_cam_view_idx_sample_position: Optional[torch.Tensor] = None

    def set_video_condition(self, state_t: int, gt_frames: torch.Tensor, condition_locations: Sequence = (),
                            random_min_num_conditional_frames_per_view: Optional[int] = None,
                            random_max_num_conditional_frames_per_view: Optional[int] = None,
                            num_conditional_frames_per_view: Optional[int] = None, condition_cam_idx: Optional[int] = None,
                            view_condition_dropout_max: int = 0,
                            conditional_frames_probs: Optional[Dict[int, float]] = None) -> "MultiViewCondition":
        locs = validate_condition_locations(condition_locations)
        assert len(locs) > 0, "condition_locations must be provided"
        B, _, T, H, W = gt_frames.shape
        assert T > 1 and T % state_t == 0, f"T={T} must be a multiple of state_t={state_t}; images are not supported"
        V = T // state_t
        mask = torch.zeros(B, 1, V, state_t, H, W, dtype=gt_frames.dtype, device=gt_frames.device)
        droppable = list(range(V))
        if ConditionLocation.REF_CAM in locs:
            pos = self.ref_cam_view_idx_sample_position
            pos = int(pos.view(-1)[0]) if isinstance(pos, torch.Tensor) else int(pos)
            mask[:, :, pos] = 1
            droppable.remove(pos)
        elif ConditionLocation.ANY_CAM in locs:
            if condition_cam_idx is None:
                # a latent frame per sample picks the camera from the view-index table (draws like the reference: one value per
                # sample; the samples of a batch must agree, their first frames belong to the same view)
                t_sel = torch.randint(0, state_t, size=(B,))
                cams = self.view_indices_B_T[torch.arange(B), t_sel]
                assert (cams == cams[0]).all(), f"the conditioning camera must be the same for all samples, got {cams}"
                condition_cam_idx = int(cams[0])
            mask[:, :, condition_cam_idx] = 1
            droppable.remove(condition_cam_idx)
        if ConditionLocation.FIRST_RANDOM_N in locs:
            lo, hi = random_min_num_conditional_frames_per_view, random_max_num_conditional_frames_per_view
            if num_conditional_frames_per_view is None and lo is not None and lo == hi:
                num_conditional_frames_per_view = lo
            if num_conditional_frames_per_view is not None:
                n_B = [int(num_conditional_frames_per_view)] * B
            elif conditional_frames_probs is not None:
                n_B = random.choices(list(conditional_frames_probs), weights=list(conditional_frames_probs.values()), k=B)
            else:
                assert lo is not None and hi is not None
                n_B = torch.randint(lo, hi + 1, (B,)).tolist()
            for i, n in enumerate(n_B):
                if n > 0:
                    mask[i, :, :, : int(n)] = 1
        if view_condition_dropout_max > 0:
            random.shuffle(droppable)
            for v in droppable[: random.randint(0, view_condition_dropout_max)]:
                mask[:, :, v] = 0
        return replace(self, state_t=state_t, gt_frames=gt_frames,
                       condition_video_input_mask_B_C_T_H_W=mask.view(B, 1, T, H, W))

    def edit_for_inference(self, condition_locations: Sequence = (), is_cfg_conditional: bool = True,
                           num_conditional_frames_per_view: int = 1) -> "MultiViewCondition":
        c = self.set_video_condition(self.state_t, self.gt_frames, condition_locations, 0, 0,
                                     num_conditional_frames_per_view, view_condition_dropout_max=0)
        if not is_cfg_conditional:
            u = c.use_video_condition
            c = replace(c, use_video_condition=torch.ones_like(u, dtype=torch.bool) if isinstance(u, torch.Tensor) else True)
        return c

    def broadcast(self, process_group) -> "MultiViewCondition":
        """Rank-0's condition to all ranks; every view's frames are split over the group."""
        if self._is_broadcasted or process_group is None or cp._size_rank(process_group)[0] == 1:
            return self
        gt, mask, vidx = self.gt_frames, self.condition_video_input_mask_B_C_T_H_W, self.view_indices_B_T
        stripped = replace(self, gt_frames=None, condition_video_input_mask_B_C_T_H_W=None, view_indices_B_T=None)
        base = Text2WorldCondition.broadcast(stripped, process_group)
        V = gt.shape[2] // self.state_t
        gt = _unviews(cp.broadcast_split_tensor(_views(gt, V), seq_dim=3, cp_group=process_group))
        mask = _unviews(cp.broadcast_split_tensor(_views(mask, V), seq_dim=3, cp_group=process_group))
        if vidx is not None:
            vidx = _unviews(cp.broadcast_split_tensor(_views(vidx, V, dim=1), seq_dim=2, cp_group=process_group), dim=1)
        return replace(base, gt_frames=gt, condition_video_input_mask_B_C_T_H_W=mask, view_indices_B_T=vidx)


class MultiViewConditioner(GeneralConditioner):
    condition_cls = MultiViewCondition


def default_multiview_conditioner(text_dropout: float = 0.2) -> MultiViewConditioner:
    return MultiViewConditioner(
        fps=ReMapkey(input_key="fps", output_key="fps"),
        padding_mask=ReMapkey(input_key="padding_mask", output_key="padding_mask"),
        text=TextAttr(input_key="t5_text_embeddings", dropout_rate=text_dropout),
        use_video_condition=BooleanFlag(input_key="fps", output_key="use_video_condition", dropout_rate=0.0),
        view_indices_B_T=ReMapkey(input_key="latent_view_indices_B_T", output_key="view_indices_B_T"),
        ref_cam_view_idx_sample_position=ReMapkey(input_key="ref_cam_view_idx_sample_position",
                                                  output_key="ref_cam_view_idx_sample_position"),
    )


# ---- guidance ---------------------------------------------------------------------------------------------------------
class MomentumBuffer:
    def __init__(self, momentum: float):
        self.momentum, self.running_average = momentum, 0

    def update(self, value: torch.Tensor):
        self.running_average = value + self.momentum * self.running_average


def project(v0: torch.Tensor, v1: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Components of v0 parallel and orthogonal to v1 (per sample, float64 inside)."""
    dims = list(range(1, v0.ndim))
    a, b = v0.double(), torch.nn.functional.normalize(v1.double(), dim=dims)
    par = (a * b).sum(dim=dims, keepdim=True) * b
    return par.to(v0.dtype), (a - par).to(v0.dtype)


def adaptive_projected_guidance(pred_cond: torch.Tensor, pred_uncond: torch.Tensor, guidance_scale: float,
                                momentum_buffer: Optional[MomentumBuffer] = None, eta: float = 1.0,
                                norm_threshold: float = 0.0) -> torch.Tensor:
    diff = pred_cond - pred_uncond
    if momentum_buffer is not None:
        momentum_buffer.update(diff)
        diff = momentum_buffer.running_average
    if norm_threshold > 0:
        n = diff.norm(p=2, dim=list(range(1, diff.ndim)), keepdim=True)
        diff = diff * torch.minimum(torch.ones_like(n), norm_threshold / n)
    par, orth = project(diff, pred_cond)
    return pred_cond + (guidance_scale - 1) * (orth + eta * par)


# ---- model ---------------------------------------------------------------------------------------------------------------
@dataclass
class MultiviewRFConfig(Video2WorldRFConfig):
    min_num_conditional_frames_per_view: int = 1
    max_num_conditional_frames_per_view: int = 2
    train_sample_views_range: Optional[Tuple[int, int]] = None
    condition_locations: List[str] = field(default_factory=lambda: ["first_random_n"])
    state_t: int = 8
    view_condition_dropout_max: int = 0
    tokens_per_view: int = 512
    use_apg: bool = False
    apg_momentum: float = -0.75
    apg_eta: float = 0.0
    apg_norm_threshold: float = 7.5


class _MultiviewMixin:
    """What the rectified-flow model and the noise-level model share: one tokenizer call per view (or one view per rank), view
    sub-sampling, latent view indices, the per-view context-parallel split and prompt embeddings computed online per view."""

    _plain_model = Text2WorldModelRectifiedFlow      # whose ``get_data_and_condition`` gives (raw, latent, condition) without frames
    empty_string_text_embeddings: Optional[torch.Tensor] = None
    neg_text_embeddings: Optional[torch.Tensor] = None

    def _latent_scale(self) -> float:
        return 1.0

    def build_net(self):
        net = MultiViewDiT(self.config.net).to(self.device_)
        net.init_weights()
        if self.config.use_lora:
            from .lora import add_lora
            add_lora(net, self.config.lora_rank, self.config.lora_alpha, self.config.lora_target_modules)
        return net

    # ---- tokenizer: one view at a time, or one view per rank ----------------------------------------------------
    def _pixel_frames_per_view(self) -> int:
        return self.tokenizer.get_pixel_num_frames(self.state_t)

    def _distribute_views(self, x: torch.Tensor, V: int, fn: Callable) -> torch.Tensor:
        """Rank r of the context-parallel group processes view r; results are all-gathered (views <= group size)."""
        size, rank = cp._size_rank(self.cp_group)
        xv = _views(x, V).movedim(2, 0).contiguous()                      # V B C T H W
        pad = torch.zeros((size,) + tuple(xv.shape[1:]), dtype=xv.dtype, device=xv.device)
        pad[:V] = xv
        pad = cp.broadcast(pad, self.cp_group)
        local = fn(pad[rank])                                              # B C T' H W
        outs = [torch.empty_like(local) for _ in range(size)]
        dist.all_gather(outs, local.contiguous(), group=self.cp_group)
        return torch.cat(outs[:V], dim=2)

    @torch.no_grad()
    def encode(self, state: torch.Tensor) -> torch.Tensor:
        V = state.shape[2] // self._pixel_frames_per_view()
        size, _ = cp._size_rank(self.cp_group)
        k = self._latent_scale()
        if 4 < V <= size:
            return self._distribute_views(state, V, self.tokenizer.encode) * k
        return batch_to_views(self.tokenizer.encode(views_to_batch(state, V)), V) * k

    @torch.no_grad()
    def decode(self, latent: torch.Tensor) -> torch.Tensor:
        V = latent.shape[2] // self.state_t
        size, _ = cp._size_rank(self.cp_group)
        latent = latent / self._latent_scale()
        if 4 < V <= size:
            return self._distribute_views(latent, V, self.tokenizer.decode)
        return batch_to_views(self.tokenizer.decode(views_to_batch(latent, V)), V)

    # ---- data ----------------------------------------------------------------------------------------------------
    def sample_first_n_views(self, batch: Dict, n_views: int) -> Dict:
        """Keep the first ``n_views`` cameras of every per-view field."""
        total = int(batch["sample_n_views"]) if "sample_n_views" in batch else None
        if total is not None and n_views == total:
            return batch
        fpv = int(batch["num_video_frames_per_view"])
        out = dict(batch)
        key = self.config.input_data_key
        if key in batch:
            out[key] = batch[key][:, :, : fpv * n_views]
        if self.config.input_latent_key in batch:
            out[self.config.input_latent_key] = batch[self.config.input_latent_key][:, :, : self.state_t * n_views]
        if "view_indices" in batch:
            out["view_indices"] = batch["view_indices"][:, : fpv * n_views]
        for k in ("t5_text_embeddings", "t5_text_mask"):
            if k in batch:
                out[k] = batch[k][:, : self.config.tokens_per_view * n_views]
        if "ai_caption" in batch:
            out["ai_caption"] = [" -- ".join(c.split(" -- ")[:n_views]) for c in batch["ai_caption"]]
        if "camera_keys_selection" in batch:
            out["camera_keys_selection"] = batch["camera_keys_selection"][:n_views]
        if "sample_n_views" in batch:
            out["sample_n_views"] = batch["sample_n_views"] * 0 + n_views
        return out

    def _preprocess_databatch(self, batch: Dict) -> Dict:
        rng = self.config.train_sample_views_range
        if batch.get(TRAIN_SAMPLING_APPLIED_KEY) or rng is None:
            return batch
        n = batch.get(TRAIN_SAMPLE_N_VIEWS_KEY)
        if n is None:
            n = random.randint(*rng)
            if cp._size_rank(self.cp_group)[0] > 1:
                n = cp.broadcast(n, self.cp_group)
        if n < 1:
            return batch
        out = self.sample_first_n_views(batch, int(n))
        out[TRAIN_SAMPLING_APPLIED_KEY] = True
        return out

    def with_latent_view_indices(self, batch: Dict) -> Dict:
        """Adds ``latent_view_indices_B_T``: the camera id of every latent frame."""
        batch = self._preprocess_databatch(batch)
        out = dict(batch)
        if "view_indices" in batch:
            fpv = int(batch["num_video_frames_per_view"])
            vi = batch["view_indices"]
            V = vi.shape[1] // fpv
            out["latent_view_indices_B_T"] = vi.view(vi.shape[0], V, fpv)[:, :, : self.state_t].reshape(vi.shape[0], -1)
        else:
            key = self.config.input_latent_key if self.config.input_latent_key in batch else self.config.input_data_key
            B = batch[key].shape[0]
            T = batch[key].shape[2]
            V = T // (self.state_t if key == self.config.input_latent_key else self._pixel_frames_per_view())
            out["latent_view_indices_B_T"] = torch.arange(V).repeat_interleave(self.state_t).unsqueeze(0).expand(B, -1).clone()
        if "ref_cam_view_idx_sample_position" not in out:
            out["ref_cam_view_idx_sample_position"] = torch.zeros(1, dtype=torch.int64)
        return out

    def get_data_and_condition(self, batch: Dict):
        b = self.with_latent_view_indices(batch)
        raw, latent, condition = self._plain_model.get_data_and_condition(self, b)
        c = self.config
        condition = condition.set_video_condition(
            state_t=c.state_t, gt_frames=latent.to(**self.tensor_kwargs), condition_locations=c.condition_locations,
            random_min_num_conditional_frames_per_view=c.min_num_conditional_frames_per_view,
            random_max_num_conditional_frames_per_view=c.max_num_conditional_frames_per_view,
            view_condition_dropout_max=c.view_condition_dropout_max, conditional_frames_probs=c.conditional_frames_probs)
        return raw, latent, condition

    def _net_kwargs(self, condition) -> Dict:
        kw = super()._net_kwargs(condition)
        kw["view_indices_B_T"] = getattr(condition, "view_indices_B_T", None)
        return kw

    # ---- context parallel: split the frames of each view ------------------------------------------------------------
    def broadcast_split_for_model_parallelsim(self, x0, condition, eps, t):
        def fold(z):
            return None if z is None else views_to_batch(z, z.shape[2] // self.state_t).contiguous()

        size = cp._size_rank(self.cp_group)[0]
        if size == 1 or condition.data_type != DataType.VIDEO:
            return super().broadcast_split_for_model_parallelsim(x0, condition, eps, t)
        V = (x0 if x0 is not None else condition.gt_frames).shape[2] // self.state_t
        t_folded = False
        if t is not None and t.ndim == 2 and t.shape[-1] != 1:
            t = t.view(t.shape[0], V, -1).reshape(t.shape[0] * V, -1)
            t_folded = True
        x0f, condition, epsf, t = super().broadcast_split_for_model_parallelsim(fold(x0), condition, fold(eps), t)
        x0 = None if x0f is None else batch_to_views(x0f, V)
        eps = None if epsf is None else batch_to_views(epsf, V)
        if t_folded:
            t = t.view(t.shape[0] // V, -1)
        return x0, condition, eps, t

    # ---- prompt embeddings computed online -------------------------------------------------------------------------------
    def compute_empty_and_negative_text_embeddings(self) -> None:
        """Embeddings of the blank prompt (the filler of views without a caption, and what a dropped prompt becomes) and of the
        default negative prompt, computed once."""
        from ..config import DEFAULT_NEGATIVE_PROMPT
        key = self.config.input_caption_key
        if self.empty_string_text_embeddings is None:
            self.empty_string_text_embeddings = self.text_encoder.compute_text_embeddings_online({key: [" "]}, key)
        if self.neg_text_embeddings is None:
            self.neg_text_embeddings = self.text_encoder.compute_text_embeddings_online({key: [DEFAULT_NEGATIVE_PROMPT]}, key)

    def compute_text_embeddings_online_multiview(self, batch: Dict) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """(prompt, negative prompt, dropped prompt) embeddings ``[B, V L, D]``. One caption per sample: it describes the front
        camera (``front_cam_view_idx_sample_position``) and every other view gets the blank prompt's embedding. ``V`` captions
        joined by `` -- `` (batch size 1): one per view, and the negative prompt is repeated for every view."""
        self.compute_empty_and_negative_text_embeddings()
        key, cap_key = self.config.input_data_key, self.config.input_caption_key
        fpv = self._pixel_frames_per_view() if batch.get(IS_PREPROCESSED_KEY) is True else int(batch["num_video_frames_per_view"])
        B, V = batch[key].shape[0], batch[key].shape[2] // fpv
        captions = batch[cap_key][0].split(" -- ")
        assert len(captions) in (1, V), f"Expected 1 or {V} captions, got {len(captions)}"
        empty, enc = self.empty_string_text_embeddings, self.text_encoder
        L = empty.shape[1]
        if len(captions) == 1:
            front = enc.compute_text_embeddings_online(batch, cap_key)                      # [B, L, D]
            assert front.shape[1] == L, f"the prompt embedding should have {L} tokens, got {tuple(front.shape)}"
            pos = empty.clone().repeat(B, V, 1).view(B, V, L, -1)
            neg = pos.clone()
            for b in range(B):
                v = int(batch["front_cam_view_idx_sample_position"][b])
                pos[b, v] = front[b]
                neg[b, v] = self.neg_text_embeddings[0]
            pos, neg = pos.flatten(1, 2), neg.flatten(1, 2)
        else:
            if len(batch[cap_key]) != 1:
                raise NotImplementedError(f"Expected batch size of 1, got {len(batch[cap_key])}")
            pos = torch.cat([enc.compute_text_embeddings_online({cap_key: [c]}, cap_key) for c in captions], dim=1)
            neg = self.neg_text_embeddings[:1].repeat(B, V, 1)
        dropped = empty.clone().repeat(B, V, 1)
        embedders = getattr(self.conditioner, "embedders", None)
        text = embedders["text"] if embedders is not None and "text" in embedders else None
        if not getattr(text, "use_empty_string", False):
            dropped = dropped * 0.0
        return pos, neg, dropped

    def inplace_compute_text_embeddings_online(self, batch: Dict) -> None:
        pos, neg, dropped = self.compute_text_embeddings_online_multiview(batch)
        if getattr(self.config, "online_text_embeddings_as_dict", False):
            batch["t5_text_embeddings"] = {"text_embeddings": pos, "dropout_text_embeddings": dropped}
            batch["neg_t5_text_embeddings"] = {"text_embeddings": neg, "dropout_text_embeddings": dropped}
        else:
            batch["t5_text_embeddings"], batch["neg_t5_text_embeddings"] = pos, neg
        batch["t5_text_mask"] = torch.ones(pos.shape[0], pos.shape[1], device=pos.device)

    # ---- sampling -----------------------------------------------------------------------------------------------------
    def _multiview_sampling_conditions(self, b: Dict, cond, uncond):
        """Conditions of the two guidance branches for a batch that carries latent view indices: the clean frames of every view,
        the inference-time mask, split for context parallelism."""
        n = b.get(NUM_CONDITIONAL_FRAMES_KEY, 1)
        _, x0, _ = self._plain_model.get_data_and_condition(self, b)
        x0 = x0.to(**self.tensor_kwargs)
        locs = self.config.condition_locations
        cond = replace(cond, state_t=self.state_t, gt_frames=x0).edit_for_inference(locs, True, n)
        uncond = replace(uncond, state_t=self.state_t, gt_frames=x0).edit_for_inference(locs, False, n)
        _, cond, _, _ = self.broadcast_split_for_model_parallelsim(x0, cond, None, None)
        _, uncond, _, _ = self.broadcast_split_for_model_parallelsim(x0, uncond, None, None)
        return cond, uncond

    def _regroup_gathered_views(self, out: torch.Tensor) -> torch.Tensor:
        size = cp._size_rank(self.cp_group)[0]
        if size > 1 and self.net.is_context_parallel_enabled:
            # the gather concatenated rank-major: (rank, view, t) -> (view, rank, t)
            B, C, T, H, W = out.shape
            V = T // self.state_t
            out = out.view(B, C, size, V, self.state_t // size, H, W).transpose(2, 3).reshape(B, C, T, H, W)
        return out


class MultiviewVid2VidModelRectifiedFlow(_MultiviewMixin, Video2WorldModelRectifiedFlow):
    def __init__(self, config: MultiviewRFConfig, **kw):
        if config.conditioner is None:
            config.conditioner = default_multiview_conditioner(config.text_dropout)
        super().__init__(config, **kw)
        self.state_t = config.state_t
        if self.text_encoder is not None and getattr(config, "compute_text_embeddings_online", True):
            self.compute_empty_and_negative_text_embeddings()

    def training_step(self, data_batch: Dict, iteration: int):
        if self.text_encoder is not None and "t5_text_embeddings" not in data_batch:
            self.inplace_compute_text_embeddings_online(data_batch)
        return super().training_step(data_batch, iteration)

    def get_velocity_fn_from_batch(self, data_batch: Dict, guidance: float = 1.5, is_negative_prompt: bool = False):
        b = self.with_latent_view_indices(data_batch)
        cond, uncond = self._conditions_for_sampling(b, is_negative_prompt)
        cond, uncond = self._multiview_sampling_conditions(b, cond, uncond)
        if not self.config.use_apg:
            return self._batched_cfg_fn(cond, uncond, guidance, t2w_formula=False)
        buf = MomentumBuffer(self.config.apg_momentum)

        def velocity_fn(noise, noise_x, timestep):
            c = self.denoise(noise, noise_x, timestep, cond)
            u = self.denoise(noise, noise_x, timestep, uncond)
            return adaptive_projected_guidance(c, u, guidance + 1.0, buf, self.config.apg_eta, self.config.apg_norm_threshold)

        return velocity_fn

    @torch.no_grad()
    def generate_samples_from_batch(self, data_batch: Dict, *args, **kw) -> torch.Tensor:
        return self._regroup_gathered_views(super().generate_samples_from_batch(self.with_latent_view_indices(data_batch), *args, **kw))


# ---- noise-level (EDM-era) twin ---------------------------------------------------------------------------------------------
USE_APG_KEY = "use_apg"


@dataclass
class MultiviewVid2VidModelConfig(edm.EDMConfig):
    min_num_conditional_frames_per_view: int = 1
    max_num_conditional_frames_per_view: int = 2
    train_sample_views_range: Optional[Tuple[int, int]] = None
    condition_locations: List[str] = field(default_factory=list)
    state_t: int = 8
    view_condition_dropout_max: int = 0
    tokens_per_view: int = 512
    apg_momentum: float = -0.75
    apg_eta: float = 0.0
    apg_norm_threshold: float = 7.5
    online_text_embeddings_as_dict: bool = True

class MultiviewVid2VidModel(_MultiviewMixin, edm.Video2WorldModel):
    """Multi-camera model on the noise-level (EDM) preconditioning. Sampling guides the clean-latent predictions; a batch with
    ``use_apg: True`` switches classifier-free guidance for adaptive projected guidance with the configured momentum, eta
    and norm threshold (the guidance scale is passed to it as given)."""

    _plain_model = edm.DiffusionModel

    def __init__(self, config, **kw):
        if config.conditioner is None:
            config.conditioner = default_multiview_conditioner(config.text_dropout)
        super().__init__(config, **kw)
        self.state_t = config.state_t
        if self.text_encoder is not None:
            self.compute_empty_and_negative_text_embeddings()

    def _latent_scale(self) -> float:
        return self.sigma_data

    def training_step(self, data_batch: Dict, iteration: int):
        if self.text_encoder is not None and "t5_text_embeddings" not in data_batch:
            self.inplace_compute_text_embeddings_online(data_batch)
        return super().training_step(data_batch, iteration)

    def _prepare_sampling_conditions(self, data_batch, cond, uncond):
        return self._multiview_sampling_conditions(data_batch, cond, uncond)

    def _guidance_combiner(self, data_batch: Dict, guidance: float) -> Callable:
        if data_batch.get(USE_APG_KEY) is not True:
            return super()._guidance_combiner(data_batch, guidance)
        buf, c = MomentumBuffer(self.config.apg_momentum), self.config
        return lambda cond_x0, uncond_x0: adaptive_projected_guidance(cond_x0, uncond_x0, guidance, buf, c.apg_eta, c.apg_norm_threshold)

    @torch.no_grad()
    def generate_samples_from_batch(self, data_batch: Dict, *args, **kw) -> torch.Tensor:
        return self._regroup_gathered_views(super().generate_samples_from_batch(self.with_latent_view_indices(data_batch), *args, **kw))

