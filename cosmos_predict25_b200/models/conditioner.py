"""Conditioning: embedder registry with per-embedder dropout, and the immutable condition records
the network consumes.

Parity targets: ``GeneralConditioner`` / ``TextAttr`` / ``ReMapkey`` / ``BooleanFlag`` /
``Text2WorldCondition`` (cosmos_predict2/_src/predict2/conditioner.py:105-573) and
``Video2WorldCondition`` (cosmos_predict2/_src/predict2/configs/video2world/defaults/conditioner.py:39-169).

A condition is a frozen dataclass; every edit returns a new record. Text dropout zeroes the
embedding (it does not substitute an empty-prompt embedding). Video conditioning marks the first
n latent frames of each sample as clean: the mask is a [B,1,T,H,W] tensor that is both a network
input channel and the selector for frame replacement in the denoiser.
"""

from __future__ import annotations

import copy
import random
from dataclasses import dataclass, fields, replace
from enum import Enum
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn

from ..parallel import context_parallel as cp


class DataType(Enum):
    IMAGE = "image"
    VIDEO = "video"
    MIX = "mix"


@dataclass(frozen=True)
class Text2WorldCondition:
    crossattn_emb: Optional[torch.Tensor] = None
    data_type: DataType = DataType.VIDEO
    padding_mask: Optional[torch.Tensor] = None
    fps: Optional[torch.Tensor] = None
    _is_broadcasted: bool = False

    def to_dict(self, skip_underscore: bool = True) -> Dict[str, Any]:
        return {f.name: getattr(self, f.name) for f in fields(self) if not (skip_underscore and f.name.startswith("_"))}

    @property
    def is_broadcasted(self) -> bool:
        return self._is_broadcasted

    def broadcast(self, process_group) -> "Text2WorldCondition":
        """Make all ranks of a context-parallel group hold rank-0's condition."""
        if self._is_broadcasted or process_group is None:
            return self
        size, _ = cp._size_rank(process_group)
        if size == 1:
            return self
        kw = self.to_dict(skip_underscore=False)
        for k, v in list(kw.items()):
            if k.startswith("_") or k in ("gt_frames", "condition_video_input_mask_B_C_T_H_W"):
                continue
            if isinstance(v, torch.Tensor):
                kw[k] = cp.broadcast(v, process_group)
            elif v is not None and not isinstance(v, DataType):
                kw[k] = cp.broadcast(v, process_group)
        kw["_is_broadcasted"] = True
        return type(self)(**kw)


@dataclass(frozen=True)
class Video2WorldCondition(Text2WorldCondition):
    use_video_condition: Union[bool, torch.Tensor] = False
    gt_frames: Optional[torch.Tensor] = None
    condition_video_input_mask_B_C_T_H_W: Optional[torch.Tensor] = None

    def set_video_condition(self, gt_frames: torch.Tensor, random_min_num_conditional_frames: int,
                            random_max_num_conditional_frames: int,
                            num_conditional_frames: Optional[Union[int, torch.Tensor]] = None,
                            conditional_frames_probs: Optional[Dict[int, float]] = None) -> "Video2WorldCondition":
        """Attach clean frames and the mask selecting the first n latent frames of each sample.

        Images (T == 1) never condition. For video either a fixed n, a categorical draw from
        ``conditional_frames_probs`` ({frames: probability}) or a uniform draw in [min, max]."""
        B, _, T, H, W = gt_frames.shape
        if T == 1:
            n_B = [0] * B
        elif num_conditional_frames is not None:
            if isinstance(num_conditional_frames, torch.Tensor):
                n_B = (torch.ones(B, dtype=torch.int32) * num_conditional_frames.cpu()).tolist()
            else:
                n_B = [int(num_conditional_frames)] * B
        elif conditional_frames_probs is not None:
            n_B = random.choices(list(conditional_frames_probs.keys()), weights=list(conditional_frames_probs.values()), k=B)
        else:
            n_B = torch.randint(random_min_num_conditional_frames, random_max_num_conditional_frames + 1, (B,)).tolist()
        mask = torch.zeros(B, 1, T, H, W, dtype=gt_frames.dtype, device=gt_frames.device)
        for i, n in enumerate(n_B):
            if n > 0:
                mask[i, :, : int(n)] = 1
        return replace(self, gt_frames=gt_frames, condition_video_input_mask_B_C_T_H_W=mask)

    def edit_for_inference(self, is_cfg_conditional: bool = True, num_conditional_frames: int = 1) -> "Video2WorldCondition":
        c = self.set_video_condition(self.gt_frames, 0, 0, num_conditional_frames=num_conditional_frames)
        if not is_cfg_conditional:
            # the unconditional branch still sees the clean frames
            uvc = c.use_video_condition
            uvc = torch.ones_like(uvc, dtype=torch.bool) if isinstance(uvc, torch.Tensor) else True
            c = replace(c, use_video_condition=uvc)
        return c

    def broadcast(self, process_group) -> "Video2WorldCondition":
        if self._is_broadcasted or process_group is None:
            return self
        size, _ = cp._size_rank(process_group)
        if size == 1:
            return self
        base = Text2WorldCondition.broadcast(self, process_group)
        gt, mask = self.gt_frames, self.condition_video_input_mask_B_C_T_H_W
        T = gt.shape[2]
        if T > 1:
            gt = cp.broadcast_split_tensor(gt, seq_dim=2, cp_group=process_group)
            mask = cp.broadcast_split_tensor(mask, seq_dim=2, cp_group=process_group)
        return replace(base, gt_frames=gt, condition_video_input_mask_B_C_T_H_W=mask)


class Video2WorldConditionV2(Video2WorldCondition):
    """Variant whose samples WITHOUT the video-condition flag get no conditioning frames at all (the mask is zero for them), where
    the first version keeps the frames and lets the model multiply them by the flag; at inference both guidance branches see the
    requested number of frames (configs/video2world/defaults/conditioner.py:172-209 of the reference)."""

    def set_video_condition(self, gt_frames, random_min_num_conditional_frames, random_max_num_conditional_frames,
                            num_conditional_frames=None, conditional_frames_probs=None) -> "Video2WorldConditionV2":
        c = super().set_video_condition(gt_frames, random_min_num_conditional_frames, random_max_num_conditional_frames,
                                        num_conditional_frames, conditional_frames_probs)
        uvc = self.use_video_condition
        if isinstance(uvc, torch.Tensor):
            keep = uvc.to(c.condition_video_input_mask_B_C_T_H_W.device).bool().view(-1, 1, 1, 1, 1)
            mask = c.condition_video_input_mask_B_C_T_H_W * keep.to(c.condition_video_input_mask_B_C_T_H_W.dtype)
        else:
            mask = c.condition_video_input_mask_B_C_T_H_W if uvc else torch.zeros_like(c.condition_video_input_mask_B_C_T_H_W)
        return replace(c, condition_video_input_mask_B_C_T_H_W=mask)

    def edit_for_inference(self, is_cfg_conditional: bool = True, num_conditional_frames: int = 1) -> "Video2WorldConditionV2":
        return Video2WorldCondition.set_video_condition(self, self.gt_frames, 0, 0, num_conditional_frames=num_conditional_frames)


# --------------------------------------------------------------------------------------------
# embedders
# --------------------------------------------------------------------------------------------
class AbstractEmbModel(nn.Module):
    """One conditioning input: reads ``input_key`` from the batch, may drop it with probability
    ``dropout_rate`` per sample, and emits {output_key: tensor}."""

    def __init__(self, input_key=None, output_key=None, dropout_rate: float = 0.0, is_trainable: bool = False):
        super().__init__()
        self.input_key = input_key
        self.output_key = output_key
        self.dropout_rate = dropout_rate
        self.is_trainable = is_trainable

    def random_dropout_input(self, x: Optional[torch.Tensor], dropout_rate: Optional[float] = None, key: Optional[str] = None):
        if x is None:
            return None
        rate = self.dropout_rate if dropout_rate is None else dropout_rate
        # one host-side draw per sample for EVERY embedder, also at rate 0: the same seed then drops the same samples as in the
        # reference (conditioner.py:215-223 there), whose generator advances the same way
        keep = torch.bernoulli((1.0 - rate) * torch.ones(x.shape[0]))
        if rate <= 0.0:
            return x
        return x * keep.to(x.device).type_as(x).view(-1, *([1] * (x.ndim - 1)))

    def details(self) -> str:
        return f"{type(self).__name__}(in={self.input_key}, out={self.output_key}, dropout={self.dropout_rate})"


class TextAttr(AbstractEmbModel):
    """Text embedding [B, L, C] -> ``crossattn_emb``. A dropped sample becomes zeros or, with ``use_empty_string``, the embedding
    of the empty prompt (a tensor file read once through easy_io, or ``set_empty_string_embeddings``); ``*mask*`` entries are
    never dropped (conditioner.py:238-289 of the reference)."""

    def __init__(self, input_key="t5_text_embeddings", dropout_rate: float = 0.0, use_empty_string: bool = False,
                 empty_string_embeddings_path: Optional[str] = None, credential_path: Optional[str] = None):
        super().__init__(input_key, "crossattn_emb", dropout_rate)
        self.use_empty_string = use_empty_string
        self.empty_string_embeddings_path = empty_string_embeddings_path
        self.credential_path = credential_path
        self._empty = None

    def set_empty_string_embeddings(self, emb: torch.Tensor) -> None:
        self._empty = emb

    def _empty_string_embeddings(self) -> torch.Tensor:
        if self._empty is None:
            if not self.empty_string_embeddings_path:
                raise ValueError("use_empty_string needs the empty prompt's embedding: give empty_string_embeddings_path or call "
                                 "set_empty_string_embeddings")
            from ..utils.easy_io import easy_io
            kw = {}
            if str(self.empty_string_embeddings_path).startswith("s3://"):
                kw["backend_args"] = {"backend": "s3", "s3_credential_path": self.credential_path}
            self._empty = easy_io.load(self.empty_string_embeddings_path, **kw)
        return self._empty

    def random_dropout_input(self, x, dropout_rate=None, key=None):
        if key is not None and "mask" in key:
            return x
        if not self.use_empty_string or x is None:
            return super().random_dropout_input(x, dropout_rate, key)
        rate = self.dropout_rate if dropout_rate is None else dropout_rate
        keep = torch.bernoulli((1.0 - rate) * torch.ones(x.shape[0])).to(x.device).type_as(x).view(-1, *([1] * (x.ndim - 1)))
        empty = self._empty_string_embeddings().to(dtype=x.dtype, device=x.device).expand(x.shape)
        return keep * x + (1.0 - keep) * empty

    def forward(self, emb: torch.Tensor) -> Dict[str, torch.Tensor]:
        return {"crossattn_emb": emb}


class TextAttrEmptyStringDrop(TextAttr):
    """``TextAttr`` that always replaces a dropped prompt by the empty prompt's embedding (conditioner.py:291-335 of the reference,
    which reads that embedding from a fixed bucket path; here the path is an argument)."""

    def __init__(self, input_key="t5_text_embeddings", dropout_rate: float = 0.0, empty_string_embeddings_path: Optional[str] = None,
                 credential_path: Optional[str] = None):
        super().__init__(input_key, dropout_rate, True, empty_string_embeddings_path, credential_path)

    def _empty_string_embeddings(self) -> torch.Tensor:
        e = super()._empty_string_embeddings()
        if isinstance(e, (list, tuple)):
            e = e[0]
        return e if e.ndim == 3 else e.unsqueeze(0)


class ReMapkey(AbstractEmbModel):
    """Pass a batch entry through under another name (fps, padding_mask), optionally cast."""

    def __init__(self, input_key: str, output_key: Optional[str] = None, dropout_rate: float = 0.0, dtype: Optional[str] = None):
        super().__init__(input_key, output_key or input_key, dropout_rate)
        self.dtype = {None: None, "float": torch.float32, "bfloat16": torch.bfloat16, "half": torch.float16,
                      "float16": torch.float16, "int": torch.int32, "long": torch.int64}[dtype]

    def forward(self, x):
        if isinstance(x, torch.Tensor) and self.dtype is not None:
            x = x.to(self.dtype)
        return {self.output_key: x}


class BooleanFlag(AbstractEmbModel):
    """A per-sample boolean that is True unless dropped (e.g. ``use_video_condition``)."""

    def __init__(self, input_key: str, output_key: Optional[str] = None, dropout_rate: float = 0.0):
        super().__init__(input_key, output_key or input_key, dropout_rate)

    def random_dropout_input(self, x, dropout_rate=None, key=None):
        rate = self.dropout_rate if dropout_rate is None else dropout_rate
        return bool(torch.bernoulli((1.0 - rate) * torch.ones(1)).item())

    def forward(self, flag):
        return {self.output_key: torch.tensor(bool(flag))}


class GeneralConditioner(nn.Module):
    """Runs every embedder on the batch and assembles a condition record."""

    KEY2DIM = {"crossattn_emb": 1}
    condition_cls = Text2WorldCondition

    def __init__(self, **embedders: AbstractEmbModel):
        super().__init__()
        self.embedders = nn.ModuleDict()
        for name, emb in embedders.items():
            assert isinstance(emb, AbstractEmbModel), f"{name} must derive from AbstractEmbModel"
            if not emb.is_trainable:
                for p in emb.parameters():
                    p.requires_grad = False
                emb.eval()
            self.embedders[name] = emb

    def _collect(self, batch: Dict, override_dropout_rate: Optional[Dict[str, float]] = None) -> Dict[str, Any]:
        override = override_dropout_rate or {}
        for name in override:
            assert name in self.embedders, f"unknown embedder {name}"
        out: Dict[str, List] = {}
        for name, emb in self.embedders.items():
            rate = override.get(name)
            with torch.set_grad_enabled(emb.is_trainable and torch.is_grad_enabled()):
                if isinstance(emb.input_key, str):
                    res = emb(emb.random_dropout_input(batch.get(emb.input_key), rate))
                else:
                    res = emb(*[emb.random_dropout_input(batch.get(k), rate, k) for k in emb.input_key])
            for k, v in res.items():
                out.setdefault(k, []).append(v)
        merged = {}
        for k, vs in out.items():
            if len(vs) == 1 or not isinstance(vs[0], torch.Tensor):
                merged[k] = vs[0]
            else:
                merged[k] = torch.cat(vs, dim=self.KEY2DIM.get(k, -1))
        return merged

    def forward(self, batch: Dict, override_dropout_rate: Optional[Dict[str, float]] = None):
        out = self._collect(batch, override_dropout_rate)
        valid = {f.name for f in fields(self.condition_cls)}
        return self.condition_cls(**{k: v for k, v in out.items() if k in valid})

    def get_condition_uncondition(self, batch: Dict) -> Tuple[Any, Any]:
        """(all conditions applied, all droppable conditions dropped)."""
        cond = {n: 0.0 for n in self.embedders}
        uncond = {n: (1.0 if e.dropout_rate > 1e-4 else 0.0) for n, e in self.embedders.items()}
        return self(batch, cond), self(batch, uncond)

    def get_condition_with_negative_prompt(self, batch: Dict) -> Tuple[Any, Any]:
        """Like ``get_condition_uncondition`` but the unconditional text is the negative prompt's
        embedding (``neg_t5_text_embeddings``) instead of zeros."""
        cond = {n: 0.0 for n in self.embedders}
        uncond = {n: (0.0 if isinstance(e, TextAttr) else (1.0 if e.dropout_rate > 1e-4 else 0.0))
                  for n, e in self.embedders.items()}
        neg = dict(batch)
        if isinstance(neg.get("neg_t5_text_embeddings"), torch.Tensor):
            neg["t5_text_embeddings"] = neg["neg_t5_text_embeddings"]
        return self(batch, cond), self(neg, uncond)


class VideoConditioner(GeneralConditioner):
    condition_cls = Text2WorldCondition


class Video2WorldConditioner(GeneralConditioner):
    condition_cls = Video2WorldCondition


class Video2WorldConditionerV2(GeneralConditioner):
    condition_cls = Video2WorldConditionV2


def default_video2world_conditioner(text_dropout: float = 0.2) -> Video2WorldConditioner:
    """Embedder set of the 2.5 configs: fps, padding mask, text (dropout 0.2 for 2B, 0.1 for 14B) and
    the ``use_video_condition`` flag with dropout 0
    (cosmos_predict2/_src/predict2/configs/video2world/defaults/conditioner.py:228-351)."""
    return Video2WorldConditioner(
        fps=ReMapkey("fps", "fps", 0.0),
        padding_mask=ReMapkey("padding_mask", "padding_mask", 0.0),
        text=TextAttr("t5_text_embeddings", text_dropout),
        use_video_condition=BooleanFlag("fps", "use_video_condition", 0.0),
    )


def default_text2world_conditioner(text_dropout: float = 0.2) -> VideoConditioner:
    return VideoConditioner(
        fps=ReMapkey("fps", "fps", 0.0),
        padding_mask=ReMapkey("padding_mask", "padding_mask", 0.0),
        text=TextAttr("t5_text_embeddings", text_dropout),
    )
