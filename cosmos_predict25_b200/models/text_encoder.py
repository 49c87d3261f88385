"""Text conditioning: Cosmos-Reason1 / Qwen2.5-VL language tower -> per-layer normalised hidden states.

Contract (cosmos_predict2/_src/predict2/text_encoders/text_encoder.py:67-216): the prompt is wrapped in a
chat template (system: "You are a helpful assistant who will provide prompts to an image generator."),
tokenised, padded with the pad id or truncated to 512 tokens, run through the decoder-only LLM; the hidden
states of layers 1..L are each normalised over the feature dim ((h - mean) / (std + 1e-8)) and combined:
``full_concat`` -> [B, 512, L*hidden] (28 x 3584 = 100352 for the 7B model), ``mean_pooling`` -> [B,512,hidden],
``pool_every_n_layers_and_concat``.

The language tower here is a self-contained PyTorch implementation of the Qwen2 decoder (GQA attention
with rotary embeddings, SwiGLU MLP, RMSNorm; reference network: cosmos_predict2/_src/reason1/networks/qwen2_5_vl.py)
that loads Hugging Face-format weights. For text-only prompts the multimodal rotary embedding of
Qwen2.5-VL degenerates to ordinary 1-D RoPE, which is what is implemented. When no weights are available
(offline builds, tests) ``HashTextEncoder`` provides deterministic pseudo-embeddings with the same shape
contract so that pipelines can run end to end; its output carries no semantics.
"""

from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import dataclass, field
from typing import Tuple, Dict, List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

NUM_EMBEDDING_PADDING_TOKENS = 512
SYSTEM_PROMPT = "You are a helpful assistant who will provide prompts to an image generator."


class EmbeddingConcatStrategy:
    FULL_CONCAT = "full_concat"
    MEAN_POOLING = "mean_pooling"
    POOL_EVERY_N_LAYERS_AND_CONCAT = "pool_every_n_layers_and_concat"


@dataclass
class QwenConfig:
    """Language-tower hyper-parameters; defaults = Qwen2.5-VL-7B / Cosmos-Reason1-7B."""

    vocab_size: int = 152064
    hidden_size: int = 3584
    intermediate_size: int = 18944
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1000000.0
    tie_word_embeddings: bool = False
    pad_token_id: int = 151643


@dataclass
class TextEncoderConfig:
    compute_online: bool = False
    embedding_concat_strategy: str = EmbeddingConcatStrategy.FULL_CONCAT
    n_layers_per_group: int = 5
    ckpt_path: str = "nvidia/Cosmos-Reason1.1-7B"
    tokenizer_path: str = "Qwen/Qwen2.5-VL-7B-Instruct"
    model: QwenConfig = field(default_factory=QwenConfig)


class QwenRMSNorm(nn.Module):
    def __init__(self, dim, eps):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        dt = x.dtype
        x = x.float()
        return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps)).to(dt) * self.weight


def _rotate_half(x):
    a, b = x.chunk(2, dim=-1)
    return torch.cat((-b, a), dim=-1)


class QwenAttention(nn.Module):
    def __init__(self, c: QwenConfig):
        super().__init__()
        self.h, self.kv, self.hd = c.num_attention_heads, c.num_key_value_heads, c.hidden_size // c.num_attention_heads
        self.q_proj = nn.Linear(c.hidden_size, self.h * self.hd, bias=True)
        self.k_proj = nn.Linear(c.hidden_size, self.kv * self.hd, bias=True)
        self.v_proj = nn.Linear(c.hidden_size, self.kv * self.hd, bias=True)
        self.o_proj = nn.Linear(self.h * self.hd, c.hidden_size, bias=False)
        self.cp_group = None   # set by QwenLanguageModel.forward for all-gather-KV context parallelism

    def forward(self, x, cos, sin, mask):
        B, S, _ = x.shape
        # head counts are inferred from the projection width so that column-sharded (tensor-parallel) projections work
        q = self.q_proj(x).view(B, S, -1, self.hd).transpose(1, 2)
        k = self.k_proj(x).view(B, S, -1, self.hd).transpose(1, 2)
        v = self.v_proj(x).view(B, S, -1, self.hd).transpose(1, 2)
        q = q * cos + _rotate_half(q) * sin
        k = k * cos + _rotate_half(k) * sin
        if self.cp_group is not None:
            # queries stay sequence-sharded; keys / values of the whole sequence are gathered (before the GQA repeat: less traffic)
            k, v = _gather_seq(k, self.cp_group), _gather_seq(v, self.cp_group)
        rep = self.h // self.kv
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=mask, is_causal=mask is None)
        return self.o_proj(o.transpose(1, 2).reshape(B, S, -1))


def _gather_seq(t: torch.Tensor, group) -> torch.Tensor:
    """All-gather [B, heads, S_loc, hd] along the sequence in rank order."""
    import torch.distributed as dist
    parts = [torch.empty_like(t) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, t.contiguous(), group=group)
    return torch.cat(parts, dim=2)


class QwenMLP(nn.Module):
    def __init__(self, c: QwenConfig):
        super().__init__()
        self.gate_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.up_proj = nn.Linear(c.hidden_size, c.intermediate_size, bias=False)
        self.down_proj = nn.Linear(c.intermediate_size, c.hidden_size, bias=False)

    def forward(self, x):
        return self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))


class QwenLayer(nn.Module):
    def __init__(self, c: QwenConfig):
        super().__init__()
        self.self_attn = QwenAttention(c)
        self.mlp = QwenMLP(c)
        self.input_layernorm = QwenRMSNorm(c.hidden_size, c.rms_norm_eps)
        self.post_attention_layernorm = QwenRMSNorm(c.hidden_size, c.rms_norm_eps)

    def forward(self, x, cos, sin, mask):
        x = x + self.self_attn(self.input_layernorm(x), cos, sin, mask)
        return x + self.mlp(self.post_attention_layernorm(x))


class QwenLanguageModel(nn.Module):
    """Decoder-only tower returning every hidden state (embedding output + one per layer)."""

    def __init__(self, c: QwenConfig):
        super().__init__()
        self.config = c
        self.embed_tokens = nn.Embedding(c.vocab_size, c.hidden_size)
        self.layers = nn.ModuleList([QwenLayer(c) for _ in range(c.num_hidden_layers)])
        self.norm = QwenRMSNorm(c.hidden_size, c.rms_norm_eps)

    def rope(self, S: int, device, dtype):
        hd = self.config.hidden_size // self.config.num_attention_heads
        inv = 1.0 / (self.config.rope_theta ** (torch.arange(0, hd, 2, device=device, dtype=torch.float32) / hd))
        ang = torch.outer(torch.arange(S, device=device, dtype=torch.float32), inv)
        emb = torch.cat([ang, ang], -1)
        return emb.cos()[None, None].to(dtype), emb.sin()[None, None].to(dtype)

    @torch.no_grad()
    def forward(self, input_ids: Optional[torch.Tensor], attention_mask: Optional[torch.Tensor] = None, cp_group=None,
                inputs_embeds: Optional[torch.Tensor] = None, rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> List[torch.Tensor]:
        """Every hidden state [B, S, hidden]. With ``cp_group`` (every rank passes the same ``input_ids``) the sequence is
        split into contiguous ranges over the group: embeddings, RoPE rows and causal-mask rows are sliced, each attention
        all-gathers keys / values (the reference's all-gather-KV context parallelism of the VLM tower,
        cosmos_reason1 qwen2_5_vl.py:1032-1034,1267-1281), and the hidden states are gathered back at the end."""
        import torch.distributed as dist
        cp = dist.get_world_size(cp_group) if cp_group is not None and dist.is_initialized() else 1
        # ``inputs_embeds`` (token embeddings with vision features scattered in) and ``rope`` (cos, sin [B, 1, S, head_dim] from
        # 3-D multimodal positions) are supplied by the vision-language wrapper (models/qwen_vl.py)
        x = self.embed_tokens(input_ids) if inputs_embeds is None else inputs_embeds
        B, S, _ = x.shape
        cos, sin = self.rope(S, x.device, x.dtype) if rope is None else rope
        mask = None
        if attention_mask is not None or cp > 1:
            causal = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
            mask = causal[None, None].expand(B, 1, S, S)
            if attention_mask is not None:
                mask = mask & attention_mask[:, None, None, :].bool()
        if cp > 1:
            assert S % cp == 0, f"sequence {S} does not divide over {cp} ranks"
            r, n = dist.get_rank(cp_group), S // cp
            x, mask = x[:, r * n:(r + 1) * n], mask[:, :, r * n:(r + 1) * n]
            cos_q, sin_q = cos[:, :, r * n:(r + 1) * n], sin[:, :, r * n:(r + 1) * n]
        else:
            cos_q, sin_q = cos, sin
        for layer in self.layers:
            layer.self_attn.cp_group = cp_group if cp > 1 else None
        try:
            hidden = [x]
            for i, layer in enumerate(self.layers):
                x = layer(x, cos_q, sin_q, mask)   # keys are rotated with their own (local) positions before the gather
                hidden.append(self.norm(x) if i == len(self.layers) - 1 else x)
        finally:
            for layer in self.layers:
                layer.self_attn.cp_group = None
        if cp > 1:
            gathered = []
            for h in hidden:
                parts = [torch.empty_like(h) for _ in range(cp)]
                dist.all_gather(parts, h.contiguous(), group=cp_group)
                gathered.append(torch.cat(parts, dim=1))
            hidden = gathered
        return hidden

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Accepts Hugging Face Qwen2 / Qwen2.5-VL key names (``model.layers.N...``, ``model.language_model...``)."""
        own = self.state_dict()
        mapped = {}
        for k, v in sd.items():
            if k.endswith("._extra_state"):
                continue
            for prefix in ("model.language_model.", "language_model.model.", "language_model.", "model.", ""):
                kk = k[len(prefix):] if k.startswith(prefix) else None
                if kk is not None and kk in own:
                    mapped[kk] = v
                    break
        missing = [k for k in own if k not in mapped]
        if missing:
            raise KeyError(f"text-encoder checkpoint lacks {len(missing)} tensors, e.g. {missing[:3]}")
        self.load_state_dict(mapped, strict=True)


def mean_normalize(t: torch.Tensor) -> torch.Tensor:
    return (t - t.mean(dim=-1, keepdim=True)) / (t.std(dim=-1, keepdim=True) + 1e-8)


def combine_hidden_states(hidden: Sequence[torch.Tensor], strategy: str, n_layers_per_group: int = 5) -> torch.Tensor:
    """``hidden`` = [embedding output, layer 1, ..., layer L]; layers 1..L are used."""
    normed = [mean_normalize(h) for h in hidden[1:]]
    if strategy == EmbeddingConcatStrategy.FULL_CONCAT:
        return torch.cat(normed, dim=-1)
    if strategy == EmbeddingConcatStrategy.MEAN_POOLING:
        return torch.stack(normed).mean(0)
    if strategy == EmbeddingConcatStrategy.POOL_EVERY_N_LAYERS_AND_CONCAT:
        groups = [torch.stack(normed[i:i + n_layers_per_group]).mean(0) for i in range(0, len(normed), n_layers_per_group)]
        return torch.cat(groups, dim=-1)
    raise ValueError(f"invalid embedding_concat_strategy {strategy}")


def build_chat_text(prompt: str) -> str:
    """ChatML rendering of the two-turn conversation (system + user), no generation prompt."""
    return (f"<|im_start|>system\n{SYSTEM_PROMPT}<|im_end|>\n<|im_start|>user\n{prompt}<|im_end|>\n")


class TextEncoder:
    """Online prompt -> embedding. ``tokenizer`` must map text -> list[int] (a Hugging Face tokenizer works)."""

    def __init__(self, config: TextEncoderConfig, device="cuda", tokenizer=None, model: Optional[QwenLanguageModel] = None,
                 dtype=torch.bfloat16):
        self.config = config
        self.device = torch.device(device)
        self.model = model
        self.tokenizer = tokenizer
        if self.model is None:
            self.model = self._load_model(dtype)
        if self.tokenizer is None:
            self.tokenizer = self._load_tokenizer()
        self.model.eval().requires_grad_(False).to(self.device)

    def _load_model(self, dtype) -> QwenLanguageModel:
        from ..utils.checkpoint_db import get_checkpoint_path
        path = get_checkpoint_path(self.config.ckpt_path)
        with torch.device("meta"):
            m = QwenLanguageModel(self.config.model)
        m.to_empty(device="cpu")
        sd: Dict[str, torch.Tensor] = {}
        if os.path.isdir(path):
            from safetensors.torch import load_file
            for f in sorted(os.listdir(path)):
                if f.endswith(".safetensors"):
                    sd.update(load_file(os.path.join(path, f)))
                elif f.endswith((".pt", ".bin")):
                    sd.update(torch.load(os.path.join(path, f), map_location="cpu", weights_only=False))
        else:
            sd = torch.load(path, map_location="cpu", weights_only=False)
        m.load_hf_state_dict(sd)
        return m.to(dtype)

    def _load_tokenizer(self):
        from transformers import AutoTokenizer
        from ..utils.checkpoint_db import get_checkpoint_path
        try:
            return AutoTokenizer.from_pretrained(get_checkpoint_path(self.config.tokenizer_path))
        except Exception:
            return AutoTokenizer.from_pretrained(self.config.tokenizer_path)

    def tokenize(self, prompt: str) -> List[int]:
        text = build_chat_text(prompt)
        ids = self.tokenizer(text)["input_ids"] if callable(self.tokenizer) else self.tokenizer.encode(text)
        pad = getattr(self.tokenizer, "pad_token_id", None)
        pad = self.config.model.pad_token_id if pad is None else pad
        n = NUM_EMBEDDING_PADDING_TOKENS
        return (list(ids) + [pad] * (n - len(ids)))[:n]

    @torch.no_grad()
    def compute_text_embeddings_online(self, data_batch: Dict, input_caption_key: str = "ai_caption") -> torch.Tensor:
        prompts = data_batch[input_caption_key]
        prompts = [prompts] if isinstance(prompts, str) else list(prompts)
        ids = torch.tensor([self.tokenize(p) for p in prompts], dtype=torch.long, device=self.device)
        hidden = self.model(ids)
        return combine_hidden_states(hidden, self.config.embedding_concat_strategy, self.config.n_layers_per_group)

    def encode_prompts(self, prompts: Sequence[str]) -> torch.Tensor:
        return self.compute_text_embeddings_online({"p": list(prompts)}, "p")


class HashTextEncoder:
    """Deterministic pseudo-embeddings with the shape contract of the real encoder ([B, 512, dim]); for offline
    pipelines and tests only. Each (prompt, token position) seeds a reproducible normal vector."""

    def __init__(self, dim: int = 100352, n_tokens: int = NUM_EMBEDDING_PADDING_TOKENS, device="cpu", dtype=torch.bfloat16):
        self.dim, self.n_tokens, self.device, self.dtype = dim, n_tokens, torch.device(device), dtype

    def encode_prompts(self, prompts: Sequence[str]) -> torch.Tensor:
        outs = []
        for p in prompts:
            seed = int.from_bytes(hashlib.sha256(p.encode()).digest()[:8], "little") % (2 ** 63)
            g = torch.Generator().manual_seed(seed)
            outs.append(torch.randn(self.n_tokens, self.dim, generator=g))
        return torch.stack(outs).to(self.device, self.dtype)

    def compute_text_embeddings_online(self, data_batch: Dict, input_caption_key: str = "ai_caption") -> torch.Tensor:
        prompts = data_batch[input_caption_key]
        return self.encode_prompts([prompts] if isinstance(prompts, str) else list(prompts))
