"""T5 encoder (the T5-XXL / "t5-11b" text tower of the earlier Cosmos models) with a loader for Hugging Face checkpoints.

Parity target: cosmos_predict2/_src/imaginaire/modules/nlp/t5xxl/t5encoder.py:44-120 (tokenise to 512 tokens, encode, cut to
``max_seq_len``, zero everything after the valid tokens, return embeddings + mask). The reference delegates the network to
``transformers.T5EncoderModel``; here the tower is this package's own (layer norm and relative-position modules shared with the
umT5 tower of ``wan_encoders.py``). T5 v1.0 shares ONE relative-position table between all layers and uses a ReLU feed-forward;
v1.1 / umT5 checkpoints use the gated GELU form: both are covered by ``T5Config``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .wan_encoders import T5LayerNorm, T5RelativeEmbedding


@dataclass
class T5Config:
    vocab_size: int = 32128
    d_model: int = 1024
    d_kv: int = 128
    num_heads: int = 128
    d_ff: int = 65536
    num_layers: int = 24
    num_buckets: int = 32
    max_distance: int = 128
    feed_forward: str = "relu"            # "relu" (T5 v1.0) | "gated-gelu" (v1.1, umT5)
    eps: float = 1e-6


class _T5Block(nn.Module):
    def __init__(self, c: T5Config):
        super().__init__()
        inner = c.d_kv * c.num_heads
        self.num_heads = c.num_heads
        self.norm1, self.norm2 = T5LayerNorm(c.d_model, c.eps), T5LayerNorm(c.d_model, c.eps)
        self.q, self.k, self.v = (nn.Linear(c.d_model, inner, bias=False) for _ in range(3))
        self.o = nn.Linear(inner, c.d_model, bias=False)
        self.gated = c.feed_forward == "gated-gelu"
        self.wi = nn.Linear(c.d_model, c.d_ff, bias=False)
        self.wg = nn.Linear(c.d_model, c.d_ff, bias=False) if self.gated else None
        self.wo = nn.Linear(c.d_ff, c.d_model, bias=False)

    def forward(self, x, bias):
        B, S, _ = x.shape
        h = self.norm1(x)
        q, k, v = (lin(h).view(B, S, self.num_heads, -1).transpose(1, 2) for lin in (self.q, self.k, self.v))
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=bias.to(q.dtype), scale=1.0)      # T5 does not scale the scores
        x = x + self.o(o.transpose(1, 2).reshape(B, S, -1))
        h = self.norm2(x)
        h = F.gelu(self.wg(h), approximate="tanh") * self.wi(h) if self.gated else F.relu(self.wi(h))
        return x + self.wo(h)


class T5EncoderTower(nn.Module):
    def __init__(self, config: T5Config):
        super().__init__()
        c = self.config = config
        self.shared = nn.Embedding(c.vocab_size, c.d_model)
        self.relative_attention_bias = T5RelativeEmbedding(c.num_buckets, c.num_heads, True, c.max_distance)
        self.blocks = nn.ModuleList([_T5Block(c) for _ in range(c.num_layers)])
        self.final_layer_norm = T5LayerNorm(c.d_model, c.eps)

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        x = self.shared(input_ids)
        S = x.shape[1]
        bias = self.relative_attention_bias(S, S).to(x.dtype)                                     # [1, heads, S, S], all layers
        if attention_mask is not None:
            bias = bias.masked_fill(~attention_mask.view(-1, 1, 1, S).bool(), torch.finfo(x.dtype).min)
        for blk in self.blocks:
            x = blk(x, bias)
        return self.final_layer_norm(x)

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """``transformers.T5EncoderModel`` names -> this tower."""
        out: Dict[str, torch.Tensor] = {}
        for k, v in sd.items():
            k = k.removeprefix("encoder.") if not k.startswith("encoder.embed_tokens") else "shared.weight"
            if k in ("shared.weight", "embed_tokens.weight"):
                out["shared.weight"] = v
            elif k == "final_layer_norm.weight":
                out[k] = v
            elif k.startswith("block."):
                _, i, _, j, *rest = k.split(".")
                name = ".".join(rest)
                if name == "SelfAttention.relative_attention_bias.weight":
                    out["relative_attention_bias.embedding.weight"] = v
                elif name.startswith("SelfAttention."):
                    out[f"blocks.{i}.{name.split('.')[1]}.weight"] = v
                elif name == "layer_norm.weight":
                    out[f"blocks.{i}.norm{1 + int(j)}.weight"] = v
                elif name.startswith("DenseReluDense."):
                    part = name.split(".")[1]
                    out[f"blocks.{i}.{ {'wi': 'wi', 'wi_0': 'wg', 'wi_1': 'wi', 'wo': 'wo'}[part] }.weight"] = v
        self.load_state_dict(out, strict=True)


class T5Encoder:
    """Prompts -> ``(embeddings [B, max_seq_len, d_model], mask [B, max_seq_len])``; positions after the valid tokens are zero."""

    def __init__(self, tower: T5EncoderTower, tokenizer, max_seq_len: int = 512, model_seq_len: int = 512, device="cpu",
                 dtype=torch.float32):
        self.tower = tower.to(device, dtype).eval().requires_grad_(False)
        self.tokenizer, self.max_seq_len, self.model_seq_len, self.device = tokenizer, max_seq_len, model_seq_len, torch.device(device)

    @torch.no_grad()
    def encode(self, texts: List[str]) -> Tuple[torch.Tensor, torch.Tensor]:
        tok = self.tokenizer(texts, return_tensors="pt", padding="max_length", max_length=self.model_seq_len, truncation=True)
        ids, mask = tok["input_ids"].to(self.device), tok["attention_mask"].to(self.device)
        out = self.tower(ids, mask)[:, : self.max_seq_len]
        mask = mask[:, : self.max_seq_len]
        return out * mask.unsqueeze(-1).to(out.dtype), mask
