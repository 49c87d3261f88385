"""OpenAI-CLIP (ViT variants): image and text towers under the parameter names of the released ``.pt`` checkpoints.

Parity target: cosmos_predict2/_src/imaginaire/modules/image_embeddings.py:232-575 (``CLIP.encode_image`` / ``encode_text`` /
``forward`` and ``build_model``, which sizes the network from the shapes in a state dict). The ResNet image towers of the original
release (RN50 ...) are not restated: the framework's callers use the ViT checkpoints. Attention runs through torch's fused
scaled-dot-product call; the blocks are pre-norm with the x * sigmoid(1.702 x) activation.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F


class _LN(nn.LayerNorm):
    def forward(self, x):
        return super().forward(x.float()).type_as(x)


class _Attention(nn.Module):
    """Same parameters as ``nn.MultiheadAttention`` (``in_proj_weight`` [3D, D], ``in_proj_bias``, ``out_proj``)."""

    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.heads = heads
        self.in_proj_weight = nn.Parameter(torch.empty(3 * dim, dim))
        self.in_proj_bias = nn.Parameter(torch.zeros(3 * dim))
        self.out_proj = nn.Linear(dim, dim)
        nn.init.normal_(self.in_proj_weight, std=dim ** -0.5)

    def forward(self, x, causal: bool):
        B, S, D = x.shape
        q, k, v = F.linear(x, self.in_proj_weight, self.in_proj_bias).view(B, S, 3, self.heads, D // self.heads).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=causal)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, D))


class _Block(nn.Module):
    def __init__(self, dim: int, heads: int):
        super().__init__()
        self.ln_1, self.ln_2 = _LN(dim), _LN(dim)
        self.attn = _Attention(dim, heads)
        self.mlp = nn.ModuleDict(dict(c_fc=nn.Linear(dim, 4 * dim), c_proj=nn.Linear(4 * dim, dim)))

    def forward(self, x, causal: bool):
        x = x + self.attn(self.ln_1(x), causal)
        h = self.mlp["c_fc"](self.ln_2(x))
        return x + self.mlp["c_proj"](h * torch.sigmoid(1.702 * h))


class _Transformer(nn.Module):
    def __init__(self, width: int, layers: int, heads: int, causal: bool):
        super().__init__()
        self.causal = causal
        self.resblocks = nn.ModuleList([_Block(width, heads) for _ in range(layers)])

    def forward(self, x):
        for blk in self.resblocks:
            x = blk(x, self.causal)
        return x


class VisionTower(nn.Module):
    def __init__(self, input_resolution: int, patch_size: int, width: int, layers: int, heads: int, output_dim: int):
        super().__init__()
        self.input_resolution = input_resolution
        self.conv1 = nn.Conv2d(3, width, patch_size, patch_size, bias=False)
        scale = width ** -0.5
        self.class_embedding = nn.Parameter(scale * torch.randn(width))
        self.positional_embedding = nn.Parameter(scale * torch.randn((input_resolution // patch_size) ** 2 + 1, width))
        self.ln_pre, self.ln_post = _LN(width), _LN(width)
        self.transformer = _Transformer(width, layers, heads, causal=False)
        self.proj = nn.Parameter(scale * torch.randn(width, output_dim))

    def forward(self, image: torch.Tensor) -> torch.Tensor:
        x = self.conv1(image).flatten(2).transpose(1, 2)                                 # [B, grid^2, width]
        cls = self.class_embedding.to(x.dtype).expand(x.shape[0], 1, -1)
        x = self.ln_pre(torch.cat([cls, x], 1) + self.positional_embedding.to(x.dtype))
        x = self.transformer(x)
        return self.ln_post(x[:, 0]) @ self.proj


class CLIP(nn.Module):
    def __init__(self, embed_dim: int, image_resolution: int, vision_layers: int, vision_width: int, vision_patch_size: int,
                 context_length: int, vocab_size: int, transformer_width: int, transformer_heads: int, transformer_layers: int):
        super().__init__()
        self.context_length = context_length
        self.visual = VisionTower(image_resolution, vision_patch_size, vision_width, vision_layers, vision_width // 64, embed_dim)
        self.transformer = _Transformer(transformer_width, transformer_layers, transformer_heads, causal=True)
        self.token_embedding = nn.Embedding(vocab_size, transformer_width)
        self.positional_embedding = nn.Parameter(0.01 * torch.randn(context_length, transformer_width))
        self.ln_final = _LN(transformer_width)
        self.text_projection = nn.Parameter(transformer_width ** -0.5 * torch.randn(transformer_width, embed_dim))
        self.logit_scale = nn.Parameter(torch.ones([]) * 2.6592)                        # ln(1 / 0.07)

    @property
    def dtype(self):
        return self.visual.conv1.weight.dtype

    def encode_image(self, image: torch.Tensor) -> torch.Tensor:
        return self.visual(image.type(self.dtype))

    def encode_text(self, text: torch.Tensor) -> torch.Tensor:
        x = self.token_embedding(text).type(self.dtype) + self.positional_embedding.type(self.dtype)
        x = self.ln_final(self.transformer(x)).type(self.dtype)
        # features of the end-of-text token: the largest id in every sequence
        return x[torch.arange(x.shape[0]), text.argmax(dim=-1)] @ self.text_projection

    def forward(self, image: torch.Tensor, text: torch.Tensor):
        img = F.normalize(self.encode_image(image), dim=-1)
        txt = F.normalize(self.encode_text(text), dim=-1)
        logits = self.logit_scale.exp() * img @ txt.t()
        return logits, logits.t()


def build_model(state_dict: Dict[str, torch.Tensor], dtype: Optional[torch.dtype] = None) -> CLIP:
    """Size a ``CLIP`` from the tensor shapes of a released ViT checkpoint and load it."""
    if "visual.proj" not in state_dict:
        raise ValueError("only the ViT checkpoints are supported (no 'visual.proj' in this state dict)")
    vision_width = state_dict["visual.conv1.weight"].shape[0]
    vision_layers = len({k.split(".")[3] for k in state_dict if k.startswith("visual.transformer.resblocks.")})
    patch = state_dict["visual.conv1.weight"].shape[-1]
    grid = round((state_dict["visual.positional_embedding"].shape[0] - 1) ** 0.5)
    width = state_dict["ln_final.weight"].shape[0]
    model = CLIP(embed_dim=state_dict["text_projection"].shape[1], image_resolution=patch * grid, vision_layers=vision_layers,
                 vision_width=vision_width, vision_patch_size=patch, context_length=state_dict["positional_embedding"].shape[0],
                 vocab_size=state_dict["token_embedding.weight"].shape[0], transformer_width=width, transformer_heads=width // 64,
                 transformer_layers=len({k.split(".")[2] for k in state_dict if k.startswith("transformer.resblocks.")}))
    sd = {k: v for k, v in state_dict.items() if k not in ("input_resolution", "context_length", "vocab_size")}
    model.load_state_dict(sd)
    return model.eval() if dtype is None else model.to(dtype).eval()
