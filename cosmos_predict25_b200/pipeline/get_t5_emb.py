"""Prompt -> T5 embedding, the pre-processing step of the T5-conditioned (predict2-era) models.

Parity target: ``CosmosT5TextEncoder`` / ``get_text_embedding`` / ``CosmosT5TextEncoderConfig``
(cosmos_predict2/_src/predict2/inference/get_t5_emb.py:28-180): tokenise with truncation and padding to ``max_length``, run the
encoder, zero everything after each prompt's last token, optionally return the boolean mask; a module-level encoder is created
on first use and reused. The encoder is this package's own T5 tower (``models/t5_xxl.py``) loaded from a Hugging Face checkpoint
directory (``config.json`` + ``*.safetensors`` or ``pytorch_model*.bin``); transformers is used for the tokenizer only.

Where the checkpoint comes from: ``model_name`` if it is a directory, else ``$COSMOS_T5_MODEL_DIR``, else
``<cache_dir>/<model_name>``, else ``checkpoints/<model_name>``, else (unless ``local_files_only``) the Hugging Face hub.
"""

from __future__ import annotations

import glob
import json
import os
from dataclasses import dataclass
from typing import ClassVar, List, Optional, Tuple, Union

import torch

from ..models.t5_xxl import T5Config, T5EncoderTower

T5_MODEL_DIR = "checkpoints/google-t5/t5-11b"


def _resolve(model_name: str, cache_dir: Optional[str], local_files_only: bool) -> str:
    cands = [model_name, os.environ.get("COSMOS_T5_MODEL_DIR", ""), os.path.join(cache_dir or "", model_name) if cache_dir else "",
             os.path.join("checkpoints", model_name)]
    for c in cands:
        if c and os.path.isfile(os.path.join(c, "config.json")):
            return c
    if local_files_only:
        raise FileNotFoundError(f"no local copy of {model_name} (looked in {[c for c in cands if c]})")
    from huggingface_hub import snapshot_download
    return snapshot_download(model_name, cache_dir=cache_dir)


def _load_tower(path: str) -> T5EncoderTower:
    hf = json.load(open(os.path.join(path, "config.json")))
    cfg = T5Config(vocab_size=hf["vocab_size"], d_model=hf["d_model"], d_kv=hf["d_kv"], num_heads=hf["num_heads"], d_ff=hf["d_ff"],
                   num_layers=hf["num_layers"], num_buckets=hf.get("relative_attention_num_buckets", 32),
                   max_distance=hf.get("relative_attention_max_distance", 128),
                   feed_forward="gated-gelu" if "gated" in hf.get("feed_forward_proj", "relu") else "relu",
                   eps=hf.get("layer_norm_epsilon", 1e-6))
    tower = T5EncoderTower(cfg)
    sd = {}
    files = sorted(glob.glob(os.path.join(path, "*.safetensors")))
    if files:
        from safetensors.torch import load_file
        for f in files:
            sd.update(load_file(f))
    else:
        for f in sorted(glob.glob(os.path.join(path, "pytorch_model*.bin"))):
            sd.update(torch.load(f, map_location="cpu", weights_only=True))
    if not sd:
        raise FileNotFoundError(f"no weight files in {path}")
    sd = {k: v for k, v in sd.items() if k.startswith(("encoder.", "shared."))}
    if "shared.weight" in sd:
        sd.pop("encoder.embed_tokens.weight", None)
    tower.load_hf_state_dict(sd)
    return tower


class CosmosT5TextEncoder(torch.nn.Module):
    def __init__(self, model_name: str = "google-t5/t5-11b", device: str = "cuda", cache_dir=None, local_files_only=False,
                 tower: Optional[T5EncoderTower] = None, tokenizer=None):
        super().__init__()
        if tower is None or tokenizer is None:
            path = _resolve(model_name, cache_dir, local_files_only)
            if tokenizer is None:
                from transformers import T5TokenizerFast
                tokenizer = T5TokenizerFast.from_pretrained(path, local_files_only=True)
            if tower is None:
                tower = _load_tower(path)
        self.tokenizer = tokenizer
        self.text_encoder = tower.to(device).eval().requires_grad_(False)
        self.device = device

    @torch.inference_mode()
    def encode_prompts(self, prompts: Union[str, List[str]], max_length: int = 512, return_mask: bool = False
                       ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        if isinstance(prompts, str):
            prompts = [prompts]
        if not prompts:
            raise ValueError("The input prompt list is empty.")
        enc = self.tokenizer(list(prompts), return_tensors="pt", truncation=True, padding="max_length", max_length=max_length)
        ids, mask = enc["input_ids"].to(self.device), enc["attention_mask"].to(self.device)
        out = self.text_encoder(ids, mask)
        out = out * mask.unsqueeze(-1).to(out.dtype)          # positions after a prompt's last token are zero
        return (out, mask.bool()) if return_mask else out


@dataclass
class CosmosT5TextEncoderConfig:
    CKPT_PATH: ClassVar[str] = T5_MODEL_DIR
    NUM_TOKENS: ClassVar[int] = 512
    EMBED_DIM: ClassVar[int] = 1024
    ckpt_path: str = T5_MODEL_DIR
    num_tokens: int = 512
    embed_dim: int = 1024


cosmos_encoder: Optional[CosmosT5TextEncoder] = None


def get_text_embedding(prompts: Union[str, List[str]], encoder: Optional[CosmosT5TextEncoder] = None, device: str = "cuda",
                       max_length: int = 512, return_mask: bool = False, cache_dir: Optional[str] = None,
                       local_files_only: bool = False, text_encoder_class: str = "T5"):
    """Embeddings ``[B, max_length, D]`` (and the mask with ``return_mask``). Without ``encoder`` a module-level one is created on
    first use and kept."""
    assert text_encoder_class == "T5", f"text_encoder_class {text_encoder_class} is not supported"
    global cosmos_encoder
    if encoder is None:
        if cosmos_encoder is None:
            cosmos_encoder = CosmosT5TextEncoder(device=device, cache_dir=cache_dir, local_files_only=local_files_only)
        encoder = cosmos_encoder
    return encoder.encode_prompts(prompts, max_length=max_length, return_mask=return_mask)
