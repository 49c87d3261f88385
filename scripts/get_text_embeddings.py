"""Pre-compute caption embeddings for a local dataset: ``<dataset>/metas/*.txt`` -> ``<dataset>/<out>/*.pt``.

Usage:  python scripts/get_text_embeddings.py --dataset_path datasets/my_videos [--encoder reason1|hash] [--out embeddings]

Parity: scripts/get_t5_embeddings.py / get_t5_embeddings_from_groot_dataset.py of the reference (T5-XXL there; the 2.5 models
condition on the Reason1 / Qwen2.5-VL language tower, so that is the default here). ``--encoder hash`` writes the
deterministic pseudo-embeddings used by offline tests.
"""

import argparse
import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))   # repository root
import os

import torch


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset_path", required=True)
    ap.add_argument("--caption_dir", default="metas")
    ap.add_argument("--out", default="embeddings")
    ap.add_argument("--encoder", default="reason1", choices=["reason1", "hash"])
    ap.add_argument("--checkpoint", default=None, help="text-encoder checkpoint directory (reason1)")
    ap.add_argument("--max_length", type=int, default=512)
    ap.add_argument("--dim", type=int, default=100352, help="embedding width of the hash encoder")
    a = ap.parse_args(argv)
    from cosmos_predict25_b200.models.text_encoder import HashTextEncoder, TextEncoder, TextEncoderConfig
    if a.encoder == "hash":
        enc = HashTextEncoder(a.dim, a.max_length)
    else:
        enc = TextEncoder(TextEncoderConfig(ckpt_path=a.checkpoint) if a.checkpoint else TextEncoderConfig(),
                          device="cuda" if torch.cuda.is_available() else "cpu")
    src, dst = os.path.join(a.dataset_path, a.caption_dir), os.path.join(a.dataset_path, a.out)
    os.makedirs(dst, exist_ok=True)
    names = sorted(f for f in os.listdir(src) if f.endswith(".txt"))
    for i, name in enumerate(names):
        with open(os.path.join(src, name)) as f:
            prompt = f.read().strip()
        emb = enc.encode_prompts([prompt])[0].cpu()
        torch.save(emb, os.path.join(dst, name[:-4] + ".pt"))
        if i % 50 == 0:
            print(f"[{i + 1}/{len(names)}] {name}: {tuple(emb.shape)}")
    print(f"wrote {len(names)} embeddings to {dst}")


if __name__ == "__main__":
    main()
