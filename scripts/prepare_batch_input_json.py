"""Build the json-lines batch file the inference CLI consumes from a folder of inputs.

Usage:  python scripts/prepare_batch_input_json.py --input_dir assets/ --output batch.jsonl [--prompt_dir prompts/] [--default_prompt "..."]

Every image / video in ``input_dir`` becomes one sample ``{"name", "input_path", "prompt", "inference_type"}``; the prompt is
read from ``<prompt_dir>/<stem>.txt`` when present (parity: scripts/prepare_batch_input_json.py of the reference).
"""

import argparse
import json
import os

IMAGE_EXT = (".png", ".jpg", ".jpeg", ".webp", ".bmp")
VIDEO_EXT = (".mp4", ".mov", ".avi", ".mkv", ".webm")


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--prompt_dir", default=None)
    ap.add_argument("--default_prompt", default="")
    a = ap.parse_args(argv)
    rows = []
    for f in sorted(os.listdir(a.input_dir)):
        ext = os.path.splitext(f)[1].lower()
        if ext not in IMAGE_EXT + VIDEO_EXT:
            continue
        stem = os.path.splitext(f)[0]
        prompt = a.default_prompt
        for d in filter(None, (a.prompt_dir, a.input_dir)):
            p = os.path.join(d, stem + ".txt")
            if os.path.exists(p):
                prompt = open(p).read().strip()
                break
        rows.append({"name": stem, "input_path": os.path.abspath(os.path.join(a.input_dir, f)), "prompt": prompt,
                     "inference_type": "image2world" if ext in IMAGE_EXT else "video2world"})
    with open(a.output, "w") as fh:
        for r in rows:
            fh.write(json.dumps(r) + "\n")
    print(f"wrote {len(rows)} samples to {a.output}")
    return rows


if __name__ == "__main__":
    main()
