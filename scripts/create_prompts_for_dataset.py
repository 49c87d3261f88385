"""Write one caption file per video: ``<dataset>/videos/*.mp4`` -> ``<dataset>/metas/*.txt``.

Usage:  python scripts/create_prompts_for_dataset.py --dataset_path datasets/cosmos_nemo_assets --prompt "A video of sks teal robot."

Parity: scripts/create_prompts_for_nemo_assets.py of the reference (a fixed prompt for every clip of a small post-training set).
"""

import argparse
import os


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--dataset_path", default="datasets/cosmos_nemo_assets")
    ap.add_argument("--prompt", default="A video of sks teal robot.")
    ap.add_argument("--overwrite", action="store_true")
    a = ap.parse_args(argv)
    vids, metas = os.path.join(a.dataset_path, "videos"), os.path.join(a.dataset_path, "metas")
    os.makedirs(metas, exist_ok=True)
    n = 0
    for f in sorted(os.listdir(vids)):
        if not f.lower().endswith((".mp4", ".mov", ".avi", ".mkv", ".webm")):
            continue
        out = os.path.join(metas, os.path.splitext(f)[0] + ".txt")
        if os.path.exists(out) and not a.overwrite:
            continue
        with open(out, "w") as fh:
            fh.write(a.prompt)
        n += 1
    print(f"wrote {n} prompt files to {metas}")
    return n


if __name__ == "__main__":
    main()
