"""Dump frames of every video of a folder as jpg images (for image-conditioned evaluation sets).

Usage:  python scripts/extract_images_from_videos.py --input_dir videos/ --output_dir frames/ [--every 10] [--first_only]
(parity: scripts/extract_images_from_videos.py of the reference)
"""

import argparse
import os


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--every", type=int, default=1)
    ap.add_argument("--first_only", action="store_true")
    a = ap.parse_args(argv)
    import cv2
    os.makedirs(a.output_dir, exist_ok=True)
    n = 0
    for f in sorted(os.listdir(a.input_dir)):
        if not f.lower().endswith((".mp4", ".mov", ".avi", ".mkv", ".webm")):
            continue
        cap = cv2.VideoCapture(os.path.join(a.input_dir, f))
        i = 0
        while True:
            good, frame = cap.read()
            if not good:
                break
            if i % a.every == 0:
                cv2.imwrite(os.path.join(a.output_dir, f"{os.path.splitext(f)[0]}_{i:06d}.jpg"), frame)
                n += 1
                if a.first_only:
                    break
            i += 1
        cap.release()
    print(f"wrote {n} images to {a.output_dir}")
    return n


if __name__ == "__main__":
    main()
