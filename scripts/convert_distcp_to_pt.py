"""Convert a distributed checkpoint (``.../checkpoints/iter_XXXXXXXXX/model``) into single-file checkpoints.

Usage:  python scripts/convert_distcp_to_pt.py <distcp dir or s3:// uri> <output dir> [--no-ema]

Writes ``model.pt`` (all keys) and, unless ``--no-ema``, ``model_ema_fp32.pt`` / ``model_ema_bf16.pt`` holding the EMA weights
renamed ``net_ema.* -> net.*`` (the layout inference loads). An ``s3://`` input is first synchronised to ``<output dir>/model``
through the unified file API (parity: scripts/convert_distcp_to_pt.py of the reference, which shells out to s5cmd).
"""

import argparse
import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))   # repository root
import os
from pathlib import Path


def fetch_s3(uri: str, dst: Path) -> Path:
    from cosmos_predict25_b200.utils.easy_io import easy_io
    uri = uri.rstrip("/")
    uri = uri[: -len("/model")] if uri.endswith("/model") else uri
    dst.mkdir(parents=True, exist_ok=True)
    for rel in easy_io.list_dir_or_file(f"{uri}/model", list_dir=False, recursive=True):
        easy_io.copyfile_to_local(f"{uri}/model/{rel}", str(dst / rel))
    return dst


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("input_dir", help="S3 URI of the checkpoint or path to the distcp directory")
    ap.add_argument("output_dir", type=Path)
    ap.add_argument("--no-ema", action="store_true", help="do not export the EMA weights")
    a = ap.parse_args(argv)
    from cosmos_predict25_b200.checkpoint.dcp import convert_distcp_to_pt
    a.output_dir.mkdir(parents=True, exist_ok=True)
    for name in ("model.pt", "model_ema_fp32.pt", "model_ema_bf16.pt"):
        (a.output_dir / name).unlink(missing_ok=True)
    src = fetch_s3(a.input_dir, a.output_dir / "model") if a.input_dir.startswith("s3://") else Path(a.input_dir)
    paths = convert_distcp_to_pt(str(src), str(a.output_dir))
    if a.no_ema:
        for k in ("ema_fp32", "ema_bf16"):
            if k in paths:
                os.remove(paths.pop(k))
    for k, p in paths.items():
        print(f"{k}: {p}")
    return paths


if __name__ == "__main__":
    main()
