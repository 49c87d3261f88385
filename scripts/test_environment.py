"""Check that this machine can run the framework: Python, PyTorch + CUDA, the in-tree sm_100a extension, optional packages.

Usage:  python scripts/test_environment.py [--training]     (parity: scripts/test_environment.py of the reference)
"""

import argparse
import os as _os
import sys as _sys

_sys.path.insert(0, _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__))))   # repository root
import importlib
import os
import sys

GREEN, RED, YELLOW, END = "\033[92m", "\033[91m", "\033[93m", "\033[0m"


def ok(msg):
    print(f"{GREEN}[SUCCESS]{END} {msg}")


def bad(msg):
    print(f"{RED}[ERROR]{END} {msg}")


def warn(msg):
    print(f"{YELLOW}[WARNING]{END} {msg}")


def check_packages(packages, required=True) -> bool:
    good = True
    for pkg in packages:
        alts = pkg if isinstance(pkg, tuple) else (pkg,)
        for name in alts:
            try:
                m = importlib.import_module(name)
                ok(f"{name} found" + (f" (v{m.__version__})" if hasattr(m, "__version__") else ""))
                break
            except ImportError:
                continue
        else:
            (bad if required else warn)(f"none of {', '.join(alts)} found")
            good = good and not required
    return good


def main(argv=None) -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--training", action="store_true", help="also check the packages only training needs")
    a = ap.parse_args(argv)
    good = True
    if sys.version_info < (3, 10):
        bad(f"Python >= 3.10 required, found {sys.version.split()[0]}")
        good = False
    else:
        ok(f"Python {sys.version.split()[0]}")
    good &= check_packages(["torch", "numpy", "einops", "pydantic", "yaml"])
    check_packages(["cv2", "PIL", "transformers", "fastapi", ("boto3",), "wandb"], required=False)
    if a.training:
        check_packages(["pandas", "pyarrow"], required=False)
    import torch
    if torch.cuda.is_available():
        cap = torch.cuda.get_device_capability(0)
        name = torch.cuda.get_device_name(0)
        (ok if cap[0] == 10 else warn)(f"GPU 0: {name} (sm_{cap[0]}{cap[1]}); the kernels of this framework target sm_100a")
    else:
        warn("no CUDA device visible: only the CPU reference paths will run")
    try:
        from cosmos_predict25_b200.ops import native
        if os.path.exists(native.lib_path()):
            ok(f"extension built: {native.lib_path()}")
            if torch.cuda.is_available():
                native.load()
                ok(f"extension loaded, {len([n for n in dir(torch.ops.cosmos_b200) if not n.startswith('_')])} operators registered")
        else:
            bad("extension not built: run `python -m cosmos_predict25_b200.ops.build`")
            good = False
    except Exception as e:
        bad(f"extension check failed: {e}")
        good = False
    print(f"{GREEN}environment OK{END}" if good else f"{RED}environment incomplete{END}")
    return 0 if good else 1


if __name__ == "__main__":
    sys.exit(main())
