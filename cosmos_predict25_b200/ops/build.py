"""Builds the in-tree sm_100a extension ``_C.so`` with explicit nvcc / g++ command lines.

Kernels (``csrc/*.cu``) do not include torch headers and compile in seconds each; only the binding
files (``csrc/bindings*.cpp``) see torch. Objects are cached by content hash under ``_build/`` so the
"does it build" check is incremental. Usage: ``python -m cosmos_predict25_b200.ops.build [--force]``.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
BUILD = os.path.join(HERE, "_build")
OUT = os.path.join(HERE, "_C.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v"]


def _nvcc() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else (shutil.which("nvcc") or "nvcc")


def _hash(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()[:16]


def _run(cmd, log_path=None):
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + r.stdout)
    if r.returncode != 0:
        raise RuntimeError(f"command failed: {' '.join(cmd)}\n{r.stdout[-4000:]}")
    return r.stdout


def build_extension(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension

    os.makedirs(BUILD, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh"))]
    cu = sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))
    cpp = sorted(f for f in os.listdir(CSRC) if f.endswith(".cpp"))
    torch_inc = []
    for p in cpp_extension.include_paths("cuda") if "device_type" in cpp_extension.include_paths.__code__.co_varnames \
            else cpp_extension.include_paths(True):
        torch_inc += ["-I", p]
    cuda_home = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    abi = int(torch._C._GLIBCXX_USE_CXX11_ABI)
    jobs = []
    objs = []
    for f in cu:
        src = os.path.join(CSRC, f)
        tag = _hash([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD, f"{f}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-I", CSRC, "-c", src, "-o", obj], os.path.join(BUILD, f + ".log")))
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H",
                 "-I", CSRC, "-I", os.path.join(cuda_home, "include"), *torch_inc, "-w"]
    for f in cpp:
        src = os.path.join(CSRC, f)
        tag = _hash([src] + headers, " ".join(cxx_flags) + torch.__version__)
        obj = os.path.join(BUILD, f"{f}.{tag}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((["g++", *cxx_flags, "-c", src, "-o", obj], os.path.join(BUILD, f + ".log")))
    if jobs or not os.path.exists(OUT) or force:
        with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
            list(ex.map(lambda j: _run(*j), jobs))
        lib_dir = os.path.join(os.path.dirname(torch.__file__), "lib")
        link = ["g++", "-shared", "-o", OUT, *objs, "-L", lib_dir, "-L", os.path.join(cuda_home, "lib64"),
                "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-lcudart",
                f"-Wl,-rpath,{lib_dir}", f"-Wl,-rpath,{os.path.join(cuda_home, 'lib64')}"]
        _run(link, os.path.join(BUILD, "link.log"))
        # drop stale objects
        keep = set(objs)
        for f in os.listdir(BUILD):
            p = os.path.join(BUILD, f)
            if f.endswith(".o") and p not in keep:
                os.remove(p)
    if verbose:
        for f in sorted(os.listdir(BUILD)):
            if f.endswith(".cu.log"):
                with open(os.path.join(BUILD, f)) as fh:
                    sys.stdout.write(fh.read())
    return OUT


def resource_usage() -> str:
    """ptxas register / spill / shared-memory report of the last build (one block per source file)."""
    out = []
    for f in sorted(os.listdir(BUILD)) if os.path.isdir(BUILD) else []:
        if f.endswith(".cu.log"):
            with open(os.path.join(BUILD, f)) as fh:
                out.append(f"== {f}\n" + fh.read())
    return "\n".join(out)


if __name__ == "__main__":
    path = build_extension(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print(path)
