"""Test helpers for code that is written against this package: ``RunIf`` (a ``pytest.mark.skipif`` assembled from requirements)
and ``run_command`` (a shell command with retries).

Parity target: cosmos_predict2/_src/imaginaire/utils/helper_test.py:30-170 (same module name, so ``from ...utils.helper_test import
RunIf`` keeps working). The GPU model comes from torch's device name instead of NVML; only B200 is a target of this package, the
other names are reported so that ``supported_arch`` lists written for the reference skip here as intended.
"""

from __future__ import annotations

import importlib.util
import subprocess
import sys
import time
from pathlib import Path
from typing import List, Optional, Union

import pytest
import torch
from packaging.version import Version


def get_gpu_architecture() -> str:
    if not torch.cuda.is_available():
        return "Other"
    name = torch.cuda.get_device_name(0)
    for tag, arch in (("B200", "B200"), ("H100", "H100"), ("H200", "H100"), ("A100", "A100"), ("L40S", "L40S")):
        if tag in name:
            return arch
    return "Other"


def RunIf(min_gpus: int = 0, min_torch: Optional[str] = None, max_torch: Optional[str] = None, min_python: Optional[str] = None,
          supported_arch: Optional[Union[str, List[str]]] = None, requires_file: Optional[Union[str, List[str]]] = None,
          requires_package: Optional[Union[str, List[str]]] = None, **kwargs):
    """``@RunIf(min_gpus=2, requires_package="cv2")`` skips the test unless every requirement holds; the reason lists the ones
    that do not. Extra keyword arguments go to ``pytest.mark.skipif``."""
    as_list = lambda x: [x] if isinstance(x, str) else list(x or [])
    torch_version = Version(torch.__version__.split("+")[0])
    unmet = []
    if min_gpus and torch.cuda.device_count() < min_gpus:
        unmet.append(f"GPUs>={min_gpus}")
    if min_torch and torch_version < Version(min_torch):
        unmet.append(f"torch>={min_torch}")
    if max_torch and torch_version >= Version(max_torch):
        unmet.append(f"torch<{max_torch}")
    if min_python and Version(".".join(map(str, sys.version_info[:3]))) < Version(min_python):
        unmet.append(f"python>={min_python}")
    if supported_arch and get_gpu_architecture() not in as_list(supported_arch):
        unmet.append(f"supported_arch arch={','.join(as_list(supported_arch))}")
    missing = [f for f in as_list(requires_file) if not Path(f).exists()]
    if missing:
        unmet.append(f"requires file={','.join(missing)}")
    for package in as_list(requires_package):
        if importlib.util.find_spec(package) is None:
            unmet.append(f"Package {package} is not installed.")
    return pytest.mark.skipif(condition=bool(unmet), reason=f"Requires: [{' + '.join(unmet)}]", **kwargs)


def run_command(cmd: str, max_retry_counter: int = 3, is_raise: bool = True, capture_output: bool = True) -> subprocess.CompletedProcess:
    """Run ``cmd`` in a shell; on a non-zero exit wait a second and try again, up to ``max_retry_counter`` retries; then raise
    (``is_raise``) or return the last result."""
    attempt = 0
    while True:
        result = subprocess.run(cmd, shell=True, capture_output=capture_output, text=True)
        if result.returncode == 0 or attempt >= max_retry_counter:
            break
        attempt += 1
        time.sleep(1)
    if result.returncode != 0 and is_raise:
        raise RuntimeError(f"command failed after {attempt} retries (exit {result.returncode}): {cmd}\n{(result.stderr or '')[-2000:]}")
    return result
