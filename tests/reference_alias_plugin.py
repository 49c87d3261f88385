"""pytest plugin for running the reference's OWN test files against this package: the module names those files import are
mapped onto this package's modules (``COSMOS_ALIAS_JSON``: {reference module name: module name here}); ancestors of the mapped
names become empty packages, so nothing of the reference's implementation is importable. Used by
``tests/test_cpu_reference_suites.py`` in a sub-process."""

import importlib
import json
import os
import sys
import types


def _install():
    for ref_name, own_name in json.loads(os.environ.get("COSMOS_ALIAS_JSON", "{}")).items():
        parts = ref_name.split(".")
        for i in range(1, len(parts)):
            anc = ".".join(parts[:i])
            if anc not in sys.modules:
                pkg = types.ModuleType(anc)
                pkg.__path__ = []
                sys.modules[anc] = pkg
        mod = importlib.import_module(own_name)
        sys.modules[ref_name] = mod
        setattr(sys.modules[".".join(parts[:-1])], parts[-1], mod)


def _cuda_calls_stay_on_the_host():
    """Some of those files place tensors with ``.cuda()``; without a GPU (``COSMOS_ALIAS_NO_CUDA=1``) that call is the identity
    and the process group is gloo."""
    import torch
    if os.environ.get("COSMOS_ALIAS_NO_CUDA") != "1" or torch.cuda.is_available():
        return
    torch.Tensor.cuda = lambda self, *a, **k: self
    torch.nn.Module.cuda = lambda self, *a, **k: self


_install()
_cuda_calls_stay_on_the_host()


def pytest_configure(config):
    for marker in ("L0", "L1", "L2", "GPU", "CPU"):
        config.addinivalue_line("markers", f"{marker}: marker of the reference's test files")
