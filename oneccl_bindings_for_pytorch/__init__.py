"""Drop-in import name of the `ccl` backend.

`import oneccl_bindings_for_pytorch` registers backend "ccl" with `torch.distributed` for CUDA
and CPU tensors and publishes `torch.distributed.ProcessGroupCCL`, exactly as importing the
reference package does for XPU and CPU (oneccl_bindings_for_pytorch/__init__.py:1-43 of
intel/torch-ccl). Attributes kept from the reference: `cwd`, `__version__`, `git_version`,
`is_available(tensors)`. The implementation lives in `torch_ccl_b200`.
"""
import os

import torch  # noqa: F401  (torch must be imported before the extension)

cwd = os.path.dirname(os.path.abspath(__file__))
if not os.path.exists(os.path.join(cwd, "version.py")):
    raise RuntimeError("oneccl_bindings_for_pytorch is not installed!")

from .version import __version__, git_version  # noqa: E402
from torch_ccl_b200 import _C as ccl_lib  # noqa: E402  (importing registers the backend)
from torch_ccl_b200 import (  # noqa: E402,F401
    flight_recorder,
    get_backend,
    ops,
    reparse_env,
    stats,
)

__all__ = ["is_available", "stats", "flight_recorder", "reparse_env", "get_backend", "ops"]


def is_available(tensors):
    """True when every tensor is contiguous and no two live on the same device index."""
    devices = set()
    for tensor in tensors:
        if not tensor.is_contiguous():
            return False
        device = tensor.get_device()
        if device in devices:
            return False
        devices.add(device)
    return True
