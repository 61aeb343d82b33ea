"""Locate and load the compiled libraries (built in-tree by ``build.py``)."""
from __future__ import annotations

import importlib.machinery
import importlib.util
import os
import sys

LIB_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib")
CORE_LIB = os.path.join(LIB_DIR, "libsparse_mla_b200.so")
TORCH_EXT = os.path.join(LIB_DIR, "flash_mla_cuda.so")


def load_torch_extension():
    """Import ``flash_mla_cuda`` so that ``torch.ops.flash_mla.*`` is registered."""
    if "flash_mla_cuda" in sys.modules:
        return sys.modules["flash_mla_cuda"]
    if not (os.path.exists(TORCH_EXT) and os.path.exists(CORE_LIB)):
        raise ImportError(
            f"flash_mla: compiled libraries not found under {LIB_DIR}; run "
            "`python forks-flash-mla-int_b200/build.py` (needs nvcc with sm_100a support). "
            "There is no CPU fallback.")
    import torch  # noqa: F401  (libtorch must be loaded before the extension)

    loader = importlib.machinery.ExtensionFileLoader("flash_mla_cuda", TORCH_EXT)
    spec = importlib.util.spec_from_file_location("flash_mla_cuda", TORCH_EXT, loader=loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    sys.modules["flash_mla_cuda"] = mod
    return mod
