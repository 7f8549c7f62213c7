"""CUDA kernels (sm_100a) and their Python launchers.

``native()`` returns the compiled extension module, building it in-tree on
first use.  On a machine with a GPU a missing or unloadable extension is an
error, never a silent fallback to PyTorch ops.
"""
from __future__ import annotations

import importlib
import threading

_lock = threading.Lock()
_mod = None


def native():
    global _mod
    if _mod is None:
        with _lock:
            if _mod is None:
                import torch  # noqa: F401  (loads libcudart before the extension)

                import os

                from . import build as _build

                # GRACE_CHECKED=1: the variant compiled with index / offset checks (see ops/build.py)
                checked = os.environ.get("GRACE_CHECKED", "") not in ("", "0")
                _build.ensure_built(checked)
                _mod = importlib.import_module("grace_b200._C_checked" if checked else "grace_b200._C")
    return _mod


def available() -> bool:
    import torch

    return torch.cuda.is_available()
