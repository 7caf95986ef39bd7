"""Loader of the native extension.

Importing this module never fails on a machine without the built library; the first call of
:func:`ext` does.  On a GPU box a missing extension is a hard error (no silent PyTorch
fallback): ops raise instead of running something slower.
"""
from __future__ import annotations

import importlib
import threading

import torch

_lock = threading.Lock()
_mod = None
_err = None


def ext():
    """Return the ``helix_a2a_b200._C`` module (registers ``torch.ops.helix_a2a_b200``)."""
    global _mod, _err
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is None:
            try:
                _mod = importlib.import_module("helix_a2a_b200._C")
            except ImportError as e:  # not built yet
                _err = e
                raise RuntimeError(
                    "helix_a2a_b200 native extension is not built; run "
                    "`python -m helix_a2a_b200._build` (needs nvcc) first") from e
    return _mod


def available() -> bool:
    try:
        ext()
        return True
    except RuntimeError:
        return False


def ops():
    ext()
    return torch.ops.helix_a2a_b200
