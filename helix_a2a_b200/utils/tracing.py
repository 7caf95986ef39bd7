"""Optional NVTX ranges and debug checks (both off by default).

``HELIX_A2A_NVTX=1`` wraps the library's public calls and the model stacks' layers in NVTX ranges so
that an external timeline tool can attribute GPU time; ``HELIX_A2A_DEBUG=1`` makes the exchange ops
pre-fill their outputs with NaN (done in the binding) and makes :func:`check_written` verify, after a
synchronisation, that every row was written.  The reference has neither
(its profiling is an external ``nsys`` wrapper, ``benchmark/sbatch/pipeline_bench.sbatch:167-173``).
"""
from __future__ import annotations

import contextlib

import torch

from . import env


def nvtx_enabled() -> bool:
    return env.nvtx() and torch.cuda.is_available()


@contextlib.contextmanager
def nvtx_range(name: str):
    if nvtx_enabled():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


def debug_enabled() -> bool:
    return env.debug()


def check_written(t: torch.Tensor, what: str) -> None:
    """In debug mode: synchronise and raise if ``t`` still holds the NaN poison."""
    if not debug_enabled() or not t.is_cuda or not t.is_floating_point():
        return
    torch.cuda.synchronize(t.device)
    if torch.isnan(t).any():
        raise RuntimeError(f"helix debug: {what} has rows the kernel did not write")
