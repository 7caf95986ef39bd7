"""Install the Helix DCP hook at import time, without touching vLLM's files.

The reference overwrites ``vllm/v1/attention/ops/dcp_alltoall.py`` on disk
(``install_in_container.sh:36-54``) because the attention backends bind ``dcp_a2a_lse_reduce``
with ``from ... import`` when they are first imported.  A meta-path finder gets in earlier: it
lets the stock module load, then swaps the two public functions before any backend sees them.
It also wraps ``Worker.compile_or_warm_up_model`` so that the workspace exists before CUDA-graph
capture starts (stock vLLM never calls ``dcp_a2a_ensure_initialized``; the reference asks the
integrator to, ``patches/dcp_alltoall_helix.py:119-135``), and ``Worker.execute_model`` so that the status
of the native exchange is read after every step (``HELIX_A2A_HOOK_CHECK=0`` switches that off).

``install()`` works in the current process.  vLLM's worker processes are separate interpreters:
put ``helix_a2a_b200/vllm_patch/autoload`` on ``PYTHONPATH`` (``autoload_env()`` returns the
environment for that) and its ``sitecustomize`` calls ``install()`` in every one of them.

This module imports neither torch nor vLLM: it must stay cheap, it runs at interpreter start.
"""
from __future__ import annotations

import importlib.abc
import importlib.util
import os
import sys

DCP_MODULE = "vllm.v1.attention.ops.dcp_alltoall"
WORKER_MODULE = "vllm.v1.worker.gpu_worker"
_TARGETS = (DCP_MODULE, WORKER_MODULE)


def _patch_dcp_module(module) -> None:
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hx
    stock = getattr(module, "dcp_a2a_lse_reduce", None)
    if stock is not None and stock is not hx.dcp_a2a_lse_reduce and hx._stock_reduce is None:
        hx._stock_reduce = stock
    module.dcp_a2a_lse_reduce = hx.dcp_a2a_lse_reduce
    module.dcp_a2a_ensure_initialized = hx.dcp_a2a_ensure_initialized
    module.__helix_hooked__ = True


def _patch_worker_module(module) -> None:
    worker = getattr(module, "Worker", None)
    warm = getattr(worker, "compile_or_warm_up_model", None) if worker is not None else None
    if warm is None or getattr(warm, "__helix_hooked__", False):
        return

    def compile_or_warm_up_model(self, *args, **kwargs):
        _ensure_before_capture()
        return warm(self, *args, **kwargs)

    compile_or_warm_up_model.__helix_hooked__ = True
    compile_or_warm_up_model.__wrapped__ = warm
    worker.compile_or_warm_up_model = compile_or_warm_up_model

    step = getattr(worker, "execute_model", None)
    if step is not None and not getattr(step, "__helix_hooked__", False):
        def execute_model(self, *args, **kwargs):
            out = step(self, *args, **kwargs)
            _check_after_step()
            return out

        execute_model.__helix_hooked__ = True
        execute_model.__wrapped__ = step
        worker.execute_model = execute_model


def _ensure_before_capture() -> None:
    """Create the workspace while ranks are still in lock step (model loaded, nothing captured yet)."""
    if os.environ.get("HELIX_A2A_BACKEND", "nccl").lower() != "native":
        return
    from vllm.distributed.parallel_state import get_dcp_group
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hx
    try:
        group = get_dcp_group()
    except AssertionError:      # no DCP group in this deployment
        return
    hx.dcp_a2a_ensure_initialized(group)


def _check_after_step() -> None:
    """A device-side wait of the native exchange that ran out must stop the engine, not go on serving the
    NaN rows it left.  Once per step the status block is polled WITHOUT waiting for the GPU (a 32-byte copy to
    pinned memory is requested and the previous one inspected), so a failure stops the engine one or two steps
    late; ``HELIX_A2A_HOOK_CHECK=sync`` reads it with a synchronisation every step (costs ~0.25 ms per step of a
    small model: the engine's asynchronous scheduling stalls), ``=0`` switches the check off."""
    if os.environ.get("HELIX_A2A_BACKEND", "nccl").lower() != "native":
        return
    from helix_a2a_b200.utils import env as _env
    mode = _env.hook_check_mode()
    if mode == "off":
        return
    from helix_a2a_b200.vllm_patch import dcp_alltoall_helix as hx
    if mode == "sync":
        hx.dcp_a2a_check_status(raise_on_error=True)
    else:
        hx.dcp_a2a_poll_status(raise_on_error=True)


class _PatchingLoader(importlib.abc.Loader):
    def __init__(self, inner, patch):
        self._inner = inner
        self._patch = patch

    def create_module(self, spec):
        return self._inner.create_module(spec)

    def exec_module(self, module):
        self._inner.exec_module(module)
        self._patch(module)


class HelixHookFinder(importlib.abc.MetaPathFinder):
    """Finds nothing itself: asks the remaining finders, then wraps the loader of the two targets."""

    def find_spec(self, fullname, path=None, target=None):
        if fullname not in _TARGETS:
            return None
        for finder in sys.meta_path:
            if finder is self or not hasattr(finder, "find_spec"):
                continue
            spec = finder.find_spec(fullname, path, target)
            if spec is not None and spec.loader is not None:
                patch = _patch_dcp_module if fullname == DCP_MODULE else _patch_worker_module
                spec.loader = _PatchingLoader(spec.loader, patch)
                return spec
        return None


def install() -> bool:
    """Register the finder (idempotent); modules that are already imported are patched in place."""
    if any(isinstance(f, HelixHookFinder) for f in sys.meta_path):
        return False
    sys.meta_path.insert(0, HelixHookFinder())
    if DCP_MODULE in sys.modules:
        _patch_dcp_module(sys.modules[DCP_MODULE])
        from helix_a2a_b200.vllm_patch.dcp_alltoall_helix import apply_runtime_patch
        apply_runtime_patch()          # backends that already bound the stock function
    if WORKER_MODULE in sys.modules:
        _patch_worker_module(sys.modules[WORKER_MODULE])
    return True


def uninstall() -> None:
    sys.meta_path[:] = [f for f in sys.meta_path if not isinstance(f, HelixHookFinder)]


def autoload_dir() -> str:
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "autoload")


def autoload_env(env=None) -> dict:
    """A copy of ``env`` (default: this process's) whose ``PYTHONPATH`` makes every child interpreter
    install the hook at start-up: the autoload directory first, then the directory that holds the package."""
    out = dict(os.environ if env is None else env)
    pkg_parent = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    parts = [autoload_dir(), pkg_parent] + [p for p in out.get("PYTHONPATH", "").split(os.pathsep) if p]
    seen, uniq = set(), []
    for p in parts:
        if p not in seen:
            seen.add(p)
            uniq.append(p)
    out["PYTHONPATH"] = os.pathsep.join(uniq)
    out.setdefault("HELIX_A2A_VLLM_HOOK", "1")
    return out
