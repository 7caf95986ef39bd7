"""DCP all-to-all + LSE reduce for vLLM, backed by the fused Helix kernel.

Same hook as the reference's drop-in (``patches/dcp_alltoall_helix.py:391-448``) and as the
module it replaces in vLLM 0.22 (``vllm/v1/attention/ops/dcp_alltoall.py``)::

    dcp_a2a_lse_reduce(cp_attn_out [B,H,D], cp_attn_lse [B,H], cp_group, ctx=None,
                       return_lse=False, is_lse_base_on_e=True) -> [B, H/N, D] (, [B, H/N])
    dcp_a2a_ensure_initialized(cp_group)     # before CUDA-graph capture

Backend switch, read at import like the reference (``patches/dcp_alltoall_helix.py:40,49``):
``HELIX_A2A_BACKEND=nccl`` (default) is two ``all_to_all_single`` + the stand-alone combine kernel
(``dcp_lse_combine``; ``HELIX_A2A_NCCL_IMPL=stock`` calls the function of the replaced vLLM module instead);
``native`` runs ONE kernel that
reads ``cp_attn_out`` / ``cp_attn_lse`` in place (no permute / pad / zeros copies), exchanges over
NVLink and applies the LSE-weighted combine on the receive side.  Base-2 LSEs (FlashInfer) are
combined natively instead of being converted to base e and back
(``patches/dcp_alltoall_helix.py:564-567,591-593``).

A device-side wait that runs out of time does not hang the GPU: the kernel records a status, fills the rows it
could not complete with NaN and returns.  ``dcp_a2a_check_status()`` turns that status into a
``HelixTimeoutError``; the import hook calls it after every engine step, so a failed exchange stops the
server instead of serving garbage.  The waits of this hook default to 30 s (``HELIX_A2A_HOOK_TIMEOUT_MS``):
ranks may be far apart during warm-up.

``apply_runtime_patch()`` swaps the function into the vLLM modules that imported it; the
``install`` module next to this file rewrites vLLM's file on disk instead.
"""
from __future__ import annotations

import logging
import os
from typing import Optional

import torch
import torch.distributed as dist

import helix_a2a_b200 as _helix
from helix_a2a_b200.ops import reference_math as _rm
from helix_a2a_b200.utils import env as _env

logger = logging.getLogger(__name__)

_HELIX_BACKEND = _env.backend()
# What "nccl" means: "own" = two all_to_all_single + a torch combine, as in the reference's hook
# (patches/dcp_alltoall_helix.py:455-504); "stock" = the function of the vLLM module this hook replaced.
_NCCL_IMPL = _env.nccl_impl()
_HOOK_TIMEOUT_MS = _env.hook_timeout_ms()
_workspace: Optional[torch.Tensor] = None
_workspace_key = None
_stock_reduce = None     # vLLM's original function, when it could be imported


def _lse_weighted_combine(outputs, lses, return_lse: bool = False, is_lse_base_on_e: bool = True):
    """Torch reference combine: ``[N,B,H,D]`` + ``[N,B,H]`` -> ``[B,H,D]`` (same rules as the
    reference's ``_lse_weighted_combine``, ``patches/dcp_alltoall_helix.py:142-207``)."""
    res = _rm.lse_combine(outputs, lses, return_lse=return_lse, base2=not is_lse_base_on_e)
    if return_lse:
        return res[0].to(outputs.dtype), res[1]
    return res.to(outputs.dtype)


def dcp_lse_combine(recv_output: torch.Tensor, recv_lse: torch.Tensor, return_lse: bool = False,
                    is_lse_base_on_e: bool = True):
    """``recv_output [N, B, H, D]`` + ``recv_lse [N, B, H]`` -> ``[B, H, D]`` (+ global LSE ``[B, H]``).

    Same contract as the reference's ``dcp_lse_combine_triton`` (``patches/dcp_alltoall_helix.py:323-384``);
    on CUDA tensors it is the library's hand-written combine kernel, on CPU tensors the torch oracle."""
    return _helix.lse_combine(recv_output, recv_lse, return_lse=return_lse, base2=not is_lse_base_on_e)


dcp_lse_combine_triton = dcp_lse_combine   # the reference's public name; there is no Triton behind it here


def dcp_a2a_check_status(raise_on_error: bool = True) -> dict:
    """Status of the native exchange on this rank (synchronises the current stream).  Raises
    ``helix_a2a_b200.HelixTimeoutError`` if a device-side wait ran out since the workspace was (re)initialised;
    the workspace then needs ``helix_a2a_b200.reset_workspace`` on every rank before it is used again."""
    if _workspace is None or _workspace_key is None:
        return {"code": 0, "name": "ok"}
    cp_size, cp_rank, _ = _workspace_key
    return _helix.check_status(_workspace, cp_rank, cp_size, raise_on_error=raise_on_error)


_poller = None
_poller_key = None


def dcp_a2a_poll_status(raise_on_error: bool = True):
    """Non-blocking form of :func:`dcp_a2a_check_status` for a call once per engine step: looks at the status copy
    requested by the previous call (if it has arrived) and requests the next one; never waits for the GPU.  A
    failure surfaces one or two steps late as ``HelixTimeoutError``."""
    global _poller, _poller_key
    if _workspace is None or _workspace_key is None:
        return None
    if _poller is None or _poller_key is not _workspace_key:
        cp_size, cp_rank, _ = _workspace_key
        _poller = _helix.StatusPoller(_workspace, cp_rank, cp_size)
        _poller_key = _workspace_key
    return _poller.poll(raise_on_error=raise_on_error)


def _mnnvl_setting():
    v = _env.use_mnnvl()
    return False if v == "0" else True if v == "1" else "auto"


def _init_workspace(cp_rank: int, cp_size: int, cp_group, device: torch.device):
    """Collective over the DCP group: allocate, initialise, barrier.  Never inside graph capture."""
    global _workspace, _workspace_key
    cpu_group = getattr(cp_group, "cpu_group", None)
    if device.type == "cpu":
        ws = _helix.allocate_workspace(cp_size, cp_rank, device="cpu", cpu_group=cpu_group)
    else:
        mnnvl = _mnnvl_setting()
        if mnnvl is False and cp_size > 1:
            logger.warning("HELIX_A2A_USE_MNNVL=0 gives every process private rows; peers cannot be reached")
        ws = _helix.allocate_workspace(cp_size, cp_rank, mnnvl=True if mnnvl == "auto" else mnnvl, cpu_group=cpu_group)
        _helix.init_workspace(ws, cp_rank, cp_size)
    if cpu_group is not None:
        dist.barrier(cpu_group)
    else:
        dist.barrier(cp_group.device_group)
    _workspace, _workspace_key = ws, (cp_size, cp_rank, str(device))
    logger.info("helix workspace ready: rank %d / %d, %s", cp_rank, cp_size, getattr(ws, "_helix_kind", "?"))
    # one line on stderr as well: inside a serving engine this logger is usually not configured, and an
    # operator wants to see which exchange a worker really runs
    import sys
    print(f"helix_a2a_b200: DCP workspace ready (backend=native, cp_rank={cp_rank}, cp_size={cp_size}, "
          f"{getattr(ws, '_helix_kind', 'device')} rows, {ws.shape[1] * 8 >> 20} MiB per rank)", file=sys.stderr, flush=True)
    return ws


def _get_workspace(cp_rank: int, cp_size: int, cp_group, device: torch.device):
    if _workspace is not None and _workspace_key == (cp_size, cp_rank, str(device)):
        return _workspace
    if device.type == "cuda" and torch.cuda.is_current_stream_capturing():
        raise RuntimeError(
            "the helix workspace is not initialised and cannot be initialised inside CUDA graph capture "
            "(allocation exchanges handles over the DCP group); call dcp_a2a_ensure_initialized(cp_group) "
            "before capture, e.g. during model warm-up")
    return _init_workspace(cp_rank, cp_size, cp_group, device)


def dcp_a2a_ensure_initialized(cp_group, device: Optional[torch.device] = None) -> None:
    """Pre-initialise the workspace for the native backend (no-op otherwise / when already done)."""
    if _HELIX_BACKEND != "native" or cp_group.world_size == 1:
        return
    dev = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    _get_workspace(cp_group.rank_in_group, cp_group.world_size, cp_group, torch.device(dev))


def _nccl_reduce(cp_attn_out, cp_attn_lse, cp_group, return_lse, is_lse_base_on_e):
    """Stock path: two all_to_all_single + combine (``patches/dcp_alltoall_helix.py:455-504``)."""
    N = cp_group.world_size
    B, H, D = cp_attn_out.shape
    Hl = H // N
    so = cp_attn_out.contiguous().view(B, N, Hl, D).permute(1, 0, 2, 3).contiguous()
    sl = cp_attn_lse.contiguous().view(B, N, Hl).permute(1, 0, 2).contiguous()
    ro, rl = torch.empty_like(so), torch.empty_like(sl)
    w1 = dist.all_to_all_single(ro.view(-1), so.view(-1), group=cp_group.device_group, async_op=True)
    w2 = dist.all_to_all_single(rl.view(-1), sl.view(-1), group=cp_group.device_group, async_op=True)
    w1.wait()
    w2.wait()
    return dcp_lse_combine(ro, rl, return_lse=return_lse, is_lse_base_on_e=is_lse_base_on_e)


def dcp_a2a_lse_reduce(cp_attn_out: torch.Tensor, cp_attn_lse: torch.Tensor, cp_group, ctx=None,
                       return_lse: bool = False, is_lse_base_on_e: bool = True):
    """Combine partial attention outputs across DCP ranks; returns the head-scattered ``[B, H/N, D]``."""
    world = cp_group.world_size
    if world == 1:
        return (cp_attn_out, cp_attn_lse) if return_lse else cp_attn_out
    if _HELIX_BACKEND == "native":
        rank = cp_group.rank_in_group
        ws = _get_workspace(rank, world, cp_group, cp_attn_out.device)
        lse = cp_attn_lse if cp_attn_lse.dtype == torch.float32 else cp_attn_lse.float()
        return _helix.alltoall_combine(cp_attn_out.contiguous(), lse.contiguous(), ws, rank, world,
                                       return_lse=return_lse, base2=not is_lse_base_on_e,
                                       timeout_ms=_HOOK_TIMEOUT_MS)
    if _stock_reduce is not None and _NCCL_IMPL == "stock":
        return _stock_reduce(cp_attn_out, cp_attn_lse, cp_group, ctx, return_lse, is_lse_base_on_e)
    return _nccl_reduce(cp_attn_out, cp_attn_lse, cp_group, return_lse, is_lse_base_on_e)


_PATCH_TARGETS = (
    "vllm.v1.attention.ops.dcp_alltoall",
    "vllm.v1.attention.backends.flash_attn",
    "vllm.v1.attention.backends.flashinfer",
    "vllm.model_executor.layers.attention.mla_attention",
)


def apply_runtime_patch() -> list:
    """Replace ``dcp_a2a_lse_reduce`` in the vLLM modules that bound it at import; returns their names."""
    global _stock_reduce
    import importlib
    patched = []
    for name in _PATCH_TARGETS:
        try:
            mod = importlib.import_module(name)
        except Exception:  # noqa: BLE001  (module absent in this vLLM build)
            continue
        fn = getattr(mod, "dcp_a2a_lse_reduce", None)
        if fn is None or fn is dcp_a2a_lse_reduce:
            continue
        if _stock_reduce is None and name.endswith("dcp_alltoall"):
            _stock_reduce = fn
        setattr(mod, "dcp_a2a_lse_reduce", dcp_a2a_lse_reduce)
        patched.append(name)
    return patched
