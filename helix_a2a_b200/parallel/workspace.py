"""Workspace allocation: policy, handle exchange over ``torch.distributed`` and the CPU stand-in.

The physical allocation, export / import and mapping are done by the C++ allocator
(``csrc/vmm_workspace.cpp``); this module only decides *which* kind of workspace to make
and moves the handle bytes between ranks.  It covers what the reference does in
``helix_a2a/mnnvl.py:549-678`` (``should_use_mnnvl`` policy, ``allocate_mnnvl_workspace``)
with three differences: POSIX-fd handles work on x86 without opt-in when a process group is
given, descriptors can travel over a Unix socket when ``pidfd_getfd`` is not permitted, and a
CPU (gloo) workspace exists so the whole API runs without a GPU.
"""
from __future__ import annotations

import logging
import os
import platform
import socket
import threading
import uuid
from typing import Any, List, Optional

import torch
import torch.distributed as dist

from ..utils import env

logger = logging.getLogger(__name__)

B200_SM_COUNT = 148


def _sm_count(device=None) -> int:
    if torch.cuda.is_available():
        return torch.cuda.get_device_properties(device if device is not None else torch.cuda.current_device()).multi_processor_count
    return B200_SM_COUNT


def ref_max_channels(cp_size: int, sm_count: Optional[int] = None) -> int:
    """``max(SMs / (2 * ceil(cp / 8)), 1)`` — the reference's channel bound (``csrc/helix_alltoall.cu:590-603``)."""
    sm = _sm_count() if sm_count is None else sm_count
    return max(sm // (((cp_size + 7) // 8) * 2), 1)


def workspace_bytes(cp_size: int, sm_count: Optional[int] = None) -> int:
    """Bytes per rank: ``512 KiB * cp * maxCh + 2 * 256 B * cp * maxCh`` (``csrc/helix_alltoall.cu:605-614``)."""
    if cp_size < 1:
        raise ValueError("cp_size must be >= 1")
    ch = ref_max_channels(cp_size, sm_count)
    return 512 * 1024 * cp_size * ch + 2 * 256 * cp_size * ch


def _allgather(obj: Any, group) -> List[Any]:
    out: List[Any] = [None] * dist.get_world_size(group=group)
    dist.all_gather_object(out, obj, group=group)
    return out


def is_multi_node(cpu_group) -> bool:
    return len(set(_allgather(socket.gethostname(), cpu_group))) > 1


def should_use_mnnvl(cpu_group, mnnvl_param="auto") -> bool:
    """Decide between a peer-mapped VMM workspace (True) and private device memory (False).

    ``mnnvl_param=True`` forces VMM.  ``"auto"`` follows ``HELIX_A2A_USE_MNNVL``
    (``0/false/no/off`` -> device memory, ``1/true/yes/on`` -> VMM); when that is unset too the
    answer is VMM whenever a process group with more than one rank is available, because on
    a single NVSwitch box POSIX-fd handles need nothing special and on aarch64 multi-node
    NVLink systems fabric handles are used.  (The reference enables "auto" only on aarch64,
    ``helix_a2a/mnnvl.py:589-607``.)
    """
    if mnnvl_param is True:
        return True
    if mnnvl_param is False:
        return False
    e = env.use_mnnvl()
    if e == "0":
        return False
    if e == "1":
        return True
    if cpu_group is None:
        return False
    if dist.get_world_size(group=cpu_group) < 2:
        return False
    if is_multi_node(cpu_group) and "aarch64" not in platform.machine().lower():
        logger.info("ranks span several x86 hosts: no NVLink between them, using device memory")
        return False
    return True


class VmmWorkspaceHandle:
    """The Python-side share of a VMM allocation.  The rows stay mapped until this handle is closed AND every
    tensor made from it is gone (the tensors' storages hold shares too); unmapping synchronises the device first.
    Peers may still be storing into this rank's row: barrier over the group before closing a workspace."""

    def __init__(self, handle: int, kind: str, transport: str):
        self._h = handle
        self.kind = kind
        self.transport = transport

    def close(self):
        if self._h:
            from ..ops._ext import ext
            try:
                ext().vmm_destroy(self._h)
            finally:
                self._h = 0

    def __del__(self):
        try:
            self.close()
        except Exception:  # interpreter shutdown
            pass


def _pick_kind(device_index: int, cpu_group) -> str:
    t = env.handle_transport()
    if t == "fabric":
        return "fabric"
    if t in ("pidfd", "scm"):
        return "posix_fd"
    from ..ops._ext import ext
    if is_multi_node(cpu_group) and ext().vmm_fabric_supported(device_index):
        return "fabric"
    return "posix_fd"


def allocate_vmm_workspace(cp_size: int, cp_rank: int, cpu_group, device: Optional[torch.device] = None) -> torch.Tensor:
    """Allocate one row per rank and map all rows into every process.

    Returns an int64 tensor ``[cp_size, elems]`` whose row ``r`` is rank ``r``'s physical
    memory (stride between rows is the mapped slot size, not ``elems``).  All ranks of
    ``cpu_group`` must call this together.
    """
    from ..ops._ext import ext
    C = ext()
    if cpu_group is None:
        raise ValueError("a peer-mapped workspace needs a process group (cpu_group=...) for the handle exchange")
    if dist.get_world_size(group=cpu_group) != cp_size:
        raise ValueError("cpu_group size must equal cp_size")
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    ws_bytes = workspace_bytes(cp_size, _sm_count(dev))
    sizes = _allgather(ws_bytes, cpu_group)
    if any(s != ws_bytes for s in sizes):
        raise RuntimeError(f"ranks disagree on the workspace size: {sizes}")

    kind = _pick_kind(dev.index, cpu_group)
    h = C.vmm_create(cp_size, cp_rank, dev.index, ws_bytes, 1 if kind == "fabric" else 0)
    transport = kind
    try:
        C.vmm_map_local(h)
        if kind == "fabric":
            blobs = _allgather(bytes(C.vmm_export_fabric(h)), cpu_group)
            for r, blob in enumerate(blobs):
                if r != cp_rank:
                    C.vmm_map_peer_fabric(h, r, blob)
        else:
            fd = C.vmm_export_fd(h)
            transport = env.handle_transport()
            if transport not in ("pidfd", "scm"):
                transport = "pidfd"
            fds: List[Optional[int]] = [None] * cp_size
            if transport == "pidfd":
                pairs = _allgather((os.getpid(), fd), cpu_group)
                try:
                    for r, (pid, rfd) in enumerate(pairs):
                        if r != cp_rank:
                            fds[r] = C.vmm_dup_fd_from_pid(pid, rfd)
                    ok = True
                except RuntimeError as e:
                    logger.warning("pidfd_getfd not usable (%s); passing descriptors over a Unix socket", e)
                    ok = False
                oks = _allgather(ok, cpu_group)
                if not all(oks):
                    for f in fds:
                        if f is not None:
                            C.close_fd(f)
                    fds = [None] * cp_size
                    transport = "scm"
            if transport == "scm":
                name = f"helix-a2a-{uuid.uuid4().hex}"
                names = _allgather(name, cpu_group)
                t = threading.Thread(target=C.vmm_send_fd_unix, args=(name, fd, cp_size - 1, 60000), daemon=True)
                t.start()
                for r in range(cp_size):
                    if r != cp_rank:
                        fds[r] = C.vmm_recv_fd_unix(names[r], 60000)
                t.join()
            for r in range(cp_size):
                if r != cp_rank:
                    C.vmm_map_peer_fd(h, r, fds[r])
                    C.close_fd(fds[r])
        dist.barrier(group=cpu_group)   # nobody unmaps / exits before every import is done
    except Exception:
        C.vmm_destroy(h)
        raise
    ws = C.vmm_tensor(h, dev.index)
    ws._helix_handle = VmmWorkspaceHandle(h, kind, transport)
    ws._helix_kind = f"vmm-{transport}"
    logger.info("rank %d: peer-mapped workspace %s stride=%d kind=%s", cp_rank, list(ws.shape), ws.stride(0), ws._helix_kind)
    return ws


def allocate_single_process_workspace(devices: List[int], cp_size: Optional[int] = None) -> List[torch.Tensor]:
    """One process driving several GPUs: rows of all devices mapped in one range.

    Returns one ``[cp, elems]`` view per device (same addresses, different ``device``).
    """
    from ..ops._ext import ext
    C = ext()
    cp = len(devices) if cp_size is None else cp_size
    ws_bytes = workspace_bytes(cp, _sm_count(devices[0]))
    h = C.vmm_create_single_process(list(devices), ws_bytes)
    handle = VmmWorkspaceHandle(h, "single_process", "none")
    views = []
    for d in devices:
        t = C.vmm_tensor(h, d)
        t._helix_handle = handle
        t._helix_kind = "vmm-single-process"
        views.append(t)
    return views


def allocate_device_workspace(cp_size: int, device="cuda") -> torch.Tensor:
    """Private device memory: all ``cp_size`` rows live in this process.

    Usable for cp=1, for input-validation tests and for single-GPU emulation where one
    launch plays every rank (the reference's ``mnnvl=False`` path, ``helix_a2a/__init__.py:75-79``).
    """
    elems = (workspace_bytes(cp_size, _sm_count(device if torch.device(device).index is not None else None)) + 7) // 8
    ws = torch.zeros(cp_size, elems, dtype=torch.long, device=device)
    ws._helix_kind = "device"
    return ws


class CpuWorkspace(torch.Tensor):
    """Stand-in workspace for the CPU (gloo) backend: carries the process group."""

    @staticmethod
    def make(cp_size: int, cp_rank: int, group) -> "CpuWorkspace":
        t = torch.zeros(cp_size, 8, dtype=torch.long).as_subclass(CpuWorkspace)
        t._helix_group = group
        t._helix_kind = "cpu-gloo"
        t._helix_rank = cp_rank
        return t
