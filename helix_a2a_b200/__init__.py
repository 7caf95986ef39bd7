"""helix_a2a_b200 — Blackwell-native (B200, sm_100a) Helix context-parallel decode library.

Public API (same four calls as the reference's ``helix_a2a/__init__.py:23-121`` plus the
fused paths)::

    workspace_size(cp_size) -> int
    allocate_workspace(cp_size, cp_rank, device="cuda", *, mnnvl=False, cpu_group=None) -> Tensor
    init_workspace(workspace, cp_rank, cp_size) -> None
    alltoall(partial_o, softmax_stats, workspace, cp_rank, cp_size) -> (Tensor, Tensor)
    alltoall_combine(attn_out, lse, workspace, cp_rank, cp_size, ...) -> Tensor
    lse_combine(outputs, lses, ...) -> Tensor                 # stand-alone combine kernel
    check_status / reset_workspace / debug_info
"""
from ._version import __version__
from .api import (
    HelixTimeoutError,
    alltoall,
    alltoall_combine,
    alltoall_combine_oproj,
    alltoall_combine_oproj_fits,
    allocate_workspace,
    check_status,
    StatusPoller,
    debug_info,
    exchange_trace,
    init_workspace,
    init_workspace_all_rows,
    lse_combine,
    reset_workspace,
    workspace_size,
)

__all__ = [
    "workspace_size",
    "allocate_workspace",
    "init_workspace",
    "alltoall",
    "alltoall_combine",
    "alltoall_combine_oproj",
    "alltoall_combine_oproj_fits",
    "lse_combine",
    "check_status",
    "StatusPoller",
    "reset_workspace",
    "debug_info",
    "exchange_trace",
    "init_workspace_all_rows",
    "HelixTimeoutError",
    "__version__",
]
