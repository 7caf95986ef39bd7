"""Public API: the reference's four calls plus the fused B200 paths.

Reference surface (``helix_a2a/__init__.py:23-121``)::

    workspace_size(cp_size) -> int
    allocate_workspace(cp_size, cp_rank, device="cuda", *, mnnvl=False, cpu_group=None) -> Tensor
    init_workspace(workspace, cp_rank, cp_size) -> None
    alltoall(partial_o, softmax_stats, workspace, cp_rank, cp_size) -> (Tensor, Tensor)

Additions: :func:`alltoall_combine` (exchange with the LSE-weighted combine fused into the
receive side, taking the attention output in its native ``[B, H, D]`` layout),
:func:`check_status` / :func:`reset_workspace` (bounded waits report instead of hanging) and
:func:`debug_info`.
"""
from __future__ import annotations

import logging
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .ops import reference_math as rm
from .parallel import cpu_backend, workspace as ws_mod
from .parallel.workspace import CpuWorkspace
from .utils.tracing import check_written, nvtx_range

logger = logging.getLogger(__name__)

STATUS_NAMES = {
    0: "ok",
    1: "timeout: a receiver never saw a line's flag (peer did not send)",
    2: "timeout: a sender's ring never drained (peer's receiver is stuck or absent)",
    3: "timeout: receiver barrier",
    4: "timeout: fused o_proj never saw its activation tile",
    5: "timeout: TMA / MMA barrier",
    6: "bad argument",
}


class HelixTimeoutError(RuntimeError):
    """A device-side wait ran out of its time limit; the workspace must be reset before reuse."""

    def __init__(self, code: int, peer: int, channel: int, entry: int):
        self.code, self.peer, self.channel, self.entry = code, peer, channel, entry
        super().__init__(f"helix exchange failed: {STATUS_NAMES.get(code, code)} "
                         f"(peer={peer}, channel={channel}, entry={entry})")


def workspace_size(cp_size: int) -> int:
    """Workspace size **in bytes** per rank for a CP group of ``cp_size`` ranks.

    ``512 KiB * cp * maxCh + 2 * 256 B * cp * maxCh`` with ``maxCh = max(SMs / (2 ceil(cp/8)), 1)``;
    without a GPU the SM count of a B200 (148) is assumed.
    """
    if torch.cuda.is_available():
        from .ops._ext import ops
        return int(ops().get_helix_workspace_size_per_rank(cp_size))
    return ws_mod.workspace_bytes(cp_size)


def allocate_workspace(cp_size: int, cp_rank: int, device="cuda", *, mnnvl=False,
                       cpu_group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Allocate the ``[cp_size, elems]`` int64 workspace.

    ``mnnvl=False``: private device memory (every row in this process; enough for cp=1,
    validation tests and single-GPU emulation).  ``mnnvl=True`` / ``"auto"``: rows are
    created with CUDA VMM and mapped into every rank of ``cpu_group`` (policy in
    :func:`helix_a2a_b200.parallel.workspace.should_use_mnnvl`).  ``device="cpu"`` returns the
    stand-in used by the gloo backend.

    After allocation call :func:`init_workspace` and then a barrier over the group before the
    first exchange, exactly as with the reference (``helix_a2a/__init__.py:52-58``).
    """
    if torch.device(device).type == "cpu":
        return CpuWorkspace.make(cp_size, cp_rank, cpu_group)
    if mnnvl is True or (isinstance(mnnvl, str) and mnnvl == "auto"):
        if ws_mod.should_use_mnnvl(cpu_group, mnnvl):
            return ws_mod.allocate_vmm_workspace(cp_size, cp_rank, cpu_group,
                                                 None if str(device) == "cuda" else torch.device(device))
    return ws_mod.allocate_device_workspace(cp_size, device)


def init_workspace(workspace: torch.Tensor, cp_rank: int, cp_size: int) -> None:
    """Reset the local row: rings to all-ones, counters and status to zero.  Synchronous.

    All ranks must finish this before any rank exchanges: put a barrier after it.
    """
    if isinstance(workspace, CpuWorkspace):
        return
    from .ops._ext import ops
    ops().initialize_helix_workspace(workspace, cp_rank, cp_size)
    torch.cuda.current_stream(workspace.device).synchronize()


def init_workspace_all_rows(workspace: torch.Tensor, cp_size: int) -> None:
    """Single-process workspaces (emulation): reset every row."""
    for r in range(cp_size):
        init_workspace(workspace, r, cp_size)


def reset_workspace(workspace: torch.Tensor, cp_rank: int, cp_size: int,
                    group: Optional[dist.ProcessGroup] = None) -> None:
    """Recovery after a :class:`HelixTimeoutError`: re-initialise the local row, then barrier."""
    torch.cuda.synchronize(workspace.device) if workspace.is_cuda else None
    if group is not None:
        dist.barrier(group=group)   # nobody is still sending into a row that is being cleared
    init_workspace(workspace, cp_rank, cp_size)
    if group is not None:
        dist.barrier(group=group)


def alltoall(partial_o: torch.Tensor, softmax_stats: torch.Tensor, workspace: torch.Tensor,
             cp_rank: int, cp_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Helix all-to-all with the reference's contract.

    ``partial_o [..., cp_size, D]`` (fp16 / bf16), ``softmax_stats [..., cp_size, S]`` (fp32,
    S even); slice ``[..., j, :]`` goes to rank j.  Returns tensors of the same shapes where
    slice ``[..., p, :]`` came from rank p.
    """
    if isinstance(workspace, CpuWorkspace):
        return cpu_backend.alltoall(partial_o, softmax_stats, workspace._helix_group, cp_size)
    from .ops._ext import ops
    with nvtx_range("helix.alltoall"):
        ro, rs = ops().alltoall_helix_native(partial_o, softmax_stats, workspace, cp_rank, cp_size)
    check_written(ro, "alltoall output")
    return ro, rs


_STATS_MODES = {"lse": 0, "max_sumexp": 1}


def alltoall_combine(attn_out: torch.Tensor, lse: torch.Tensor, workspace: torch.Tensor,
                     cp_rank: int, cp_size: int, *, return_lse: bool = False, base2: bool = False,
                     stats_mode: str = "lse", layout: str = "native", timeout_ms: int = 0):
    """Exchange + LSE-weighted combine in one kernel.

    ``layout="native"``: ``attn_out [B, H, D]`` and ``lse [B, H]`` (or stats ``[B, H, 2]``) as an
    attention kernel produces them; heads ``[j*H/N, (j+1)*H/N)`` are combined on rank j and the
    result is ``[B, H/N, D]`` (+ global LSE ``[B, H/N]``).  ``layout="entries"``:
    ``partial_o [..., cp, D]`` / ``softmax_stats [..., cp, 2]`` in the reference's exchange
    layout; the result is ``[..., D]``.
    """
    if stats_mode not in _STATS_MODES:
        raise ValueError(f"stats_mode must be one of {list(_STATS_MODES)}")
    if isinstance(workspace, CpuWorkspace):
        if layout != "native":
            ro, rs = cpu_backend.alltoall(attn_out, lse, workspace._helix_group, cp_size)
            l = rm.stats_to_lse(rs, stats_mode, base2)              # [..., cp]
            shp, D = ro.shape[:-2], ro.shape[-1]
            res, g = rm.lse_combine(ro.movedim(-2, 0).reshape(cp_size, 1, -1, D),
                                    l.movedim(-1, 0).reshape(cp_size, 1, -1), return_lse=True, base2=base2)
            out = res.reshape(*shp, D).to(attn_out.dtype)
            return (out, g.reshape(*shp)) if return_lse else out
        return cpu_backend.alltoall_combine(attn_out, lse, workspace._helix_group, cp_size,
                                            return_lse=return_lse, base2=base2, stats_mode=stats_mode)
    if cp_size == 1 and layout == "native" and lse.dim() == 2:
        # nothing to exchange or combine
        return (attn_out, lse) if return_lse else attn_out
    from .ops._ext import ops
    with nvtx_range("helix.alltoall_combine"):
        out, glse = ops().alltoall_combine(attn_out, lse, workspace, cp_rank, cp_size,
                                           0 if layout == "native" else 1, return_lse, base2,
                                           _STATS_MODES[stats_mode], False, 0, timeout_ms)
    check_written(out, "alltoall_combine output")
    return (out, glse) if return_lse else out


def alltoall_combine_oproj(attn_out: torch.Tensor, lse: torch.Tensor, w_o, workspace: torch.Tensor,
                           cp_rank: int, cp_size: int, *, base2: bool = False, timeout_ms: int = 0) -> torch.Tensor:
    """Exchange + LSE combine + o_proj in one kernel launch.

    ``attn_out [B, H, D]`` (bf16), ``lse [B, H]`` (fp32), ``w_o [hidden, (H/N) * D]`` (this rank's K-slice of the
    o_proj weight, bf16, or its ``ops.oproj.PackedOprojWeight`` form) -> ``y [B, hidden]`` (this rank's partial
    sum).  GEMM CTAs request their weights first, then receive and combine the rows of their own heads straight
    into the tensor-core operand in shared memory; the combined activation never goes through global memory.
    On CPU tensors, or when the shape does not fit (more than 64 tokens, a head wider than 512 dims, more GEMM
    CTAs than SMs), the exchange and the GEMM run as two launches.
    """
    from .ops import oproj as _oproj
    B = attn_out.shape[0]
    if isinstance(workspace, CpuWorkspace) or not attn_out.is_cuda or cp_size == 1:
        x = alltoall_combine(attn_out, lse, workspace, cp_rank, cp_size, base2=base2) if cp_size > 1 else attn_out
        return _oproj.oproj(x.reshape(B, -1), w_o)
    from .ops._ext import ops
    try:
        if isinstance(w_o, _oproj.PackedOprojWeight):
            return ops().alltoall_combine_oproj_packed(attn_out, lse, w_o.packed, w_o.hidden, workspace, cp_rank, cp_size,
                                                       base2, timeout_ms)
        y, _ = ops().alltoall_combine_oproj(attn_out, lse, w_o, workspace, cp_rank, cp_size, base2, False, timeout_ms)
        return y
    except RuntimeError as e:
        if "does not fit" not in str(e):
            raise
        x = alltoall_combine(attn_out, lse, workspace, cp_rank, cp_size, base2=base2)
        return _oproj.oproj(x.reshape(B, -1), w_o)


def alltoall_combine_oproj_fits(tokens: int, heads_local: int, head_dim: int, hidden: int, cp_size: int) -> bool:
    """Would :func:`alltoall_combine_oproj` run as ONE kernel for these sizes on the current GPU?

    ``heads_local`` = heads this rank combines (H / cp), ``hidden`` = rows of its o_proj weight.  The rules are the
    launcher's (``csrc/fused_exchange_oproj.cu::fused_fits``): at most 64 tokens and 8 ranks, heads of at most 232
    dims, head groups of at most 512 K-columns, and ``hidden / 128 x groups`` GEMM CTAs resident at once beside at
    least one sender CTA.  False without the extension or a GPU.
    """
    from .ops import _ext
    if not torch.cuda.is_available() or not _ext.available():
        return False
    return bool(_ext.ext().fused_oproj_fits(int(tokens), int(heads_local), int(head_dim), int(hidden), int(cp_size)))


def lse_combine(outputs: torch.Tensor, lses: torch.Tensor, *, return_lse: bool = False, base2: bool = False,
                layout: str = "NBHD"):
    """LSE-weighted combine of per-rank partial attention outputs that are already on this rank.

    ``layout="NBHD"``: ``outputs [N, ..., D]`` with ``lses [N, ...]`` (what two NCCL all-to-alls leave);
    ``layout="BHND"``: ``outputs [..., N, D]`` with ``lses [..., N]`` (what :func:`alltoall` returns; pass
    ``recv_stats[..., 0]``).  Returns ``[..., D]`` in the input dtype, plus the global LSE with ``return_lse``.
    NaN and infinite LSEs count as "no contribution"; a row without any contribution is zero with LSE ``-inf``.

    On CUDA tensors this is one hand-written kernel (``csrc/lse_combine.cu``), the counterpart of the
    reference's Triton ``dcp_lse_combine_triton`` (``patches/dcp_alltoall_helix.py:210-384``); the fused
    :func:`alltoall_combine` does the same arithmetic while the rows arrive and needs no separate call.
    """
    if layout not in ("NBHD", "BHND"):
        raise ValueError("layout must be 'NBHD' or 'BHND'")
    if not outputs.is_cuda:
        o = outputs if layout == "NBHD" else outputs.movedim(-2, 0)
        l = lses if layout == "NBHD" else lses.movedim(-1, 0)
        res = rm.lse_combine(o, l, return_lse=return_lse, base2=base2)
        if return_lse:
            return res[0].to(outputs.dtype), res[1]
        return res.to(outputs.dtype)
    from .ops._ext import ops
    out, g = ops().lse_combine(outputs, lses.float(), 0 if layout == "NBHD" else -2, return_lse, base2)
    return (out, g) if return_lse else out


def check_status(workspace: torch.Tensor, cp_rank: int, cp_size: int, *, raise_on_error: bool = True) -> dict:
    """Read the status block of the local row (synchronises the current stream)."""
    if isinstance(workspace, CpuWorkspace):
        return {"code": 0, "name": "ok"}
    from .ops._ext import ops
    s = ops().read_status(workspace, cp_rank, cp_size).tolist()
    info = {"code": int(s[0]), "peer": int(s[1]), "channel": int(s[2]), "entry": int(s[3]),
            "name": STATUS_NAMES.get(int(s[0]), str(s[0]))}
    if raise_on_error and info["code"] != 0:
        raise HelixTimeoutError(info["code"], info["peer"], info["channel"], info["entry"])
    return info


class StatusPoller:
    """Watches the status block of the local row WITHOUT synchronising: every :meth:`poll` first looks at the copy
    the previous poll requested (if it has arrived in pinned host memory) and then requests a fresh one on the
    current stream (a 32-byte device-to-host copy and an event, no host wait).  A failure is therefore seen one or
    two polls late, which is the price of not stalling a serving engine once per step; :func:`check_status` is the
    blocking, immediate form.  Raises :class:`HelixTimeoutError` like it."""

    def __init__(self, workspace: torch.Tensor, cp_rank: int, cp_size: int):
        from .ops._ext import ext
        self._cpu = isinstance(workspace, CpuWorkspace) or not workspace.is_cuda
        if self._cpu:
            return
        off = int(ext().layout(int(cp_size), ws_mod._sm_count(workspace.device))["status_offset"])
        assert off % 8 == 0
        self._view = workspace[cp_rank, off // 8: off // 8 + 4]          # code, peer, channel, entry
        self._host = torch.zeros(4, dtype=torch.int64).pin_memory()
        self._event = torch.cuda.Event()
        self._pending = False

    def poll(self, raise_on_error: bool = True) -> Optional[dict]:
        """Returns the decoded status when a requested copy has arrived (None otherwise)."""
        if self._cpu:
            return {"code": 0, "name": "ok"}
        info = None
        if self._pending and self._event.query():
            self._pending = False
            s = self._host.tolist()
            info = {"code": int(s[0]), "peer": int(s[1]), "channel": int(s[2]), "entry": int(s[3]),
                    "name": STATUS_NAMES.get(int(s[0]), str(s[0]))}
            if raise_on_error and info["code"] != 0:
                raise HelixTimeoutError(info["code"], info["peer"], info["channel"], info["entry"])
        if not self._pending:
            self._host.copy_(self._view, non_blocking=True)
            self._event.record()
            self._pending = True
        return info


def exchange_trace(workspace: torch.Tensor) -> torch.Tensor:
    """Device timeline of the LAST exchange launch on the workspace's device (needs ``HELIX_A2A_EXCHANGE_TRACE=1`` set
    before the first call): an ``[n, 8]`` int64 tensor of ``%globaltimer`` stamps, one row per CTA (= channel) in
    launch order: kernel entry, after the wait on the previous kernel, first line posted, last line posted, first
    peer message complete, last peer message complete, exit, unused.  Rows of CTAs that were not launched are zero."""
    from .ops._ext import ops
    return ops().exchange_trace(workspace)


def debug_info(workspace: Optional[torch.Tensor] = None) -> dict:
    """Launch shape chosen by the auto-tuner for the last call, and the workspace kind."""
    from .ops._ext import ext
    info = dict(ext().last_launch_info())
    if workspace is not None:
        info["workspace_kind"] = getattr(workspace, "_helix_kind", "unknown")
        info["workspace_shape"] = list(workspace.shape)
        info["workspace_row_stride_bytes"] = workspace.stride(0) * 8
    return info
