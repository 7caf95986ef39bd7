"""Environment knobs of the library, all under the ``HELIX_A2A_`` prefix.

The first four keep the names and meanings the reference uses
(``csrc/helix_alltoall.cu:541-548``, ``csrc/torch_binding.cpp:25-32``,
``helix_a2a/mnnvl.py:577-607``, ``patches/dcp_alltoall_helix.py:40``); the rest
are new.  Unlike the reference, values are read on every call (cheap) so tests
can flip them without re-importing.
"""
from __future__ import annotations

import os

_TRUE = ("1", "true", "yes", "on")
_FALSE = ("0", "false", "no", "off")


def enable_pdl() -> bool:
    """``HELIX_A2A_ENABLE_PDL=1``: launch with programmatic stream serialization."""
    return os.environ.get("HELIX_A2A_ENABLE_PDL", "0").strip() == "1"


def channel_count() -> int:
    """``HELIX_A2A_CHANNEL_COUNT``: 0 / unset = auto-tune, else a fixed channel count."""
    v = os.environ.get("HELIX_A2A_CHANNEL_COUNT", "0").strip()
    try:
        return max(int(v), 0)
    except ValueError:
        return 0


def use_mnnvl() -> str:
    """``HELIX_A2A_USE_MNNVL``: ``"0"`` device memory, ``"1"`` peer-mapped VMM, ``"auto"``."""
    v = os.environ.get("HELIX_A2A_USE_MNNVL", "auto").strip().lower()
    if v in _FALSE:
        return "0"
    if v in _TRUE:
        return "1"
    return "auto"


def backend() -> str:
    """``HELIX_A2A_BACKEND``: ``nccl`` (default) or ``native`` for the vLLM hook."""
    return os.environ.get("HELIX_A2A_BACKEND", "nccl").strip().lower()


def timeout_ms() -> int:
    """``HELIX_A2A_TIMEOUT_MS``: time limit of every device-side wait (default 2000 ms)."""
    try:
        return max(int(os.environ.get("HELIX_A2A_TIMEOUT_MS", "2000")), 1)
    except ValueError:
        return 2000


def handle_transport() -> str:
    """``HELIX_A2A_HANDLE_TRANSPORT``: ``auto`` | ``pidfd`` | ``scm`` | ``fabric`` - how the VMM handles of the
    workspace rows travel between ranks (POSIX fd duplicated with ``pidfd_getfd``, POSIX fd sent over a Unix
    socket, or fabric handles).  There is no cudaIpc transport: rows must sit at ``base + rank * stride`` and an
    IPC mapping lands wherever the driver puts it."""
    v = os.environ.get("HELIX_A2A_HANDLE_TRANSPORT", "auto").strip().lower()
    if v not in ("auto", "pidfd", "scm", "fabric"):
        raise ValueError(f"HELIX_A2A_HANDLE_TRANSPORT={v!r}: expected auto, pidfd, scm or fabric")
    return v


def debug() -> bool:
    return os.environ.get("HELIX_A2A_DEBUG", "0").strip() in _TRUE


def oproj_streamk() -> str:
    """``HELIX_A2A_OPROJ_STREAMK``: ``1`` / ``0`` forces / forbids the stream-K o_proj kernel for calls
    that leave the choice to the library; unset = the library's heuristic.  Read by the extension."""
    return os.environ.get("HELIX_A2A_OPROJ_STREAMK", "auto").strip().lower()


def oproj_trace() -> bool:
    """``HELIX_A2A_OPROJ_TRACE=1``: the stream-K o_proj kernel records ``%globaltimer`` stamps per CTA."""
    return os.environ.get("HELIX_A2A_OPROJ_TRACE", "0").strip() == "1"


def nccl_impl() -> str:
    """``HELIX_A2A_NCCL_IMPL``: what ``HELIX_A2A_BACKEND=nccl`` runs inside the vLLM hook - ``own``
    (default: two ``all_to_all_single`` + torch combine) or ``stock`` (the replaced vLLM function)."""
    return os.environ.get("HELIX_A2A_NCCL_IMPL", "own").strip().lower()


def vllm_hook_enabled() -> bool:
    """``HELIX_A2A_VLLM_HOOK=0`` keeps the start-up shim (``vllm_patch/autoload``) from installing the import hook."""
    return os.environ.get("HELIX_A2A_VLLM_HOOK", "1").strip() != "0"


def mla_variant() -> str:
    """``HELIX_A2A_MLA_VARIANT``: ``ws`` (default: producer warps + math warps) or ``lockstep`` (all warps
    walk the phases of a tile together; the only one with the ``HELIX_A2A_MLA_PROF=1`` cycle profile)."""
    return os.environ.get("HELIX_A2A_MLA_VARIANT", "ws").strip().lower()


def attn_trace() -> bool:
    """``HELIX_A2A_ATTN_TRACE=1``: the GQA decode attention kernel records four ``%globaltimer`` stamps per
    CTA (entry, first data, end of streaming, exit; the SM id rides in the low byte of the second)."""
    return os.environ.get("HELIX_A2A_ATTN_TRACE", "0").strip() == "1"


def mla_prof() -> bool:
    """``HELIX_A2A_MLA_PROF=1``: the lockstep MLA kernel sums ``clock64`` per phase of its tile loop
    (read back with ``ops().attn_trace``)."""
    return os.environ.get("HELIX_A2A_MLA_PROF", "0").strip() == "1"


def nvtx() -> bool:
    """``HELIX_A2A_NVTX=1``: NVTX ranges around the Python-level ops (``utils/tracing.py``)."""
    return os.environ.get("HELIX_A2A_NVTX", "0").strip() == "1"


def oproj_prepack() -> bool:
    """``HELIX_A2A_OPROJ_PREPACK=0``: the model stacks keep the plain ``[hidden, K]`` o_proj weights instead of
    packing them once into the tile-major, pre-swizzled layout (``ops.oproj.prepack_weight``)."""
    return os.environ.get("HELIX_A2A_OPROJ_PREPACK", "1").strip() != "0"
