"""Environment knobs of the library, all under the ``HELIX_A2A_`` prefix.

The first four keep the names and meanings the reference uses
(``csrc/helix_alltoall.cu:541-548``, ``csrc/torch_binding.cpp:25-32``,
``helix_a2a/mnnvl.py:577-607``, ``patches/dcp_alltoall_helix.py:40``); the rest are new.  Unlike the
reference, values are read on every call (cheap) so tests can flip them without re-importing.

The functions below are the knobs that Python code reads; every Python reader goes through them.
``EXTENSION_KNOBS`` lists the ones the native extension reads itself with ``getenv`` (on every call of
the op concerned); they are here so that one place names every knob.
"""
from __future__ import annotations

import os

_TRUE = ("1", "true", "yes", "on")
_FALSE = ("0", "false", "no", "off")

#: knob -> (default, meaning); read by the C++ bindings (``csrc/binding.cpp``, ``csrc/binding_ops.cpp``)
EXTENSION_KNOBS = {
    "HELIX_A2A_ENABLE_PDL": ("0", "1: every kernel is launched with programmatic stream serialization"),
    "HELIX_A2A_CHANNEL_COUNT": ("0", "0 / unset: the auto-tuner picks the exchange's channel count; n: exactly n"),
    "HELIX_A2A_TIMEOUT_MS": ("2000", "time limit of every device-side wait of a call that does not pass its own"),
    "HELIX_A2A_DEBUG": ("0", "1: exchange outputs are pre-filled with NaN so that an unwritten row shows"),
    "HELIX_A2A_BULK_LINES": ("24", "lines per channel and call from which the exchange gives more of a CTA's warps to receiving"),
    "HELIX_A2A_BULK_SEND_WARPS": ("4 / 6", "sender warps per CTA for such calls (two ranks / more ranks)"),
    "HELIX_A2A_OPROJ_STREAMK": ("unset", "1 / 0: force / forbid the stream-K o_proj kernel where the library would choose"),
    "HELIX_A2A_OPROJ_TRACE": ("0", "1: the stream-K o_proj kernel records %globaltimer stamps per CTA"),
    "HELIX_A2A_EXCHANGE_TRACE": ("0", "1: the exchange kernel records per-channel %globaltimer stamps (api.exchange_trace)"),
    "HELIX_A2A_ATTN_TRACE": ("0", "1: the GQA decode kernel records per-CTA %globaltimer stamps, SM id and chunk counts"),
    "HELIX_A2A_ATTN_DYN_PCT": ("unset", "percent of every long (sequence, kv head) pair handed out dynamically; 0: fixed shares"),
    "HELIX_A2A_ATTN_DYN_CHUNK": ("unset", "blocks of 16 tokens per dynamically drawn chunk"),
    "HELIX_A2A_ATTN_DYN_MIN_BLOCKS": ("unset", "only (sequence, kv head) pairs with at least this many 16-token blocks get a pool (default 64)"),
    "HELIX_A2A_MLA_VARIANT": ("ws", "ws: producer + math warps; lockstep: all warps walk a tile's phases together"),
    "HELIX_A2A_MLA_PROF": ("0", "1: the lockstep MLA kernel sums clock64 per phase of its tile loop"),
}


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


def hook_timeout_ms() -> int:
    """``HELIX_A2A_HOOK_TIMEOUT_MS``: time limit of the waits of calls made through the vLLM hook (default 30 s:
    ranks of a serving engine can be far apart during warm-up)."""
    try:
        return max(int(os.environ.get("HELIX_A2A_HOOK_TIMEOUT_MS", "30000")), 1)
    except ValueError:
        return 30000


def oproj_library() -> bool:
    """``HELIX_A2A_OPROJ_LIBRARY=0``: ``ops.oproj`` never hands a large-token product to cuBLAS
    (``torch.nn.functional.linear``); default: it does above the measured crossover."""
    return os.environ.get("HELIX_A2A_OPROJ_LIBRARY", "1").strip() != "0"


def hook_check_mode() -> str:
    """``HELIX_A2A_HOOK_CHECK``: how the import hook watches the exchange's status after every engine step:
    ``poll`` (default, any other value) = without waiting for the GPU, a failure is seen one or two steps late;
    ``sync`` = read with a synchronisation every step; ``off`` (``0``) = not at all."""
    v = os.environ.get("HELIX_A2A_HOOK_CHECK", "1").strip().lower()
    return "off" if v in ("0", "off") else "sync" if v == "sync" else "poll"


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
    """``HELIX_A2A_DEBUG=1``: NaN-poisoned outputs plus a check that every row was written."""
    return os.environ.get("HELIX_A2A_DEBUG", "0").strip() in _TRUE


def nccl_impl() -> str:
    """``HELIX_A2A_NCCL_IMPL``: what ``HELIX_A2A_BACKEND=nccl`` runs inside the vLLM hook - ``own``
    (default: two ``all_to_all_single`` + the combine kernel) or ``stock`` (the replaced vLLM function)."""
    return os.environ.get("HELIX_A2A_NCCL_IMPL", "own").strip().lower()


def nvtx() -> bool:
    """``HELIX_A2A_NVTX=1``: NVTX ranges around the Python-level ops (``utils/tracing.py``)."""
    return os.environ.get("HELIX_A2A_NVTX", "0").strip() == "1"


def oproj_prepack() -> bool:
    """``HELIX_A2A_OPROJ_PREPACK=0``: the model stacks keep the plain ``[hidden, K]`` o_proj weights instead of
    packing them once into the tile-major, pre-swizzled layout (``ops.oproj.prepack_weight``)."""
    return os.environ.get("HELIX_A2A_OPROJ_PREPACK", "1").strip() != "0"
