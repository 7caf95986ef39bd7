"""vLLM decode-context-parallel (DCP) integration of the Helix exchange."""
from .dcp_alltoall_helix import (  # noqa: F401
    dcp_a2a_ensure_initialized,
    dcp_a2a_lse_reduce,
    _lse_weighted_combine,
    apply_runtime_patch,
)
