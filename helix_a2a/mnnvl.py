"""Names of the reference's allocator module (``helix_a2a/mnnvl.py:72,549,615``) on top of the C++ VMM allocator."""
from helix_a2a_b200.parallel.workspace import (  # noqa: F401
    allocate_vmm_workspace,
    should_use_mnnvl,
    VmmWorkspaceHandle as HelixMnnvlHandle,
)


def is_cuda_driver_available() -> bool:
    """The driver API is reached through the CUDA runtime, so it is available whenever the extension is."""
    from helix_a2a_b200.ops._ext import available
    return available()


def allocate_mnnvl_workspace(cp_size, cp_rank, cpu_group, mnnvl=True):
    import helix_a2a_b200 as h
    return h.allocate_workspace(cp_size, cp_rank, mnnvl=mnnvl, cpu_group=cpu_group)
