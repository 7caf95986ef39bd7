"""Thin wrappers with the reference's names (``helix_a2a/_ops.py:16-37``)."""
from typing import Tuple

import torch

from helix_a2a_b200.ops._ext import ops as _ops


def get_workspace_size_per_rank(cp_size: int) -> int:
    return int(_ops().get_helix_workspace_size_per_rank(cp_size))


def initialize_workspace(workspace: torch.Tensor, cp_rank: int, cp_size: int) -> None:
    _ops().initialize_helix_workspace(workspace, cp_rank, cp_size)


def alltoall_native(partial_o, softmax_stats, workspace, cp_rank: int, cp_size: int) -> Tuple[torch.Tensor, torch.Tensor]:
    return _ops().alltoall_helix_native(partial_o, softmax_stats, workspace, cp_rank, cp_size)
