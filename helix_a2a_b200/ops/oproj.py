"""o_proj for decode: ``y[tokens, hidden] = x[tokens, K] @ w[hidden, K]^T``.

CUDA tensors run the tcgen05 / TMEM kernel (``csrc/oproj_gemm.cu``); CPU tensors use a plain
matmul.  In the reference this is vLLM's cuBLAS linear layer.
"""
from __future__ import annotations

import torch


def oproj(x: torch.Tensor, w: torch.Tensor, *, splits: int = 0) -> torch.Tensor:
    """``x [tokens, K]`` bf16, ``w [hidden, K]`` bf16 (``nn.Linear`` weight layout) -> bf16 ``[tokens, hidden]``.

    ``splits``: 0 lets the library pick (stream-K over all SMs when the plain grid would leave
    some idle), -1 forces the stream-K kernel, ``n >= 1`` forces the plain kernel with ``n`` K splits.
    """
    if not x.is_cuda:
        return (x.float() @ w.float().t()).to(x.dtype)
    from ._ext import ops
    return ops().oproj(x, w, splits)


def check_compute_status(like: torch.Tensor) -> None:
    """Raise if an attention / GEMM kernel gave up on a bounded wait since the last check."""
    from ._ext import ops
    code = int(ops().read_error_flag(like))
    if code != 0:
        ops().clear_error_flag(like)
        raise RuntimeError(f"helix compute kernel reported status {code} (a bounded wait ran out)")
