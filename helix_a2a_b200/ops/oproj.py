"""o_proj for decode: ``y[tokens, hidden] = x[tokens, K] @ w[hidden, K]^T``.

CUDA tensors run the tcgen05 / TMEM kernel (``csrc/oproj_gemm.cu``); CPU tensors use a plain
matmul.  In the reference this is vLLM's cuBLAS linear layer.
"""
from __future__ import annotations

from typing import Optional

import torch


def oproj(x: torch.Tensor, w, *, splits: int = 0, library: Optional[bool] = None) -> torch.Tensor:
    """``x [tokens, K]`` bf16, ``w [hidden, K]`` bf16 (``nn.Linear`` weight layout) -> bf16 ``[tokens, hidden]``.

    ``splits``: 0 lets the library pick (stream-K over all SMs when the plain grid would leave
    some idle), -1 forces the stream-K kernel, ``n >= 1`` forces the plain kernel with ``n`` K splits.

    The hand-written kernel is built for decode: few tokens, bound by streaming W once (swap-AB, one 128-row slab
    of W per CTA, every CTA reads all of x).  With many tokens the product is compute-bound and every slab's CTA
    re-reads x, and cuBLAS is faster (measured on B200 inside CUDA graphs, hidden 8192: level up to 8 tokens, 10-40 %
    ahead at 32-64 tokens, 2x at 128).  So with ``splits=0`` and a plain weight matrix calls of 32 tokens or more go to
    ``torch.nn.functional.linear``; ``library=False`` (or ``HELIX_A2A_OPROJ_LIBRARY=0``) keeps the hand-written
    kernel for every size.  Packed weights always use the hand-written kernel (the plain matrix is not kept).
    """
    if isinstance(w, PackedOprojWeight):
        if not x.is_cuda:
            return (x.float() @ unpack_weight(w).float().t()).to(x.dtype)
        from ._ext import ops
        return ops().oproj_packed(x, w.packed, w.hidden, w.K, max(splits, 0))
    if not x.is_cuda:
        return (x.float() @ w.float().t()).to(x.dtype)
    if splits == 0 and library is not False and library_gemm_pays(x.shape[0], w.shape[1]):
        return torch.nn.functional.linear(x, w)
    from ._ext import ops
    return ops().oproj(x, w, splits)


def library_gemm_pays(tokens: int, K: int) -> bool:
    """The measured crossover between the decode kernel and cuBLAS (see :func:`oproj`)."""
    from ..utils import env as _env
    if not _env.oproj_library():
        return False
    del K          # the crossover does not depend on it: 32 tokens at K = 1024 ... 8192
    return tokens >= 32


class PackedOprojWeight:
    """A ``[hidden, K]`` bf16 weight re-laid for the o_proj kernel: per 128-row slab, ``K / 64`` atoms
    (padded with zeros to a multiple of 4) of ``128 rows x 128 bytes``, each atom stored exactly as the
    tensor core reads it from shared memory (16-byte chunk ``c`` of row ``r`` sits at chunk ``c ^ (r & 7)``).
    One pipeline stage of the kernel is then a single contiguous bulk copy instead of several strided
    tensor copies that open a DRAM page for 128 bytes at a time.  Weights are static, so this is done once."""

    def __init__(self, packed: torch.Tensor, hidden: int, K: int):
        self.packed, self.hidden, self.K = packed, hidden, K

    @property
    def shape(self):
        return (self.hidden, self.K)


def packed_atoms(K: int) -> int:
    return ((K + 63) // 64 + 3) // 4 * 4


def prepack_weight(w: torch.Tensor) -> PackedOprojWeight:
    """``w [hidden, K]`` bf16 (any row stride, e.g. a CP rank's column slice of W_o) -> ``PackedOprojWeight``."""
    hidden, K = w.shape
    if hidden % 128 or K % 64 or w.dtype != torch.bfloat16:
        raise ValueError("prepack_weight needs a bfloat16 [hidden % 128 == 0, K % 64 == 0] matrix")
    na = packed_atoms(K)
    wp = torch.zeros(hidden, na * 64, dtype=w.dtype, device=w.device)
    wp[:, :K] = w
    # [slab, row, atom, chunk, 8 elements] -> [slab, atom, row, chunk', 8] with chunk' = chunk ^ (row & 7)
    t = wp.view(hidden // 128, 128, na, 8, 8).permute(0, 2, 1, 3, 4).contiguous()
    r = torch.arange(128, device=w.device).view(1, 1, 128, 1, 1)
    c = torch.arange(8, device=w.device).view(1, 1, 1, 8, 1)
    src_chunk = (c ^ (r & 7)).expand(t.shape[0], na, 128, 8, 8)      # position c' holds source chunk c' ^ (r & 7)
    t = torch.gather(t, 3, src_chunk.contiguous())
    return PackedOprojWeight(t.contiguous().view(torch.uint8).reshape(-1), hidden, K)


def unpack_weight(pw: PackedOprojWeight) -> torch.Tensor:
    """Inverse of ``prepack_weight`` (tests, debugging)."""
    na = packed_atoms(pw.K)
    t = pw.packed.view(torch.bfloat16).view(pw.hidden // 128, na, 128, 8, 8)
    r = torch.arange(128, device=t.device).view(1, 1, 128, 1, 1)
    c = torch.arange(8, device=t.device).view(1, 1, 1, 8, 1)
    t = torch.gather(t, 3, (c ^ (r & 7)).expand_as(t).contiguous())   # the swizzle is its own inverse
    return t.permute(0, 2, 1, 3, 4).reshape(pw.hidden, na * 64)[:, :pw.K].contiguous()


def check_compute_status(like: torch.Tensor) -> None:
    """Raise if an attention / GEMM kernel gave up on a bounded wait since the last check."""
    from ._ext import ops
    code = int(ops().read_error_flag(like))
    if code != 0:
        ops().clear_error_flag(like)
        raise RuntimeError(f"helix compute kernel reported status {code} (a bounded wait ran out)")
