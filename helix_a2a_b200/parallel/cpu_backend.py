"""CPU implementation of the exchange and the fused exchange+combine over ``torch.distributed``.

Works on CPU tensors with a gloo process group (and on any device with any backend that has
``all_to_all_single``).  It is the oracle for the CUDA kernels, the backend of the CPU
correctness configuration (world size 2, fp32, 1e-5 against single-device attention) and the
host-side fault-injection target.  The reference has no CPU path at all; its only oracle is
NCCL ``all_to_all_single`` on GPUs (``tests/test_alltoall.py:274-297``).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import reference_math as rm


def _a2a(t: torch.Tensor, group) -> torch.Tensor:
    """``t [N, ...]``: chunk j goes to rank j; returns ``[N, ...]`` with chunk i from rank i."""
    out = torch.empty_like(t)
    dist.all_to_all_single(out.view(-1), t.contiguous().view(-1), group=group)
    return out


def alltoall(partial_o: torch.Tensor, softmax_stats: torch.Tensor, group, cp_size: int
             ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Reference contract: ``recv[..., p, :]`` is what rank p had at ``[..., me, :]``."""
    if partial_o.shape[-2] != cp_size or softmax_stats.shape[-2] != cp_size:
        raise RuntimeError("second-to-last dimension must equal cp_size")
    if partial_o.shape[:-2] != softmax_stats.shape[:-2]:
        raise RuntimeError("partial_o and softmax_stats must have matching dimensions except last two")
    if cp_size == 1:
        return partial_o.clone(), softmax_stats.clone()
    D, S = partial_o.shape[-1], softmax_stats.shape[-1]
    o = partial_o.reshape(-1, cp_size, D).transpose(0, 1).contiguous()
    s = softmax_stats.reshape(-1, cp_size, S).transpose(0, 1).contiguous()
    ro = _a2a(o, group).transpose(0, 1).contiguous().view(partial_o.shape)
    rs = _a2a(s, group).transpose(0, 1).contiguous().view(softmax_stats.shape)
    return ro, rs


def alltoall_combine(attn_out: torch.Tensor, lse: torch.Tensor, group, cp_size: int, *,
                     return_lse: bool = False, base2: bool = False, stats_mode: str = "lse",
                     out_dtype: Optional[torch.dtype] = None):
    """``attn_out [B,H,D]``, ``lse [B,H]`` (or stats ``[B,H,2]``) -> ``[B,H/N,D]`` combined.

    Heads ``[j*H/N, (j+1)*H/N)`` go to rank j; the combine is the fp32 oracle.
    """
    B, H, D = attn_out.shape
    if lse.dim() == 3:
        lse = rm.stats_to_lse(lse, stats_mode, base2)
    N = cp_size
    if H % N:
        raise RuntimeError("number of heads must be divisible by cp_size")
    Hl = H // N
    out_dtype = attn_out.dtype if out_dtype is None else out_dtype
    if N == 1:
        o, l = attn_out.unsqueeze(0), lse.unsqueeze(0)
    else:
        so = attn_out.view(B, N, Hl, D).permute(1, 0, 2, 3).contiguous()
        sl = lse.float().view(B, N, Hl).permute(1, 0, 2).contiguous()
        o, l = _a2a(so, group), _a2a(sl, group)
    res = rm.lse_combine(o, l, return_lse=return_lse, base2=base2)
    if return_lse:
        return res[0].to(out_dtype), res[1]
    return res.to(out_dtype)
