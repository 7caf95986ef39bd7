"""Split-KV paged decode attention (per-rank partial output + LSE).

``gqa_decode`` runs the hand-written sm_100a kernel (``csrc/decode_attn_gqa.cu``); on CPU
tensors it falls back to the fp32 oracle so that the model code runs without a GPU.  In the
reference this step belongs to vLLM's attention backends
(``benchmark/sbatch/run_gb200_aiperf_v3.sbatch:95``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from . import reference_math as rm


def gqa_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
               seq_lens: torch.Tensor, *, scale: Optional[float] = None, lse_base2: bool = False,
               layout: str = "HND", splits: int = 0, max_seq_len: int = 0,
               kv_stable: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Decode attention of ``q [B, Hq, 128]`` over each sequence's local KV pages.

    ``k_cache`` / ``v_cache``: ``[pages, Hkv, page, 128]`` (``layout="HND"``) or
    ``[pages, page, Hkv, 128]`` (``"NHD"``), bf16.  ``block_table [B, max_pages]`` int32,
    ``seq_lens [B]`` int32 (tokens of the LOCAL shard).  Returns ``o [B, Hq, 128]`` (bf16,
    normalised) and ``lse [B, Hq]`` (fp32; natural log, or base 2 with ``lse_base2``).
    ``splits=0`` lets the library pick the number of KV splits from ``max_seq_len``.
    ``kv_stable=True`` is a promise about the kernel launched just before this one on the stream: it
    writes at most the newest token of each sequence (the cache append) and ``q``.  With
    ``HELIX_A2A_ENABLE_PDL=1`` the first K/V tiles are then fetched while that kernel is still draining.
    """
    scale = 1.0 / math.sqrt(q.shape[-1]) if scale is None else scale
    if not q.is_cuda:
        kc = k_cache if layout == "HND" else k_cache.permute(0, 2, 1, 3)
        vc = v_cache if layout == "HND" else v_cache.permute(0, 2, 1, 3)
        o, lse = rm.paged_decode_attention_reference(q, kc, vc, block_table, seq_lens, scale, lse_base2)
        return o.to(q.dtype), lse
    from ._ext import ops
    if max_seq_len <= 0:
        max_seq_len = block_table.shape[1] * (k_cache.shape[2] if layout == "HND" else k_cache.shape[1])
    return ops().gqa_decode(q, k_cache, v_cache, block_table, seq_lens, float(scale), lse_base2,
                            layout == "HND", splits, max_seq_len, kv_stable)


def mla_decode(q_nope: torch.Tensor, q_pe: torch.Tensor, ckv_fp8: torch.Tensor, scales: torch.Tensor,
               kpe: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor, *, scale: float,
               lse_base2: bool = False, ctas: int = 0, max_seq_len: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """MLA decode attention in the absorbed (latent) form over a block-scaled fp8 cache.

    ``q_nope [B, 128, 512]`` (already multiplied by W_uk) and ``q_pe [B, 128, 64]`` in bf16;
    ``ckv_fp8 [pages, page, 512]`` e4m3 with ``scales [pages, page, 4]`` (one fp32 per 128 latent
    values) and ``kpe [pages, page, 64]`` bf16 rope keys.  Scores are
    ``(q_nope . ckv + q_pe . kpe) * scale``, values are the dequantised latent.  Returns the
    normalised partial ``o [B, 128, 512]`` (bf16) and ``lse [B, 128]``: exactly what the exchange
    takes for the MLA shape.
    """
    if not q_nope.is_cuda:
        B = q_nope.shape[0]
        page = ckv_fp8.shape[1]
        lat = rm.dequantize_fp8_blockscaled(ckv_fp8, scales, 128)
        outs, lses = [], []
        for b in range(B):
            n = int(seq_lens[b])
            npg = (n + page - 1) // page
            idx = block_table[b, :npg].long()
            c = lat[idx].reshape(-1, 512)[:n]
            k = kpe[idx].reshape(-1, 64)[:n]
            o, l = rm.mla_partial_attention(q_nope[b:b + 1], q_pe[b:b + 1], c, k, scale, lse_base2)
            outs.append(o)
            lses.append(l)
        return torch.cat(outs).to(q_nope.dtype), torch.cat(lses)
    from ._ext import ops
    if max_seq_len <= 0:
        max_seq_len = block_table.shape[1] * ckv_fp8.shape[1]
    return ops().mla_decode(q_nope, q_pe, ckv_fp8, scales, kpe, block_table, seq_lens, float(scale), lse_base2,
                            ctas, max_seq_len)
