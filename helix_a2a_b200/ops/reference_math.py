"""Plain-PyTorch fp32 oracles for every op in the library.

These functions are the numerical ground truth for the CUDA kernels and the
CPU backend: full softmax attention, split-KV partial attention producing
``(o, lse)``, the LSE-weighted combine, paged-KV gather helpers, block-scaled
fp8 quantisation of an MLA latent cache and the o_proj matmul.

The combine follows the edge-case rules of the reference's torch combine
(``patches/dcp_alltoall_helix.py:142-207``): NaN / +-inf LSEs count as
``-inf``, an all ``-inf`` column uses max 0, NaN weights become 0 and the
weight sum is clamped at 1e-10.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

LOG2E = 1.4426950408889634
LN2 = 0.6931471805599453


def full_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                   scale: Optional[float] = None) -> torch.Tensor:
    """Decode attention of ``q [T, H, D]`` against ``k, v [S, Hkv, D(v)]`` (no mask).

    ``H`` must be a multiple of ``Hkv`` (GQA); returns ``[T, H, Dv]`` in fp32.
    """
    o, _ = partial_attention(q, k, v, scale)
    return o


def partial_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                      scale: Optional[float] = None,
                      base2: bool = False) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention over one KV shard: returns normalised ``o [T,H,Dv]`` and ``lse [T,H]``.

    ``lse`` is ``log(sum(exp(s)))`` (natural log) or, with ``base2``, the same
    quantity expressed in base 2 (``lse_e * log2(e)``).  An empty shard gives
    ``o = 0`` and ``lse = -inf``.
    """
    T, H, D = q.shape
    S, Hkv, _ = k.shape
    Dv = v.shape[-1]
    g = H // Hkv
    scale = (1.0 / math.sqrt(D)) if scale is None else scale
    qf = q.float().view(T, Hkv, g, D)
    kf = k.float()
    vf = v.float()
    if S == 0:
        return (torch.zeros(T, H, Dv, dtype=torch.float32, device=q.device),
                torch.full((T, H), float("-inf"), dtype=torch.float32, device=q.device))
    s = torch.einsum("thgd,shd->thgs", qf, kf) * scale
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.einsum("thgs,shd->thgd", p, vf).reshape(T, H, Dv)
    lse = lse.reshape(T, H)
    if base2:
        lse = lse * LOG2E
    return o, lse


def sanitize_lse(lses: torch.Tensor) -> torch.Tensor:
    """NaN and +-inf become -inf (a shard that contributes nothing)."""
    bad = torch.isnan(lses) | torch.isinf(lses)
    return torch.where(bad, torch.full_like(lses, float("-inf")), lses)


def lse_combine(outputs: torch.Tensor, lses: torch.Tensor, *,
                return_lse: bool = False, base2: bool = False):
    """Combine ``outputs [N,B,H,D]`` with ``lses [N,B,H]`` into ``[B,H,D]`` (fp32).

    ``out = sum_n w_n o_n / sum_n w_n`` with ``w_n = exp(lse_n - max_n lse_n)``.
    """
    out_f = outputs.float()
    l = sanitize_lse(lses.float())
    m, _ = l.max(dim=0)
    m = torch.where(m == float("-inf"), torch.zeros_like(m), m)
    d = l - m.unsqueeze(0)
    w = torch.pow(2.0, d) if base2 else torch.exp(d)
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    wsum = w.sum(dim=0, keepdim=True)
    wn = w / wsum.clamp(min=1e-10)
    res = (out_f * wn.unsqueeze(-1)).sum(dim=0)
    if return_lse:
        g = (torch.log2(wsum.squeeze(0)) if base2 else torch.log(wsum.squeeze(0))) + m
        return res, g
    return res


def stats_to_lse(stats: torch.Tensor, stats_mode: str = "lse", base2: bool = False) -> torch.Tensor:
    """Turn a ``[..., 2]`` softmax-stats pair into one LSE per entry.

    ``"lse"``: slot 0 already is the LSE (slot 1 is padding).
    ``"max_sumexp"``: slot 0 is the running max, slot 1 the sum of exponentials.
    """
    if stats_mode == "lse":
        return stats[..., 0]
    if stats_mode == "max_sumexp":
        s = stats[..., 1]
        return stats[..., 0] + (torch.log2(s) if base2 else torch.log(s))
    raise ValueError(f"unknown stats_mode {stats_mode!r}")


def alltoall_reference(send_o_all: torch.Tensor, send_s_all: torch.Tensor):
    """Exchange oracle on stacked per-rank tensors.

    ``send_o_all [N, E, N, D]``: rank r's ``partial_o`` is ``send_o_all[r]``; the
    result ``recv[r, e, p] = send[p, e, r]`` is what rank r receives.
    """
    return send_o_all.transpose(0, 2).contiguous(), send_s_all.transpose(0, 2).contiguous()


def head_scatter_combine_reference(outs: torch.Tensor, lses: torch.Tensor, *,
                                   return_lse: bool = False, base2: bool = False):
    """Oracle of the fused exchange+combine on stacked per-rank inputs.

    ``outs [N, B, H, D]``, ``lses [N, B, H]`` are every rank's split-KV partials.
    Rank r ends with heads ``[r*H/N, (r+1)*H/N)`` fully combined.  Returns
    ``[N, B, H/N, D]`` (index 0 = receiving rank) and optionally ``[N, B, H/N]``.
    """
    N, B, H, D = outs.shape
    Hl = H // N
    res, glse = lse_combine(outs, lses, return_lse=True, base2=base2)  # [B,H,D]
    res = res.view(B, N, Hl, D).permute(1, 0, 2, 3).contiguous()
    if return_lse:
        return res, glse.view(B, N, Hl).permute(1, 0, 2).contiguous()
    return res


def oproj_reference(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``y[B, hidden] = x[B, K] @ w[hidden, K]^T`` in fp32."""
    return x.float() @ w.float().t()


# ----------------------------------------------------------------------------------------
# paged KV helpers
# ----------------------------------------------------------------------------------------

def gather_paged_kv(cache: torch.Tensor, block_table: torch.Tensor, seq_len: int) -> torch.Tensor:
    """Gather ``seq_len`` tokens of one sequence from ``cache [pages, Hkv, page, D]``.

    Returns ``[seq_len, Hkv, D]``.  ``block_table`` is the 1-D list of page ids.
    """
    page = cache.shape[2]
    n_pages = (seq_len + page - 1) // page
    pages = cache[block_table[:n_pages].long()]              # [n, Hkv, page, D]
    toks = pages.permute(0, 2, 1, 3).reshape(n_pages * page, cache.shape[1], cache.shape[3])
    return toks[:seq_len]


def paged_decode_attention_reference(q, k_cache, v_cache, block_tables, seq_lens,
                                     scale=None, base2=False):
    """Split-KV decode oracle: ``q [B,H,D]`` against each sequence's local pages.

    Returns ``o [B,H,Dv]`` fp32 and ``lse [B,H]`` fp32.
    """
    B = q.shape[0]
    outs, lses = [], []
    for b in range(B):
        n = int(seq_lens[b])
        k = gather_paged_kv(k_cache, block_tables[b], n)
        v = gather_paged_kv(v_cache, block_tables[b], n)
        o, l = partial_attention(q[b:b + 1], k, v, scale, base2)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs, 0), torch.cat(lses, 0)


# ----------------------------------------------------------------------------------------
# MLA latent cache: block-scaled fp8 e4m3
# ----------------------------------------------------------------------------------------

FP8_E4M3_MAX = 448.0


def quantize_fp8_blockscaled(x: torch.Tensor, block: int = 128):
    """Quantise the last dim of ``x`` to e4m3 with one fp32 scale per ``block`` elements.

    The last dim is zero-padded up to a multiple of ``block`` for the scale
    computation only; returns ``(x_fp8 [..., D], scales [..., ceil(D/block)])``
    with ``x ~= x_fp8.float() * scales.repeat_interleave(block)[..., :D]``.
    """
    D = x.shape[-1]
    nb = (D + block - 1) // block
    xf = x.float()
    pad = nb * block - D
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    xb = xf.view(*x.shape[:-1], nb, block)
    amax = xb.abs().amax(dim=-1).clamp(min=1e-12)
    scale = amax / FP8_E4M3_MAX
    q = (xb / scale.unsqueeze(-1)).clamp(-FP8_E4M3_MAX, FP8_E4M3_MAX)
    q = q.view(*x.shape[:-1], nb * block)[..., :D].to(torch.float8_e4m3fn)
    return q, scale


def dequantize_fp8_blockscaled(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    D = q.shape[-1]
    s = scale.repeat_interleave(block, dim=-1)[..., :D]
    return q.float() * s


def mla_partial_attention(q_nope: torch.Tensor, q_pe: torch.Tensor, ckv: torch.Tensor,
                          kpe: torch.Tensor, scale: float, base2: bool = False):
    """MLA decode in the absorbed ("latent") form over one KV shard.

    ``q_nope [T,H,R]`` (already multiplied by W_uk), ``q_pe [T,H,P]``, latent
    ``ckv [S,R]`` and rope keys ``kpe [S,P]``.  Scores are
    ``(q_nope.ckv + q_pe.kpe) * scale``; values are the latent itself, so the
    output is ``[T,H,R]`` plus ``lse [T,H]``.
    """
    T, H, R = q_nope.shape
    S = ckv.shape[0]
    if S == 0:
        return (torch.zeros(T, H, R, dtype=torch.float32, device=q_nope.device),
                torch.full((T, H), float("-inf"), dtype=torch.float32, device=q_nope.device))
    s = (torch.einsum("thr,sr->ths", q_nope.float(), ckv.float())
         + torch.einsum("thp,sp->ths", q_pe.float(), kpe.float())) * scale
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.unsqueeze(-1))
    o = torch.einsum("ths,sr->thr", p, ckv.float())
    if base2:
        lse = lse * LOG2E
    return o, lse
