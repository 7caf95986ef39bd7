"""The fp32 oracles agree with each other (split-KV + combine == full attention, edge cases)."""
import math

import pytest
import torch

from helix_a2a_b200.ops import reference_math as rm


@pytest.mark.parametrize("shards", [1, 2, 4, 8])
@pytest.mark.parametrize("base2", [False, True])
def test_split_kv_combine_equals_full_attention(shards, base2):
    torch.manual_seed(0)
    T, H, Hkv, D, S = 4, 8, 2, 64, 256
    q, k, v = torch.randn(T, H, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
    full = rm.full_attention(q, k, v)
    outs, lses = [], []
    for ks, vs in zip(k.chunk(shards), v.chunk(shards)):
        o, l = rm.partial_attention(q, ks, vs, base2=base2)
        outs.append(o)
        lses.append(l)
    res, glse = rm.lse_combine(torch.stack(outs), torch.stack(lses), return_lse=True, base2=base2)
    assert (res - full).abs().max() < 1e-5
    _, lse_full = rm.partial_attention(q, k, v, base2=base2)
    assert (glse - lse_full).abs().max() < 1e-4


def test_combine_edge_cases():
    N, B, H, D = 3, 2, 4, 8
    o = torch.randn(N, B, H, D)
    l = torch.randn(N, B, H)
    l[0, 0, 0] = float("-inf")      # an empty shard
    l[1, 0, 1] = float("nan")       # NaN counts as -inf
    l[2, 0, 2] = float("inf")       # +inf counts as -inf too
    l[:, 1, 3] = float("-inf")      # every shard empty -> output 0, LSE -inf
    res, g = rm.lse_combine(o, l, return_lse=True)
    assert torch.isfinite(res).all()
    assert (res[1, 3] == 0).all() and g[1, 3] == float("-inf")
    w = torch.softmax(l[1:, 0, 0], 0)
    assert torch.allclose(res[0, 0], w[0] * o[1, 0, 0] + w[1] * o[2, 0, 0], atol=1e-6)


def test_stats_to_lse_modes():
    m, s = torch.randn(5, 3), torch.rand(5, 3) + 0.5
    st = torch.stack([m, s], -1)
    assert torch.allclose(rm.stats_to_lse(st, "max_sumexp"), m + torch.log(s))
    assert torch.allclose(rm.stats_to_lse(st, "max_sumexp", base2=True), m + torch.log2(s))
    assert torch.equal(rm.stats_to_lse(st, "lse"), m)


def test_head_scatter_reference_matches_per_rank_combine():
    N, B, H, D = 4, 3, 8, 16
    outs, lses = torch.randn(N, B, H, D), torch.randn(N, B, H)
    res = rm.head_scatter_combine_reference(outs, lses)
    Hl = H // N
    for r in range(N):
        sl = slice(r * Hl, (r + 1) * Hl)
        want = rm.lse_combine(outs[:, :, sl], lses[:, :, sl])
        assert torch.allclose(res[r], want, atol=1e-6)


def test_paged_attention_reference_matches_dense():
    torch.manual_seed(1)
    B, H, Hkv, D, page = 3, 8, 2, 32, 16
    seq = [5, 48, 33]
    n_pages = 16
    kc, vc = torch.randn(n_pages, Hkv, page, D), torch.randn(n_pages, Hkv, page, D)
    bt = torch.stack([torch.randperm(n_pages)[:4] for _ in range(B)]).int()
    q = torch.randn(B, H, D)
    o, l = rm.paged_decode_attention_reference(q, kc, vc, bt, torch.tensor(seq))
    for b in range(B):
        k = rm.gather_paged_kv(kc, bt[b], seq[b])
        assert k.shape == (seq[b], Hkv, D)
        ob, lb = rm.partial_attention(q[b:b + 1], k, rm.gather_paged_kv(vc, bt[b], seq[b]))
        assert torch.allclose(o[b], ob[0], atol=1e-6) and torch.allclose(l[b], lb[0], atol=1e-6)


def test_fp8_blockscaled_roundtrip():
    x = torch.randn(7, 576) * 3
    q, s = rm.quantize_fp8_blockscaled(x, 128)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (7, 5)
    back = rm.dequantize_fp8_blockscaled(q, s, 128)
    assert ((back - x).abs() <= x.abs() * 0.07 + 1e-3).all()


def test_mla_partial_attention_is_attention_over_concat():
    T, H, R, P, S = 2, 4, 32, 8, 40
    qn, qp, ckv, kpe = torch.randn(T, H, R), torch.randn(T, H, P), torch.randn(S, R), torch.randn(S, P)
    scale = 1 / math.sqrt(R + P)
    o, l = rm.mla_partial_attention(qn, qp, ckv, kpe, scale)
    q = torch.cat([qn, qp], -1)
    k = torch.cat([ckv, kpe], -1).unsqueeze(1)
    o2, l2 = rm.partial_attention(q, k, ckv.unsqueeze(1), scale)
    assert torch.allclose(o, o2, atol=1e-5) and torch.allclose(l, l2, atol=1e-5)


def test_e4m3_bit_move_matches_float8_for_every_code():
    """The MLA kernels decode e4m3 without a conversion instruction: the byte s.eeee.mmm, moved to
    s.000.0eeee.mmm.0000, read as bf16, is 2^-120 times its value (subnormals and zero included).
    Mirror of ``e4m3x2_to_bf16x2_scaled`` in csrc/decode_attn_mla.cu on all 256 codes."""
    import torch
    codes = torch.arange(256, dtype=torch.int32)
    x = codes << 8                                            # the byte in the high byte of a 16-bit half
    bits = ((x >> 4) & 0x07FF) | (x & 0x8000)
    as_bf16 = bits.to(torch.int16).view(torch.bfloat16).to(torch.float64)   # exact
    got = as_bf16 * 2.0 ** 64 * 2.0 ** 56                     # the two multiplies of the kernel (scale 1)
    want = torch.arange(256, dtype=torch.uint8).view(torch.float8_e4m3fn).to(torch.float64)
    finite = ~torch.isnan(want)
    assert finite.sum() == 254
    assert torch.equal(got[finite], want[finite])
    # the first multiply alone stays inside bf16's normal range for every finite code but zero
    mid = (as_bf16 * 2.0 ** 64)[finite]
    nz = mid != 0
    assert (mid[nz].abs() >= 2.0 ** -126).all() and (mid[nz].abs() < 2.0 ** 20).all()


def test_streamk_partition_arithmetic():
    """Mirror of the unit partition of the stream-K o_proj kernel (csrc/oproj_gemm.cu): CTA c owns units
    [c U / G, (c + 1) U / G); the CTAs that meet a slab are found in closed form, and a slab is written
    directly only by a CTA that covers all of it."""
    for slabs, kb_total, G in [(64, 32, 148), (64, 4, 148), (4, 1, 4), (9, 4, 7), (56, 64, 148), (3, 5, 15)]:
        U = slabs * kb_total
        if G > U:
            continue
        start = [c * U // G for c in range(G + 1)]
        assert all(start[c + 1] > start[c] for c in range(G))            # every CTA has work
        for m in range(slabs):
            t0, t1 = m * kb_total, m * kb_total + kb_total - 1
            c_first = ((t0 + 1) * G + U - 1) // U - 1
            c_last = ((t1 + 1) * G + U - 1) // U - 1
            owners = [c for c in range(G) if start[c] <= t1 and start[c + 1] > t0]
            assert owners == list(range(c_first, c_last + 1)), (slabs, kb_total, G, m)
            whole = [c for c in owners if start[c] <= t0 and start[c + 1] > t1]
            assert (len(owners) == 1) == bool(whole)
            # piece slots: the CTA that starts the slab uses slot 1, continuations slot 0 - never both for one slab
            assert start[c_first] <= t0 and all(start[c] > t0 for c in owners[1:])


def test_oproj_weight_prepack_layout_and_roundtrip():
    """Packed layout = per slab, per 64-column atom, 128 rows x 128 bytes with chunk c of row r at c ^ (r & 7)."""
    import torch
    from helix_a2a_b200.ops.oproj import oproj, packed_atoms, prepack_weight, unpack_weight
    torch.manual_seed(0)
    hidden, K = 256, 320                       # 5 atoms -> padded to 8
    w_full = torch.randn(hidden, 1024).bfloat16()
    w = w_full[:, 128:128 + K]                 # a column slice, as a CP rank holds it
    pw = prepack_weight(w)
    na = packed_atoms(K)
    assert na == 8 and pw.packed.numel() == (hidden // 128) * na * 16384
    flat = pw.packed.view(torch.bfloat16)
    for (row, col) in [(0, 0), (5, 9), (127, 63), (128, 64), (200, 319), (255, 130)]:
        slab, r, atom, c, e = row // 128, row % 128, col // 64, (col % 64) // 8, col % 8
        off = ((slab * na + atom) * 128 + r) * 64 + ((c ^ (r & 7)) * 8) + e
        assert flat[off] == w[row, col], (row, col)
    # padding atoms are zero, and the inverse gives the matrix back
    assert (flat.view(hidden // 128, na, 128 * 64)[:, 5:] == 0).all()
    assert torch.equal(unpack_weight(pw), w.contiguous())
    x = torch.randn(3, K).bfloat16()
    assert torch.equal(oproj(x, pw), oproj(x, w.contiguous()))
