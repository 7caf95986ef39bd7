"""Numerics of the decode attention and o_proj kernels against plain PyTorch fp32 references."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def built(native_built):
    from helix_a2a_b200.ops._ext import ext
    ext()
    return True


def _paged_case(B, Hq, Hkv, seq_lens, page=16, layout="HND", seed=0):
    torch.manual_seed(seed)
    D = 128
    max_blocks = max((s + page - 1) // page for s in seq_lens)
    n_pages = B * max_blocks + 3
    perm = torch.randperm(n_pages)[:B * max_blocks].view(B, max_blocks).int()
    shape = (n_pages, Hkv, page, D) if layout == "HND" else (n_pages, page, Hkv, D)
    kc = torch.randn(shape, device="cuda").bfloat16()
    vc = torch.randn(shape, device="cuda").bfloat16()
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    return q, kc, vc, perm.cuda(), torch.tensor(seq_lens, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("layout", ["HND", "NHD"])
@pytest.mark.parametrize("seq_lens,splits", [([5], 1), ([16, 17, 300], 1), ([1000, 37, 512, 2048], 3),
                                             ([4096, 4000], 0), ([129] * 5, 4)])
def test_gqa_decode_matches_fp32_reference(built, layout, seq_lens, splits):
    from helix_a2a_b200.ops import attention, reference_math as rm
    from helix_a2a_b200.ops.oproj import check_compute_status
    B, Hq, Hkv = len(seq_lens), 64, 8
    q, kc, vc, bt, sl = _paged_case(B, Hq, Hkv, seq_lens, layout=layout, seed=len(seq_lens))
    o, lse = attention.gqa_decode(q, kc, vc, bt, sl, layout=layout, splits=splits, max_seq_len=max(seq_lens))
    torch.cuda.synchronize()
    check_compute_status(q)
    kr = kc if layout == "HND" else kc.permute(0, 2, 1, 3)
    vr = vc if layout == "HND" else vc.permute(0, 2, 1, 3)
    o_ref, lse_ref = rm.paged_decode_attention_reference(q.float(), kr.float(), vr.float(), bt, sl, 1 / math.sqrt(128))
    assert (o.float() - o_ref).abs().max() < 2e-2
    assert (lse - lse_ref).abs().max() < 2e-3


@pytest.mark.parametrize("seq_lens", [[8192, 300, 4096], [40000]])
def test_gqa_decode_early_kv_prefetch_under_programmatic_launch(built, monkeypatch, seq_lens):
    """kv_stable: K/V tiles are requested before the wait on the preceding kernel; q comes from that kernel."""
    from helix_a2a_b200.ops import attention, reference_math as rm
    from helix_a2a_b200.ops.oproj import check_compute_status
    monkeypatch.setenv("HELIX_A2A_ENABLE_PDL", "1")
    q0, kc, vc, bt, sl = _paged_case(len(seq_lens), 64, 8, seq_lens, seed=11)
    big = torch.randn(64 << 20, device="cuda")
    for _ in range(3):
        big.mul_(1.0001)                       # keeps the GPU busy so that q's producer is still in flight
        q = (q0.float() * 2.0).bfloat16()      # q is produced by the kernel right before the attention
        o, lse = attention.gqa_decode(q, kc, vc, bt, sl, max_seq_len=max(seq_lens), kv_stable=True)
    torch.cuda.synchronize()
    check_compute_status(q)
    o_ref, lse_ref = rm.paged_decode_attention_reference(q.float(), kc.float(), vc.float(), bt, sl, 1 / math.sqrt(128))
    assert (o.float() - o_ref).abs().max() < 2e-2
    assert (lse - lse_ref).abs().max() < 2e-3


@pytest.mark.parametrize("seq_lens,pct,chunk,ahead", [([40000], 25, 4, 8), ([8192, 300, 4096], 30, 4, 1),
                                                      ([20000, 20000], 12, 8, 2), ([16384] * 8, 30, 8, 4),
                                                      ([5000, 0, 70000], 40, 12, 3), ([131072], 50, 2, 2)])
def test_gqa_decode_dynamic_tail_matches_fp32_reference(built, monkeypatch, seq_lens, pct, chunk, ahead):
    """Part of every long pair is handed out chunk by chunk to whichever CTA finishes its fixed share first; the result
    must not depend on who took what, and the counters must be back at zero for the next launch."""
    from helix_a2a_b200.ops import attention, reference_math as rm
    from helix_a2a_b200.ops.oproj import check_compute_status
    monkeypatch.setenv("HELIX_A2A_ATTN_DYN_PCT", str(pct))
    monkeypatch.setenv("HELIX_A2A_ATTN_DYN_CHUNK", str(chunk))
    monkeypatch.setenv("HELIX_A2A_ATTN_DYN_AHEAD", str(ahead))
    monkeypatch.setenv("HELIX_A2A_ATTN_DYN_MIN_BLOCKS", "8")
    q, kc, vc, bt, sl = _paged_case(len(seq_lens), 64, 8, seq_lens, seed=3)
    o_ref, lse_ref = rm.paged_decode_attention_reference(q.float(), kc.float(), vc.float(), bt, sl, 1 / math.sqrt(128))
    for _ in range(4):                                # repeated launches reuse the library's counters
        o, lse = attention.gqa_decode(q, kc, vc, bt, sl, max_seq_len=max(seq_lens))
        torch.cuda.synchronize()
        check_compute_status(q)
        live = sl > 0
        assert (o.float() - o_ref)[live].abs().max() < 2e-2
        assert (lse - lse_ref)[live].abs().max() < 2e-3
    # the same call with fixed shares only gives the same answer to rounding
    monkeypatch.setenv("HELIX_A2A_ATTN_DYN_PCT", "0")
    o2, lse2 = attention.gqa_decode(q, kc, vc, bt, sl, max_seq_len=max(seq_lens))
    assert (o2.float() - o.float())[live].abs().max() < 1e-2


def test_gqa_decode_small_group_base2_and_empty_sequence(built):
    from helix_a2a_b200.ops import attention, reference_math as rm
    seq_lens = [0, 40, 16]
    q, kc, vc, bt, sl = _paged_case(3, 8, 2, seq_lens, page=32, seed=7)       # group of 4, page 32
    o, lse = attention.gqa_decode(q, kc, vc, bt, sl, lse_base2=True, splits=2)
    o_ref, lse_ref = rm.paged_decode_attention_reference(q.float(), kc.float(), vc.float(), bt, sl,
                                                         1 / math.sqrt(128), base2=True)
    assert (o.float() - o_ref).abs().max() < 2e-2
    assert (o[0] == 0).all() and (lse[0] == float("-inf")).all()
    assert (lse[1:] - lse_ref[1:]).abs().max() < 3e-3


@pytest.mark.parametrize("tokens", [1, 8, 17, 64, 200, 300])
@pytest.mark.parametrize("hidden,K,splits", [(8192, 1024, 0), (1024, 8192, 1), (512, 256, 2), (8192, 8192, 0),
                                             (8192, 8192, -1), (8192, 1024, -1), (512, 256, -1), (1152, 832, -1),
                                             (1024, 8192, 3), (512, 4096, 8), (1024, 2048, 4)])
def test_oproj_matches_fp32_matmul(built, monkeypatch, tokens, hidden, K, splits):
    from helix_a2a_b200.ops.oproj import oproj, check_compute_status
    monkeypatch.setenv("HELIX_A2A_OPROJ_LIBRARY", "0")     # the hand-written kernel at every size
    torch.manual_seed(tokens + hidden)
    x = torch.randn(tokens, K, device="cuda").bfloat16()
    w = (torch.randn(hidden, K, device="cuda") * 0.02).bfloat16()
    y = oproj(x, w, splits=splits)
    torch.cuda.synchronize()
    check_compute_status(x)
    ref = x.float() @ w.float().t()
    err = (y.float() - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


@pytest.mark.parametrize("hidden,K,splits,tokens", [(512, 256, 2, 300), (1024, 2048, 4, 300), (512, 256, 2, 17),
                                                    (8192, 1024, 0, 8), (512, 256, -1, 300), (1024, 8192, 3, 300)])
def test_oproj_back_to_back_under_programmatic_launch(built, monkeypatch, hidden, K, splits, tokens):
    """Launches chained by programmatic dependent launch share the split-K scratch: a launch (a 256-token slice of a
    larger call, or the next call) must not touch it before the previous one is done, not even from a CTA that has
    no k-block of its own (512 x 256 in two splits with one 256-wide stage: the second split is empty)."""
    from helix_a2a_b200.ops.oproj import oproj, check_compute_status
    monkeypatch.setenv("HELIX_A2A_ENABLE_PDL", "1")
    monkeypatch.setenv("HELIX_A2A_OPROJ_LIBRARY", "0")
    torch.manual_seed(tokens + K)
    w = (torch.randn(hidden, K, device="cuda") * 0.02).bfloat16()
    xs = [torch.randn(tokens, K, device="cuda").bfloat16() for _ in range(3)]
    ys = [oproj(x, w, splits=splits) for x in xs]          # no synchronisation in between
    torch.cuda.synchronize()
    check_compute_status(xs[0])
    for x, y in zip(xs, ys):
        ref = x.float() @ w.float().t()
        assert (y.float() - ref).abs().max() < 2e-2 * max(1.0, ref.abs().max().item())


def test_oproj_hands_compute_bound_sizes_to_the_library(built, monkeypatch):
    """splits=0 with a plain weight: above the measured crossover the product goes to cuBLAS (same result within
    bf16 rounding); below it, with packed weights, or with HELIX_A2A_OPROJ_LIBRARY=0 the hand-written kernel runs."""
    from helix_a2a_b200.ops import oproj as om
    monkeypatch.delenv("HELIX_A2A_OPROJ_LIBRARY", raising=False)
    assert not om.library_gemm_pays(8, 8192) and not om.library_gemm_pays(31, 1024)
    assert om.library_gemm_pays(32, 2048) and om.library_gemm_pays(256, 1024)
    x = torch.randn(96, 2048, device="cuda").bfloat16()
    w = (torch.randn(1024, 2048, device="cuda") * 0.02).bfloat16()
    y_lib = om.oproj(x, w)
    monkeypatch.setenv("HELIX_A2A_OPROJ_LIBRARY", "0")
    assert not om.library_gemm_pays(96, 2048)
    y_own = om.oproj(x, w)
    ref = x.float() @ w.float().t()
    assert (y_lib.float() - ref).abs().max() < 2e-2 and (y_own.float() - ref).abs().max() < 2e-2


@pytest.mark.parametrize("tokens", [1, 8, 40, 200])
@pytest.mark.parametrize("hidden,K,splits", [(8192, 1024, 0), (1024, 8192, 0), (512, 320, 1), (1152, 832, 2), (2048, 4096, 4)])
def test_oproj_prepacked_weight_matches_fp32_matmul(built, tokens, hidden, K, splits):
    """Pre-packed weights (one bulk copy per stage) give the same product; the source is a column slice."""
    from helix_a2a_b200.ops.oproj import oproj, prepack_weight, check_compute_status
    torch.manual_seed(tokens + K)
    w_full = (torch.randn(hidden, K + 128, device="cuda") * 0.02).bfloat16()
    w = w_full[:, 64:64 + K]
    x = torch.randn(tokens, K, device="cuda").bfloat16()
    pw = prepack_weight(w)
    y = oproj(x, pw, splits=splits)
    torch.cuda.synchronize()
    check_compute_status(x)
    ref = x.float() @ w.float().t()
    err = (y.float() - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err
    assert torch.equal(y, oproj(x, w, splits=max(splits, 0)) if splits else y)


def test_oproj_on_column_slice_of_full_weight(built):
    """Each CP rank multiplies by its K-slice of W_o: a strided view, no copy."""
    from helix_a2a_b200.ops.oproj import oproj
    w_full = (torch.randn(1024, 4096, device="cuda") * 0.02).bfloat16()
    x = torch.randn(9, 1024, device="cuda").bfloat16()
    w_slice = w_full[:, 1024:2048]
    y = oproj(x, w_slice)
    ref = x.float() @ w_slice.float().t()
    assert (y.float() - ref).abs().max() < 2e-2


def _mla_case(seq_lens, page=16, seed=0):
    from helix_a2a_b200.ops import reference_math as rm
    torch.manual_seed(seed)
    B = len(seq_lens)
    max_blocks = max((s + page - 1) // page for s in seq_lens) + 1
    n_pages = B * max_blocks + 2
    bt = torch.randperm(n_pages)[:B * max_blocks].view(B, max_blocks).int().cuda()
    lat = torch.randn(n_pages, page, 512, device="cuda")
    ckv, scales = rm.quantize_fp8_blockscaled(lat, 128)
    kpe = torch.randn(n_pages, page, 64, device="cuda").bfloat16()
    qn = (torch.randn(B, 128, 512, device="cuda") * 0.5).bfloat16()
    qp = (torch.randn(B, 128, 64, device="cuda") * 0.5).bfloat16()
    return qn, qp, ckv, scales, kpe, bt, torch.tensor(seq_lens, dtype=torch.int32, device="cuda")


@pytest.mark.parametrize("variant", ["lockstep", "ws"])
def test_mla_fp8_dequant_covers_every_e4m3_value(built, monkeypatch, variant):
    monkeypatch.setenv("HELIX_A2A_MLA_VARIANT", variant)
    """The kernels decode e4m3 with integer bit moves and bf16 multiplies: check all 254 finite byte values
    (subnormals, zero, both signs), small and large block scales, through the attention output itself:
    with one token per sequence the output IS that token's dequantised latent row."""
    from helix_a2a_b200.ops import attention
    page = 16
    finite = [b for b in range(256) if (b & 0x7F) != 0x7F]
    B = 8
    codes = torch.tensor(finite, dtype=torch.uint8).repeat(3)[:512]
    ckv = torch.zeros(B, page, 512, dtype=torch.uint8, device="cuda")
    scales = torch.ones(B, page, 4, device="cuda")
    sc_vals = [1.0, 2.0 ** -20, 2.0 ** 20, 3.3e-3, 777.0, 0.37, 2.0 ** 40, 1.5]
    for b in range(B):
        ckv[b, 0] = codes.roll(b * 37).cuda()
        scales[b, 0] = torch.tensor([sc_vals[b], sc_vals[(b + 1) % B], sc_vals[(b + 2) % B], sc_vals[(b + 3) % B]])
    kpe = torch.zeros(B, page, 64, device="cuda").bfloat16()
    bt = torch.arange(B, dtype=torch.int32, device="cuda").view(B, 1)
    sl = torch.ones(B, dtype=torch.int32, device="cuda")
    qn = torch.zeros(B, 128, 512, device="cuda").bfloat16()
    qp = torch.zeros(B, 128, 64, device="cuda").bfloat16()
    o, _ = attention.mla_decode(qn, qp, ckv.view(torch.float8_e4m3fn), scales, kpe, bt, sl, scale=0.1, max_seq_len=1)
    torch.cuda.synchronize()
    want = ckv[:, 0].view(torch.float8_e4m3fn).float() * scales[:, 0].repeat_interleave(128, dim=-1)
    got = o[:, 0].float()                                     # every head sees the same single token
    tol = want.abs() * 2.0 ** -7 + 1e-30                     # two bf16 roundings (scale, product)
    assert ((got - want).abs() <= tol).all(), ((got - want).abs() / (want.abs() + 1e-30)).max()
    assert (o.float() == got[:, None, :]).all()


@pytest.mark.parametrize("seq_lens,ctas", [([32], 1), ([100, 7, 64], 1), ([1000, 333], 3), ([4096, 2000, 17, 0], 0),
                                           ([700] * 5, 7)])
@pytest.mark.parametrize("variant", ["lockstep", "ws"])
def test_mla_fp8_decode_matches_fp32_reference(built, monkeypatch, seq_lens, ctas, variant):
    import math
    monkeypatch.setenv("HELIX_A2A_MLA_VARIANT", variant)
    from helix_a2a_b200.ops import attention, reference_math as rm
    from helix_a2a_b200.ops.oproj import check_compute_status
    qn, qp, ckv, scales, kpe, bt, sl = _mla_case(seq_lens, seed=len(seq_lens))
    scale = 1.0 / math.sqrt(128 + 64)
    o, lse = attention.mla_decode(qn, qp, ckv, scales, kpe, bt, sl, scale=scale, ctas=ctas, max_seq_len=max(seq_lens))
    torch.cuda.synchronize()
    check_compute_status(qn)
    lat = rm.dequantize_fp8_blockscaled(ckv, scales, 128)
    for b, n in enumerate(seq_lens):
        if n == 0:
            assert (o[b] == 0).all() and (lse[b] == float("-inf")).all()
            continue
        npg = (n + 15) // 16
        idx = bt[b, :npg].long()
        c = lat[idx].reshape(-1, 512)[:n]
        k = kpe[idx].reshape(-1, 64)[:n].float()
        o_ref, l_ref = rm.mla_partial_attention(qn[b:b + 1].float(), qp[b:b + 1].float(), c, k, scale)
        assert (o[b].float() - o_ref[0]).abs().max() < 3e-2, (b, n)
        assert (lse[b] - l_ref[0]).abs().max() < 5e-3, (b, n)
