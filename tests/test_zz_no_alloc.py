"""The allocation-free C entry point of the decode attention, called through its exported symbol.

Some hosts of this library cannot obtain device memory when they need attention: a serving engine
that gave all free HBM to its KV cache at start-up, an engine that funnels every device allocation
through its own pool, or a plain C / C++ program without a tensor library.  For them the library
exports `helix_gqa_decode_noalloc`, whose scratch memory is a fixed array inside the library image.
This test drives that symbol with raw pointers (ctypes, no torch op in between) and checks its
output against the regular op on two calls in a row; the second call also proves that the state the
first call left in the shared scratch does not leak into the next result.

The file name sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import glob
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(native_built):
    from helix_a2a_b200.ops._ext import ext
    ext()
    path = glob.glob(os.path.join(ROOT, "helix_a2a_b200", "_C*.so"))[0]
    L = ctypes.CDLL(path)
    L.helix_gqa_decode_noalloc.restype = ctypes.c_int
    L.helix_gqa_decode_noalloc.argtypes = [
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_int64,            # q, strides
        ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int64,           # k, v, pages
        ctypes.c_int64, ctypes.c_int64, ctypes.c_int64,             # cache strides: page, head, token
        ctypes.c_void_p, ctypes.c_int64, ctypes.c_void_p,           # block table, stride, seq_lens
        ctypes.c_void_p, ctypes.c_void_p,                           # o, lse
        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int,   # batch, Hq, Hkv, page, max_seq_len
        ctypes.c_float, ctypes.c_int, ctypes.c_void_p]              # scale, base2, stream
    L.helix_noalloc_read_error.restype = ctypes.c_int
    L.helix_noalloc_read_error.argtypes = [ctypes.c_void_p]
    L.helix_noalloc_last_error.restype = ctypes.c_char_p
    return L


def _case(seq_lens, seed, Hq=64, Hkv=8, page=16):
    torch.manual_seed(seed)
    B, D = len(seq_lens), 128
    max_blocks = max((s + page - 1) // page for s in seq_lens)
    n_pages = B * max_blocks + 5
    bt = torch.randperm(n_pages)[:B * max_blocks].view(B, max_blocks).int().cuda()
    kc = torch.randn(n_pages, Hkv, page, D, device="cuda").bfloat16()
    vc = torch.randn(n_pages, Hkv, page, D, device="cuda").bfloat16()
    q = torch.randn(B, Hq, D, device="cuda").bfloat16()
    sl = torch.tensor(seq_lens, dtype=torch.int32, device="cuda")
    return q, kc, vc, bt, sl


def _call(lib, q, kc, vc, bt, sl, max_len):
    B, Hq, D = q.shape
    o = torch.full((B, Hq, D), float("nan"), device="cuda", dtype=torch.bfloat16)
    lse = torch.full((B, Hq), float("nan"), device="cuda", dtype=torch.float32)
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.helix_gqa_decode_noalloc(
        q.data_ptr(), q.stride(0), q.stride(1), kc.data_ptr(), vc.data_ptr(), kc.shape[0],
        kc.stride(0), kc.stride(1), kc.stride(2), bt.data_ptr(), bt.stride(0), sl.data_ptr(),
        o.data_ptr(), lse.data_ptr(), B, Hq, kc.shape[1], kc.shape[2], max_len,
        1.0 / math.sqrt(D), 0, ctypes.c_void_p(stream))
    assert rc == 0, lib.helix_noalloc_last_error()
    assert lib.helix_noalloc_read_error(ctypes.c_void_p(stream)) == 0
    return o, lse


def test_noalloc_entry_matches_regular_op_twice(lib):
    from helix_a2a_b200.ops import attention, reference_math as rm
    # two different problems back to back: the second one reuses the scratch the first one dirtied
    for seq_lens, seed in (([3000, 517, 4096, 64], 1), ([2048] * 6 + [1], 2)):
        q, kc, vc, bt, sl = _case(seq_lens, seed)
        want_o, want_lse = attention.gqa_decode(q, kc, vc, bt, sl, max_seq_len=max(seq_lens))
        got_o, got_lse = _call(lib, q, kc, vc, bt, sl, max(seq_lens))
        torch.cuda.synchronize()
        assert (got_o.float() - want_o.float()).abs().max() < 2e-2
        assert (got_lse - want_lse).abs().max() < 2e-3
        # and against the plain fp32 attention, so that the check does not lean on the library's own op
        ref_o, ref_lse = rm.paged_decode_attention_reference(q.float(), kc.float(), vc.float(), bt, sl, 1 / math.sqrt(128))
        assert (got_o.float() - ref_o).abs().max() < 2e-2
        assert (got_lse - ref_lse).abs().max() < 2e-3


def test_noalloc_entry_rejects_oversized_and_bad_arguments(lib):
    q, kc, vc, bt, sl = _case([32], 3)
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    args = [q.data_ptr(), q.stride(0), q.stride(1), kc.data_ptr(), vc.data_ptr(), kc.shape[0],
            kc.stride(0), kc.stride(1), kc.stride(2), bt.data_ptr(), bt.stride(0), sl.data_ptr(),
            q.data_ptr(), q.data_ptr()]
    # batch * kv_heads beyond the built-in scratch: refused before anything is launched
    rc = lib.helix_gqa_decode_noalloc(*args, 1000, 64, 8, 16, 32, 0.1, 0, stream)
    assert rc == 2 and b"exceeds" in lib.helix_noalloc_last_error()
    # page size that is not a multiple of 16
    rc = lib.helix_gqa_decode_noalloc(*args, 1, 64, 8, 8, 32, 0.1, 0, stream)
    assert rc == 1
