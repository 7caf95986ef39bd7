#!/usr/bin/env python
"""Small fixed cases for profiler captures (one kernel, a few launches, ~1 GB on the device).

    python benchmarks/profile_case.py attn      # GQA decode, B=8, 16K tokens per sequence (537 MB of KV)
    python benchmarks/profile_case.py oproj     # o_proj, 8 tokens, K=8192, hidden 8192 (134 MB of W)
    python benchmarks/profile_case.py exchange  # fused exchange+combine, 4 ranks played by one launch
    python benchmarks/profile_case.py mla       # MLA fp8 decode, B=8, 16K tokens per sequence
    python benchmarks/profile_case.py fused     # one-kernel exchange+combine+o_proj, 8 ranks played by one launch
    python benchmarks/profile_case.py fused_rows  # the same with 64 tokens (slabs of a head group share the rows)
    python benchmarks/profile_case.py streamk   # stream-K o_proj, 8 tokens, K=8192, hidden 8192
    python benchmarks/profile_case.py combine   # stand-alone LSE combine, 8 ranks x 4096 rows x 512
"""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import torch  # noqa: E402


def main():
    which = sys.argv[1] if len(sys.argv) > 1 else "attn"
    launches = 3
    if which == "attn":
        from helix_a2a_b200.ops import attention
        B, ctx, Hq, Hkv, D, page = 8, 16384, 64, 8, 128, 16
        pages = B * ctx // page
        bt = torch.randperm(pages).int().view(B, -1).cuda()
        sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        kc = torch.randn(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        vc = torch.randn(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16)
        q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
        for _ in range(launches):
            attention.gqa_decode(q, kc, vc, bt, sl, max_seq_len=ctx)
    elif which == "oproj":
        from helix_a2a_b200.ops.oproj import oproj
        w = (torch.randn(8192, 8192, device="cuda") * 0.02).bfloat16()
        x = torch.randn(8, 8192, device="cuda").bfloat16()
        for _ in range(launches):
            oproj(x, w)
    elif which == "streamk":
        from helix_a2a_b200.ops.oproj import oproj
        w = (torch.randn(8192, 8192, device="cuda") * 0.02).bfloat16()
        x = torch.randn(8, 8192, device="cuda").bfloat16()
        for _ in range(launches):
            oproj(x, w, splits=-1)
    elif which == "combine":
        import helix_a2a_b200 as helix
        o = torch.randn(8, 32, 128, 512, device="cuda").bfloat16()
        l = torch.randn(8, 32, 128, device="cuda")
        for _ in range(launches):
            helix.lse_combine(o, l)
    elif which in ("fused", "fused_rows"):
        import helix_a2a_b200 as helix
        from helix_a2a_b200.ops._ext import ops
        # per rank: K = 1024 in two head groups, 8 slabs; "fused_rows": 64 tokens, so the slabs share the rows
        cp, B, H, D, hidden = 8, (8 if which == "fused" else 64), 64, 128, 1024
        ws = helix.allocate_workspace(cp, 0)
        helix.init_workspace_all_rows(ws, cp)
        outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
        lses = torch.randn(cp, B, H, device="cuda")
        w = (torch.randn(cp, hidden, (H // cp) * D, device="cuda") * 0.05).bfloat16()
        for _ in range(launches):
            ops().alltoall_combine_oproj(outs, lses, w, ws, 0, cp, False, True, 0)
    elif which == "mla":
        import math
        from helix_a2a_b200.ops import attention, reference_math as rm
        B, ctx, page = 8, 16384, 16
        pages = B * ctx // page
        bt = torch.randperm(pages).int().view(B, -1).cuda()
        sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
        ckv, sc = rm.quantize_fp8_blockscaled(torch.randn(pages, page, 512, device="cuda"), 128)
        kpe = torch.randn(pages, page, 64, device="cuda").bfloat16()
        qn = (torch.randn(B, 128, 512, device="cuda") * 0.3).bfloat16()
        qp = (torch.randn(B, 128, 64, device="cuda") * 0.3).bfloat16()
        for _ in range(launches):
            attention.mla_decode(qn, qp, ckv, sc, kpe, bt, sl, scale=1 / math.sqrt(192), max_seq_len=ctx)
    else:
        import helix_a2a_b200 as helix
        from helix_a2a_b200.ops._ext import ops
        cp, B, H, D = 4, 64, 128, 512
        ws = helix.allocate_workspace(cp, 0)
        helix.init_workspace_all_rows(ws, cp)
        outs = torch.randn(cp, B, H, D, device="cuda").bfloat16()
        lses = torch.randn(cp, B, H, device="cuda")
        for _ in range(launches):
            ops().alltoall_combine(outs, lses, ws, 0, cp, 0, False, False, 0, True, 0, 0)
    torch.cuda.synchronize()
    print("done", which)


if __name__ == "__main__":
    main()
