#!/usr/bin/env python
"""Per-kernel timings on one GPU: decode attention and o_proj at the shapes of the headline
benchmark, as achieved HBM bandwidth and fraction of the measured copy bandwidth.

    python benchmarks/kernel_bench.py [--iters 20] [--json results/kernels.json]

Every timed launch reads buffers that were last touched several launches ago and that are together
much larger than L2 (layers are rotated), CUDA events on the launching stream, >= 3 warm-ups.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import torch  # noqa: E402


def measured_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            d = json.load(f)
        return d["hbm_gbs"], d["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def time_rotating(fns, iters, warmup=3, graph=True):
    """Device time per call in us: the calls (one per rotating buffer, so that nothing is found in L2) are captured
    into ONE CUDA graph that is replayed ``iters`` times between two events, so the host's launch cost (10-25 us per
    op call from Python, more than a small kernel runs) is not in the number.  ``graph=False`` times eager calls."""
    for _ in range(warmup):
        for f in fns:
            f()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if not graph:
        e0.record()
        for _ in range(iters):
            for f in fns:
                f()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / (iters * len(fns)) * 1e3
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for f in fns:
            f()
        side.synchronize()
        with torch.cuda.graph(g, stream=side):
            for f in fns:
                f()
    torch.cuda.current_stream().wait_stream(side)
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize()
    e0.record()
    for _ in range(iters):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / (iters * len(fns)) * 1e3   # us


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--json", default="")
    ap.add_argument("--only", default="")
    ap.add_argument("--splits", type=int, default=0)
    ap.add_argument("--oproj-splits", type=int, default=0, help="0 = pick, -1 = stream-K, n = n K splits")
    ap.add_argument("--oproj-packed", action="store_true", help="pre-pack the weights (one bulk copy per stage)")
    args = ap.parse_args()
    from helix_a2a_b200.ops import attention
    from helix_a2a_b200.ops.oproj import oproj, check_compute_status
    hbm, tflops, src = measured_peaks()
    rows = []
    if args.only in ("", "attn"):
        for (B, ctx) in ((1, 131072), (8, 16384), (32, 4096)):
            Hq, Hkv, D, page, nl = 64, 8, 128, 16, 4
            pages = B * ctx // page
            bt = torch.randperm(pages).int().view(B, -1).cuda()
            sl = torch.full((B,), ctx, dtype=torch.int32, device="cuda")
            kcs = [torch.randn(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16) for _ in range(nl)]
            vcs = [torch.randn(pages, Hkv, page, D, device="cuda", dtype=torch.bfloat16) for _ in range(nl)]
            q = torch.randn(B, Hq, D, device="cuda", dtype=torch.bfloat16)
            fns = [(lambda l=l: attention.gqa_decode(q, kcs[l], vcs[l], bt, sl, max_seq_len=ctx, splits=args.splits))
                   for l in range(nl)]
            us = time_rotating(fns, args.iters)
            nbytes = 2 * B * ctx * Hkv * D * 2
            rows.append({"kernel": "gqa_decode", "B": B, "ctx": ctx, "us": us, "GBs": nbytes / us / 1e3,
                         "frac_of_%s_hbm" % src: nbytes / us / 1e3 / hbm})
            del kcs, vcs
            check_compute_status(q)
    if args.only in ("", "oproj"):
        for (tokens, K) in ((1, 8192), (8, 1024), (8, 8192), (64, 1024), (256, 1024)):
            hidden, nl = 8192, max(2, (512 * 1024 * 1024) // (8192 * K * 2))
            ws = [(torch.randn(hidden, K, device="cuda") * 0.02).bfloat16() for _ in range(nl)]
            x = torch.randn(tokens, K, device="cuda").bfloat16()
            wk = ws
            if args.oproj_packed:
                from helix_a2a_b200.ops.oproj import prepack_weight
                wk = [prepack_weight(w) for w in ws]
            fns = [(lambda l=l: oproj(x, wk[l], splits=args.oproj_splits, library=False)) for l in range(nl)]
            us = time_rotating(fns, args.iters)
            nbytes = hidden * K * 2 + tokens * K * 2 + tokens * hidden * 2
            rows.append({"kernel": "oproj", "tokens": tokens, "K": K, "us": us, "GBs": nbytes / us / 1e3,
                         "frac_of_%s_hbm" % src: nbytes / us / 1e3 / hbm,
                         "tflops": 2 * tokens * K * hidden / us / 1e6})
            fns2 = [(lambda l=l: torch.nn.functional.linear(x, ws[l])) for l in range(nl)]
            us2 = time_rotating(fns2, args.iters)
            rows.append({"kernel": "torch.linear (cuBLAS) for comparison", "tokens": tokens, "K": K, "us": us2,
                         "GBs": nbytes / us2 / 1e3})
            del ws
            check_compute_status(x)
    for r in rows:
        print(json.dumps(r))
    if args.json:
        os.makedirs(os.path.dirname(args.json), exist_ok=True)
        with open(args.json, "w") as f:
            json.dump(rows, f, indent=1)


if __name__ == "__main__":
    main()
