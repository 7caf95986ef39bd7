#!/usr/bin/env python
"""Per-CTA device timeline of the GQA decode attention kernel (1 GPU).  The reference has no attention kernel of its
own: vLLM supplies it, and the reference's hook starts from the attention output (patches/dcp_alltoall_helix.py:511-600).

    HELIX_A2A_ATTN_TRACE=1 python benchmarks/attn_timeline.py [--shapes 1x131072,8x16384] [--per-sm]

With the trace variable set the attention op launches the kernel instance that records %globaltimer stamps per
CTA: entry, end of the fixed share, last K/V block streamed (fixed share or pool chunk), exit, and how many pool
chunks the CTA drew.  Printed per shape as min / p10 / median / p90 / max over CTAs, in microseconds after the
first CTA's entry.  `HELIX_A2A_ATTN_DYN_PCT=0` shows the fixed shares alone.  The traced instance is a little
slower than the timed one; read shares and spreads, not absolutes.
"""
import argparse
import collections
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("HELIX_A2A_ATTN_TRACE", "1")
import torch  # noqa: E402

from helix_a2a_b200.ops import attention  # noqa: E402
from helix_a2a_b200.ops._ext import ops  # noqa: E402


def _stats(x):
    return "min %.1f p10 %.1f med %.1f p90 %.1f max %.1f" % (x.min(), x.quantile(0.1), x.median(), x.quantile(0.9), x.max())


def run(batch, ctx, per_sm):
    hq, hkv, d, page = 64, 8, 128, 16
    pages = batch * ctx // page
    bt = torch.randperm(pages).int().view(batch, -1).cuda()
    sl = torch.full((batch,), ctx, dtype=torch.int32, device="cuda")
    # three caches in turn so that no launch finds its K/V in L2
    kcs = [torch.randn(pages, hkv, page, d, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    vcs = [torch.randn(pages, hkv, page, d, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    q = torch.randn(batch, hq, d, device="cuda", dtype=torch.bfloat16)
    for _ in range(3):
        for l in range(3):
            attention.gqa_decode(q, kcs[l], vcs[l], bt, sl, max_seq_len=ctx)
        torch.cuda.synchronize()
    tr = ops().attn_trace(q).view(-1, 8).cpu()          # the stamps of the last launch
    n = int((tr[:, 3] > 0).sum())
    tr = tr[:n]
    t0 = int(tr[:, 0].min())
    us = lambda col: (tr[:, col] - t0).double() / 1e3   # noqa: E731
    entry, exit_ = us(0), us(3)
    fixed = torch.where(tr[:, 2] > 0, us(2), us(4))
    stream = torch.where(tr[:, 4] > 0, us(4), fixed)
    drawn, visits = tr[:, 5] & 0xFFFFFFFF, tr[:, 5] >> 32
    print(f"== B={batch} ctx={ctx} ctas={n} dyn_pct={os.environ.get('HELIX_A2A_ATTN_DYN_PCT', 'default')} "
          f"chunk={os.environ.get('HELIX_A2A_ATTN_DYN_CHUNK', 'default')}")
    print(" entry      ", _stats(entry))
    print(" fixed end  ", _stats(fixed))
    print(" stream end ", _stats(stream))
    print(" exit       ", _stats(exit_))
    print(" chunks drawn: total %d, per CTA min %d med %d max %d; visits to other pairs' pools: %d"
          % (int(drawn.sum()), int(drawn.min()), int(drawn.median()), int(drawn.max()), int(visits.sum())))
    if per_sm:
        by = collections.defaultdict(list)
        for sm, dur in zip((tr[:, 6] & 0xFF).tolist(), (fixed - entry).tolist()):
            by[sm].append(dur)
        cells = ["%d:%s" % (k, "/".join("%.0f" % x for x in by[k])) for k in sorted(by)]
        print(" fixed-share duration per SM (smid: us of its CTAs):")
        for i in range(0, len(cells), 12):
            print("   " + "  ".join(cells[i:i + 12]))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shapes", default="1x131072,8x16384", help="comma-separated BATCHxCONTEXT")
    ap.add_argument("--per-sm", action="store_true")
    args = ap.parse_args()
    for s in args.shapes.split(","):
        b, c = s.lower().split("x")
        run(int(b), int(c), args.per_sm)


if __name__ == "__main__":
    main()
