#!/usr/bin/env python
"""Device timeline of the one-kernel exchange + combine + o_proj (the counterpart of an nsys timeline of the
reference's pipeline, benchmark/sbatch/pipeline_bench.sbatch:167-170; the kernel stamps %globaltimer itself).

Real ranks (one per GPU):
    HELIX_A2A_EXCHANGE_TRACE=1 torchrun --nproc-per-node N benchmarks/fused_timeline.py [--tokens 1,8,32,64] [--hidden 2048]
All ranks played by one launch on one GPU (the test emulation; NVLink is then a local store):
    HELIX_A2A_EXCHANGE_TRACE=1 python benchmarks/fused_timeline.py --emulate 2 --hidden 1024

Every CTA records %globaltimer stamps.  Sender CTAs: entry, inputs ready, first and last line posted (warp 0), exit.
GEMM CTAs: entry, inputs ready (the weight slice has been requested before that), rows received and combined into
the tensor-core operand, accumulator ready, exit without the split-K fold; the slab's last CTA also stamps the end
of the fold.  Printed per token count as median / max over CTAs and calls, in microseconds after the CTA's entry.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("HELIX_A2A_EXCHANGE_TRACE", "1")
import torch  # noqa: E402

import helix_a2a_b200 as helix  # noqa: E402
from helix_a2a_b200.ops._ext import ops  # noqa: E402


def summarise(rows):
    tr = torch.cat(rows).double()
    out = {}
    t0 = tr[:, 0].min()
    for role, name, cols in ((1, "sender", {"inputs_ready": 1, "first_line_posted": 2, "last_line_posted_warp0": 3, "exit": 6}),
                             (2, "gemm", {"inputs_ready": 1, "rows_combined": 2, "accumulator_ready": 3, "exit_before_fold": 6,
                                          "fold_done": 4})):
        sel = tr[tr[:, 7] == role]
        if sel.numel() == 0:
            continue
        d = {"ctas_x_calls": int(sel.shape[0]), "entry_spread_us": round(float((sel[:, 0].max() - t0) / 1e3), 2)}
        for k, c in cols.items():
            v = sel[:, c]
            v = (v[v > 0] - sel[:, 0][v > 0]) / 1e3
            if v.numel():
                d[k] = [round(float(v.median()), 2), round(float(v.max()), 2)]
        out[name] = d
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,8,32,64")
    ap.add_argument("--hidden", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--emulate", type=int, default=0, help="play this many ranks in one launch on one GPU")
    ap.add_argument("--calls", type=int, default=10)
    args = ap.parse_args()
    H, D = args.heads, 128
    if args.emulate:
        cp, rank = args.emulate, 0
        torch.cuda.set_device(0)
        ws = helix.allocate_workspace(cp, 0)
        helix.init_workspace_all_rows(ws, cp)
    else:
        import torch.distributed as dist
        rank, cp = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        cpu_group = dist.new_group(backend="gloo")
        ws = helix.allocate_workspace(cp, rank, mnnvl=True, cpu_group=cpu_group)
        helix.init_workspace(ws, rank, cp)
        dist.barrier()
    K = H // cp * D
    for T in [int(t) for t in args.tokens.split(",")]:
        lead = (cp,) if args.emulate else ()
        o = torch.randn(*lead, T, H, D, device="cuda").bfloat16()
        lse = torch.randn(*lead, T, H, device="cuda")
        w = (torch.randn(*lead, args.hidden, K, device="cuda") * 0.05).bfloat16()

        def call():
            return ops().alltoall_combine_oproj(o, lse, w, ws, rank, cp, False, bool(args.emulate), 0)

        for _ in range(3):
            call()
        rows = []
        for _ in range(args.calls):
            torch.cuda.synchronize()
            if not args.emulate:
                dist.barrier()
            call()
            torch.cuda.synchronize()
            tr = ops().attn_trace(o).view(-1, 8)
            rows.append(tr[tr[:, 7] > 0].cpu())
        res = {"cp": cp, "tokens": T, "hidden": args.hidden, "emulated": bool(args.emulate), "rank": rank, **summarise(rows)}
        if args.emulate or rank == 0:
            print(json.dumps(res), flush=True)
    if not args.emulate:
        helix.check_status(ws, rank, cp)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
