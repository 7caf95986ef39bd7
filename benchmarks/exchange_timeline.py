#!/usr/bin/env python
"""Device timeline of the fused exchange + combine kernel on real GPUs (one rank per GPU, torchrun).

The reference looks inside a call with nsys around its benchmark (benchmark/scripts/benchmark_helix_pipeline.py:30-31,
benchmark/sbatch/pipeline_bench.sbatch:167-170); nsys is not available where this library is developed, so the
kernel stamps %globaltimer itself.

    HELIX_A2A_EXCHANGE_TRACE=1 torchrun --nproc-per-node N benchmarks/exchange_timeline.py [--shape gqa|mla] [--tokens 8,256]

Every CTA (= channel) of the kernel records %globaltimer stamps (kernel entry, first / last line posted, first /
last peer message complete, exit).  Per call this prints, as the median and the maximum over channels and ranks,
how long after kernel entry each of these happened: "first message complete" minus "first line posted" is the
one-way latency of a message through NVLink and the receive poll when the ranks enter together (a barrier precedes
every traced call); clocks of different GPUs are not compared.
"""
import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ.setdefault("HELIX_A2A_EXCHANGE_TRACE", "1")
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import helix_a2a_b200 as helix  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--shape", default="gqa", choices=["gqa", "mla"])
    ap.add_argument("--tokens", default="1,8,64,256")
    ap.add_argument("--calls", type=int, default=20)
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cpu_group = dist.new_group(backend="gloo")
    ws = helix.allocate_workspace(world, rank, mnnvl=True, cpu_group=cpu_group)
    helix.init_workspace(ws, rank, world)
    dist.barrier()
    H, D = (64, 128) if args.shape == "gqa" else (128, 512)
    for T in [int(t) for t in args.tokens.split(",")]:
        o = torch.randn(T, H, D, device="cuda").bfloat16()
        lse = torch.randn(T, H, device="cuda")
        for _ in range(5):
            helix.alltoall_combine(o, lse, ws, rank, world)
        rows = []
        for _ in range(args.calls):
            torch.cuda.synchronize()
            dist.barrier()
            helix.alltoall_combine(o, lse, ws, rank, world)
            torch.cuda.synchronize()
            tr = helix.exchange_trace(ws)
            tr = tr[tr[:, 6] > 0].double()
            rel = (tr[:, 1:7] - tr[:, :1]) / 1e3          # us after kernel entry, per channel
            rel[tr[:, 1:7] == 0] = float("nan")
            rows.append(rel)
        rel = torch.cat(rows)
        names = ["inputs_ready", "first_line_posted", "last_line_posted", "first_message_complete",
                 "last_message_complete", "exit"]
        med = [float(torch.nanmedian(rel[:, i])) for i in range(6)]
        mx = [float(rel[:, i][~torch.isnan(rel[:, i])].max()) if (~torch.isnan(rel[:, i])).any() else float("nan") for i in range(6)]
        t = torch.tensor(med + mx, dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if rank == 0:
            vals = t.tolist()
            print(json.dumps({"shape": args.shape, "cp": world, "tokens": T, "channels": int(rows[0].shape[0]),
                              "us_after_entry_median_over_channels_max_over_ranks": dict(zip(names, [round(v, 2) for v in vals[:6]])),
                              "us_after_entry_max": dict(zip(names, [round(v, 2) for v in vals[6:]]))}), flush=True)
    helix.check_status(ws, rank, world)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
