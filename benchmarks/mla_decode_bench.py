#!/usr/bin/env python
"""DeepSeek-V3-architecture MLA decode step with a block-scaled fp8 latent cache under Helix CP.

    python benchmarks/mla_decode_bench.py --ctx 131072 --batch 32 --layers 8                       # one GPU
    torchrun --nproc-per-node 8 benchmarks/mla_decode_bench.py --ctx 1048576 --batch 32 --layers 30  # cp = 8

Per step: MLA fp8 attention -> Helix exchange + combine -> o_proj, for `--layers` layers (the full
model has 61; 1M tokens x batch 32 x 61 layers of cache is 168 GB per GPU at cp = 8 and does not fit
next to the weights, so the layer count is a flag and the JSON line reports both the measured
ms per layer and the 61-layer extrapolation, labelled as such).  Device-timed, max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=131072, help="context per sequence (whole group)")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--fuse-oproj", action="store_true")
    args = ap.parse_args()
    os.environ.setdefault("HELIX_A2A_ENABLE_PDL", "1")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    cpu_group = None
    if world > 1:
        local = int(os.environ.get("LOCAL_RANK", rank))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        cpu_group = dist.new_group(backend="gloo")
    from helix_a2a_b200.models.deepseek_mla_decode import MlaDecodeConfig, MlaDecodeStack
    from helix_a2a_b200.ops.oproj import check_compute_status
    cfg = MlaDecodeConfig(n_layers=args.layers)
    stack = MlaDecodeStack(cfg, batch=args.batch, local_ctx=args.ctx // world, cp_size=world, cp_rank=rank,
                           group=cpu_group, fuse_oproj=args.fuse_oproj)
    g = torch.Generator(device="cuda").manual_seed(5)
    qn = (torch.randn(args.layers, args.batch, 128, 512, device="cuda", generator=g) * 0.3).bfloat16()
    qp = (torch.randn(args.layers, args.batch, 128, 64, device="cuda", generator=g) * 0.3).bfloat16()

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    stack.decode_step(qn, qp)
    sync()
    if not args.no_graph:
        stack.capture(qn, qp)
    for _ in range(max(args.warmup, 3)):
        stack.step(qn, qp)
    sync()
    check_compute_status(qn)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        stack.step(qn, qp)
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    check_compute_status(qn)
    if rank == 0:
        per_layer = ms / args.layers
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
            tf, src = peaks["bf16_tflops_sustained"], "measured (sustained)"
        except Exception:
            tf, src = 1400.0, "fallback"
        fl = stack.attention_flops_per_step()
        print(json.dumps({
            "bench": "mla_fp8_decode_step", "n_gpus": world, "batch": args.batch, "ctx": args.ctx,
            "layers_measured": args.layers, "ms_per_step_measured": ms, "ms_per_layer": per_layer,
            "tok_s_measured_layers": args.batch / (ms * 1e-3),
            "tok_s_61_layers_extrapolated": args.batch / (per_layer * 61 * 1e-3),
            "attention_tflops_per_gpu": fl / (ms * 1e-3) / 1e12, "frac_of_%s_bf16" % src: fl / (ms * 1e-3) / 1e12 / tf,
            "kv_gbs_per_gpu": stack.kv_bytes_per_step() / (ms * 1e-3) / 1e9,
            "cuda_graph": not args.no_graph, "one_kernel_exchange_oproj": args.fuse_oproj and world > 1,
            "dtype": "bf16 compute, fp8 e4m3 block-scaled cache", "data": "synthetic"}), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
