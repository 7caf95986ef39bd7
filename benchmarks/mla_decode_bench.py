#!/usr/bin/env python
"""DeepSeek-V3-architecture MLA decode step with a block-scaled fp8 latent cache under Helix CP.

    python benchmarks/mla_decode_bench.py --ctx 131072 --batch 32 --layers 8                       # one GPU
    torchrun --nproc-per-node 8 benchmarks/mla_decode_bench.py --ctx 1048576 --batch 32 --layers 30  # cp = 8

    ... --impl reference [--ref-dtype fp8|bf16]      # stock parts only, same shapes (see run_reference below)

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


def run_reference(args, world, rank, cpu_group):
    """The same step from stock parts: vLLM's prebuilt SM100 CUTLASS MLA decode (`sm100_cutlass_mla_decode`, pages of
    128 tokens, latent + rope in one [pages, 128, 576] cache) -> the unmodified reference's hook (its kernel + its
    Triton combine) -> torch.nn.functional.linear.  The stock kernel has no block-scaled cache: `--ref-dtype fp8`
    runs it on an unscaled e4m3 cache with e4m3 queries (its fastest mode, fewer bytes than the block-scaled
    cache), `bf16` on a bf16 cache.  Nothing of this library's kernels is used.  Prints one JSON line, or an
    `unavailable` line that says what failed."""
    import importlib.util
    import math
    import torch.nn.functional as F
    REF = os.path.join(ROOT, "baseline", "_ref")

    def unavailable(why):
        if rank == 0:
            print(json.dumps({"bench": "mla_fp8_decode_step", "impl": "reference", "unavailable": why[:300]}), flush=True)

    try:
        import vllm._custom_ops as vops
        decode, ws_size = vops.sm100_cutlass_mla_decode, vops.sm100_cutlass_mla_get_workspace_size
    except Exception as e:  # noqa: BLE001
        return unavailable(f"vllm sm100_cutlass_mla_decode not importable: {e!r}")
    hook = None
    if world > 1:
        try:
            os.environ["HELIX_A2A_BACKEND"] = "native"
            os.environ.setdefault("HELIX_A2A_USE_MNNVL", "1")
            sys.path.insert(0, REF)
            for m in [k for k in sys.modules if k == "helix_a2a" or k.startswith("helix_a2a.")]:
                del sys.modules[m]
            spec = importlib.util.spec_from_file_location("ref_dcp_alltoall_helix", os.path.join(REF, "patches", "dcp_alltoall_helix.py"))
            hook = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(hook)
        except Exception as e:  # noqa: BLE001
            return unavailable(f"reference hook import failed: {e!r}")

    class _G:
        rank_in_group, world_size = rank, world
        device_group, cpu_group_ = dist.group.WORLD if world > 1 else None, cpu_group
    _G.cpu_group = cpu_group
    L, B, H, hidden, page = args.layers, args.batch, 128, 7168, 128
    local_ctx = args.ctx // world
    dt = torch.float8_e4m3fn if args.ref_dtype == "fp8" else torch.bfloat16
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(rank)
    pages_per_seq = (local_ctx + page - 1) // page
    n_pages = B * pages_per_seq
    bt = torch.randperm(n_pages, generator=torch.Generator().manual_seed(0)).int().view(B, pages_per_seq).to(dev)
    sl = torch.full((B,), local_ctx, dtype=torch.int32, device=dev)
    try:
        caches, ws_o = [], []
        for _ in range(L):
            c = torch.empty(n_pages, page, 576, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen)
            caches.append(c.to(dt))
            del c
            ws_o.append(torch.empty(hidden, (H // world) * 512, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=gen))
        sms = torch.cuda.get_device_properties(dev).multi_processor_count
        wbuf = torch.empty(max(int(ws_size(local_ctx, B, sms, -1)), 1), dtype=torch.uint8, device=dev)
        qn = (torch.randn(L, B, H, 512, device=dev, generator=gen) * 0.3).to(dt)
        qp = (torch.randn(L, B, H, 64, device=dev, generator=gen) * 0.3).to(dt)
        scale = 1.0 / math.sqrt(128 + 64)
        if world > 1:
            hook.dcp_a2a_ensure_initialized(_G)

        def step():
            y = None
            for l in range(L):
                out = torch.empty(B, H, 512, dtype=torch.bfloat16, device=dev)
                lse = torch.empty(B, H, dtype=torch.float32, device=dev)
                decode(out, lse, qn[l], qp[l], caches[l], sl, bt, wbuf, scale, -1)
                if world > 1:
                    out = hook.dcp_a2a_lse_reduce(out, lse, _G)
                y = F.linear(out.reshape(B, -1), ws_o[l])
            return y
        step()
        torch.cuda.synchronize()
    except Exception as e:  # noqa: BLE001
        return unavailable(f"stock MLA step failed: {e!r}")

    def sync():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        try:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                step()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    step()
            torch.cuda.current_stream().wait_stream(s)
        except Exception:  # noqa: BLE001
            graph = None
            torch.cuda.synchronize()
    run = graph.replay if graph is not None else step
    for _ in range(max(args.warmup, 3)):
        run()
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    sync()
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    if rank == 0:
        fl = L * B * local_ctx * 128 * (576 + 512) * 2
        print(json.dumps({
            "bench": "mla_fp8_decode_step", "impl": "reference", "n_gpus": world, "batch": B, "ctx": args.ctx,
            "layers_measured": L, "ms_per_step_measured": ms, "ms_per_layer": ms / L,
            "tok_s_measured_layers": B / (ms * 1e-3), "attention_tflops_per_gpu": fl / (ms * 1e-3) / 1e12,
            "attention": f"vllm sm100_cutlass_mla_decode, {args.ref_dtype} cache and queries, pages of 128 (no block scales)",
            "exchange": "reference helix_a2a.alltoall + its Triton combine" if world > 1 else "none",
            "o_proj": "torch.nn.functional.linear", "cuda_graph": graph is not None, "data": "synthetic"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ctx", type=int, default=131072, help="context per sequence (whole group)")
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--fuse-oproj", action="store_true")
    ap.add_argument("--impl", default="helix", choices=["helix", "reference"])
    ap.add_argument("--ref-dtype", default="fp8", choices=["fp8", "bf16"])
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
    if args.impl == "reference":
        run_reference(args, world, rank, cpu_group)
        if world > 1:
            dist.destroy_process_group()
        return
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
            "bench": "mla_fp8_decode_step", "impl": "helix_a2a_b200", "n_gpus": world, "batch": args.batch, "ctx": args.ctx,
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
