#!/usr/bin/env python
"""Headline benchmark: decode tokens/s of the Llama-3-70B-architecture attention stack at 128K
context under Helix context parallelism (split-KV attention -> exchange + combine -> o_proj, 80
layers), one rank per GPU.

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N ...            # the unmodified reference + stock vLLM-side ops

Weak scaling: the context is 131072 tokens at every N and is split evenly over the N ranks; the
global batch is one sequence per GPU (batch 8 on 8 GPUs, the named configuration), so every GPU
streams the same 43 GB of KV cache per step.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode tok/s, Llama-3-70B-arch attention stack, 128K context (Helix a2a+combine us/step in extras)"
CTX = 131072


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx = float(r[1])
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        busy = [c for c in sm if mx and c > 0.3 * mx] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm)}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="helix", choices=["helix", "reference"])
    ap.add_argument("--layers", type=int, default=80)
    ap.add_argument("--ctx", type=int, default=CTX)
    ap.add_argument("--batch-per-gpu", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--fuse-oproj", nargs="?", const="on", default="off", choices=["on", "off", "auto"],
                    help="exchange+combine+o_proj as ONE kernel: on / auto = whenever the shape fits that kernel (for "
                         "this model: cp = 8), off = two kernels chained by programmatic dependent launch")
    ap.add_argument("--no-pdl", action="store_true", help="do not chain the kernels by programmatic dependent launch")
    return ap.parse_args()


def init_dist(n):
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world == 1 and n == 1:
        torch.cuda.set_device(0)
        return 0, 1, None, None
    if world != n:
        raise SystemExit(f"launch with torchrun --nproc-per-node {n} (WORLD_SIZE={world})")
    rank = int(os.environ["RANK"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cpu_group = dist.new_group(backend="gloo")
    return rank, world, dist.group.WORLD, cpu_group


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def barrier(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def time_op_in_graph(fn, world: int, calls: int = 20, replays: int = 20) -> float:
    """Microseconds per call of ``fn`` (a collective every rank calls), measured as a CUDA graph of ``calls``
    back-to-back calls replayed ``replays`` times: device time without host launch overhead, max over ranks.
    Both arms of the benchmark time their exchange + combine with this one function."""
    import torch
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            fn()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(calls):
                fn()
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(3):
        g.replay()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    barrier(world)
    return max_over_ranks(e0.elapsed_time(e1), world) / (replays * calls) * 1e3


def bench_config(n_layers: int, batch: int, ctx: int, world: int, page_size: int, local_ctx: int, kv_bytes: int,
                 graph: bool) -> dict:
    """The ``config`` entry of the JSON line: what is measured, with the same keys in both arms (how each arm
    computes it goes under ``extras.path``)."""
    return {"model": f"llama3-70b-arch attention stack ({n_layers} layers, 64q/8kv heads, d=128, hidden 8192)",
            "global_batch": batch, "seq_len": ctx, "parallelism": f"cp{world}", "page_size": page_size,
            "kv_tokens_per_gpu_per_seq": local_ctx,
            "l2": "inputs larger than L2 (KV cache read per step: %.1f GB per GPU)" % (kv_bytes / 1e9),
            "cuda_graph": graph}


def check_exchange_against_nccl(stack, q_layer0, rank: int, world: int, group) -> float:
    """One layer's exchange + combine on every rank against two NCCL all-to-alls + the fp32 torch combine.
    Returns the largest absolute difference over all ranks (the benchmark aborts when it is not small)."""
    import torch
    import torch.distributed as dist
    import helix_a2a_b200 as helix
    from helix_a2a_b200.ops import attention, reference_math as rm
    cfg = stack.cfg
    o, lse = attention.gqa_decode(q_layer0, stack.k_cache[0], stack.v_cache[0], stack.block_table, stack.seq_lens,
                                  scale=stack.scale, max_seq_len=stack.local_ctx)
    got = helix.alltoall_combine(o, lse, stack.workspace, rank, world)
    B, H, D = o.shape
    Hl = H // world
    so = o.view(B, world, Hl, D).permute(1, 0, 2, 3).contiguous()
    sl = lse.view(B, world, Hl).permute(1, 0, 2).contiguous()
    ro, rl = torch.empty_like(so), torch.empty_like(sl)
    dist.all_to_all_single(ro.view(-1), so.view(-1), group=group)
    dist.all_to_all_single(rl.view(-1), sl.view(-1), group=group)
    want = rm.lse_combine(ro, rl)
    err = float((got.float() - want).abs().max())
    if not (err == err):
        err = float("inf")
    return max_over_ranks(err, world)


def run_helix(args):
    import torch
    if not args.no_pdl:
        os.environ.setdefault("HELIX_A2A_ENABLE_PDL", "1")     # the library's documented knob
    rank, world, group, cpu_group = init_dist(args.gpus)
    from helix_a2a_b200.models.llama_decode import HelixDecodeStack, LlamaDecodeConfig
    from helix_a2a_b200.ops.oproj import check_compute_status
    import helix_a2a_b200 as helix

    cfg = LlamaDecodeConfig.llama3_70b(n_layers=args.layers)
    batch = args.batch_per_gpu * world
    local_ctx = args.ctx // world
    stack = HelixDecodeStack(cfg, batch=batch, local_ctx=local_ctx, cp_size=world, cp_rank=rank, group=cpu_group,
                             fuse_oproj={"on": True, "off": False, "auto": None}[args.fuse_oproj])
    gen = torch.Generator().manual_seed(7)          # same q on every rank
    q_host = [torch.randn(cfg.n_layers, batch, cfg.n_q_heads, cfg.head_dim, generator=gen).bfloat16().pin_memory()
              for _ in range(2)]
    q_dev = q_host[0].cuda()
    out_pinned = torch.empty(batch, cfg.hidden, dtype=torch.bfloat16).pin_memory()

    # warm-up: eager first (also sizes the library's scratch), then the captured graph
    stack.decode_step_device(q_dev)
    barrier(world)
    if not args.no_graph:
        stack.capture(q_dev)
    for _ in range(max(args.warmup, 3)):
        stack.decode_step_device(q_dev)
    barrier(world)
    check_compute_status(q_dev)
    exchange_err = None
    if world > 1:
        helix.check_status(stack.workspace, rank, world)
        # a wrong exchange must not print a tok/s line: compare one layer with the NCCL + torch path first
        exchange_err = check_exchange_against_nccl(stack, q_dev[0], rank, world, group)
        if not exchange_err < 2e-2:
            if rank == 0:
                print(f"bench: exchange + combine differs from the NCCL + torch path by {exchange_err}", file=sys.stderr)
            raise SystemExit(1)

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    # ---- device-timed steps -------------------------------------------------------------------
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        stack.decode_step_device(q_dev)
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps

    # ---- end to end through the public call: pinned host q in, host y out, every step -----------
    for i in range(2):
        stack.decode_step_host(q_host[i % 2], out_pinned)
    barrier(world)
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        stack.decode_step_host(q_host[i % 2], out_pinned)
    t1.record()
    barrier(world)
    ms_e2e = max_over_ranks(t0.elapsed_time(t1), world) / args.steps
    clocks = sampler.stop()
    check_compute_status(q_dev)
    if world > 1:
        helix.check_status(stack.workspace, rank, world)

    # ---- exchange + combine alone (the reference's own headline op) --------------------------------
    a2a_us = None
    if world > 1:
        o = torch.randn(batch, cfg.n_q_heads, cfg.head_dim, device="cuda").bfloat16()
        lse = torch.randn(batch, cfg.n_q_heads, device="cuda")
        a2a_us = time_op_in_graph(lambda: helix.alltoall_combine(o, lse, stack.workspace, rank, world), world)
        helix.check_status(stack.workspace, rank, world)

    if rank == 0:
        kv_bytes = 2 * cfg.n_layers * batch * local_ctx * cfg.n_kv_heads * cfg.head_dim * 2
        w_bytes = cfg.n_layers * cfg.hidden * stack.k_local * 2
        line = {
            "metric": METRIC, "value": batch / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random-init weights, KV ~ N(0,1), random q)",
            "impl": "helix_a2a_b200",
            "config": bench_config(cfg.n_layers, batch, args.ctx, world, cfg.page_size, local_ctx, kv_bytes,
                                   not args.no_graph),
            "clocks": clocks,
            "e2e": {"value": batch / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": stack.h2d_bytes_per_step(), "d2h_bytes_per_step": stack.d2h_bytes_per_step()},
            "gpu_launches": stack.kernels_per_step() * args.steps,
            "extras": {"helix_a2a_combine_us": a2a_us, "helix_a2a_combine_us_how": "CUDA graph of 20 calls, replayed",
                       "exchange_check_max_err_vs_nccl_torch": exchange_err,
                       "hbm_bytes_per_step_per_gpu": kv_bytes + w_bytes,
                       "achieved_hbm_gbs": (kv_bytes + w_bytes) / (ms * 1e-3) / 1e9,
                       "path": {"attention": "helix gqa_decode (sm_100a, TMA + mbarrier)",
                                "exchange": ("helix exchange+combine+o_proj in one kernel" if stack.fuse_oproj
                                             else "helix exchange+combine (one kernel)") if world > 1 else "none (cp=1)",
                                "o_proj": "helix tcgen05 GEMM, weights " +
                                          ("packed once at load time (tile-major, pre-swizzled bf16; same values)"
                                           if getattr(stack, "prepack_oproj", False)
                                           else "plain [hidden, K]"),
                                "pdl": os.environ.get("HELIX_A2A_ENABLE_PDL", "0") == "1"}},
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def main():
    args = parse()
    if args.impl == "reference":
        from benchmarks.reference_arm import run_reference
        run_reference(args)
    else:
        run_helix(args)


if __name__ == "__main__":
    main()
