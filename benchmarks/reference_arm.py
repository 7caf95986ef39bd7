"""Reference arm of ``bench.py``: the same decode step built only from stock parts.

Per layer: stock paged decode attention from the image (vLLM's flash-attention build, else
FlashInfer's paged decode wrapper) -> the UNMODIFIED reference's vLLM hook
``dcp_a2a_lse_reduce`` with ``HELIX_A2A_BACKEND=native`` (its ``helix_a2a.alltoall`` kernel +
its Triton combine, ``patches/dcp_alltoall_helix.py``) -> ``torch.nn.functional.linear``.  This
is the path a vLLM deployment of the reference runs; none of this library's kernels, models or
allocator is imported.  The reference package is the offline install under ``baseline/_ref``.
"""
from __future__ import annotations

import importlib.util
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")


def _unavailable(why: str) -> None:
    print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


class _Group:
    """The few attributes of vLLM's GroupCoordinator that the reference's hook reads."""

    def __init__(self, rank, world, device_group, cpu_group):
        self.rank_in_group, self.world_size = rank, world
        self.device_group, self.cpu_group = device_group, cpu_group


def _pick_attention(torch, cfg, batch, device):
    """Returns (name, fn(q, layer_index) -> (o [B,H,D], lse [B,H] fp32)) for the first stock backend that runs."""
    errors = []
    try:
        from vllm.vllm_flash_attn import flash_attn_varlen_func  # stock vLLM attention op

        def fa(q, kc, vc, bt, sl, scale, max_len):
            B = q.shape[0]
            cu = torch.arange(0, B + 1, dtype=torch.int32, device=q.device)
            out, lse = flash_attn_varlen_func(q=q, k=kc, v=vc, max_seqlen_q=1, cu_seqlens_q=cu, max_seqlen_k=max_len,
                                              seqused_k=sl, softmax_scale=scale, causal=True, block_table=bt,
                                              return_softmax_lse=True)
            return out, lse.transpose(0, 1).contiguous() if lse.shape[0] != B else lse
        return "vllm_flash_attn.flash_attn_varlen_func (NHD pages)", "NHD", fa
    except Exception as e:  # noqa: BLE001
        errors.append(f"vllm_flash_attn: {e!r}"[:160])
    try:
        import flashinfer

        state = {}

        def fi(q, kc, vc, bt, sl, scale, max_len):
            B = q.shape[0]
            if "w" not in state:
                page = kc.shape[2]
                npg = (sl + page - 1) // page
                indptr = torch.zeros(B + 1, dtype=torch.int32, device=q.device)
                indptr[1:] = torch.cumsum(npg, 0)
                indices = torch.cat([bt[b, :int(npg[b])] for b in range(B)]).int()
                last = ((sl - 1) % page + 1).int()
                wbuf = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=q.device)
                w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(wbuf, "HND", use_tensor_cores=True)
                w.plan(indptr, indices, last, cfg.n_q_heads, cfg.n_kv_heads, cfg.head_dim, page,
                       q_data_type=q.dtype, kv_data_type=kc.dtype, sm_scale=scale)
                state["w"] = w
            o, lse = state["w"].run(q, (kc, vc), return_lse=True)
            return o, lse * 0.6931471805599453      # FlashInfer returns base-2 LSE
        return "flashinfer.BatchDecodeWithPagedKVCacheWrapper (HND pages, tensor cores)", "HND", fi
    except Exception as e:  # noqa: BLE001
        errors.append(f"flashinfer: {e!r}"[:160])
    raise RuntimeError("no stock paged decode attention available: " + "; ".join(errors))


def run_reference(args) -> None:
    if not os.path.isdir(os.path.join(REF, "helix_a2a")):
        return _unavailable("baseline/_ref is missing: the reference could not be installed offline")
    os.environ["HELIX_A2A_BACKEND"] = "native"
    os.environ.setdefault("HELIX_A2A_USE_MNNVL", "1")
    sys.path.insert(0, REF)                      # the reference's helix_a2a, not this repo's shim
    for m in [k for k in sys.modules if k == "helix_a2a" or k.startswith("helix_a2a.")]:
        del sys.modules[m]
    try:
        import torch
        import torch.distributed as dist
        import torch.nn.functional as F
        import bench as _b  # noqa: F401
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"import failed: {e!r}"[:200])
    from bench import ClockSampler, METRIC, barrier, bench_config, init_dist, max_over_ranks, time_op_in_graph

    try:
        rank, world, group, cpu_group = init_dist(args.gpus)
        import helix_a2a as ref_pkg
        if os.path.realpath(os.path.dirname(ref_pkg.__file__)) != os.path.realpath(os.path.join(REF, "helix_a2a")):
            return _unavailable("imported helix_a2a is not the reference install")
        hook = None
        if world > 1:
            spec = importlib.util.spec_from_file_location("ref_dcp_alltoall_helix",
                                                          os.path.join(REF, "patches", "dcp_alltoall_helix.py"))
            hook = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(hook)
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference import failed: {e!r}"[:300])

    import math
    L, Hq, Hkv, D, hidden, page = args.layers, 64, 8, 128, 8192, 16
    batch = args.batch_per_gpu * world
    local_ctx = args.ctx // world
    Hl = Hq // world
    scale = 1.0 / math.sqrt(D)
    dev = torch.device("cuda", torch.cuda.current_device())

    class Cfg:
        n_q_heads, n_kv_heads, head_dim = Hq, Hkv, D
    try:
        att_name, layout, att = _pick_attention(torch, Cfg, batch, dev)
    except Exception as e:  # noqa: BLE001
        return _unavailable(str(e)[:300])

    gen = torch.Generator(device=dev).manual_seed(rank)
    pages_per_seq = (local_ctx + page - 1) // page
    n_pages = batch * pages_per_seq
    bt = torch.randperm(n_pages, generator=torch.Generator().manual_seed(0)).int().view(batch, pages_per_seq).to(dev)
    sl = torch.full((batch,), local_ctx, dtype=torch.int32, device=dev)
    shape = (n_pages, Hkv, page, D) if layout == "HND" else (n_pages, page, Hkv, D)
    kcs, vcs, ws_ = [], [], []
    for _ in range(L):
        kcs.append(torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen))
        vcs.append(torch.empty(shape, dtype=torch.bfloat16, device=dev).normal_(0, 1, generator=gen))
        ws_.append(torch.empty(hidden, Hl * D, dtype=torch.bfloat16, device=dev).normal_(0, 0.02, generator=gen))
    cp = _Group(rank, world, group, cpu_group)
    if world > 1:
        hook.dcp_a2a_ensure_initialized(cp)

    def step(q_all):
        y = None
        for l in range(L):
            o, lse = att(q_all[l], kcs[l], vcs[l], bt, sl, scale, local_ctx)
            if world > 1:
                o = hook.dcp_a2a_lse_reduce(o, lse.float(), cp)
            y = F.linear(o.reshape(batch, Hl * D), ws_[l])
        return y

    g7 = torch.Generator().manual_seed(7)
    q_host = [torch.randn(L, batch, Hq, D, generator=g7).bfloat16().pin_memory() for _ in range(2)]
    q_dev = q_host[0].to(dev)
    out_pinned = torch.empty(batch, hidden, dtype=torch.bfloat16).pin_memory()
    try:
        step(q_dev)
        barrier(world)
    except Exception as e:  # noqa: BLE001
        return _unavailable(f"reference step failed with {att_name}: {e!r}"[:400])

    graph, static_q, static_y = None, q_dev.clone(), None
    if not args.no_graph:
        try:
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                step(static_q)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=s):
                    static_y = step(static_q)
            torch.cuda.current_stream().wait_stream(s)
        except Exception:  # noqa: BLE001
            graph = None
            torch.cuda.synchronize()

    def run_dev():
        if graph is not None:
            graph.replay()
            return static_y
        return step(static_q)

    def run_host(qp):
        static_q.copy_(qp, non_blocking=True)
        y = run_dev()
        out_pinned.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()

    for _ in range(max(args.warmup, 3)):
        run_dev()
    barrier(world)
    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        run_dev()
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world) / args.steps
    for i in range(2):
        run_host(q_host[i % 2])
    barrier(world)
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(args.steps):
        run_host(q_host[i % 2])
    t1.record()
    barrier(world)
    ms_e2e = max_over_ranks(t0.elapsed_time(t1), world) / args.steps
    clocks = sampler.stop()

    a2a_us = None
    if world > 1:
        o = torch.randn(batch, Hq, D, device=dev).bfloat16()
        lse = torch.randn(batch, Hq, device=dev)
        try:
            a2a_us = time_op_in_graph(lambda: hook.dcp_a2a_lse_reduce(o, lse, cp), world)
        except Exception:  # noqa: BLE001  (capture refused: leave the figure out rather than report host overhead)
            a2a_us = None
            torch.cuda.synchronize()

    if rank == 0:
        kv_bytes = 2 * L * batch * local_ctx * Hkv * D * 2
        print(json.dumps({
            "metric": METRIC, "value": batch / (ms * 1e-3), "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic (random-init weights, KV ~ N(0,1), random q)",
            "impl": "reference",
            "config": bench_config(L, batch, args.ctx, world, page, local_ctx, kv_bytes, graph is not None),
            "clocks": clocks,
            "e2e": {"value": batch / (ms_e2e * 1e-3), "unit": "tok/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": L * batch * Hq * D * 2, "d2h_bytes_per_step": batch * hidden * 2},
            "gpu_launches": 0,
            "extras": {"helix_a2a_combine_us": a2a_us, "helix_a2a_combine_us_how": "CUDA graph of 20 calls, replayed",
                       "path": {"attention": att_name,
                                "exchange": "reference helix_a2a.alltoall + its Triton combine" if world > 1
                                else "none (cp=1 passthrough in the reference's hook)",
                                "o_proj": "torch.nn.functional.linear", "pdl": False}},
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()
