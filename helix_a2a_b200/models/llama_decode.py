"""Llama-3-70B-architecture decode stack under Helix context parallelism.

One decode step of the attention block of every layer on one CP rank::

    split-KV paged attention over the LOCAL KV shard   ->  (o [B, Hq, D], lse [B, Hq])
    Helix exchange + LSE combine (head scatter)        ->  x [B, Hq/N, D]
    o_proj with this rank's K-slice of W_o             ->  y [B, hidden]   (partial sum over ranks)

The KV cache of every sequence is split evenly over the ``cp_size`` ranks; each rank holds all KV
heads of its shard.  Weights are random-init (N(0, 0.02)), KV ~ N(0, 1): there is no checkpoint
loading here, the stack exists to drive and measure the kernels on the shapes of a real model.
The reference leaves all of this to vLLM (``benchmark/sbatch/run_gb200_aiperf_v3.sbatch:284-305``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import api
from ..ops import attention, oproj as oproj_mod
from ..utils import env
from ..utils.tracing import nvtx_range


@dataclass
class LlamaDecodeConfig:
    n_layers: int = 80
    n_q_heads: int = 64
    n_kv_heads: int = 8
    head_dim: int = 128
    hidden: int = 8192
    page_size: int = 16
    dtype: torch.dtype = torch.bfloat16

    @staticmethod
    def llama3_70b(**kw) -> "LlamaDecodeConfig":
        return LlamaDecodeConfig(**kw)

    @staticmethod
    def tiny(**kw) -> "LlamaDecodeConfig":
        base = dict(n_layers=2, n_q_heads=16, n_kv_heads=2, head_dim=128, hidden=256)
        base.update(kw)
        return LlamaDecodeConfig(**base)


class HelixDecodeStack:
    """KV cache shard, o_proj slices and workspace of one CP rank, plus the decode step."""

    def __init__(self, cfg: LlamaDecodeConfig, *, batch: int, local_ctx: int, cp_size: int = 1, cp_rank: int = 0,
                 group: Optional[dist.ProcessGroup] = None, device="cuda", seed: int = 0,
                 workspace: Optional[torch.Tensor] = None, kv_std: float = 1.0,
                 fuse_oproj: Optional[bool] = False):
        assert cfg.n_q_heads % cp_size == 0, "query heads must divide evenly over the CP ranks"
        self.cfg, self.batch, self.local_ctx = cfg, batch, local_ctx
        self.cp_size, self.cp_rank, self.group = cp_size, cp_rank, group
        self.device = torch.device(device)
        self.heads_local = cfg.n_q_heads // cp_size
        # exchange + combine + o_proj as one kernel: True / False, or None = whenever the shape fits that kernel
        # (a request that does not fit runs the two-kernel chain, and is counted as such)
        fits = cp_size > 1 and self.device.type == "cuda" and api.alltoall_combine_oproj_fits(
            batch, self.heads_local, cfg.head_dim, cfg.hidden, cp_size)
        self.fuse_oproj = bool(fits) if fuse_oproj is None else bool(fuse_oproj and fits)
        self.k_local = self.heads_local * cfg.head_dim
        self.scale = 1.0 / math.sqrt(cfg.head_dim)
        gen = torch.Generator(device=self.device)
        gen.manual_seed(seed * 1000 + cp_rank)
        pages_per_seq = (local_ctx + cfg.page_size - 1) // cfg.page_size
        self.n_pages = batch * pages_per_seq
        # pages of a sequence are scattered over the pool, as a paged allocator would leave them
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).int()
        self.block_table = perm.view(batch, pages_per_seq).to(self.device)
        self.seq_lens = torch.full((batch,), local_ctx, dtype=torch.int32, device=self.device)
        shape = (self.n_pages, cfg.n_kv_heads, cfg.page_size, cfg.head_dim)
        self.k_cache: List[torch.Tensor] = []
        self.v_cache: List[torch.Tensor] = []
        self.w_o: List[torch.Tensor] = []
        self.prepack_oproj = env.oproj_prepack()
        self._w_o_packed = [None] * cfg.n_layers
        for _ in range(cfg.n_layers):
            k = torch.empty(shape, dtype=cfg.dtype, device=self.device).normal_(0, kv_std, generator=gen)
            v = torch.empty(shape, dtype=cfg.dtype, device=self.device).normal_(0, kv_std, generator=gen)
            w = torch.empty(cfg.hidden, self.k_local, dtype=cfg.dtype, device=self.device).normal_(0, 0.02, generator=gen)
            self.k_cache.append(k)
            self.v_cache.append(v)
            self.w_o.append(w)
        if workspace is not None:
            self.workspace = workspace
        elif cp_size > 1:
            self.workspace = api.allocate_workspace(cp_size, cp_rank, device=device if self.device.type == "cpu" else "cuda",
                                                    mnnvl=True, cpu_group=group)
            api.init_workspace(self.workspace, cp_rank, cp_size)
            dist.barrier(group=group)
        else:
            self.workspace = None
        self._graph = None
        self._static_q = None
        self._static_y = None

    # ---- one layer / one step --------------------------------------------------------------------
    def layer(self, l: int, q: torch.Tensor) -> torch.Tensor:
        with nvtx_range(f"layer{l}.attention"):
            o, lse = attention.gqa_decode(q, self.k_cache[l], self.v_cache[l], self.block_table, self.seq_lens,
                                          scale=self.scale, max_seq_len=self.local_ctx, kv_stable=True)
        if self.cp_size > 1 and self.fuse_oproj:
            # exchange + combine + o_proj in one launch: W_o streams while the exchange is in flight
            return api.alltoall_combine_oproj(o, lse, self._oproj_weight(l), self.workspace, self.cp_rank, self.cp_size)
        if self.cp_size > 1:
            x = api.alltoall_combine(o, lse, self.workspace, self.cp_rank, self.cp_size)
        else:
            x = o
        return oproj_mod.oproj(x.reshape(self.batch, self.k_local), self._oproj_weight(l))

    def _oproj_weight(self, l: int):
        """The layer's o_proj weight in the layout the GEMM streams fastest: packed once, on first use
        (one contiguous bulk copy per pipeline stage instead of strided tensor copies); the plain matrix
        stays in ``w_o`` for the one-kernel path and for oracles.  ``prepack_oproj=False`` keeps the plain one."""
        if not self.prepack_oproj or not self.w_o[l].is_cuda or self.w_o[l].shape[0] % 128 or self.w_o[l].shape[1] % 64:
            return self.w_o[l]
        if self._w_o_packed[l] is None:
            self._w_o_packed[l] = oproj_mod.prepack_weight(self.w_o[l])
        return self._w_o_packed[l]

    def decode_step(self, q_all: torch.Tensor) -> torch.Tensor:
        """``q_all [L, B, Hq, D]`` on the device -> ``y [L, B, hidden]`` (this rank's partial sums)."""
        ys = [self.layer(l, q_all[l]) for l in range(self.cfg.n_layers)]
        return torch.stack(ys)

    def _run_layers(self, q_all: torch.Tensor, l0: int, l1: int) -> torch.Tensor:
        y = None
        for l in range(l0, l1):
            y = self.layer(l, q_all[l])
        return y

    def _step_last(self, q_all: torch.Tensor) -> torch.Tensor:
        return self._run_layers(q_all, 0, self.cfg.n_layers)

    # ---- end-to-end call: pinned host input -> host output ---------------------------------------
    def capture(self, q_example: torch.Tensor, head_layers: Optional[int] = None) -> None:
        """Capture the step in CUDA graphs (call after at least one eager warm-up step).

        Two graphs: the first ``head_layers`` layers and the rest.  ``decode_step_host`` copies the
        queries of the head layers, starts the head graph, and lets the (much larger) copy of the
        remaining layers' queries run on a second stream underneath it; the tail graph waits for that
        copy.  With one graph the whole host-to-device copy sat in front of the first kernel."""
        L = self.cfg.n_layers
        if head_layers is None:
            head_layers = min(8, L // 2)
        self._head_layers = head_layers if 0 < head_layers < L else 0
        self._static_q = torch.empty_like(q_example, device=self.device)
        self._static_q.copy_(q_example)
        self._copy_stream = torch.cuda.Stream(device=self.device)
        self._copy_done = torch.cuda.Event()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._step_last(self._static_q)
            self._graphs = []
            bounds = [(0, self._head_layers), (self._head_layers, L)] if self._head_layers else [(0, L)]
            for l0, l1 in bounds:
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=s):
                    self._static_y = self._run_layers(self._static_q, l0, l1)
                self._graphs.append(g)
        torch.cuda.current_stream(self.device).wait_stream(s)
        self._graph = self._graphs[-1]

    def _replay(self) -> None:
        for g in self._graphs:
            g.replay()

    def decode_step_device(self, q_dev: torch.Tensor) -> torch.Tensor:
        """Step on device-resident ``q``; returns the last layer's ``y`` (``[B, hidden]``)."""
        if self._graph is not None:
            self._static_q.copy_(q_dev, non_blocking=True)
            self._replay()
            return self._static_y
        return self._step_last(q_dev)

    def decode_step_host(self, q_pinned: torch.Tensor, out_pinned: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Public end-to-end step: copies ``q`` from pinned host memory, runs every layer, copies
        the result (``[B, hidden]``) back to the host and waits for it."""
        main = torch.cuda.current_stream(self.device)
        if self._graph is not None:
            k = self._head_layers
            if k:
                # the previous step ended with a synchronize, so nothing still reads _static_q
                self._static_q[:k].copy_(q_pinned[:k], non_blocking=True)
                self._copy_stream.wait_stream(main)
                with torch.cuda.stream(self._copy_stream):
                    self._static_q[k:].copy_(q_pinned[k:], non_blocking=True)
                    self._copy_done.record(self._copy_stream)
                self._graphs[0].replay()
                main.wait_event(self._copy_done)
                self._graphs[1].replay()
            else:
                self._static_q.copy_(q_pinned, non_blocking=True)
                self._replay()
            y = self._static_y
        else:
            q_dev = torch.empty_like(q_pinned, device=self.device)
            q_dev.copy_(q_pinned, non_blocking=True)
            y = self._step_last(q_dev)
        if out_pinned is None:
            out_pinned = torch.empty(y.shape, dtype=y.dtype, pin_memory=True)
        out_pinned.copy_(y, non_blocking=True)
        main.synchronize()
        return out_pinned

    # ---- accounting ------------------------------------------------------------------------------
    def kernels_per_step(self) -> int:
        return self.cfg.n_layers * ((2 if self.fuse_oproj else 3) if self.cp_size > 1 else 2)

    def h2d_bytes_per_step(self) -> int:
        c = self.cfg
        return c.n_layers * self.batch * c.n_q_heads * c.head_dim * 2

    def d2h_bytes_per_step(self) -> int:
        return self.batch * self.cfg.hidden * 2
