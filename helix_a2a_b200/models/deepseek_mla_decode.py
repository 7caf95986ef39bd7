"""DeepSeek-V3-architecture MLA decode stack under Helix context parallelism.

Per layer on one CP rank (absorbed / latent form of MLA)::

    MLA decode over the LOCAL block-scaled fp8 latent cache  ->  (o [B, 128, 512], lse [B, 128])
    Helix exchange + LSE combine (head scatter)               ->  x [B, 128/N, 512]
    o_proj with W_uv folded into W_o, this rank's K-slice     ->  y [B, hidden]  (partial sum over ranks)

128 heads, kv_lora_rank 512, rope dim 64, hidden 7168, 61 layers; cache = e4m3 latent with one fp32
scale per 128 values plus bf16 rope keys (656 bytes per token).  Weights are random-init and the
cache is quantised random data: the stack exists to drive and measure the kernels.  In the
reference this model runs inside vLLM (``benchmark/sbatch/run_gb200_aiperf_v3.sbatch:93-127``).
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.distributed as dist

from .. import api
from ..ops import attention, oproj as oproj_mod, reference_math as rm
from ..utils import env


@dataclass
class MlaDecodeConfig:
    n_layers: int = 61
    n_heads: int = 128
    kv_lora_rank: int = 512
    rope_dim: int = 64
    qk_nope_dim: int = 128
    hidden: int = 7168
    page_size: int = 16

    @staticmethod
    def tiny(**kw) -> "MlaDecodeConfig":
        base = dict(n_layers=2, hidden=256)
        base.update(kw)
        return MlaDecodeConfig(**base)


class MlaDecodeStack:
    def __init__(self, cfg: MlaDecodeConfig, *, batch: int, local_ctx: int, cp_size: int = 1, cp_rank: int = 0,
                 group: Optional[dist.ProcessGroup] = None, device="cuda", seed: int = 0, fuse_oproj: bool = False):
        assert cfg.n_heads == 128 and cfg.kv_lora_rank == 512 and cfg.rope_dim == 64, "kernel is built for the V3 shape"
        assert cfg.n_heads % cp_size == 0
        self.cfg, self.batch, self.local_ctx = cfg, batch, local_ctx
        self.cp_size, self.cp_rank, self.group, self.fuse_oproj = cp_size, cp_rank, group, fuse_oproj
        self.device = torch.device(device)
        self.heads_local = cfg.n_heads // cp_size
        self.k_local = self.heads_local * cfg.kv_lora_rank
        self.scale = 1.0 / math.sqrt(cfg.qk_nope_dim + cfg.rope_dim)
        gen = torch.Generator(device=self.device).manual_seed(seed * 1000 + cp_rank)
        pages_per_seq = (local_ctx + cfg.page_size - 1) // cfg.page_size
        self.n_pages = batch * pages_per_seq
        perm = torch.randperm(self.n_pages, generator=torch.Generator().manual_seed(seed)).int()
        self.block_table = perm.view(batch, pages_per_seq).to(self.device)
        self.seq_lens = torch.full((batch,), local_ctx, dtype=torch.int32, device=self.device)
        self.ckv: List[torch.Tensor] = []
        self.scales: List[torch.Tensor] = []
        self.kpe: List[torch.Tensor] = []
        self.w_o: List[torch.Tensor] = []
        self.prepack_oproj = env.oproj_prepack()
        self._w_o_packed = [None] * cfg.n_layers
        for _ in range(cfg.n_layers):
            # quantise in slabs to bound the fp32 temporaries
            ckv = torch.empty(self.n_pages, cfg.page_size, 512, dtype=torch.float8_e4m3fn, device=self.device)
            sc = torch.empty(self.n_pages, cfg.page_size, 4, dtype=torch.float32, device=self.device)
            step = max(1, (1 << 26) // (cfg.page_size * 512))
            for p0 in range(0, self.n_pages, step):
                n = min(step, self.n_pages - p0)
                lat = torch.empty(n, cfg.page_size, 512, device=self.device).normal_(0, 1, generator=gen)
                q8, s = rm.quantize_fp8_blockscaled(lat, 128)
                ckv[p0:p0 + n] = q8
                sc[p0:p0 + n] = s
            self.ckv.append(ckv)
            self.scales.append(sc)
            self.kpe.append(torch.empty(self.n_pages, cfg.page_size, 64, dtype=torch.bfloat16,
                                        device=self.device).normal_(0, 1, generator=gen))
            self.w_o.append(torch.empty(cfg.hidden, self.k_local, dtype=torch.bfloat16,
                                        device=self.device).normal_(0, 0.02, generator=gen))
        if cp_size > 1:
            self.workspace = api.allocate_workspace(cp_size, cp_rank, device="cpu" if self.device.type == "cpu" else "cuda",
                                                    mnnvl=True, cpu_group=group)
            api.init_workspace(self.workspace, cp_rank, cp_size)
            dist.barrier(group=group)
        else:
            self.workspace = None
        self._graph = None

    def layer(self, l: int, q_nope: torch.Tensor, q_pe: torch.Tensor) -> torch.Tensor:
        o, lse = attention.mla_decode(q_nope, q_pe, self.ckv[l], self.scales[l], self.kpe[l], self.block_table,
                                      self.seq_lens, scale=self.scale, max_seq_len=self.local_ctx)
        if self.cp_size > 1 and self.fuse_oproj:
            return api.alltoall_combine_oproj(o, lse, self.w_o[l], self.workspace, self.cp_rank, self.cp_size)
        x = api.alltoall_combine(o, lse, self.workspace, self.cp_rank, self.cp_size) if self.cp_size > 1 else o
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

    def decode_step(self, q_nope_all: torch.Tensor, q_pe_all: torch.Tensor) -> torch.Tensor:
        """``q_nope_all [L, B, 128, 512]``, ``q_pe_all [L, B, 128, 64]`` -> last layer's ``y [B, hidden]``."""
        y = None
        for l in range(self.cfg.n_layers):
            y = self.layer(l, q_nope_all[l], q_pe_all[l])
        return y

    def capture(self, q_nope_all, q_pe_all) -> None:
        self._qn, self._qp = q_nope_all.clone(), q_pe_all.clone()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self.decode_step(self._qn, self._qp)
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                self._y = self.decode_step(self._qn, self._qp)
        torch.cuda.current_stream(self.device).wait_stream(s)
        self._graph = g

    def step(self, q_nope_all, q_pe_all) -> torch.Tensor:
        if self._graph is not None:
            self._qn.copy_(q_nope_all, non_blocking=True)
            self._qp.copy_(q_pe_all, non_blocking=True)
            self._graph.replay()
            return self._y
        return self.decode_step(q_nope_all, q_pe_all)

    def kv_bytes_per_step(self) -> int:
        return self.cfg.n_layers * self.batch * self.local_ctx * (512 + 16 + 128)

    def attention_flops_per_step(self) -> int:
        return self.cfg.n_layers * self.batch * self.local_ctx * 128 * (576 + 512) * 2
