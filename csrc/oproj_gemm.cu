// Decode o_proj GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulator in TMEM).
//
// Decode batches are small (1..256 tokens) while `hidden` is large, so the product is computed
// transposed ("swap-AB"): the 128-row UMMA M dimension walks `hidden` (rows of W), the token count
// is the UMMA N dimension (padded to a multiple of 16) and D[128, n_pad] fp32 lives in TMEM.  The
// kernel is bound by streaming W once from HBM:
//   grid (hidden / 128, splits); each CTA owns one 128-row slab of W and 1/splits of K;
//   warp 0 (one lane) feeds a ring of shared-memory stages with TMA tiled loads (128-byte swizzle,
//     four [128 x 64] W boxes + four [n_pad x 64] x boxes per stage, no cluster broadcast);
//   warp 1 (one lane) issues sixteen K=16 UMMAs per stage and releases the stage with
//     tcgen05.commit; after the last stage it commits to the accumulator barrier;
//   all four warps then read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32w..32w+31)
//     and write y (bf16) or, with split-K, park an fp32 partial in scratch memory where the last
//     CTA of the slab sums the splits.
// With programmatic dependent launch the W tiles of the first stages are requested BEFORE the
// grid-dependency wait: only the activations depend on the preceding exchange kernel, so the
// weight stream overlaps it.  All mbarrier waits are bounded.
#include "oproj.h"

#include <algorithm>

#include "oproj_device.cuh"

namespace helix {
namespace {

using namespace oproj_dev;

__global__ void __launch_bounds__(kThreads, 1) oproj_kernel(const __grid_constant__ OprojParams p) {
  extern __shared__ uint8_t smem_raw[];
  oproj_cta(
      p, smem_raw, blockIdx.x, blockIdx.y, threadIdx.x, [] { __syncthreads(); },
      [](unsigned long long) {
        // with programmatic dependent launch the activations are valid once the preceding grid is done
        asm volatile("griddepcontrol.wait;" ::: "memory");
        return true;
      });
}

// ---- stream-K variant ---------------------------------------------------------------------------------
// Work units are (128-row slab of W, k-block) pairs in slab-major order; CTA c owns the contiguous unit
// range [c U / G, (c + 1) U / G), which may end one slab and begin the next.  Six warps: warp 0 feeds the
// TMA ring across slab boundaries, warp 1 issues the UMMAs (a new accumulation starts at every slab
// boundary, once the epilogue has drained TMEM), warps 2..5 read the accumulator out.  A segment that
// covers its slab's whole K range writes y directly; otherwise it parks an fp32 piece (slot 1 if it
// starts the slab, slot 0 if it continues it) and the last CTA to finish a slab sums the pieces.
constexpr int kSkThreads = 192;
constexpr int kEpiBarrier = 1;

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync %0, %1;" ::"r"(kEpiBarrier), "r"(128) : "memory"); }

__global__ void __launch_bounds__(kSkThreads, 1) oproj_streamk_kernel(const __grid_constant__ OprojParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_bar, free_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort, s_last;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  unsigned long long* tr = p.trace ? p.trace + (size_t)blockIdx.x * 8 : nullptr;
  if (tr && tid == 0) tr[0] = now_ns();
  const int stages = p.stages, atoms = p.atoms;
  const int bk = kAtomK * atoms;
  const uint32_t atom_a_bytes = kBM * kAtomK * 2, atom_b_bytes = (uint32_t)p.n_pad * kAtomK * 2;
  const uint32_t a_bytes = atom_a_bytes * atoms, b_bytes = atom_b_bytes * atoms, stage_bytes = a_bytes + b_bytes;
  const int kb_total = (p.K + bk - 1) / bk;
  const long long U = (long long)(p.hidden / kBM) * kb_total, G = gridDim.x;
  const long long u0 = (long long)blockIdx.x * U / G, u1 = (long long)(blockIdx.x + 1) * U / G;
  const int n_units = (int)(u1 - u0);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.n_pad) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
    mbar_init(&free_bar, 4);
    mbar_fence_init();
    s_abort = 0;
    tma_prefetch_desc(&p.w_map);
    tma_prefetch_desc(&p.x_map);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_slot;
  const unsigned long long deadline = now_ns() + p.timeout_ns;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (tr && tid == 0) tr[1] = now_ns();

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- producer ----------------
      auto load_w = [&](int s, long long u) {
        const int m = (int)(u / kb_total), kb = (int)(u % kb_total);
        for (int a = 0; a < atoms; ++a)
          tma_load_2d(smem + (size_t)s * stage_bytes + (size_t)a * atom_a_bytes, &p.w_map, &full_bar[s],
                      kb * bk + a * kAtomK, m * kBM);
      };
      auto load_x = [&](int s, long long u) {
        const int kb = (int)(u % kb_total);
        for (int a = 0; a < atoms; ++a)
          tma_load_2d(smem + (size_t)s * stage_bytes + a_bytes + (size_t)a * atom_b_bytes, &p.x_map, &full_bar[s],
                      kb * bk + a * kAtomK, 0);
      };
      const int pre = min(stages, n_units);
      for (int i = 0; i < pre; ++i) {       // weights first: they do not depend on the kernel before us
        mbar_expect_tx(&full_bar[i], stage_bytes);
        load_w(i, u0 + i);
      }
      asm volatile("griddepcontrol.wait;" ::: "memory");
      for (int i = 0; i < pre; ++i) load_x(i, u0 + i);
      for (int i = pre; i < n_units; ++i) {
        const int s = i % stages;
        if (!mbar_wait(&empty_bar[s], (uint32_t)(((i / stages) - 1) & 1), deadline)) {
          fail(p, &s_abort);
          break;
        }
        mbar_expect_tx(&full_bar[s], stage_bytes);
        load_w(s, u0 + i);
        load_x(s, u0 + i);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t idesc = umma_idesc_bf16(kBM, p.n_pad);
      int seg = 0;
      for (int i = 0; i < n_units; ++i) {
        const long long u = u0 + i;
        const int kb = (int)(u % kb_total);
        const bool seg_first = (i == 0 || kb == 0), seg_last = (i == n_units - 1 || kb == kb_total - 1);
        if (seg_first && i > 0) {
          // the epilogue warps must have read the previous slab's accumulator out of TMEM
          if (!mbar_wait(&free_bar, (uint32_t)((seg - 1) & 1), deadline)) {
            fail(p, &s_abort);
            break;
          }
          tc_fence_after_sync();
        }
        const int s = i % stages;
        if (!mbar_wait(&full_bar[s], (uint32_t)((i / stages) & 1), deadline)) {
          fail(p, &s_abort);
          break;
        }
        tc_fence_after_sync();
        if (tr && i == 0) tr[2] = now_ns();
        const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes), b_addr = a_addr + a_bytes;
        for (int a = 0; a < atoms; ++a) {
#pragma unroll
          for (int k = 0; k < kAtomK / 16; ++k)
            umma_bf16(tmem_d, umma_desc_k_sw128(a_addr + a * atom_a_bytes + k * 32),
                      umma_desc_k_sw128(b_addr + a * atom_b_bytes + k * 32), idesc, !(seg_first && a == 0 && k == 0));
        }
        umma_commit(&empty_bar[s]);
        if (seg_last) {
          umma_commit(&acc_bar);
          ++seg;
        }
      }
      if (tr) tr[3] = now_ns();
    }
  } else {
    // ---------------- epilogue warps 2..5: TMEM lane quadrant = warp % 4 ----------------
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const int etid = (warp - 2) * 32 + lane;       // 0..127 among the epilogue threads
    int seg = 0;
    long long u = u0;
    while (u < u1) {
      const int m = (int)(u / kb_total), kb_begin = (int)(u % kb_total);
      const int kb_end = (int)min((long long)kb_total, kb_begin + (u1 - u));
      const bool whole = (kb_begin == 0 && kb_end == kb_total);
      // only lane 0 polls; the result is broadcast so that a failed wait cannot split the warp
      int good = 1;
      if (lane == 0) {
        unsigned spins = 0;
        while (!mbar_try_wait(&acc_bar, (uint32_t)(seg & 1))) {
          if ((++spins & 63u) == 0u && (*reinterpret_cast<volatile int*>(&s_abort) || now_ns() > deadline)) {
            good = 0;
            break;
          }
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      if (!good) {
        if (lane == 0) fail(p, &s_abort);
        break;
      }
      tc_fence_after_sync();
      if (tr && etid == 0) tr[4] = now_ns();
      const int slot = (kb_begin == 0) ? 1 : 0;
      float* part = p.partial + ((size_t)(blockIdx.x * 2 + slot) * p.n_pad) * kBM;
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_d + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = c0 + j;
          if (whole) {
            if (tok < p.tokens) p.y[(int64_t)tok * p.y_stride + m * kBM + row] = __float2bfloat16(__uint_as_float(v[j]));
          } else {
            part[(size_t)tok * kBM + row] = __uint_as_float(v[j]);
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&free_bar);        // TMEM may be overwritten by the next slab
      if (!whole) {
        // count this piece; the last CTA of the slab sums all of them
        const long long t0 = (long long)m * kb_total, t1 = t0 + kb_total - 1;
        const int c_first = (int)(((t0 + 1) * G + U - 1) / U - 1), c_last = (int)(((t1 + 1) * G + U - 1) / U - 1);
        epi_sync();
        if (etid == 0) {
          int prev;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + m) : "memory");
          s_last = (prev == c_last - c_first);
        }
        epi_sync();
        if (s_last) {
          for (int tok0 = 0; tok0 < p.tokens; tok0 += 8) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            for (int c = c_first; c <= c_last; ++c) {
              const float* src = p.partial + ((size_t)(c * 2 + (c == c_first ? 1 : 0)) * p.n_pad) * kBM;
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] += __ldcg(src + (size_t)(tok0 + j) * kBM + etid);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j)
              if (tok0 + j < p.tokens)
                p.y[(int64_t)(tok0 + j) * p.y_stride + m * kBM + etid] = __float2bfloat16(acc[j]);
          }
          if (etid == 0) p.counters[m] = 0;
        }
        epi_sync();
      }
      u += (kb_end - kb_begin);
      ++seg;
    }
    if (tr && etid == 0) tr[5] = now_ns();
  }
  __syncwarp();   // the producer / issuer lane rejoins its warp before the block-wide barrier
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
}

}  // namespace

int oproj_pick_atoms(int n_pad) { return n_pad <= 64 ? 4 : (n_pad <= 128 ? 2 : 1); }

int oproj_pick_splits(int hidden, int K, int sm_count) {
  // split K only when one CTA per 128-row slab would leave SMs idle for long: each CTA should still
  // stream at least 256 KB of W
  const int m_tiles = hidden / kBM;
  int splits = std::max(1, sm_count / std::max(m_tiles, 1));
  const int kb_total = (K + 255) / 256;
  while (splits > 1 && kb_total / splits < 4) --splits;
  return std::min(splits, 8);
}

int oproj_smem_bytes(int n_pad, int stages) {
  return stages * (kBM + n_pad) * kAtomK * oproj_pick_atoms(n_pad) * 2 + 1024;
}

int oproj_pick_stages(int n_pad) {
  const int stage = (kBM + n_pad) * kAtomK * oproj_pick_atoms(n_pad) * 2;
  int s = (222 * 1024) / stage;
  return std::max(2, std::min(s, kMaxStages));
}

cudaError_t launch_oproj(const OprojParams& p, bool pdl, cudaStream_t stream) {
  if (p.tokens <= 0) return cudaSuccess;
  if (p.hidden % kBM != 0 || p.K % kAtomK != 0 || p.n_pad % 16 != 0 || p.n_pad < 16 || p.n_pad > 256 ||
      p.tokens > p.n_pad || (p.atoms != 1 && p.atoms != 2 && p.atoms != 4) || p.stages < 2 || p.stages > kMaxStages || p.splits < 1)
    return cudaErrorInvalidValue;
  const int smem = oproj_smem_bytes(p.n_pad, p.stages);
  if (p.splits > 1 && p.partial == nullptr) return cudaErrorInvalidValue;
  cudaError_t e = cudaFuncSetAttribute(oproj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.hidden / kBM, p.splits, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, oproj_kernel, p);
}


// Stream-K is picked only when the plain grid (slabs x splits) would leave more than a fifth of the SMs idle,
// there are at least 8 units per CTA to deal out, and the token tile is small (the piece fold grows with
// n_pad: at 256 tokens and K = 1024 it costs 51 us against 18 us plain).  With a fuller plain grid the two run
// level (8192 x 8192 under programmatic launch: 128 plain CTAs 26.0 us, 148 stream-K CTAs 26.6 us).
bool oproj_streamk_pays(int hidden, int K, int n_pad, int sm_count) {
  const int bk = kAtomK * oproj_pick_atoms(n_pad);
  const long long units = (long long)(hidden / kBM) * ((K + bk - 1) / bk);
  const int plain_ctas = (hidden / kBM) * oproj_pick_splits(hidden, K, sm_count);
  return n_pad <= 32 && plain_ctas * 5 < sm_count * 4 && units >= 8LL * sm_count;
}

cudaError_t launch_oproj_streamk(const OprojParams& p, bool pdl, cudaStream_t stream) {
  if (p.tokens <= 0) return cudaSuccess;
  if (p.hidden % kBM != 0 || p.K % kAtomK != 0 || p.n_pad % 16 != 0 || p.n_pad < 16 || p.n_pad > 256 ||
      p.tokens > p.n_pad || (p.atoms != 1 && p.atoms != 2 && p.atoms != 4) || p.stages < 2 || p.stages > kMaxStages ||
      p.ctas < 1 || p.partial == nullptr)
    return cudaErrorInvalidValue;
  const int smem = oproj_smem_bytes(p.n_pad, p.stages);
  cudaError_t e = cudaFuncSetAttribute(oproj_streamk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.ctas, 1, 1);
  cfg.blockDim = dim3(kSkThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, oproj_streamk_kernel, p);
}

}  // namespace helix
