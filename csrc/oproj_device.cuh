// CTA body of the decode o_proj GEMM (tcgen05.mma, accumulator in TMEM), shared by the stand-alone
// kernel and by the kernel that fuses it with the Helix exchange.  See oproj_gemm.cu for the design.
//
// `sync_cta()` synchronises the 128 threads that run this body; `wait_input(deadline)` is called by
// the producer thread after it has requested the first W tiles and before it requests any x tile: it
// returns once the activations are valid (and false if that never happened within the time limit).
#pragma once

#include "helix_common.cuh"
#include "oproj.h"
#include "sm100.cuh"

namespace helix {
namespace oproj_dev {

using namespace sm100;

constexpr int kBM = 128;    // rows of W per CTA (UMMA M)
constexpr int kAtomK = 64;  // one 128-byte swizzle atom of bf16
constexpr int kMaxStages = 6;
constexpr int kThreads = 128;

__device__ __forceinline__ void fail(const OprojParams& p, int* s_abort) {
  atomicCAS(p.error_flag, 0, (int)kTimeoutMbarrier);
  *reinterpret_cast<volatile int*>(s_abort) = 1;
}

template <class SyncCta, class WaitInput>
__device__ __forceinline__ void oproj_cta(const OprojParams& p, uint8_t* smem_raw, int m_tile, int split, int tid,
                                          SyncCta sync_cta, WaitInput wait_input) {
  __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort, s_last;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = tid >> 5, lane = tid & 31;
  const int stages = p.stages;
  const int kAtoms = p.atoms;
  const int kBK = kAtomK * kAtoms;
  const uint32_t atom_a_bytes = kBM * kAtomK * 2, atom_b_bytes = (uint32_t)p.n_pad * kAtomK * 2;
  const uint32_t a_bytes = atom_a_bytes * kAtoms, b_bytes = atom_b_bytes * kAtoms;
  const uint32_t stage_bytes = a_bytes + b_bytes;          // multiples of 1024
  const int kb_total = (p.K + kBK - 1) / kBK;   // a ragged last block is zero-filled by TMA
  const int kb_per = (kb_total + p.splits - 1) / p.splits;
  const int kb0 = split * kb_per;
  const int nkb = max(0, min(kb_total, kb0 + kb_per) - kb0);
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < p.n_pad) tmem_cols <<= 1;

  if (tid == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(&acc_bar, 1);
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
  sync_cta();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_slot;
  const unsigned long long deadline = now_ns() + p.timeout_ns;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == 0 && lane == 0) {
    // ---------------- producer ----------------
    auto load_w = [&](int s, int i) {
      if (p.w_packed != nullptr) {
        // pre-packed weights: the stage's atoms are contiguous and already swizzled
        bulk_load_1d(smem + (size_t)s * stage_bytes,
                     p.w_packed + ((size_t)m_tile * p.packed_atoms + (size_t)(kb0 + i) * kAtoms) * atom_a_bytes, a_bytes,
                     &full_bar[s]);
        return;
      }
      for (int a = 0; a < kAtoms; ++a)
        tma_load_2d(smem + (size_t)s * stage_bytes + (size_t)a * atom_a_bytes, &p.w_map, &full_bar[s],
                    (kb0 + i) * kBK + a * kAtomK, m_tile * kBM);
    };
    auto load_x = [&](int s, int i) {
      for (int a = 0; a < kAtoms; ++a)
        tma_load_2d(smem + (size_t)s * stage_bytes + a_bytes + (size_t)a * atom_b_bytes, &p.x_map, &full_bar[s],
                    (kb0 + i) * kBK + a * kAtomK, 0);
    };
    // weights first: they do not depend on the kernel before us
    const int pre = min(stages, nkb);
    for (int i = 0; i < pre; ++i) {
      mbar_expect_tx(&full_bar[i], stage_bytes);
      load_w(i, i);
    }
    if (!wait_input(deadline)) {
      fail(p, &s_abort);
    } else {
      for (int i = 0; i < pre; ++i) load_x(i, i);
    for (int i = pre; i < nkb; ++i) {
      const int s = i % stages;
      if (!mbar_wait(&empty_bar[s], (uint32_t)(((i / stages) - 1) & 1), deadline)) {
        fail(p, &s_abort);
        break;
      }
      mbar_expect_tx(&full_bar[s], stage_bytes);
      load_w(s, i);
      load_x(s, i);
    }
    }
  } else if (warp == 1 && lane == 0) {
    // ---------------- MMA issuer ----------------
    const uint32_t idesc = umma_idesc_bf16(kBM, p.n_pad);
    bool ok = true;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % stages;
      if (!mbar_wait(&full_bar[s], (uint32_t)((i / stages) & 1), deadline)) {
        fail(p, &s_abort);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
      const uint32_t b_addr = a_addr + a_bytes;
      for (int a = 0; a < kAtoms; ++a) {
#pragma unroll
        for (int k = 0; k < kAtomK / 16; ++k) {
          umma_bf16(tmem_d, umma_desc_k_sw128(a_addr + a * atom_a_bytes + k * 32),
                    umma_desc_k_sw128(b_addr + a * atom_b_bytes + k * 32), idesc, (i | a | k) != 0);
        }
      }
      umma_commit(&empty_bar[s]);          // stage reusable once these MMAs have read it
    }
    if (ok) umma_commit(&acc_bar);         // accumulator complete
  }
  if (warp >= 0) {
    // ---------------- epilogue (all four warps) ----------------
    __syncwarp();
    bool ok = true;
    if (nkb > 0) {
      // only lane 0 polls, then the result is broadcast: a failed wait must not diverge the warp
      int good = 1;
      if (lane == 0) {
        unsigned spins = 0;
        while (!mbar_try_wait(&acc_bar, 0)) {
          if ((++spins & 63u) == 0u) {
            if (*reinterpret_cast<volatile int*>(&s_abort) || now_ns() > deadline) {
              good = 0;
              break;
            }
          }
        }
      }
      good = __shfl_sync(0xffffffffu, good, 0);
      ok = good != 0;
      if (!ok && lane == 0) fail(p, &s_abort);
    } else {
      // A CTA without any k-block has nothing that orders it behind the preceding kernel (no activation tile to wait
      // for), but it writes a zero partial into scratch memory and counts itself in: under programmatic dependent
      // launch that must not happen while the preceding launch (another o_proj on the same scratch, for instance)
      // is still running.
      asm volatile("griddepcontrol.wait;" ::: "memory");
    }
    tc_fence_after_sync();
    const int row = warp * 32 + lane;                 // TMEM lane == row of the W slab
    const int hcol = m_tile * kBM + row;
    float* part = p.partial + ((size_t)(m_tile * p.splits + split) * p.n_pad) * kBM;
    if (ok) {
      for (int c0 = 0; c0 < p.n_pad; c0 += 16) {
        uint32_t v[16];
        if (nkb > 0) {
          tmem_ld_32x32b_x16(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = 0u;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = c0 + j;
          if (p.splits == 1) {
            if (tok < p.tokens) p.y[(int64_t)tok * p.y_stride + hcol] = __float2bfloat16(__uint_as_float(v[j]));
          } else {
            part[(size_t)tok * kBM + row] = __uint_as_float(v[j]);
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  sync_cta();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
  if (p.splits == 1) return;

  // ---------------- split-K: the last CTA of this slab sums the partials ----------------
  __threadfence();
  sync_cta();
  if (tid == 0) {
    const int prev = atomicAdd(&p.counters[m_tile], 1);
    s_last = (prev == p.splits - 1);
  }
  sync_cta();
  if (!s_last) return;
  __threadfence();
  const int row = tid;
  const float* base = p.partial + (size_t)m_tile * p.splits * p.n_pad * kBM;
  for (int tok0 = 0; tok0 < p.tokens; tok0 += 8) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int s = 0; s < p.splits; ++s) {
#pragma unroll
      for (int j = 0; j < 8; ++j)   // rows of the partial are padded to n_pad (a multiple of 16): always in bounds
        acc[j] += __ldcg(base + ((size_t)s * p.n_pad + tok0 + j) * kBM + row);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (tok0 + j < p.tokens) p.y[(int64_t)(tok0 + j) * p.y_stride + m_tile * kBM + row] = __float2bfloat16(acc[j]);
  }
  if (threadIdx.x == 0) p.counters[m_tile] = 0;
}

}  // namespace oproj_dev
}  // namespace helix
