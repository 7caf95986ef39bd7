// Split-KV paged decode attention for MLA (DeepSeek-V3 shape: 128 heads, latent rank 512 + 64 rope
// dims) over a block-scaled fp8 e4m3 latent cache (one fp32 scale per 128 latent values).
//
// All 128 heads share one latent KV stream, so the kernel is bound by tensor-core work, not by HBM.
// One CTA (8 warps) handles all heads of a sequence for a chunk of its tokens, 32 tokens per tile:
//   * the fp8 latent rows, their scales and the bf16 rope keys of a tile arrive by bulk async copies
//     (cp.async.bulk, completion on an mbarrier), two tiles ahead, one issuing thread per stream;
//   * all threads dequantise the tile once (integer bit moves + packed bf16 multiplies, no cvt) into bf16
//     sub-tiles of [32 tokens x 64 dims] with the 128-byte swizzle.  That single layout serves both products: it is the K-major operand of
//     S = Q K^T and, read through an MN-major descriptor, the V operand of O = P V (the latent is
//     both key and value), so nothing is transposed or stored twice;
//   * S = Q K^T runs on warp-level tensor-core MMAs with the query fragments of the warp's 16 heads
//     held in registers for the whole kernel (the accumulator of O does not live in registers);
//   * softmax in registers (base-2 domain); the running max is only re-applied when it grew by more
//     than 2^8, so O is rarely rescaled; P is written as the K-major A operand (bf16, swizzled);
//   * O[128 heads x 512] (fp32) lives in tensor memory: it fills all 512 TMEM columns.  O += P V is
//     issued by one thread as tcgen05.mma (M = 128, N = 256, twice), completion tracked with
//     tcgen05.commit, and overlaps the dequantisation and the Q K^T of the next tile (all buffers are
//     double buffered);
//   * work is split over CTAs by cutting the global tile space into equal chunks; pieces of a
//     sequence are merged by the last CTA to finish it (scratch: two partial slots per CTA).
// Every wait is bounded; on expiry the error flag is raised, TMEM is released and the kernel returns.
#include "attention.h"

#include <cuda_fp8.h>

#include <algorithm>

#include "helix_common.cuh"
#include "sm100.cuh"

namespace helix {
namespace {

using namespace sm100;

constexpr int kH = 128;           // heads
constexpr int kDn = 512;          // latent (nope) dims, also the value dims
constexpr int kDr = 64;           // rope dims
constexpr int kTile = 32;         // tokens per tile
constexpr int kBlk = 16;          // tokens per page-aligned copy unit
constexpr int kThreads = 256;
constexpr int kSub = 9;           // bf16 sub-tiles of 64 dims: 8 latent + 1 rope
constexpr int kSubBytes = kTile * 128;                   // 4096
constexpr int kKvBytes = kSub * kSubBytes;               // 36864 per buffer
constexpr int kPBytes = kH * 128;                        // 16384 per buffer (rows padded to 128 B)
constexpr int kStageLat = kTile * kDn;                   // fp8 latent bytes per stage: 16384
constexpr int kStageScl = kTile * 16;                    // 512
constexpr int kStageRope = kTile * kDr * 2;              // 4096
constexpr int kStageBytes = kStageLat + kStageScl + kStageRope;   // 20992 (multiple of 128)
constexpr int kSmem = 2 * kKvBytes + 2 * kPBytes + 2 * kStageBytes + 1024;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr float kRescaleThreshold = 8.f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// x holds two e4m3 bytes in the high bytes of its 16-bit halves; returns bf16x2(value * scale).
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2_scaled(uint32_t x, __nv_bfloat162 scale_2p56) {
  const uint32_t bits = ((x >> 4) & 0x07FF07FFu) | (x & 0x80008000u);
  const uint32_t k2p64 = 0x5F805F80u;      // bf16x2 (2^64, 2^64)
  __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&bits);
  v = __hmul2(v, *reinterpret_cast<const __nv_bfloat162*>(&k2p64));
  v = __hmul2(v, scale_2p56);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
      "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// MN-major operand stored as [rows = K index][64 elements of the MN index] with the 128-byte swizzle,
// 8-row groups 1024 bytes apart, 64-wide MN blocks `lbo_bytes` apart.
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16, bf16 x bf16 -> fp32, A K-major, B MN-major
__device__ __forceinline__ uint32_t idesc_pv(int M, int N) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

__global__ void __launch_bounds__(kThreads, 1) mla_decode_kernel(const __grid_constant__ MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[2], pv_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ float s_alpha[kH], s_l[kH], s_m[kH];
  __shared__ int s_last, s_nb[512];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv_buf = smem;                                  // 2 x 9 sub-tiles
  uint8_t* p_buf = smem + 2 * kKvBytes;                    // 2 x [128 rows x 128 B]
  uint8_t* stage_buf = p_buf + 2 * kPBytes;                // 2 x (latent fp8 | scales | rope)
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int g = lane >> 2, t = lane & 3;
  // warp w owns the 16 heads [32 (w % 4) + 16 (w / 4), +16): they sit in the TMEM lane quadrant w % 4,
  // the only one this warp may access
  const int head0 = 32 * (warp & 3) + 16 * (warp >> 2);

  if (tid == 0) {
    mbar_init(&full_bar[0], 3);      // one arrival per issuing thread (latent, scales, rope keys)
    mbar_init(&full_bar[1], 3);
    mbar_init(&pv_bar[0], 1);
    mbar_init(&pv_bar[1], 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_o = tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long deadline = now_ns() + p.timeout_ns;

  // ---- this CTA's chunk of the global tile space (sequence-major) --------------------------------
  long long total = 0;
  for (int i = tid; i < min(p.B, 512); i += kThreads) s_nb[i] = (p.seq_lens[i] + kTile - 1) / kTile;
  __syncthreads();
  for (int b = 0; b < min(p.B, 512); ++b) total += s_nb[b];
  for (int b = 512; b < p.B; ++b) total += (p.seq_lens[b] + kTile - 1) / kTile;
  const long long chunk = max((total + gridDim.x - 1) / (long long)gridDim.x, 1LL);
  const long long g0 = (long long)blockIdx.x * chunk, g1 = min(total, g0 + chunk);
  int cur_b = 0;
  long long base = 0;
  while (cur_b < p.B) {
    const long long span = (p.seq_lens[cur_b] + kTile - 1) / kTile;
    if (g0 < base + span) break;
    base += span;
    ++cur_b;
  }
  long long gcur = g0;
  const float sl2 = p.scale * kLog2e;
  uint32_t n_full[2] = {0, 0}, n_pv[2] = {0, 0};      // completed phases consumed per barrier
  bool ok = true;
  const bool prof = p.prof != nullptr && tid == 0;
  long long pc[7] = {0, 0, 0, 0, 0, 0, 0}, pt = 0;
#define MLA_PROF(slot)                 \
  if (prof) {                          \
    const long long now_c = clock64(); \
    pc[slot] += now_c - pt;            \
    pt = now_c;                        \
  }

  while (gcur < g1 && cur_b < p.B && ok) {
    const int b = cur_b;
    const int seq_len = p.seq_lens[b];
    const int n_tiles = (seq_len + kTile - 1) / kTile;
    if (n_tiles == 0) {
      ++cur_b;
      continue;
    }
    const int t_begin = (int)(gcur - base);
    const int t_end = (int)min((long long)n_tiles, (long long)t_begin + (g1 - gcur));
    const bool whole = (t_begin == 0 && t_end == n_tiles);
    const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
    const int count = t_end - t_begin;

    // ---- query fragments of this warp's 16 heads: 32 k-steps of the latent part + 4 of the rope part
    uint32_t qa[36][4];
    {
      const __nv_bfloat16* qn = p.q_nope + ((int64_t)b * kH + head0) * kDn;
      const __nv_bfloat16* qr = p.q_pe + ((int64_t)b * kH + head0) * kDr;
#pragma unroll
      for (int ks = 0; ks < 32; ++ks) {
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)g * kDn + ks * 16 + 2 * t);
        qa[ks][1] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)(g + 8) * kDn + ks * 16 + 2 * t);
        qa[ks][2] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)g * kDn + ks * 16 + 8 + 2 * t);
        qa[ks][3] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)(g + 8) * kDn + ks * 16 + 8 + 2 * t);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) {
        qa[32 + ks][0] = *reinterpret_cast<const uint32_t*>(qr + (int64_t)g * kDr + ks * 16 + 2 * t);
        qa[32 + ks][1] = *reinterpret_cast<const uint32_t*>(qr + (int64_t)(g + 8) * kDr + ks * 16 + 2 * t);
        qa[32 + ks][2] = *reinterpret_cast<const uint32_t*>(qr + (int64_t)g * kDr + ks * 16 + 8 + 2 * t);
        qa[32 + ks][3] = *reinterpret_cast<const uint32_t*>(qr + (int64_t)(g + 8) * kDr + ks * 16 + 8 + 2 * t);
      }
    }

    // producer: bulk copies of one tile (two 16-token units) into staging slot `st`
    // page ids are looked up well ahead of the copies that need them: the (dependent) block-table load
    // must not sit between a barrier and the Q K^T of the issuing warp
    auto unit_token = [&](int tile, int u) {
      // a tile past the end of the block table still copies its full size from the last valid unit
      return min(tile * kTile + u * kBlk, max(seq_len - 1, 0) / kBlk * kBlk);
    };
    auto lookup = [&](int tile, int (&pg)[2]) {
#pragma unroll
      for (int u = 0; u < 2; ++u) pg[u] = bt[unit_token(tile, u) / p.page_size];
    };
    // One issuing thread per stream (latent, scales, rope keys): issuing a bulk copy costs its thread on the
    // order of a hundred cycles, and whoever issues is late for the next barrier; spread over three warps,
    // none of them warp 0 (which also issues the MMAs), the tile loop no longer waits for one thread.
    const int stream = (lane == 0 && warp >= 1 && warp <= 3) ? warp - 1 : -1;
    auto issue = [&](int st, int tile, const int (&pg)[2]) {
      const uint32_t row_bytes = stream == 0 ? (uint32_t)kDn : stream == 1 ? 16u : (uint32_t)(kDr * 2);
      const uint8_t* src = stream == 0 ? p.ckv : stream == 1 ? reinterpret_cast<const uint8_t*>(p.scales)
                                                             : reinterpret_cast<const uint8_t*>(p.kpe);
      uint8_t* dst = stage_buf + st * kStageBytes + (stream == 0 ? 0 : stream == 1 ? kStageLat : kStageLat + kStageScl);
      const uint32_t unit_bytes = (uint32_t)kBlk * row_bytes;
      uint64_t* bar = &full_bar[st];
      mbar_expect_tx(bar, 2 * unit_bytes);
      const int tk0 = unit_token(tile, 0), tk1 = unit_token(tile, 1);
      const int64_t row0 = (int64_t)pg[0] * p.page_size + (tk0 % p.page_size);
      const int64_t row1 = (int64_t)pg[1] * p.page_size + (tk1 % p.page_size);
      if (row1 == row0 + kBlk) {                    // both units in one page: one copy
        bulk_g2s(dst, src + row0 * row_bytes, 2 * unit_bytes, bar);
      } else {
        bulk_g2s(dst, src + row0 * row_bytes, unit_bytes, bar);
        bulk_g2s(dst + unit_bytes, src + row1 * row_bytes, unit_bytes, bar);
      }
    };
    if (stream >= 0) {
      int pg[2];
      if (count > 0) {
        lookup(t_begin, pg);
        issue(0, t_begin, pg);
      }
      if (count > 1) {
        lookup(t_begin + 1, pg);
        issue(1, t_begin + 1, pg);
      }
    }

    float m_used[2] = {-INFINITY, -INFINITY};   // rows g and g + 8 of this warp's heads
    float l_run[2] = {0.f, 0.f};                 // per-lane partial sums
    bool first_tile = true;

    if (prof) pt = clock64();
    const long long loop_c0 = pt;
    for (int i = 0; i < count && ok; ++i) {
      const int tile = t_begin + i;
      const int bf = i & 1;                      // kv / P buffer and staging slot
      uint8_t* kv = kv_buf + bf * kKvBytes;
      uint8_t* pb = p_buf + bf * kPBytes;
      const uint8_t* stg = stage_buf + bf * kStageBytes;
      int pg_next[2] = {0, 0};
      if (stream >= 0 && i + 2 < count) lookup(tile + 2, pg_next);
      // (a) the P V product that last read these buffers (tile i - 2) must be complete
      if (i >= 2) {
        if (!mbar_wait(&pv_bar[bf], n_pv[bf] & 1, deadline)) ok = false;
        ++n_pv[bf];
      }
      // (b) this tile's bytes have landed.  Every thread waits for itself; a thread whose wait ran out
      // dequantises garbage into its own chunks and says so at the barrier below.
      if (ok && !mbar_wait(&full_bar[bf], n_full[bf] & 1, deadline)) ok = false;
      ++n_full[bf];
      tc_fence_after_sync();
      MLA_PROF(0)
      // (c) dequantise: 1024 chunks of 16 fp8 values, four per thread, then the rope keys.
      // No cvt instruction (they issue at a quarter of the ALU rate): an e4m3 byte s.eeee.mmm moved to s.000.0eeee.mmm.0000 IS the bf16 number
      // 2^-120 times its value, subnormals included, so two packed bf16 multiplies (by 2^64, then by
      // scale * 2^56; one product could overflow for large scales) finish the job on the FMA pipe.
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        // Eight consecutive lanes (one phase of a 16-byte shared-memory access) take four chunks of an even
        // row and the four NEXT-group chunks of the odd row below it: their loads fall in different halves of
        // the banks, and their swizzled stores in all eight 16-byte bank groups.
        const int idx = tid + r4 * kThreads;     // 0..1023
        const int q = idx >> 3, j = idx & 7;
        const int row = 2 * (q >> 3) + (j >> 2);                 // token row
        const int c = (((q & 7) ^ (j >> 2)) << 2) + (j & 3);     // 16-byte chunk of the fp8 row
        const uint4 raw = *reinterpret_cast<const uint4*>(stg + row * kDn + c * 16);
        const float sc = *reinterpret_cast<const float*>(stg + kStageLat + row * 16 + (c >> 3) * 4);
        const bool live = tile * kTile + row < seq_len;      // rows past the end must not leak into P V
        const __nv_bfloat16 s56 = __float2bfloat16_rn(live ? sc * 7.2057594037927936e16f : 0.f);   // 2^56
        const __nv_bfloat162 sc2 = __halves2bfloat162(s56, s56);
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        uint32_t out[8];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          out[2 * j] = e4m3x2_to_bf16x2_scaled(__byte_perm(w[j], 0u, 0x1404), sc2);
          out[2 * j + 1] = e4m3x2_to_bf16x2_scaled(__byte_perm(w[j], 0u, 0x3424), sc2);
        }
        uint8_t* sub = kv + (c >> 2) * kSubBytes;            // 64-dim sub-tile
        const uint32_t cc = 2u * (c & 3);
        *reinterpret_cast<uint4*>(sub + swz128(row, cc)) = make_uint4(out[0], out[1], out[2], out[3]);
        *reinterpret_cast<uint4*>(sub + swz128(row, cc + 1)) = make_uint4(out[4], out[5], out[6], out[7]);
      }
      {
        const int row = tid >> 3, c = tid & 7;               // 32 rows x 8 chunks of the rope keys
        const uint4 v = *reinterpret_cast<const uint4*>(stg + kStageLat + kStageScl + row * 128 + c * 16);
        *reinterpret_cast<uint4*>(kv + 8 * kSubBytes + swz128(row, c)) = v;
      }
      if (!__syncthreads_and(ok ? 1 : 0)) {
        ok = false;
        break;
      }
      // the staging slot is free: fetch the tile two ahead
      if (stream >= 0 && i + 2 < count) issue(bf, tile + 2, pg_next);
      MLA_PROF(1)

      // (d) S = Q K^T for this warp's 16 heads x 32 tokens.  Bound by the rate of the warp-level MMA pipe
      // (1152 MMAs per tile in ~2450 cycles); a second set of accumulators changed nothing.
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[nt][j] = 0.f;
      {
        const int mi = lane >> 3, r8 = lane & 7;
        const uint32_t krow = (uint32_t)(((mi >> 1) << 3) + r8), kcs = (uint32_t)(mi & 1);
        const uint32_t kvb = smem_u32(kv);
#pragma unroll
        for (int ks = 0; ks < 36; ++ks) {
          const uint32_t sub = kvb + (uint32_t)(ks >> 2) * kSubBytes;
          const uint32_t cc = 2u * (ks & 3) + kcs;
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4(sub + swz128(krow, cc), r0, r1, r2, r3);
          mma_bf16_16816(s[0], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r0, r1);
          mma_bf16_16816(s[1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r2, r3);
          ldmatrix_x4(sub + swz128(krow + 16u, cc), r0, r1, r2, r3);
          mma_bf16_16816(s[2], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r0, r1);
          mma_bf16_16816(s[3], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], r2, r3);
        }
      }
      MLA_PROF(2)
      // (e) online softmax; rows g (values 0, 1 of each n-tile) and g + 8 (values 2, 3)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int tok = tile * kTile + nt * 8 + 2 * t + (j & 1);
          float v = s[nt][j] * sl2;
          if (tok >= seq_len) v = -INFINITY;
          s[nt][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      float alpha[2] = {1.f, 1.f};
      bool need = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        if (mx[r] > m_used[r] + kRescaleThreshold || m_used[r] == -INFINITY) {
          const float m_new = fmaxf(m_used[r], mx[r]);
          alpha[r] = fast_exp2(m_used[r] - m_new);           // 0 for the very first tile
          l_run[r] *= alpha[r];
          need |= (m_used[r] != -INFINITY);
          m_used[r] = m_new;
        }
      }
      // (f) P = exp2(S - m) as the K-major A operand: row = head, 16-byte chunk = n-tile
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float p0 = fast_exp2(s[nt][0] - m_used[0]), p1 = fast_exp2(s[nt][1] - m_used[0]);
        const float p2 = fast_exp2(s[nt][2] - m_used[1]), p3 = fast_exp2(s[nt][3] - m_used[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        *reinterpret_cast<uint32_t*>(pb + swz128((uint32_t)(head0 + g), (uint32_t)nt) + 4 * t) = pack_bf16(p0, p1);
        *reinterpret_cast<uint32_t*>(pb + swz128((uint32_t)(head0 + g + 8), (uint32_t)nt) + 4 * t) = pack_bf16(p2, p3);
      }
      fence_proxy_async_smem();                  // P and the dequantised tile -> visible to the tensor core
      tc_fence_before_sync();
      MLA_PROF(3)
      // One barrier: P and the dequantised tile are complete, and the warps agree on whether O in tensor
      // memory has to follow new maxima first (rare after the first tiles).
      if (__syncthreads_or((need && !first_tile) ? 1 : 0)) {
        if (t == 0) {
          s_alpha[head0 + g] = alpha[0];
          s_alpha[head0 + g + 8] = alpha[1];
        }
        // every P V issued so far must have finished before O is read
        if (i >= 1) {
          const int pb_prev = (i - 1) & 1;
          if (!mbar_wait(&pv_bar[pb_prev], n_pv[pb_prev] & 1, deadline)) ok = false;
          // not consumed: the wait at step (a) of a later tile looks at the same phase again
        }
        __syncthreads();
        tc_fence_after_sync();
        if (warp < 4 && ok) {
          const float a = s_alpha[32 * warp + lane];
          for (int c0 = 0; c0 < kDn; c0 += 16) {
            uint32_t v[16];
            tmem_ld_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * a);
            tmem_st_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
          }
          tmem_st_wait();
        }
        tc_fence_before_sync();
        __syncthreads();
        tc_fence_after_sync();
      }
      // (g) O += P V on tcgen05: two N = 256 halves, two K = 16 steps each
      if (tid == 0) {
        tc_fence_after_sync();
        const uint32_t idesc = idesc_pv(kH, 256);
        const uint32_t pa = smem_u32(pb), va = smem_u32(kv);
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int ks = 0; ks < 2; ++ks)
            umma_bf16(tmem_o + (uint32_t)half * 256u, umma_desc_k_sw128(pa + ks * 32),
                      umma_desc_mn_sw128(va + (uint32_t)half * 4u * kSubBytes + (uint32_t)ks * 2048u, kSubBytes), idesc,
                      !(first_tile && ks == 0));
        umma_commit(&pv_bar[bf]);
      }
      first_tile = false;
      MLA_PROF(4)
    }
    if (prof) {
      pc[5] += count;
      pc[6] += clock64() - loop_c0;
    }

    // ---- drain: all P V products of this segment ------------------------------------------------
    if (ok) {
      for (int k = max(count - 2, 0); k < count; ++k) {
        const int bf = k & 1;
        if (!mbar_wait(&pv_bar[bf], n_pv[bf] & 1, deadline)) ok = false;
        ++n_pv[bf];
      }
    }
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    tc_fence_after_sync();
    // row sums and maxima of all 128 heads
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
    if (t == 0) {
      s_l[head0 + g] = l_run[0];
      s_l[head0 + g + 8] = l_run[1];
      s_m[head0 + g] = m_used[0];
      s_m[head0 + g + 8] = m_used[1];
    }
    __syncthreads();

    // ---- read O out of tensor memory: warps 0..3, thread = head ------------------------------------
    const int slot = (t_begin == 0) ? 1 : 0;
    float* part_o = p.part_o + (size_t)(blockIdx.x * 2 + slot) * kH * kDn;
    float* part_l = p.part_lse + (size_t)(blockIdx.x * 2 + slot) * kH;
    if (warp < 4) {
      const int h = 32 * warp + lane;
      const float L = s_l[h], M = s_m[h];
      const float inv = L > 0.f ? 1.f / L : 0.f;
      const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
      for (int c0 = 0; c0 < kDn; c0 += 16) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
        tmem_ld_wait();
        if (whole) {
          uint32_t o16[8];
#pragma unroll
          for (int j = 0; j < 8; ++j)
            o16[j] = pack_bf16(__uint_as_float(v[2 * j]) * inv, __uint_as_float(v[2 * j + 1]) * inv);
          uint4* dst = reinterpret_cast<uint4*>(p.o + ((int64_t)b * kH + h) * kDn + c0);
          dst[0] = make_uint4(o16[0], o16[1], o16[2], o16[3]);
          dst[1] = make_uint4(o16[4], o16[5], o16[6], o16[7]);
        } else {
          float4* dst = reinterpret_cast<float4*>(part_o + (size_t)h * kDn + c0);
#pragma unroll
          for (int j = 0; j < 4; ++j)
            dst[j] = make_float4(__uint_as_float(v[4 * j]) * inv, __uint_as_float(v[4 * j + 1]) * inv,
                                 __uint_as_float(v[4 * j + 2]) * inv, __uint_as_float(v[4 * j + 3]) * inv);
        }
      }
      if (whole) p.lse[(int64_t)b * kH + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
      else part_l[h] = lse2;
    }
    tc_fence_before_sync();

    if (!whole) {
      // ---- the last CTA to finish this sequence folds its pieces -----------------------------------
      const int first_cta = (int)(base / chunk);
      const int last_cta = (int)((base + n_tiles - 1) / chunk);
      const int pieces = last_cta - first_cta + 1;
      __syncthreads();
      if (tid == 0) {
        int prev;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + b) : "memory");
        s_last = (prev == pieces - 1);
      }
      __syncthreads();
      if (s_last) {
        auto piece_slot = [&](int c) { return (size_t)(c * 2 + (c == first_cta ? 1 : 0)); };
        // warp w folds heads w, w + 8, ...: lanes share out the pieces' weights, then sum 16 columns each
        for (int h = warp; h < kH; h += kThreads / 32) {
          float M = -INFINITY;
          for (int c = first_cta + lane; c <= last_cta; c += 32) M = fmaxf(M, __ldcg(p.part_lse + piece_slot(c) * kH + h));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
          float L = 0.f;
          float4 acc[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int c0 = first_cta; c0 <= last_cta; c0 += 32) {
            const int c = c0 + lane;
            float w = 0.f;
            if (c <= last_cta && M != -INFINITY) w = fast_exp2(__ldcg(p.part_lse + piece_slot(c) * kH + h) - M);
            L += w;
            const int nb = min(32, last_cta - c0 + 1);
            for (int jn = 0; jn < nb; ++jn) {
              const float wj = __shfl_sync(0xffffffffu, w, jn);
              const float4* src = reinterpret_cast<const float4*>(p.part_o + (piece_slot(c0 + jn) * kH + h) * kDn) + lane * 4;
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float4 v = __ldcg(src + j);
                acc[j].x += wj * v.x;
                acc[j].y += wj * v.y;
                acc[j].z += wj * v.z;
                acc[j].w += wj * v.w;
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
          const float inv = L > 0.f ? 1.f / L : 0.f;
          uint32_t o16[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            o16[2 * j] = pack_bf16(acc[j].x * inv, acc[j].y * inv);
            o16[2 * j + 1] = pack_bf16(acc[j].z * inv, acc[j].w * inv);
          }
          uint4* dst = reinterpret_cast<uint4*>(p.o + ((int64_t)b * kH + h) * kDn + lane * 16);
          dst[0] = make_uint4(o16[0], o16[1], o16[2], o16[3]);
          dst[1] = make_uint4(o16[4], o16[5], o16[6], o16[7]);
          if (lane == 0) {
            const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
            p.lse[(int64_t)b * kH + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
          }
        }
        if (tid == 0) p.counters[b] = 0;
      }
    }
    __syncthreads();
    tc_fence_after_sync();
    gcur += count;
    if (t_end == n_tiles) {
      base += n_tiles;
      ++cur_b;
    }
  }

  if (!ok) {
    if (tid == 0) atomicCAS(p.error_flag, 0, (int)kTimeoutMbarrier);
    // bounded grace period for copies and MMAs that may still be in flight
    const unsigned long long grace = now_ns() + 2000000ull;
    while (now_ns() < grace) {
      bool idle = true;
      for (int s = 0; s < 2; ++s) idle &= (mbar_try_wait(&full_bar[s], 0) || mbar_try_wait(&full_bar[s], 1));
      if (idle) break;
    }
  }
  // sequences without any token: output 0, LSE -inf (CTA 0 sweeps them)
  if (blockIdx.x == 0) {
    for (int bb = 0; bb < p.B; ++bb) {
      if (p.seq_lens[bb] > 0) continue;
      for (int idx = tid; idx < kH * kDn; idx += kThreads) {
        p.o[(int64_t)bb * kH * kDn + idx] = __float2bfloat16(0.f);
        if (idx < kH) p.lse[(int64_t)bb * kH + idx] = -INFINITY;
      }
    }
  }
  if (prof)
    for (int j = 0; j < 7; ++j) p.prof[(size_t)blockIdx.x * 8 + j] = (unsigned long long)pc[j];
#undef MLA_PROF
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_o, 512);
}


// ---- warp-specialised variant ------------------------------------------------------------------------
// Twelve warps.  Warps 8..11 are producers: three of their threads issue the bulk copies, all 128
// dequantise tile after tile into the two bf16 buffers and post each one on an mbarrier; they never wait for
// the math.  Warps 0..7 are the math group of the kernel above (Q fragments in registers, Q K^T on warp-level
// MMAs, softmax, P, one thread issuing P V on tcgen05).  The copies, the dequantisation and the barriers of a
// tile (about 3000 of its 5500 cycles in the lockstep kernel) now run beside Q K^T instead of in front of it.
// Registers move from the producers to the math warps with setmaxnreg (168 each at launch -> 72 / 216; with
// 40 / 232 the producers spilled and were the slower side, with the rope part of Q in registers the math warps did).
constexpr int kWsThreads = 384;
constexpr int kWsStages = 3;
constexpr int kQrBytes = kH * 128;   // rope part of Q, [128 heads x 64] bf16, 128-byte swizzle
constexpr int kWsSmem = 2 * kKvBytes + 2 * kPBytes + kWsStages * kStageBytes + kQrBytes + 1024;
constexpr int kMathBar = 1, kProdBar = 2;
constexpr int kProdThreads = 128;

__device__ __forceinline__ void bar_sync_named(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }
__device__ __forceinline__ int bar_or_named(int id, int n, int pred) {
  int r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.s32 p, %3, 0;\n"
      "bar.red.or.pred q, %1, %2, p;\n"
      "selp.s32 %0, 1, 0, q;\n"
      "}\n"
      : "=r"(r)
      : "r"(id), "r"(n), "r"(pred)
      : "memory");
  return r;
}

__global__ void __launch_bounds__(kWsThreads, 1) mla_decode_ws_kernel(const __grid_constant__ MlaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kWsStages], kv_ready[2], pv_bar[2];
  __shared__ uint32_t tmem_slot;
  __shared__ float s_alpha[kH], s_l[kH], s_m[kH];
  __shared__ int s_last, s_nb[512];

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* kv_buf = smem;                                  // 2 x 9 sub-tiles
  uint8_t* p_buf = smem + 2 * kKvBytes;                    // 2 x [128 rows x 128 B]
  uint8_t* stage_buf = p_buf + 2 * kPBytes;                // kWsStages x (latent fp8 | scales | rope)
  uint8_t* qr_buf = stage_buf + kWsStages * kStageBytes;   // rope part of Q
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    for (int i = 0; i < kWsStages; ++i) mbar_init(&full_bar[i], 3);   // one arrival per issuing thread
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_ready[i], 4);                                      // one arrival per producer warp
      mbar_init(&pv_bar[i], 1);                                        // tcgen05.commit
    }
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_o = tmem_slot;
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long deadline = now_ns() + p.timeout_ns;

  // ---- this CTA's chunk of the global tile space (sequence-major); both groups walk it the same way ----
  long long total = 0;
  for (int i = tid; i < min(p.B, 512); i += kWsThreads) s_nb[i] = (p.seq_lens[i] + kTile - 1) / kTile;
  __syncthreads();
  for (int b = 0; b < min(p.B, 512); ++b) total += s_nb[b];
  for (int b = 512; b < p.B; ++b) total += (p.seq_lens[b] + kTile - 1) / kTile;
  const long long chunk = max((total + gridDim.x - 1) / (long long)gridDim.x, 1LL);
  const long long g0 = (long long)blockIdx.x * chunk, g1 = min(total, g0 + chunk);
  int cur_b = 0;
  long long base = 0;
  while (cur_b < p.B) {
    const long long span = (p.seq_lens[cur_b] + kTile - 1) / kTile;
    if (g0 < base + span) break;
    base += span;
    ++cur_b;
  }
  long long gcur = g0;
  bool ok = true;
  int gt = 0;                    // tiles this CTA has gone through: fixes the kv buffer (parity) and the stage

  if (warp >= 8) {
    // =========================== producers ===========================
    asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
    const int ptid = tid - 256, pwarp = warp - 8;
    const int stream = (lane == 0 && pwarp < 3) ? pwarp : -1;      // latent, scales, rope keys
    uint32_t n_full[kWsStages] = {0, 0, 0}, fills[2] = {0, 0};
    while (gcur < g1 && cur_b < p.B && ok) {
      const int b = cur_b;
      const int seq_len = p.seq_lens[b];
      const int n_tiles = (seq_len + kTile - 1) / kTile;
      if (n_tiles == 0) {
        ++cur_b;
        continue;
      }
      const int t_begin = (int)(gcur - base);
      const int t_end = (int)min((long long)n_tiles, (long long)t_begin + (g1 - gcur));
      const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
      const int count = t_end - t_begin;
      auto unit_token = [&](int tile, int u) { return min(tile * kTile + u * kBlk, max(seq_len - 1, 0) / kBlk * kBlk); };
      // page ids are fetched a whole tile before the copies that need them are issued: the issuing threads
      // must not sit on a dependent global load while their group waits for them at the barrier
      auto page_of = [&](int tile, int u) { return bt[unit_token(tile, u) / p.page_size]; };
      auto issue = [&](int st, int tile, int pg0, int pg1) {
        const int tk0 = unit_token(tile, 0), tk1 = unit_token(tile, 1);
        const uint32_t row_bytes = stream == 0 ? (uint32_t)kDn : stream == 1 ? 16u : (uint32_t)(kDr * 2);
        const uint8_t* src = stream == 0 ? p.ckv : stream == 1 ? reinterpret_cast<const uint8_t*>(p.scales)
                                                               : reinterpret_cast<const uint8_t*>(p.kpe);
        uint8_t* dst = stage_buf + st * kStageBytes + (stream == 0 ? 0 : stream == 1 ? kStageLat : kStageLat + kStageScl);
        const uint32_t unit_bytes = (uint32_t)kBlk * row_bytes;
        uint64_t* bar = &full_bar[st];
        mbar_expect_tx(bar, 2 * unit_bytes);
        const int64_t row0 = (int64_t)pg0 * p.page_size + (tk0 % p.page_size);
        const int64_t row1 = (int64_t)pg1 * p.page_size + (tk1 % p.page_size);
        if (row1 == row0 + kBlk) {
          bulk_g2s(dst, src + row0 * row_bytes, 2 * unit_bytes, bar);
        } else {
          bulk_g2s(dst, src + row0 * row_bytes, unit_bytes, bar);
          bulk_g2s(dst + unit_bytes, src + row1 * row_bytes, unit_bytes, bar);
        }
      };
      if (stream >= 0)
        for (int j = 0; j < min(count, kWsStages); ++j)
          issue((gt + j) % kWsStages, t_begin + j, page_of(t_begin + j, 0), page_of(t_begin + j, 1));

      for (int j = 0; j < count; ++j) {
        const int tile = t_begin + j;
        const int st = (gt + j) % kWsStages, bf = (gt + j) & 1;
        uint8_t* kv = kv_buf + bf * kKvBytes;
        const uint8_t* stg = stage_buf + st * kStageBytes;
        int pgn0 = 0, pgn1 = 0;
        if (stream >= 0 && j + kWsStages < count) {
          pgn0 = page_of(tile + kWsStages, 0);
          pgn1 = page_of(tile + kWsStages, 1);
        }
        // the P V product that read this buffer two tiles ago must be complete
        if (fills[bf] >= 1 && !mbar_wait(&pv_bar[bf], (fills[bf] - 1) & 1, deadline)) ok = false;
        if (ok && !mbar_wait(&full_bar[st], n_full[st] & 1, deadline)) ok = false;
        ++n_full[st];
#pragma unroll 2
        for (int r8 = 0; r8 < 8; ++r8) {
          const int idx = ptid + r8 * kProdThreads;                // 0..1023, same bank-friendly map as above
          const int q = idx >> 3, j8 = idx & 7;
          const int row = 2 * (q >> 3) + (j8 >> 2);
          const int c = (((q & 7) ^ (j8 >> 2)) << 2) + (j8 & 3);
          const uint4 raw = *reinterpret_cast<const uint4*>(stg + row * kDn + c * 16);
          const float sc = *reinterpret_cast<const float*>(stg + kStageLat + row * 16 + (c >> 3) * 4);
          const bool live = tile * kTile + row < seq_len;
          const __nv_bfloat16 s56 = __float2bfloat16_rn(live ? sc * 7.2057594037927936e16f : 0.f);   // 2^56
          const __nv_bfloat162 sc2 = __halves2bfloat162(s56, s56);
          const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
          uint32_t out[8];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            out[2 * jj] = e4m3x2_to_bf16x2_scaled(__byte_perm(w[jj], 0u, 0x1404), sc2);
            out[2 * jj + 1] = e4m3x2_to_bf16x2_scaled(__byte_perm(w[jj], 0u, 0x3424), sc2);
          }
          uint8_t* sub = kv + (c >> 2) * kSubBytes;
          const uint32_t cc = 2u * (c & 3);
          *reinterpret_cast<uint4*>(sub + swz128(row, cc)) = make_uint4(out[0], out[1], out[2], out[3]);
          *reinterpret_cast<uint4*>(sub + swz128(row, cc + 1)) = make_uint4(out[4], out[5], out[6], out[7]);
        }
#pragma unroll 1
        for (int r2 = 0; r2 < 2; ++r2) {
          const int idx = ptid + r2 * kProdThreads;                // 32 rows x 8 chunks of the rope keys
          const int row = idx >> 3, c = idx & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(stg + kStageLat + kStageScl + row * 128 + c * 16);
          *reinterpret_cast<uint4*>(kv + 8 * kSubBytes + swz128(row, c)) = v;
        }
        fence_proxy_async_smem();                                  // the tensor core reads this buffer too (P V)
        // one vote per tile: the staging slot is free for the issuers, and a failed wait ends the group together
        if (bar_or_named(kProdBar, kProdThreads, ok ? 0 : 1)) {
          ok = false;
          break;
        }
        if (lane == 0) mbar_arrive(&kv_ready[bf]);
        ++fills[bf];
        if (stream >= 0 && j + kWsStages < count) issue(st, tile + kWsStages, pgn0, pgn1);
      }
      gt += count;
      gcur += count;
      if (t_end == n_tiles) {
        base += n_tiles;
        ++cur_b;
      }
    }
    if (!ok && ptid == 0) atomicCAS(p.error_flag, 0, (int)kTimeoutMbarrier);
  } else {
    // =========================== math group ===========================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int g = lane >> 2, t = lane & 3;
    const int head0 = 32 * (warp & 3) + 16 * (warp >> 2);
    const float sl2 = p.scale * kLog2e;
    uint32_t uses[2] = {0, 0};                 // P V products issued per buffer
    while (gcur < g1 && cur_b < p.B && ok) {
      const int b = cur_b;
      const int seq_len = p.seq_lens[b];
      const int n_tiles = (seq_len + kTile - 1) / kTile;
      if (n_tiles == 0) {
        ++cur_b;
        continue;
      }
      const int t_begin = (int)(gcur - base);
      const int t_end = (int)min((long long)n_tiles, (long long)t_begin + (g1 - gcur));
      const bool whole = (t_begin == 0 && t_end == n_tiles);
      const int count = t_end - t_begin;

      // ---- query fragments of this warp's 16 heads: the 32 k-steps of the latent part stay in registers; the
      // rope part (4 k-steps) sits in shared memory and is re-read with ldmatrix every tile, which keeps the math
      // warps inside their 232 registers
      uint32_t qa[32][4];
      {
        const __nv_bfloat16* qn = p.q_nope + ((int64_t)b * kH + head0) * kDn;
        const __nv_bfloat16* qr = p.q_pe + ((int64_t)b * kH + head0) * kDr;
#pragma unroll
        for (int ks = 0; ks < 32; ++ks) {
          qa[ks][0] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)g * kDn + ks * 16 + 2 * t);
          qa[ks][1] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)(g + 8) * kDn + ks * 16 + 2 * t);
          qa[ks][2] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)g * kDn + ks * 16 + 8 + 2 * t);
          qa[ks][3] = *reinterpret_cast<const uint32_t*>(qn + (int64_t)(g + 8) * kDn + ks * 16 + 8 + 2 * t);
        }
        __syncwarp();                       // the previous segment's tiles are done with these rows
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {    // 16 rows x 8 chunks of 16 bytes, four per lane
          const int idx = lane + 32 * r4, row = idx >> 3, c = idx & 7;
          const uint4 v = *reinterpret_cast<const uint4*>(qr + (int64_t)row * kDr + c * 8);
          *reinterpret_cast<uint4*>(qr_buf + swz128((uint32_t)(head0 + row), (uint32_t)c)) = v;
        }
        __syncwarp();
      }

      float m_used[2] = {-INFINITY, -INFINITY};   // rows g and g + 8 of this warp's heads
      float l_run[2] = {0.f, 0.f};                 // per-lane partial sums
      bool first_tile = true;

      for (int i = 0; i < count && ok; ++i) {
        const int tile = t_begin + i;
        const int bf = (gt + i) & 1;
        uint8_t* kv = kv_buf + bf * kKvBytes;
        uint8_t* pb = p_buf + bf * kPBytes;
        // the P buffer is free once the P V product that used it two tiles ago is complete
        if (uses[bf] >= 1 && !mbar_wait(&pv_bar[bf], (uses[bf] - 1) & 1, deadline)) ok = false;
        // the producers have posted this tile
        if (ok && !mbar_wait(&kv_ready[bf], uses[bf] & 1, deadline)) ok = false;
        tc_fence_after_sync();
      // (d) S = Q K^T for this warp's 16 heads x 32 tokens, bound by the rate of the warp-level MMA pipe
      float s[4][4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) s[nt][j] = 0.f;
      {
        const int mi = lane >> 3, r8 = lane & 7;
        const uint32_t krow = (uint32_t)(((mi >> 1) << 3) + r8), kcs = (uint32_t)(mi & 1);
        const uint32_t kvb = smem_u32(kv);
        const uint32_t qrow = (uint32_t)(head0 + ((mi & 1) << 3) + r8), qcs = (uint32_t)(mi >> 1);
        const uint32_t qrb = smem_u32(qr_buf);
#pragma unroll
        for (int ks = 0; ks < 36; ++ks) {
          const uint32_t sub = kvb + (uint32_t)(ks >> 2) * kSubBytes;
          const uint32_t cc = 2u * (ks & 3) + kcs;
          uint32_t a0, a1, a2, a3;
          if (ks < 32) {
            a0 = qa[ks < 32 ? ks : 0][0], a1 = qa[ks < 32 ? ks : 0][1], a2 = qa[ks < 32 ? ks : 0][2], a3 = qa[ks < 32 ? ks : 0][3];
          } else {
            ldmatrix_x4(qrb + swz128(qrow, 2u * (uint32_t)(ks - 32) + qcs), a0, a1, a2, a3);
          }
          uint32_t r0, r1, r2, r3;
          ldmatrix_x4(sub + swz128(krow, cc), r0, r1, r2, r3);
          mma_bf16_16816(s[0], a0, a1, a2, a3, r0, r1);
          mma_bf16_16816(s[1], a0, a1, a2, a3, r2, r3);
          ldmatrix_x4(sub + swz128(krow + 16u, cc), r0, r1, r2, r3);
          mma_bf16_16816(s[2], a0, a1, a2, a3, r0, r1);
          mma_bf16_16816(s[3], a0, a1, a2, a3, r2, r3);
        }
      }
      // (e) online softmax; rows g (values 0, 1 of each n-tile) and g + 8 (values 2, 3)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int tok = tile * kTile + nt * 8 + 2 * t + (j & 1);
          float v = s[nt][j] * sl2;
          if (tok >= seq_len) v = -INFINITY;
          s[nt][j] = v;
          mx[j >> 1] = fmaxf(mx[j >> 1], v);
        }
      float alpha[2] = {1.f, 1.f};
      bool need = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        if (mx[r] > m_used[r] + kRescaleThreshold || m_used[r] == -INFINITY) {
          const float m_new = fmaxf(m_used[r], mx[r]);
          alpha[r] = fast_exp2(m_used[r] - m_new);           // 0 for the very first tile
          l_run[r] *= alpha[r];
          need |= (m_used[r] != -INFINITY);
          m_used[r] = m_new;
        }
      }
      // (f) P = exp2(S - m) as the K-major A operand: row = head, 16-byte chunk = n-tile
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const float p0 = fast_exp2(s[nt][0] - m_used[0]), p1 = fast_exp2(s[nt][1] - m_used[0]);
        const float p2 = fast_exp2(s[nt][2] - m_used[1]), p3 = fast_exp2(s[nt][3] - m_used[1]);
        l_run[0] += p0 + p1;
        l_run[1] += p2 + p3;
        *reinterpret_cast<uint32_t*>(pb + swz128((uint32_t)(head0 + g), (uint32_t)nt) + 4 * t) = pack_bf16(p0, p1);
        *reinterpret_cast<uint32_t*>(pb + swz128((uint32_t)(head0 + g + 8), (uint32_t)nt) + 4 * t) = pack_bf16(p2, p3);
      }
        fence_proxy_async_smem();                  // P -> visible to the tensor core
        tc_fence_before_sync();
        // One barrier of the math group: P is complete, and the warps agree on whether O in tensor memory has
        // to follow new maxima first (rare after the first tiles) or whether somebody's wait ran out.
        if (bar_or_named(kMathBar, kThreads, (!ok || (need && !first_tile)) ? 1 : 0)) {
          if (bar_or_named(kMathBar, kThreads, ok ? 0 : 1)) {
            ok = false;
            break;
          }
          if (t == 0) {
            s_alpha[head0 + g] = alpha[0];
            s_alpha[head0 + g + 8] = alpha[1];
          }
          // every P V issued so far must have finished before O is read: the latest one used the other buffer
          if (uses[bf ^ 1] >= 1 && !mbar_wait(&pv_bar[bf ^ 1], (uses[bf ^ 1] - 1) & 1, deadline)) ok = false;
          bar_sync_named(kMathBar, kThreads);
          tc_fence_after_sync();
          if (warp < 4 && ok) {
            const float a = s_alpha[32 * warp + lane];
            for (int c0 = 0; c0 < kDn; c0 += 16) {
              uint32_t v[16];
              tmem_ld_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * a);
              tmem_st_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
            }
            tmem_st_wait();
          }
          tc_fence_before_sync();
          bar_sync_named(kMathBar, kThreads);
          tc_fence_after_sync();
        }
        // (g) O += P V on tcgen05: two N = 256 halves, two K = 16 steps each
        if (tid == 0) {
          tc_fence_after_sync();
          const uint32_t idesc = idesc_pv(kH, 256);
          const uint32_t pa = smem_u32(pb), va = smem_u32(kv);
#pragma unroll
          for (int half = 0; half < 2; ++half)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks)
              umma_bf16(tmem_o + (uint32_t)half * 256u, umma_desc_k_sw128(pa + ks * 32),
                        umma_desc_mn_sw128(va + (uint32_t)half * 4u * kSubBytes + (uint32_t)ks * 2048u, kSubBytes), idesc,
                        !(first_tile && ks == 0));
          umma_commit(&pv_bar[bf]);
        }
        ++uses[bf];
        first_tile = false;
      }

      // ---- drain: the latest P V product on each buffer ----------------------------------------------
      for (int bb = 0; bb < 2; ++bb)
        if (ok && uses[bb] >= 1 && !mbar_wait(&pv_bar[bb], (uses[bb] - 1) & 1, deadline)) ok = false;
      if (bar_or_named(kMathBar, kThreads, ok ? 0 : 1)) {
        ok = false;
        break;
      }
      tc_fence_after_sync();
      // row sums and maxima of all 128 heads
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
      }
      if (t == 0) {
        s_l[head0 + g] = l_run[0];
        s_l[head0 + g + 8] = l_run[1];
        s_m[head0 + g] = m_used[0];
        s_m[head0 + g + 8] = m_used[1];
      }
      bar_sync_named(kMathBar, kThreads);

      // ---- read O out of tensor memory: warps 0..3, thread = head ------------------------------------
      const int slot = (t_begin == 0) ? 1 : 0;
      float* part_o = p.part_o + (size_t)(blockIdx.x * 2 + slot) * kH * kDn;
      float* part_l = p.part_lse + (size_t)(blockIdx.x * 2 + slot) * kH;
      if (warp < 4) {
        const int h = 32 * warp + lane;
        const float L = s_l[h], M = s_m[h];
        const float inv = L > 0.f ? 1.f / L : 0.f;
        const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
        for (int c0 = 0; c0 < kDn; c0 += 16) {
          uint32_t v[16];
          tmem_ld_32x32b_x16(tmem_o + ((uint32_t)(32 * warp) << 16) + (uint32_t)c0, v);
          tmem_ld_wait();
          if (whole) {
            uint32_t o16[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
              o16[j] = pack_bf16(__uint_as_float(v[2 * j]) * inv, __uint_as_float(v[2 * j + 1]) * inv);
            uint4* dst = reinterpret_cast<uint4*>(p.o + ((int64_t)b * kH + h) * kDn + c0);
            dst[0] = make_uint4(o16[0], o16[1], o16[2], o16[3]);
            dst[1] = make_uint4(o16[4], o16[5], o16[6], o16[7]);
          } else {
            float4* dst = reinterpret_cast<float4*>(part_o + (size_t)h * kDn + c0);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              dst[j] = make_float4(__uint_as_float(v[4 * j]) * inv, __uint_as_float(v[4 * j + 1]) * inv,
                                   __uint_as_float(v[4 * j + 2]) * inv, __uint_as_float(v[4 * j + 3]) * inv);
          }
        }
        if (whole) p.lse[(int64_t)b * kH + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
        else part_l[h] = lse2;
      }
      tc_fence_before_sync();

      if (!whole) {
        // ---- the last CTA to finish this sequence folds its pieces -----------------------------------
        const int first_cta = (int)(base / chunk);
        const int last_cta = (int)((base + n_tiles - 1) / chunk);
        const int pieces = last_cta - first_cta + 1;
        bar_sync_named(kMathBar, kThreads);
        if (tid == 0) {
          int prev;
          asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(p.counters + b) : "memory");
          s_last = (prev == pieces - 1);
        }
        bar_sync_named(kMathBar, kThreads);
        if (s_last) {
          auto piece_slot = [&](int c) { return (size_t)(c * 2 + (c == first_cta ? 1 : 0)); };
          // warp w folds heads w, w + 8, ...: lanes share out the pieces' weights, then sum 16 columns each
          for (int h = warp; h < kH; h += kThreads / 32) {
            float M = -INFINITY;
            for (int c = first_cta + lane; c <= last_cta; c += 32) M = fmaxf(M, __ldcg(p.part_lse + piece_slot(c) * kH + h));
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
            float L = 0.f;
            float4 acc[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int c0 = first_cta; c0 <= last_cta; c0 += 32) {
              const int c = c0 + lane;
              float w = 0.f;
              if (c <= last_cta && M != -INFINITY) w = fast_exp2(__ldcg(p.part_lse + piece_slot(c) * kH + h) - M);
              L += w;
              const int nb = min(32, last_cta - c0 + 1);
              for (int jn = 0; jn < nb; ++jn) {
                const float wj = __shfl_sync(0xffffffffu, w, jn);
                const float4* src = reinterpret_cast<const float4*>(p.part_o + (piece_slot(c0 + jn) * kH + h) * kDn) + lane * 4;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float4 v = __ldcg(src + j);
                  acc[j].x += wj * v.x;
                  acc[j].y += wj * v.y;
                  acc[j].z += wj * v.z;
                  acc[j].w += wj * v.w;
                }
              }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
            const float inv = L > 0.f ? 1.f / L : 0.f;
            uint32_t o16[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              o16[2 * j] = pack_bf16(acc[j].x * inv, acc[j].y * inv);
              o16[2 * j + 1] = pack_bf16(acc[j].z * inv, acc[j].w * inv);
            }
            uint4* dst = reinterpret_cast<uint4*>(p.o + ((int64_t)b * kH + h) * kDn + lane * 16);
            dst[0] = make_uint4(o16[0], o16[1], o16[2], o16[3]);
            dst[1] = make_uint4(o16[4], o16[5], o16[6], o16[7]);
            if (lane == 0) {
              const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
              p.lse[(int64_t)b * kH + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
            }
          }
          if (tid == 0) p.counters[b] = 0;
        }
      }
      bar_sync_named(kMathBar, kThreads);
      tc_fence_after_sync();
      gt += count;
      gcur += count;
      if (t_end == n_tiles) {
        base += n_tiles;
        ++cur_b;
      }
    }
    if (!ok && tid == 0) atomicCAS(p.error_flag, 0, (int)kTimeoutMbarrier);
    // sequences without any token: output 0, LSE -inf (CTA 0 sweeps them)
    if (blockIdx.x == 0) {
      for (int bb = 0; bb < p.B; ++bb) {
        if (p.seq_lens[bb] > 0) continue;
        for (int idx = tid; idx < kH * kDn; idx += kThreads) {
          p.o[(int64_t)bb * kH * kDn + idx] = __float2bfloat16(0.f);
          if (idx < kH) p.lse[(int64_t)bb * kH + idx] = -INFINITY;
        }
      }
    }
  }
  if (!ok) {
    // bounded grace period for copies that may still be in flight
    const unsigned long long grace = now_ns() + 2000000ull;
    while (now_ns() < grace) {
      bool idle = true;
      for (int st = 0; st < kWsStages; ++st) idle &= (mbar_try_wait(&full_bar[st], 0) || mbar_try_wait(&full_bar[st], 1));
      if (idle) break;
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem_o, 512);
}

}  // namespace

int mla_pick_ctas(int B, int max_seq_len, int sm_count) {
  const long long tiles = (long long)std::max(B, 1) * std::max((max_seq_len + kTile - 1) / kTile, 1);
  long long ctas = std::min<long long>(sm_count, std::max<long long>(tiles / 16, 1));
  return (int)std::min<long long>(ctas, kMlaMaxCtas);
}

cudaError_t launch_mla_decode(const MlaDecodeParams& p, bool pdl, cudaStream_t stream) {
  if (p.B <= 0) return cudaSuccess;
  if (p.page_size % kBlk != 0 || p.ctas < 1 || p.ctas > kMlaMaxCtas) return cudaErrorInvalidValue;
  const bool ws = p.variant == 1;
  auto kernel = ws ? mla_decode_ws_kernel : mla_decode_kernel;
  const int smem = ws ? kWsSmem : kSmem;
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.ctas, 1, 1);
  cfg.blockDim = dim3(ws ? kWsThreads : kThreads, 1, 1);
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
  return cudaLaunchKernelEx(&cfg, kernel, p);
}

}  // namespace helix
