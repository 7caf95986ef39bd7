// Split-KV paged decode attention, GQA (group <= 8 query heads per KV head, head_dim 128, bf16).
//
// Decode attention is bound by streaming the KV cache from HBM once.  The kernel is organised
// around that stream:
//   * grid (split, kv head, sequence); every warp of a CTA owns its own 3-stage ring of 16-token
//     KV blocks in shared memory and walks blocks warp, warp + W, ... of the split, so warps never
//     synchronise with each other while streaming;
//   * K and V blocks arrive by TMA tiled loads (cp.async.bulk.tensor, 128-byte swizzle, one
//     [16 x 64] box per half row) that complete on the warp's mbarrier; the paged layout is
//     handled by the tensor map (coordinates: d, token in page, kv head, page), so both
//     [pages, heads, page, d] and [pages, page, heads, d] caches work;
//   * the 8 query heads of the group form the (padded) 16-row A operand of m16n8k16 tensor-core
//     MMAs: S = Q K^T per block, online softmax in registers in the base-2 domain, then O += P V
//     with V fragments read by transposing ldmatrix from the swizzled tile;
//   * the warps' partial (max, sum, O) are merged through shared memory; with several KV splits
//     each CTA parks a normalised partial in scratch memory and the last CTA of a (sequence,
//     kv head) folds the splits — no second launch.
// Every mbarrier wait is bounded; on expiry the kernel raises the error flag and leaves.
#include "attention.h"

#include <algorithm>

#include "helix_common.cuh"
#include "sm100.cuh"

namespace helix {
namespace {

using namespace sm100;

constexpr int kD = 128;           // head dim
constexpr int kBlockTok = 16;     // tokens per KV block (one MMA k-step of P V)
constexpr int kWarps = 4;
constexpr int kStages = 3;
constexpr int kTileBytes = kBlockTok * kD * 2;        // 4096: one K (or V) block
constexpr int kStageBytes = 2 * kTileBytes;           // K + V
constexpr int kSmemPipe = kWarps * kStages * kStageBytes;   // 98304
constexpr int kSmemBytes = kSmemPipe + 1024;          // + alignment slack
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__global__ void __launch_bounds__(kWarps * 32, 2) gqa_decode_kernel(const __grid_constant__ GqaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kWarps][kStages];
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ int s_last;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int group = p.Hq / p.Hkv;                       // <= 8
  const int g = lane >> 2, t = lane & 3;

  if (threadIdx.x == 0) {
    for (int w = 0; w < kWarps; ++w)
      for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[w][s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
  }
  __syncthreads();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long deadline = now_ns() + p.timeout_ns;

  const int seq_len = p.seq_lens[b];
  const int n_blocks = (seq_len + kBlockTok - 1) / kBlockTok;
  const int per_split = (n_blocks + p.splits - 1) / p.splits;
  const int kb_begin = split * per_split;
  const int kb_end = min(n_blocks, kb_begin + per_split);
  const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
  uint8_t* my_smem = smem + warp * (kStages * kStageBytes);

  // ---- Q fragments (A operand, rows = heads of the group, rows >= group are zero) ----------
  uint32_t qa[8][2];
  {
    const __nv_bfloat16* qrow = p.q + (int64_t)b * p.q_stride_b + (int64_t)(kvh * group + g) * p.q_stride_h;
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      qa[ks][0] = 0u;
      qa[ks][1] = 0u;
      if (g < group) {
        qa[ks][0] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 2 * t);
        qa[ks][1] = *reinterpret_cast<const uint32_t*>(qrow + ks * 16 + 8 + 2 * t);
      }
    }
  }

  auto issue = [&](int stage, int kb) {
    const int tok0 = kb * kBlockTok;
    const int page = bt[tok0 / p.page_size];
    const int tip = tok0 % p.page_size;
    uint8_t* dst = my_smem + stage * kStageBytes;
    uint64_t* bar = &full_bar[warp][stage];
    mbar_expect_tx(bar, kStageBytes);
    tma_load_4d(dst, &p.k_map, bar, 0, tip, kvh, page);
    tma_load_4d(dst + 2048, &p.k_map, bar, 64, tip, kvh, page);
    tma_load_4d(dst + kTileBytes, &p.v_map, bar, 0, tip, kvh, page);
    tma_load_4d(dst + kTileBytes + 2048, &p.v_map, bar, 64, tip, kvh, page);
  };

  const int my_first = kb_begin + warp;
  const int my_count = my_first < kb_end ? (kb_end - my_first + kWarps - 1) / kWarps : 0;
  if (lane == 0) {
    for (int i = 0; i < kStages && i < my_count; ++i) issue(i, my_first + i * kWarps);
  }

  float m_run = -INFINITY, l_run = 0.f;      // for head g (quad-uniform), base-2 domain
  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  const float sl2 = p.scale * kLog2e;
  bool ok = true;

  // per-lane ldmatrix row / chunk selectors
  const int mi = lane >> 3, r8 = lane & 7;
  const uint32_t k_row = (uint32_t)(((mi >> 1) << 3) + r8), k_csel = (uint32_t)(mi & 1);
  const uint32_t v_row = (uint32_t)(((mi & 1) << 3) + r8), v_csel = (uint32_t)(mi >> 1);

  for (int it = 0; it < my_count; ++it) {
    const int stage = it % kStages;
    const int kb = my_first + it * kWarps;
    if (!mbar_wait(&full_bar[warp][stage], (uint32_t)((it / kStages) & 1), deadline)) {
      ok = false;
      break;
    }
    const uint32_t kbase = smem_u32(my_smem + stage * kStageBytes);
    const uint32_t vbase = kbase + kTileBytes;

    // S = Q K^T for 16 tokens: two n-tiles of 8 tokens
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint32_t c16 = 2u * ks + k_csel;
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4(kbase + (c16 >> 3) * 2048u + swz128(k_row, c16 & 7u), r0, r1, r2, r3);
      mma_bf16_16816(s[0], qa[ks][0], 0u, qa[ks][1], 0u, r0, r1);
      mma_bf16_16816(s[1], qa[ks][0], 0u, qa[ks][1], 0u, r2, r3);
    }
    // scale, mask the tail of the sequence, online softmax (rows g of the quad)
    float mx = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int tok = kb * kBlockTok + nt * 8 + 2 * t + j;
        float v = s[nt][j] * sl2;
        if (tok >= seq_len) v = -INFINITY;
        s[nt][j] = v;
        mx = fmaxf(mx, v);
      }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m_run, mx);       // finite: a block always holds >= 1 valid token
    const float alpha = exp2f(m_run - m_new);   // 0 on the first block (m_run = -inf)
    float psum = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt)
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[nt][j] = exp2f(s[nt][j] - m_new);
        psum += s[nt][j];
      }
    psum += __shfl_xor_sync(0xffffffffu, psum, 1);
    psum += __shfl_xor_sync(0xffffffffu, psum, 2);
    l_run = l_run * alpha + psum;
    m_run = m_new;
    const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]);
    const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]);
    // O = O * alpha + P V
#pragma unroll
    for (int jj = 0; jj < 8; ++jj) {
      const uint32_t c16 = 2u * jj + v_csel;
      uint32_t r0, r1, r2, r3;
      ldmatrix_x4_trans(vbase + (c16 >> 3) * 2048u + swz128(v_row, c16 & 7u), r0, r1, r2, r3);
      o_acc[2 * jj][0] *= alpha;
      o_acc[2 * jj][1] *= alpha;
      o_acc[2 * jj + 1][0] *= alpha;
      o_acc[2 * jj + 1][1] *= alpha;
      mma_bf16_16816(o_acc[2 * jj], pa0, 0u, pa2, 0u, r0, r1);
      mma_bf16_16816(o_acc[2 * jj + 1], pa0, 0u, pa2, 0u, r2, r3);
    }
    // this stage is free again: fetch the block kStages iterations ahead
    __syncwarp();
    if (lane == 0 && it + kStages < my_count) issue(stage, kb + kStages * kWarps);
  }
  if (!ok) {
    if (lane == 0) atomicCAS(p.error_flag, 0, (int)kTimeoutMbarrier);
    // bounded grace period for copies that may still be in flight into this warp's ring
    const unsigned long long grace = now_ns() + 2000000ull;
    for (int s = 0; s < kStages; ++s) {
      unsigned spins = 0;
      while (!mbar_try_wait(&full_bar[warp][s], 0) && !mbar_try_wait(&full_bar[warp][s], 1)) {
        if ((++spins & 255u) == 0u && now_ns() > grace) break;
      }
    }
  }
  __syncthreads();   // every warp is done with its ring: reuse it for the merge

  // ---- merge the warps' partials ---------------------------------------------------------------
  float* s_o = reinterpret_cast<float*>(smem);           // [kWarps][8][kD]
  if (g < 8) {
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) {
      float2 v = make_float2(o_acc[nt][0], o_acc[nt][1]);
      *reinterpret_cast<float2*>(&s_o[(warp * 8 + g) * kD + nt * 8 + 2 * t]) = v;
    }
    if (t == 0) {
      s_m[warp][g] = m_run;
      s_l[warp][g] = l_run;
    }
  }
  __syncthreads();

  const int Hq = p.Hq;
  for (int idx = threadIdx.x; idx < group * kD; idx += blockDim.x) {
    const int hg = idx / kD, d = idx - hg * kD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][hg]);
    float L = 0.f, O = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < kWarps; ++w) {
        const float sc = exp2f(s_m[w][hg] - M);
        L += s_l[w][hg] * sc;
        O += s_o[(w * 8 + hg) * kD + d] * sc;
      }
    }
    const float out = L > 0.f ? O / L : 0.f;
    const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
    const int h = kvh * group + hg;
    if (p.splits == 1) {
      p.o[((int64_t)b * Hq + h) * kD + d] = __float2bfloat16(out);
      if (d == 0) p.lse[(int64_t)b * Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
    } else {
      p.part_o[(((int64_t)b * Hq + h) * p.splits + split) * kD + d] = out;
      if (d == 0) p.part_lse[((int64_t)b * Hq + h) * p.splits + split] = lse2;
    }
  }
  if (p.splits == 1) return;

  // ---- the last CTA of this (sequence, kv head) folds the splits ---------------------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&p.counters[b * p.Hkv + kvh], 1);
    s_last = (prev == p.splits - 1);
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < group * kD; idx += blockDim.x) {
    const int hg = idx / kD, d = idx - hg * kD;
    const int h = kvh * group + hg;
    const float* pl = p.part_lse + ((int64_t)b * Hq + h) * p.splits;
    const float* po = p.part_o + ((int64_t)b * Hq + h) * p.splits * kD + d;
    float M = -INFINITY;
    for (int s = 0; s < p.splits; ++s) M = fmaxf(M, __ldcg(pl + s));
    float L = 0.f, O = 0.f;
    if (M != -INFINITY) {
      for (int s = 0; s < p.splits; ++s) {
        const float w = exp2f(__ldcg(pl + s) - M);
        L += w;
        O += w * __ldcg(po + (int64_t)s * kD);
      }
    }
    p.o[((int64_t)b * Hq + h) * kD + d] = __float2bfloat16(L > 0.f ? O / L : 0.f);
    if (d == 0) {
      const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
      p.lse[(int64_t)b * Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
    }
  }
  if (threadIdx.x == 0) p.counters[b * p.Hkv + kvh] = 0;   // ready for the next launch
}

}  // namespace

int gqa_pick_splits(int B, int Hkv, int max_seq_len, int sm_count) {
  const int ctas_base = std::max(B * Hkv, 1);
  const int blocks = std::max((max_seq_len + kBlockTok - 1) / kBlockTok, 1);
  // aim for ~4 waves of 2 CTAs per SM, but keep at least 8 blocks per warp in a split
  int want = (sm_count * 2 * 4 + ctas_base - 1) / ctas_base;
  int max_by_len = std::max(blocks / (kWarps * 8), 1);
  return std::max(1, std::min(want, max_by_len));
}

cudaError_t launch_gqa_decode(const GqaDecodeParams& p, bool pdl, cudaStream_t stream) {
  if (p.B <= 0) return cudaSuccess;
  if (p.Hq % p.Hkv != 0 || p.Hq / p.Hkv > 8 || p.page_size % kBlockTok != 0 || p.splits < 1)
    return cudaErrorInvalidValue;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gqa_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    if (dev < 64) attr_set[dev] = true;
  }
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.splits, p.Hkv, p.B);
  cfg.blockDim = dim3(kWarps * 32, 1, 1);
  cfg.dynamicSmemBytes = kSmemBytes;
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
  return cudaLaunchKernelEx(&cfg, gqa_decode_kernel, p);
}

}  // namespace helix
