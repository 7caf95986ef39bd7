// Split-KV paged decode attention, GQA (group <= 8 query heads per KV head, head_dim 128, bf16).
//
// Decode attention is bound by streaming the KV cache from HBM once.  The kernel is organised
// around that stream:
//   * balanced partition: the 16-token KV blocks of all (sequence, kv head) pairs form one linear
//     index space that is cut into gridDim.x equal contiguous chunks (two CTAs per SM), so every
//     CTA streams the same number of bytes whatever the batch size or the sequence lengths; a
//     chunk may end one pair and begin the next;
//   * every warp of a CTA owns its own 3-stage ring of KV blocks in shared memory and walks blocks
//     warp, warp + W, ... of the CTA's segment, so warps never synchronise while streaming;
//   * K and V blocks arrive by TMA tiled loads (cp.async.bulk.tensor, 128-byte swizzle, one
//     [16 x 64] box per half row) that complete on the warp's mbarrier; the paged layout is
//     handled by the tensor map (coordinates: d, token in page, kv head, page), so both
//     [pages, heads, page, d] and [pages, page, heads, d] caches work;
//   * the 8 query heads of the group form the (padded) 16-row A operand of m16n8k16 tensor-core
//     MMAs: S = Q K^T per block, online softmax in registers in the base-2 domain (the running
//     max is only re-applied when it moves), then O += P V with V fragments read by transposing
//     ldmatrix from the swizzled tile;
//   * the first loads of a CTA's next segment are issued before the epilogue of the current one;
//   * the warps' partial (max, sum, O) are merged through shared memory; a segment that does not
//     cover its whole pair parks a normalised partial in scratch memory (two slots per CTA) and
//     the last CTA to finish a pair folds the pieces — no second launch.
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
constexpr int kMergeBytes = kWarps * 4 * kD * 4;        // 8192: warps' partial O of four heads
constexpr int kSmemBytes = kSmemPipe + kMergeBytes + 1024;   // + alignment slack
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ int blocks_of(int seq_len) { return (seq_len + kBlockTok - 1) / kBlockTok; }

__global__ void __launch_bounds__(kWarps * 32, 2) gqa_decode_kernel(const __grid_constant__ GqaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kWarps][kStages];
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ int s_last;

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.Hq / p.Hkv;                       // <= 8
  const int g = lane >> 2, t = lane & 3;
  const int Hq = p.Hq, Hkv = p.Hkv;

  if (threadIdx.x == 0) {
    for (int w = 0; w < kWarps; ++w)
      for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[w][s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
  }
  __syncthreads();
  const bool early_kv = p.kv_stable != 0;
  if (!early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long t_entry = now_ns();
  const unsigned long long deadline = t_entry + p.timeout_ns;
  unsigned long long t_first = 0, t_stream = 0;

  // ---- this CTA's chunk [g0, g1) of the global block space (pair-major: pair = b * Hkv + kvh) ----
  long long total = 0;
  {
    // block counts of up to 512 sequences are fetched by all threads at once; longer batches
    // fall back to a serial walk for the remainder
    __shared__ int s_nb[512];
    for (int i = threadIdx.x; i < min(p.B, 512); i += blockDim.x) s_nb[i] = blocks_of(p.seq_lens[i]);
    __syncthreads();
    for (int b = 0; b < min(p.B, 512); ++b) total += s_nb[b];
    for (int b = 512; b < p.B; ++b) total += blocks_of(p.seq_lens[b]);
    total *= Hkv;
  }
  const long long chunk = max((total + gridDim.x - 1) / (long long)gridDim.x, 1LL);
  const long long g0 = (long long)blockIdx.x * chunk;
  const long long g1 = min(total, g0 + chunk);

  uint8_t* my_smem = smem + warp * (kStages * kStageBytes);
  const float sl2 = p.scale * kLog2e;
  const int mi = lane >> 3, r8 = lane & 7;
  const uint32_t k_row = (uint32_t)(((mi >> 1) << 3) + r8), k_csel = (uint32_t)(mi & 1);
  const uint32_t v_row = (uint32_t)(((mi & 1) << 3) + r8), v_csel = (uint32_t)(mi >> 1);
  int it_ring = 0;           // TMA iterations issued so far by this warp: fixes stage and parity
  bool ok = true;

  // ---- segment cursor: a segment is the part of one (sequence, kv head) pair inside [g0, g1) ----
  struct Seg {
    int b, kvh, kb_begin, kb_end, n_blocks, seq_len;
    long long pair_start;
    bool valid;
  };
  int cur_b = 0;
  long long base = 0;        // global index of block 0 of (cur_b, kvh = 0)
  while (cur_b < p.B) {
    const long long span = (long long)blocks_of(p.seq_lens[cur_b]) * Hkv;
    if (g0 < base + span) break;
    base += span;
    ++cur_b;
  }
  long long gcur = g0;
  auto next_segment = [&]() {
    Seg sg;
    sg.valid = false;
    while (gcur < g1 && cur_b < p.B) {
      const int seq_len = p.seq_lens[cur_b];
      const int n_blocks = blocks_of(seq_len);
      if (n_blocks == 0) {
        ++cur_b;
        continue;
      }
      sg.b = cur_b;
      sg.seq_len = seq_len;
      sg.n_blocks = n_blocks;
      sg.kvh = (int)((gcur - base) / n_blocks);
      sg.kb_begin = (int)((gcur - base) - (long long)sg.kvh * n_blocks);
      sg.kb_end = (int)min((long long)n_blocks, (long long)sg.kb_begin + (g1 - gcur));
      sg.pair_start = base + (long long)sg.kvh * n_blocks;
      sg.valid = true;
      gcur += (sg.kb_end - sg.kb_begin);
      if (sg.kvh == Hkv - 1 && sg.kb_end == n_blocks) {   // the next segment starts the next sequence
        base += (long long)n_blocks * Hkv;
        ++cur_b;
      }
      break;
    }
    return sg;
  };

  auto issue = [&](const Seg& sg, int ring, int kb, int page) {
    const int tip = (kb * kBlockTok) % p.page_size;
    uint8_t* dst = my_smem + (ring % kStages) * kStageBytes;
    uint64_t* bar = &full_bar[warp][ring % kStages];
    mbar_expect_tx(bar, kStageBytes);
    tma_load_4d(dst, &p.k_map, bar, 0, tip, sg.kvh, page);
    tma_load_4d(dst + 2048, &p.k_map, bar, 64, tip, sg.kvh, page);
    tma_load_4d(dst + kTileBytes, &p.v_map, bar, 0, tip, sg.kvh, page);
    tma_load_4d(dst + kTileBytes + 2048, &p.v_map, bar, 64, tip, sg.kvh, page);
  };
  // first loads of a segment; called while the previous segment is still being merged, so the
  // ramp of one segment hides behind the epilogue of the one before
  auto prologue = [&](const Seg& sg) {
    const int32_t* bt = p.block_table + (int64_t)sg.b * p.bt_stride;
    const int my_first = sg.kb_begin + warp;
    const int my_count = my_first < sg.kb_end ? (sg.kb_end - my_first + kWarps - 1) / kWarps : 0;
    int pg[kStages];
#pragma unroll
    for (int i = 0; i < kStages; ++i)
      pg[i] = i < my_count ? bt[((my_first + i * kWarps) * kBlockTok) / p.page_size] : 0;
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < kStages; ++i)
        if (i < my_count) issue(sg, it_ring + i, my_first + i * kWarps, pg[i]);
    }
  };

  float* s_o = reinterpret_cast<float*>(smem + kSmemPipe);   // [kWarps][4][kD]: merge buffer, not part of the rings

  Seg cur = next_segment();
  if (early_kv) {
    // old KV does not depend on the kernel before us: request the first tiles, then wait for it (q does depend).
    // A segment that reaches the newest token waits first: that token's K/V row may still be on its way.
    const bool touches_newest = cur.valid && cur.kb_end == cur.n_blocks;
    if (touches_newest) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (cur.valid) prologue(cur);
    if (!touches_newest) asm volatile("griddepcontrol.wait;" ::: "memory");
  } else if (cur.valid) {
    prologue(cur);
  }
  while (cur.valid) {
    const int b = cur.b, kvh = cur.kvh, seq_len = cur.seq_len, n_blocks = cur.n_blocks;
    const int kb_begin = cur.kb_begin, kb_end = cur.kb_end;
    const bool whole = (kb_begin == 0 && kb_end == n_blocks);
    const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
    // page ids are looked up one iteration ahead of the TMA that needs them, so the (dependent)
    // block-table load never stalls the warp in front of a copy
    auto page_of = [&](int kb) { return bt[(kb * kBlockTok) / p.page_size]; };
    const int my_first = kb_begin + warp;
    const int my_count = my_first < kb_end ? (kb_end - my_first + kWarps - 1) / kWarps : 0;
    int next_page = kStages < my_count ? page_of(my_first + kStages * kWarps) : 0;

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

    float m_run = -INFINITY, l_run = 0.f;      // for head g (quad-uniform max, per-lane partial sum)
    float o_acc[16][4];
#pragma unroll
    for (int i = 0; i < 16; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;

    for (int it = 0; it < my_count; ++it) {
      const int ring = it_ring + it;
      const int stage = ring % kStages;
      const int kb = my_first + it * kWarps;
      if (!mbar_wait(&full_bar[warp][stage], (uint32_t)((ring / kStages) & 1), deadline)) {
        ok = false;
        break;
      }
      if (p.trace != nullptr && t_first == 0) t_first = now_ns();
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
      // the running max only moves when some row saw a larger score: skip the rescale otherwise
      const bool grow = __any_sync(0xffffffffu, mx > m_run);
      float alpha = 1.f;
      if (grow) {
        const float m_new = fmaxf(m_run, mx);     // finite: a block always holds >= 1 valid token
        alpha = fast_exp2(m_run - m_new);         // 0 on the first block (m_run = -inf)
        m_run = m_new;
        l_run *= alpha;
      }
      float psum = 0.f;
#pragma unroll
      for (int nt = 0; nt < 2; ++nt)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          s[nt][j] = fast_exp2(s[nt][j] - m_run);
          psum += s[nt][j];
        }
      l_run += psum;                              // per-lane partial; the quad is reduced at the end
      const uint32_t pa0 = pack_bf16(s[0][0], s[0][1]);
      const uint32_t pa2 = pack_bf16(s[1][0], s[1][1]);
      // O = O * alpha + P V
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const uint32_t c16 = 2u * jj + v_csel;
        uint32_t r0, r1, r2, r3;
        ldmatrix_x4_trans(vbase + (c16 >> 3) * 2048u + swz128(v_row, c16 & 7u), r0, r1, r2, r3);
        if (grow) {
          o_acc[2 * jj][0] *= alpha;
          o_acc[2 * jj][1] *= alpha;
          o_acc[2 * jj + 1][0] *= alpha;
          o_acc[2 * jj + 1][1] *= alpha;
        }
        mma_bf16_16816(o_acc[2 * jj], pa0, 0u, pa2, 0u, r0, r1);
        mma_bf16_16816(o_acc[2 * jj + 1], pa0, 0u, pa2, 0u, r2, r3);
      }
      // this stage is free again: fetch the block kStages iterations ahead
      __syncwarp();
      if (lane == 0 && it + kStages < my_count) issue(cur, ring + kStages, kb + kStages * kWarps, next_page);
      if (it + 1 + kStages < my_count) next_page = page_of(kb + (kStages + 1) * kWarps);
    }
    it_ring += my_count;
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
    l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
    // The vote makes a timeout of one warp a decision of the whole CTA, so no warp is ever left
    // alone at a barrier; it also orders this merge after the reads of the previous one.
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    if (p.trace != nullptr) t_stream = now_ns();
    // start streaming the next segment before the epilogue of this one
    const Seg nxt = next_segment();
    if (nxt.valid) prologue(nxt);

    // ---- merge the warps' partials, four heads per round -------------------------------------------
    const int slot = (kb_begin == 0) ? 1 : 0;   // slot 1: the piece that starts its pair, slot 0: a continuation
    float* part_o = p.part_o + ((size_t)(blockIdx.x * 2 + slot) * 8) * kD;
    float* part_l = p.part_lse + (size_t)(blockIdx.x * 2 + slot) * 8;
    if (t == 0) {
      s_m[warp][g] = m_run;
      s_l[warp][g] = l_run;
    }
#pragma unroll
    for (int round = 0; round < 2; ++round) {
      if (round == 1) __syncthreads();          // round 0's reads are done
      if ((g >> 2) == round) {
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
          float2 v = make_float2(o_acc[nt][0], o_acc[nt][1]);
          *reinterpret_cast<float2*>(&s_o[(warp * 4 + (g & 3)) * kD + nt * 8 + 2 * t]) = v;
        }
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < 4 * kD; idx += blockDim.x) {
        const int hg = round * 4 + idx / kD, d = idx % kD;
        if (hg >= group) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) M = fmaxf(M, s_m[w][hg]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
          for (int w = 0; w < kWarps; ++w) {
            const float sc = fast_exp2(s_m[w][hg] - M);
            L += s_l[w][hg] * sc;
            O += s_o[(w * 4 + (hg & 3)) * kD + d] * sc;
          }
        }
        const float out = L > 0.f ? O / L : 0.f;
        const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
        const int h = kvh * group + hg;
        if (whole) {
          p.o[((int64_t)b * Hq + h) * kD + d] = __float2bfloat16(out);
          if (d == 0) p.lse[(int64_t)b * Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
        } else {
          part_o[hg * kD + d] = out;
          if (d == 0) part_l[hg] = lse2;
        }
      }
    }

    if (!whole) {
      // ---- the last CTA to finish this pair folds its pieces ---------------------------------------
      const int first_cta = (int)(cur.pair_start / chunk);
      const int last_cta = (int)((cur.pair_start + n_blocks - 1) / chunk);
      const int pieces = last_cta - first_cta + 1;
      // Publish this piece and count it with ONE acquire-release atomic by thread 0 after a CTA
      // barrier (the barrier orders the other threads' partial stores before it, the release makes
      // them visible device-wide; the acquire side lets the last arrival read everybody's pieces).
      __syncthreads();
      if (threadIdx.x == 0) {
        int prev;
        asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                     : "=r"(prev) : "l"(p.counters + (b * Hkv + kvh)) : "memory");
        s_last = (prev == pieces - 1);
      }
      __syncthreads();
      if (s_last) {
        // warp w folds heads 2w and 2w + 1: lanes first share out the pieces' weights, then every
        // lane sums four columns with eight independent 16-byte loads in flight
        auto piece_slot = [&](int c) { return (size_t)(c * 2 + (c == first_cta ? 1 : 0)); };
        for (int hh = 0; hh < 2; ++hh) {
          const int hg = warp * 2 + hh;
          if (hg >= group) continue;
          float M = -INFINITY;
          for (int c = first_cta + lane; c <= last_cta; c += 32)
            M = fmaxf(M, __ldcg(p.part_lse + piece_slot(c) * 8 + hg));
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
          float L = 0.f;
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          for (int c0 = first_cta; c0 <= last_cta; c0 += 32) {
            const int c = c0 + lane;
            float w = 0.f;
            if (c <= last_cta && M != -INFINITY) w = fast_exp2(__ldcg(p.part_lse + piece_slot(c) * 8 + hg) - M);
            L += w;
            const int nb = min(32, last_cta - c0 + 1);
            for (int j0 = 0; j0 < nb; j0 += 8) {
              float4 v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (j0 + j < nb)
                  v[j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + (piece_slot(c0 + j0 + j) * 8 + hg) * kD) + lane);
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (j0 + j < nb) {
                  const float wj = __shfl_sync(0xffffffffu, w, j0 + j);
                  acc.x += wj * v[j].x;
                  acc.y += wj * v[j].y;
                  acc.z += wj * v[j].z;
                  acc.w += wj * v[j].w;
                }
              }
            }
          }
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
          const float inv = L > 0.f ? 1.f / L : 0.f;
          const int h = kvh * group + hg;
          uint2 packed;
          packed.x = pack_bf16(acc.x * inv, acc.y * inv);
          packed.y = pack_bf16(acc.z * inv, acc.w * inv);
          *reinterpret_cast<uint2*>(p.o + ((int64_t)b * Hq + h) * kD + lane * 4) = packed;
          if (lane == 0) {
            const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
            p.lse[(int64_t)b * Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
          }
        }
        if (threadIdx.x == 0) p.counters[b * Hkv + kvh] = 0;   // ready for the next launch
      }
    }
    cur = nxt;
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

  if (p.trace != nullptr && threadIdx.x == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    p.trace[blockIdx.x * 4 + 0] = t_entry;
    p.trace[blockIdx.x * 4 + 1] = (t_first << 8) | (unsigned long long)(smid & 0xffu);   // low byte: SM id
    p.trace[blockIdx.x * 4 + 2] = t_stream;
    p.trace[blockIdx.x * 4 + 3] = now_ns();
  }

  // sequences without any token: output 0, LSE -inf (CTA 0 sweeps them)
  if (blockIdx.x == 0) {
    for (int bb = 0; bb < p.B; ++bb) {
      if (p.seq_lens[bb] > 0) continue;
      for (int idx = threadIdx.x; idx < Hq * kD; idx += blockDim.x) {
        p.o[(int64_t)bb * Hq * kD + idx] = __float2bfloat16(0.f);
        if (idx < Hq) p.lse[(int64_t)bb * Hq + idx] = -INFINITY;
      }
    }
  }
}

}  // namespace

// Number of CTAs for a launch: two per SM, but never so many that a CTA streams fewer than
// 32 blocks (its fixed ramp + merge cost is worth about that much streaming).
int gqa_pick_ctas(int B, int Hkv, int max_seq_len, int sm_count) {
  const long long blocks = (long long)std::max(B, 1) * Hkv * std::max((max_seq_len + kBlockTok - 1) / kBlockTok, 1);
  long long ctas = std::min<long long>(2LL * sm_count, std::max<long long>(blocks / 32, 1));
  return (int)std::min<long long>(ctas, kGqaMaxCtas);
}

cudaError_t launch_gqa_decode(const GqaDecodeParams& p, bool pdl, cudaStream_t stream) {
  if (p.B <= 0) return cudaSuccess;
  if (p.Hq % p.Hkv != 0 || p.Hq / p.Hkv > 8 || p.page_size % kBlockTok != 0 || p.ctas < 1 || p.ctas > kGqaMaxCtas)
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
  cfg.gridDim = dim3(p.ctas, 1, 1);
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
