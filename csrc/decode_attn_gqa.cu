// Split-KV paged decode attention, GQA (group <= 8 query heads per KV head, head_dim 128, bf16).
//
// Decode attention is bound by streaming the KV cache from HBM once.  The kernel is organised
// around that stream:
//   * fixed shares: the 16-token KV blocks of all (sequence, kv head) pairs form one linear index
//     space that is cut into gridDim.x equal contiguous shares (two CTAs per SM), so every CTA
//     streams the same number of bytes whatever the batch size or the sequence lengths; a share
//     may end one pair and begin the next;
//   * dynamic tail: SMs do not stream equally fast (the spread is about +-10 % and follows the SM,
//     not the data), so the last dyn_pct percent of every long pair stay out of the fixed shares
//     and form that pair's pool of small chunks.  A CTA that has finished its share draws chunks
//     with one atomic each: first from the pool of the pair it was working on - it then simply
//     keeps accumulating into the same running softmax state, no extra partial result - and, when
//     that pool is empty, from the other pools in turn (one parked partial per visited pool);
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
//   * the first loads of the next segment are issued before the epilogue of the current one;
//   * when a CTA leaves a pair, its warps' partial (max, sum, O) are merged through shared memory
//     and parked as one normalised piece in scratch memory, unless the CTA saw the whole pair; every
//     piece adds its block count to the pair's counter, and the CTA whose piece completes the pair
//     folds all pieces - no second launch, and nobody ever waits for another CTA.
// Every mbarrier wait is bounded; on expiry the kernel raises the error flag and leaves.
#include "attention.h"

#include <algorithm>
#include <climits>

#include "helix_common.cuh"
#include "sm100.cuh"

namespace helix {
namespace {

using namespace sm100;

constexpr int kD = 128;           // head dim
constexpr int kBlockTok = 16;     // tokens per KV block (one MMA k-step of P V)
constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr int kTileBytes = kBlockTok * kD * 2;        // 4096: one K (or V) block
constexpr int kStageBytes = 2 * kTileBytes;           // K + V
constexpr int kSmemPipe = kWarps * kStages * kStageBytes;   // 196608
constexpr int kMergeBytes = kWarps * 4 * kD * 4;        // 16384: warps' partial O of four heads / piece list of a fold
constexpr int kSmemBytes = kSmemPipe + kMergeBytes + 1024;   // + alignment slack
constexpr int kMaxList = kMergeBytes / 4;               // pieces one fold can list
constexpr int kQueue = 16;                              // drawn chunks a CTA can have published at a time
static_assert(2 * kGqaMaxCtas <= kMaxList, "a fold lists at most one fixed piece and one helper piece per CTA");
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

__host__ __device__ __forceinline__ int blocks_of(int seq_len) { return (seq_len + kBlockTok - 1) / kBlockTok; }

// blocks of a pair with `nb` blocks that go to its dynamic pool (a whole number of chunks, always < nb)
__host__ __device__ __forceinline__ int dyn_chunks_of(int nb, int pct, int chunk, int min_blocks) {
  if (pct <= 0 || chunk <= 0 || nb < min_blocks) return 0;
  return (int)(((long long)nb * pct / 100) / chunk);
}

__device__ __forceinline__ int ld_relaxed(const int* p) {
  int v;
  asm volatile("ld.relaxed.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int atom_add_acq_rel(int* p, int v) {
  int prev;
  asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;" : "=r"(prev) : "l"(p), "r"(v) : "memory");
  return prev;
}

// The CTA whose piece completed a pair folds all pieces listed in s_list (piece slots) into the final output.
// Warp w folds head w: lanes first share out the pieces' weights, then every lane sums four columns with
// sixteen independent 16-byte loads in flight.  Kept out of line so that its registers do not weigh on the
// streaming loop.
struct FoldArgs {
  const float* part_o;
  const float* part_lse;
  __nv_bfloat16* o;
  float* lse;
  int Hq, lse_base2;
};
__device__ __noinline__ void fold_pieces(FoldArgs p, const int* s_list, int n_pieces, int st_b, int st_kvh, int group,
                                         int warp, int lane) {
  for (int hg = warp; hg < group; hg += kWarps) {
    float M = -INFINITY;
    for (int i = lane; i < n_pieces; i += 32) M = fmaxf(M, __ldcg(p.part_lse + (size_t)s_list[i] * 8 + hg));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    float L = 0.f;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int c0 = 0; c0 < n_pieces; c0 += 32) {
      const int i = c0 + lane;
      float w = 0.f;
      int my_slot = 0;
      if (i < n_pieces) {
        my_slot = s_list[i];
        if (M != -INFINITY) w = fast_exp2(__ldcg(p.part_lse + (size_t)my_slot * 8 + hg) - M);
      }
      L += w;
      const int nbatch = min(32, n_pieces - c0);
      for (int j0 = 0; j0 < nbatch; j0 += 16) {
        float4 v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j0 + j < nbatch) {
            const int sl = __shfl_sync(0xffffffffu, my_slot, j0 + j);
            v[j] = __ldcg(reinterpret_cast<const float4*>(p.part_o + ((size_t)sl * 8 + hg) * kD) + lane);
          }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (j0 + j < nbatch) {
            const float x = __shfl_sync(0xffffffffu, w, j0 + j);
            acc.x += x * v[j].x;
            acc.y += x * v[j].y;
            acc.z += x * v[j].z;
            acc.w += x * v[j].w;
          }
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) L += __shfl_xor_sync(0xffffffffu, L, o);
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int h = st_kvh * group + hg;
    uint2 packed;
    packed.x = pack_bf16(acc.x * inv, acc.y * inv);
    packed.y = pack_bf16(acc.z * inv, acc.w * inv);
    *reinterpret_cast<uint2*>(p.o + ((int64_t)st_b * p.Hq + h) * kD + lane * 4) = packed;
    if (lane == 0) {
      const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
      p.lse[(int64_t)st_b * p.Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1) gqa_decode_kernel(const __grid_constant__ GqaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kWarps][kStages];
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ int s_flag;                         // CTA-wide broadcast word (last arrival, scan result, list length)
  __shared__ int s_dynblk[2];                    // pool blocks the warps streamed in this segment (two slots, alternating)
  __shared__ int s_cursor[2];                    // next block of the segment's queue to hand to a warp (alternating)
  __shared__ int s_chunk_base[kQueue];           // first KV block of a drawn chunk (-1: the pool was empty)
  __shared__ int s_chunk_ready[kQueue];          // tag of the chunk whose base is valid in that slot
  __shared__ int s_closed;                       // tag of the segment whose pool is known to be empty
  __shared__ int s_nb[kGqaSeqTable];             // KV blocks of each sequence
  __shared__ unsigned short s_nc[kGqaSeqTable];  // chunks in each of its pairs' pools

  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
  const int group = p.Hq / p.Hkv;                       // <= 8
  const int g = lane >> 2, t = lane & 3;
  const int Hq = p.Hq, Hkv = p.Hkv;
  const int G = gridDim.x;

  if (tid == 0) {
    for (int w = 0; w < kWarps; ++w)
      for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[w][s], 1);
    mbar_fence_init();
    tma_prefetch_desc(&p.k_map);
    tma_prefetch_desc(&p.v_map);
    s_dynblk[0] = 0;
    s_dynblk[1] = 0;
    s_cursor[0] = 0;
    s_cursor[1] = 0;
    s_closed = 0;
    for (int i = 0; i < kQueue; ++i) s_chunk_ready[i] = 0;
  }
  const bool early_kv = p.kv_stable != 0;
  if (!early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long t_entry = now_ns();
  const unsigned long long deadline = t_entry + p.timeout_ns;
  unsigned long long t_static = 0, t_dyn = 0;
  unsigned n_drawn = 0, n_visits = 0;

  // ---- per-sequence tables and totals ------------------------------------------------------------
  const int cd = p.dyn_chunk;
  const bool dyn_on = p.dyn_pct > 0 && cd > 0 && p.B <= kGqaSeqTable && p.max_helper > 0;
  const int n_tab = min(p.B, kGqaSeqTable);
  for (int i = tid; i < n_tab; i += kThreads) s_nb[i] = blocks_of(p.seq_lens[i]);
  __syncthreads();
  int total_s = 0;                               // blocks in the fixed shares (the host checked that this fits an int)
  {
    long long total = 0;
    for (int b = 0; b < n_tab; ++b) total += s_nb[b];
    for (int b = kGqaSeqTable; b < p.B; ++b) total += blocks_of(p.seq_lens[b]);
    // A pair only gets a pool if what stays in the fixed shares is longer than any share.  A CTA's share then
    // never holds such a pair from its first block to its last fixed block, so the share's two piece slots
    // (one for a pair it continues, one for a pair it starts) still suffice; and some share ends inside the
    // pair, so the pair has at least one CTA that stays on its pool until the pool is empty.
    const long long share_max = (total * Hkv + G - 1) / G;
    for (int b = 0; b < n_tab; ++b) {
      const int nb = s_nb[b];
      int nc = dyn_on ? dyn_chunks_of(nb, p.dyn_pct, cd, p.dyn_min_blocks) : 0;
      if (nb - nc * cd <= share_max || nc > 65535) nc = 0;
      if (tid == 0) s_nc[b] = (unsigned short)nc;
      total_s += nb - nc * cd;
    }
    for (int b = kGqaSeqTable; b < p.B; ++b) total_s += blocks_of(p.seq_lens[b]);
    total_s *= Hkv;
  }
  __syncthreads();
  auto seq_nb = [&](int b) { return b < kGqaSeqTable ? s_nb[b] : blocks_of(p.seq_lens[b]); };
  auto seq_nc = [&](int b) { return (dyn_on && b < kGqaSeqTable) ? (int)s_nc[b] : 0; };
  auto seq_ns = [&](int b) { return seq_nb(b) - seq_nc(b) * cd; };

  const int share = max((total_s + G - 1) / G, 1);
  const int g0 = (int)min((long long)blockIdx.x * share, (long long)total_s);
  const int g1 = min(total_s, g0 + share);

  const int P = p.B * Hkv;
  int* const done_ctr = p.counters;              // [P]
  int* const pool_ctr = p.counters + P;          // [P]
  int* const exit_ctr = p.counters + 2 * P;
  int* const helper_pair = exit_ctr + 8;         // [max_helper]: pair + 1 of the piece parked in each helper slot

  uint8_t* my_smem = smem + warp * (kStages * kStageBytes);
  const float sl2 = p.scale * kLog2e;
  const int mi = lane >> 3, r8 = lane & 7;
  const uint32_t k_row = (uint32_t)(((mi >> 1) << 3) + r8), k_csel = (uint32_t)(mi & 1);
  const uint32_t v_row = (uint32_t)(((mi & 1) << 3) + r8), v_csel = (uint32_t)(mi >> 1);
  int it_ring = 0;           // TMA iterations consumed so far by this warp: fixes stage and parity
  bool ok = true;

  // ---- segments: blocks of one pair that this CTA streams in one go ---------------------------------
  // [kb_begin, kb_end) are blocks of the fixed share, handed to the warps one at a time through a cursor in
  // shared memory (warps do not stream equally fast either); with `pool` the warps then go on drawing chunks of
  // cd blocks from the pair's pool until it is empty.
  struct Seg {
    int b, kvh, kb_begin, kb_end, n_blocks, seq_len;
    int slot;                // piece slot, should this segment open a new running state
    bool pool, valid;
  };
  int cur_b = 0;
  int base = 0;              // share-space index of block 0 of (cur_b, kvh = 0)
  while (cur_b < p.B) {
    const int span = seq_ns(cur_b) * Hkv;
    if (g0 < base + span) break;
    base += span;
    ++cur_b;
  }
  int gcur = g0;
  auto next_static = [&]() {
    Seg sg;
    sg.valid = false;
    sg.pool = false;
    while (gcur < g1 && cur_b < p.B) {
      const int ns = seq_ns(cur_b);
      if (ns == 0) {
        ++cur_b;
        continue;
      }
      sg.b = cur_b;
      sg.seq_len = p.seq_lens[cur_b];
      sg.n_blocks = seq_nb(cur_b);
      sg.kvh = (gcur - base) / ns;
      sg.kb_begin = (gcur - base) - sg.kvh * ns;
      sg.kb_end = min(ns, sg.kb_begin + (g1 - gcur));
      sg.slot = blockIdx.x * 2 + (sg.kb_begin == 0 ? 1 : 0);   // slot 1: the piece that starts its pair
      sg.valid = true;
      gcur += (sg.kb_end - sg.kb_begin);
      sg.pool = gcur >= g1 && seq_nc(cur_b) > 0;    // the share ends here: carry on with this pair's pool
      if (sg.kvh == Hkv - 1 && sg.kb_end == ns) {   // the next segment starts the next sequence
        base += ns * Hkv;
        ++cur_b;
      }
      break;
    }
    return sg;
  };
  int n_pieces_parked = 0;   // helper slots this CTA has used
  auto pool_seg = [&](int pair) {
    Seg sg;
    sg.b = pair / Hkv;
    sg.kvh = pair % Hkv;
    sg.n_blocks = seq_nb(sg.b);
    sg.seq_len = p.seq_lens[sg.b];
    sg.kb_begin = sg.kb_end = 0;
    sg.slot = 2 * G + blockIdx.x * kGqaMaxVisits + n_pieces_parked;
    sg.pool = true;
    sg.valid = true;
    return sg;
  };
  // probe of the pools after `start` (one per thread); stale answers are fine: a pool never refills
  auto probe = [&](int start, int off, int exclude) {
    bool avail = false;
    if (off + tid < P) {
      const int q = (int)(((long long)start + off + tid) % P);
      const int nc = seq_nc(q / Hkv);
      if (nc > 0 && q != exclude) avail = ld_relaxed(pool_ctr + q) < nc;
    }
    return avail;
  };
  // Pick a pool that (probably) still has chunks, starting at pair `start`.  Uniform over the CTA.
  auto pick_pool = [&](int start, bool have_pre, bool pre) {
    for (int off = 0; off < P; off += kThreads) {
      const bool avail = (off == 0 && have_pre) ? pre : probe(start, off, -1);
      if (tid == 0) s_flag = INT_MAX;
      __syncthreads();
      if (avail) atomicMin(&s_flag, off + tid);
      __syncthreads();
      const int f = s_flag;
      __syncthreads();
      if (f != INT_MAX) return (int)(((long long)start + f) % P);
    }
    return -1;
  };

  // ---- per-warp loader: which block comes next, and the loads in flight -------------------------------
  // The blocks of a segment form the CTA's queue: first the blocks of the fixed share, then the chunks drawn
  // from the pair's pool.  Warps take one block at a time from a cursor in shared memory, so a warp that
  // streams faster takes more.  The warp that takes queue position t0 + k * cd (t0 = `ahead` chunks before the
  // end of what the queue holds) draws chunk k from the pool with a global atomic and publishes its first
  // block a few blocks later, when the atomic's round trip (several microseconds under load) is over; so the
  // queue is refilled `ahead` chunks before it runs dry and nobody waits for an atomic.
  int ld_mode = 2;           // 0: taking blocks from the queue, 2: nothing more
  int ld_base = 0, ld_len = 0, ld_kvh = 0, ld_nc = 0, ld_ns = 0, ld_par = 0, ld_t0 = 0, ld_tag = 0;
  bool ld_pool = false;
  const int32_t* ld_bt = p.block_table;
  int* ld_ctr = pool_ctr;
  int c_raw = 0;                                 // lane 0: result of this warp's draw in flight
  bool pd_valid = false;
  int pd_k = 0, pd_age = 0;
  int pend_kb = 0, pend_page = 0;
  bool pend_valid = false;
  int issued = 0, consumed = 0, my_dyn = 0;
  int kq0 = 0, kq1 = 0, kq2 = 0;                 // block index of the load in each ring stage
  const int ahead = max(p.dyn_ahead, 1);

  auto publish_pending = [&]() {
    if (!pd_valid) return;
    const int c = __shfl_sync(0xffffffffu, c_raw, 0);          // waits for the atomic if it is still in flight
    const int base_kb = c < ld_nc ? ld_ns + c * cd : -1;
    if (lane == 0) {
      s_chunk_base[pd_k % kQueue] = base_kb;
      __threadfence_block();
      *reinterpret_cast<volatile int*>(&s_chunk_ready[pd_k % kQueue]) = ld_tag + pd_k + 1;
      if (base_kb < 0) *reinterpret_cast<volatile int*>(&s_closed) = ld_tag;
    }
    pd_valid = false;
  };
  auto issue_draw = [&](int k) {
    publish_pending();                                         // one draw in flight per warp
    ++n_drawn;
    if (*reinterpret_cast<volatile int*>(&s_closed) == ld_tag) {
      if (lane == 0) {                                         // the pool is known to be empty: no atomic needed
        s_chunk_base[k % kQueue] = -1;
        __threadfence_block();
        *reinterpret_cast<volatile int*>(&s_chunk_ready[k % kQueue]) = ld_tag + k + 1;
      }
      return;
    }
    if (lane == 0) c_raw = atomicAdd(ld_ctr, 1);
    pd_valid = true;
    pd_k = k;
    pd_age = 0;
  };
  auto gen_advance = [&]() {
    pend_valid = false;
    if (ld_mode == 0) {
      int i = 0;
      if (lane == 0) i = atomicAdd(&s_cursor[ld_par], 1);
      i = __shfl_sync(0xffffffffu, i, 0);
      if (pd_valid && ++pd_age >= 3) publish_pending();
      if (ld_pool) {
        const int t = i - ld_t0;
        if (t >= 0 && t % cd == 0) issue_draw(t / cd);
      }
      if (i < ld_len) {
        pend_kb = ld_base + i;
        pend_valid = true;
      } else if (!ld_pool) {
        ld_mode = 2;
      } else {
        if (p.trace != nullptr && t_static == 0) t_static = now_ns();
        const int j = (i - ld_len) / cd, off = (i - ld_len) % cd;
        volatile int* rdy = reinterpret_cast<volatile int*>(&s_chunk_ready[j % kQueue]);
        if (*rdy != ld_tag + j + 1) {
          publish_pending();                 // never wait while holding a result that others may be waiting for
          unsigned spins = 0;
          while (*rdy != ld_tag + j + 1) {
            if ((++spins & 255u) == 0u && now_ns() > deadline) {
              ok = false;
              break;
            }
          }
        }
        const int base_kb = ok ? *reinterpret_cast<volatile int*>(&s_chunk_base[j % kQueue]) : -1;
        if (base_kb < 0) {
          ld_mode = 2;
          publish_pending();                 // leaving: hand over what this warp still holds
        } else {
          pend_kb = base_kb + off;
          ++my_dyn;
          pend_valid = true;
        }
      }
    }
    // the page id is looked up one block ahead of the copy that needs it, so the (dependent) block-table
    // load never stalls the warp in front of a copy
    if (pend_valid) pend_page = ld_bt[(pend_kb * kBlockTok) / p.page_size];
  };
  auto issue_pending = [&]() {
    const int ring = it_ring + issued;
    const int stage = ring % kStages;
    if (lane == 0) {
      const int tip = (pend_kb * kBlockTok) % p.page_size;
      uint8_t* dst = my_smem + stage * kStageBytes;
      uint64_t* bar = &full_bar[warp][stage];
      mbar_expect_tx(bar, kStageBytes);
      tma_load_4d(dst, &p.k_map, bar, 0, tip, ld_kvh, pend_page);
      tma_load_4d(dst + 2048, &p.k_map, bar, 64, tip, ld_kvh, pend_page);
      tma_load_4d(dst + kTileBytes, &p.v_map, bar, 0, tip, ld_kvh, pend_page);
      tma_load_4d(dst + kTileBytes + 2048, &p.v_map, bar, 64, tip, ld_kvh, pend_page);
    }
    if (stage == 0) kq0 = pend_kb;
    else if (stage == 1) kq1 = pend_kb;
    else kq2 = pend_kb;
    ++issued;
    gen_advance();
  };
  // Point the loader at a segment and request its first blocks.  Called while the previous segment is still
  // being merged, so the ramp of one segment hides behind the epilogue of the one before.
  auto seg_begin = [&](const Seg& sg) {
    ld_mode = 0;
    ld_par ^= 1;
    ld_tag += 1 << 16;
    ld_base = sg.kb_begin;
    ld_len = sg.kb_end - sg.kb_begin;
    ld_kvh = sg.kvh;
    ld_pool = sg.pool;
    ld_nc = seq_nc(sg.b);
    ld_ns = sg.n_blocks - ld_nc * cd;
    ld_t0 = ld_len - ahead * cd;
    ld_bt = p.block_table + (int64_t)sg.b * p.bt_stride;
    ld_ctr = pool_ctr + (sg.b * Hkv + sg.kvh);
    issued = consumed = 0;
    my_dyn = 0;
    // chunks whose drawing position lies before the start of the queue are drawn right away, one per warp
    if (ld_pool && ld_t0 < 0 && warp < min((-ld_t0 + cd - 1) / cd, kWarps)) issue_draw(warp);
    gen_advance();
    while (issued < kStages && pend_valid) issue_pending();
  };

  float* s_o = reinterpret_cast<float*>(smem + kSmemPipe);   // [kWarps][4][kD]: merge buffer, not part of the rings
  int* s_list = reinterpret_cast<int*>(smem + kSmemPipe);    // the same bytes list a fold's pieces

  Seg cur = next_static();
  if (early_kv) {
    // old KV does not depend on the kernel before us: request the first tiles, then wait for it (q does depend).
    // A segment that reaches the newest token, or that draws from a pool (the counters are re-armed by the
    // launch before this one), waits first.
    const bool wait_first = cur.valid && (cur.kb_end == cur.n_blocks || cur.pool);
    if (wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
    if (cur.valid) seg_begin(cur);
    if (!wait_first) asm volatile("griddepcontrol.wait;" ::: "memory");
  } else if (cur.valid) {
    seg_begin(cur);
  }
  int n_attempts = 0;
  if (!cur.valid && dyn_on) {          // no fixed share (more CTAs than blocks): go straight to the pools
    const int q = pick_pool(blockIdx.x % max(P, 1), false, false);
    ++n_attempts;
    if (q >= 0) {
      cur = pool_seg(q);
      seg_begin(cur);
    }
  }

  // ---- running state of the pair this CTA is accumulating ------------------------------------------
  bool st_active = false;
  int st_b = 0, st_kvh = 0, st_slot = 0, st_blocks = 0, st_nb = 0;
  uint32_t qa[8][2];
  float m_run = -INFINITY, l_run = 0.f;      // for head g (quad-uniform max, per-lane partial sum)
  float o_acc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  int dpar = 0;

  while (cur.valid) {
    const int b = cur.b, kvh = cur.kvh, seq_len = cur.seq_len;
    if (!st_active) {
      st_active = true;
      st_b = b;
      st_kvh = kvh;
      st_slot = cur.slot;
      st_blocks = 0;
      st_nb = cur.n_blocks;
      // Q fragments (A operand, rows = heads of the group, rows >= group are zero)
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
    // a look at the other pools now tells, when this segment is done, where to go next without a round trip
    const bool pre = cur.pool ? probe(b * Hkv + kvh + 1, 0, b * Hkv + kvh) : false;

    while (consumed < issued) {
      const int ring = it_ring + consumed;
      const int stage = ring % kStages;
      if (!mbar_wait(&full_bar[warp][stage], (uint32_t)((ring / kStages) & 1), deadline)) {
        ok = false;
        break;
      }
      const int kb = stage == 0 ? kq0 : (stage == 1 ? kq1 : kq2);
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
      l_run += psum;                              // per-lane partial; the quad is reduced at the flush
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
      ++consumed;
      // this stage is free again: fetch the block kStages ahead
      __syncwarp();
      if (pend_valid) issue_pending();
    }
    it_ring += consumed;
    dpar ^= 1;
    if (lane == 0 && my_dyn != 0) atomicAdd(&s_dynblk[dpar], my_dyn);
    // The vote makes a timeout of one warp a decision of the whole CTA, so no warp is ever left
    // alone at a barrier; it also orders the next merge after the reads of the previous one and
    // publishes the warps' pool block counts.
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    if (p.trace != nullptr) t_dyn = now_ns();
    st_blocks += (cur.kb_end - cur.kb_begin) + s_dynblk[dpar];
    // ---- pick the next segment and start streaming it before the epilogue of this one ---------------
    Seg nxt = next_static();
    if (!nxt.valid && dyn_on && n_pieces_parked < kGqaMaxVisits && n_attempts < 2 * kGqaMaxVisits) {
      const int q = pick_pool(b * Hkv + kvh + 1, cur.pool, pre);
      ++n_attempts;
      if (q >= 0) nxt = pool_seg(q);
    }
    if (nxt.valid) seg_begin(nxt);
    if (tid == 0) {                       // the next use of these slots is two barriers away
      s_dynblk[dpar] = 0;
      s_cursor[dpar] = 0;
    }

    const bool leave = !nxt.valid || nxt.b != st_b || nxt.kvh != st_kvh;
    if (leave && st_blocks == 0) st_active = false;      // a pool that turned out to be empty: nothing to park
    if (leave && st_blocks != 0) {
      // ---- leave the pair: merge the warps' partials, four heads per round --------------------------
      const bool whole = (st_blocks == st_nb);
      const bool helper = st_slot >= 2 * G;
      if (helper) {
        ++n_pieces_parked;
        ++n_visits;
      }
      float* part_o = p.part_o + (size_t)st_slot * 8 * kD;
      float* part_l = p.part_lse + (size_t)st_slot * 8;
      float l_quad = l_run;
      l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 1);
      l_quad += __shfl_xor_sync(0xffffffffu, l_quad, 2);
      if (t == 0) {
        s_m[warp][g] = m_run;
        s_l[warp][g] = l_quad;
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
        for (int idx = tid; idx < 4 * kD; idx += kThreads) {
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
          const int h = st_kvh * group + hg;
          if (whole) {
            p.o[((int64_t)st_b * Hq + h) * kD + d] = __float2bfloat16(out);
            if (d == 0) p.lse[(int64_t)st_b * Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
          } else {
            part_o[hg * kD + d] = out;
            if (d == 0) part_l[hg] = lse2;
          }
        }
      }

      if (!whole) {
        // Publish this piece and count its blocks with ONE acquire-release atomic by thread 0 after a CTA
        // barrier (the barrier orders the other threads' partial stores before it, the release makes
        // them visible device-wide; the acquire side lets the arrival that completes the pair read
        // everybody's pieces).
        const int pair = st_b * Hkv + st_kvh;
        __syncthreads();
        if (tid == 0) {
          if (helper) helper_pair[st_slot - 2 * G] = pair + 1;
          const int prev = atom_add_acq_rel(done_ctr + pair, st_blocks);
          s_flag = (prev + st_blocks == st_nb);
        }
        __syncthreads();
        const bool completes = s_flag != 0;
        if (completes) {
          // ---- this piece completed the pair: fold all of its pieces ---------------------------------
          __syncthreads();                    // everybody has read the verdict before s_flag is reused
          // pieces from the fixed shares: one per CTA whose share overlaps the pair's fixed blocks
          const int ns = st_nb - seq_nc(st_b) * cd;
          int sp0 = 0;
          for (int bb = 0; bb < st_b; ++bb) sp0 += seq_ns(bb);
          sp0 = sp0 * Hkv + st_kvh * ns;
          const int i0 = sp0 / share, i1 = (sp0 + ns - 1) / share;
          const int n_fixed = i1 - i0 + 1;
          for (int i = tid; i < n_fixed; i += kThreads) s_list[i] = (i0 + i) * 2 + (i == 0 ? 1 : 0);
          if (tid == 0) s_flag = n_fixed;
          __syncthreads();
          // pieces parked by CTAs that came over from other pairs
          if (dyn_on) {
            const int n_slots = min(G * kGqaMaxVisits, p.max_helper);
            for (int i = tid; i < n_slots; i += kThreads) {
              if (ld_relaxed(helper_pair + i) == pair + 1) {
                const int k = atomicAdd(&s_flag, 1);
                if (k < kMaxList) s_list[k] = 2 * G + i;
                helper_pair[i] = 0;                        // ready for the next launch
              }
            }
            __syncthreads();
          }
          const int n_pieces = min(s_flag, kMaxList);
          fold_pieces(FoldArgs{p.part_o, p.part_lse, p.o, p.lse, Hq, p.lse_base2}, s_list, n_pieces, st_b, st_kvh, group,
                      warp, lane);
          if (tid == 0) done_ctr[pair] = 0;   // ready for the next launch
          __syncthreads();                    // the list is read; the merge buffer may be reused
        }
      }
      // the running state is consumed: a fresh one starts with the next segment
      st_active = false;
      m_run = -INFINITY;
      l_run = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
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
  } else if (dyn_on && warp == 0) {
    // the last CTA to leave re-arms the pools for the next launch: nobody draws or probes any more
    int last = 0;
    if (lane == 0) last = (atom_add_acq_rel(exit_ctr, 1) == G - 1);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      for (int i = lane; i < P; i += 32) pool_ctr[i] = 0;
      if (lane == 0) *exit_ctr = 0;
    }
  }

  if (p.trace != nullptr && tid == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    unsigned long long* tr = p.trace + (size_t)blockIdx.x * 8;
    tr[0] = t_entry;
    tr[1] = smid;
    tr[2] = t_static;      // warp 0 left the fixed share for the pool (0: never)
    tr[3] = now_ns();
    tr[4] = t_dyn;         // end of the last segment's streaming
    tr[5] = (unsigned long long)n_drawn | ((unsigned long long)n_visits << 32);   // warp 0's chunks, CTA's helper pieces
  }

  // sequences without any token: output 0, LSE -inf (CTA 0 sweeps them)
  if (blockIdx.x == 0) {
    for (int bb = 0; bb < p.B; ++bb) {
      if (p.seq_lens[bb] > 0) continue;
      for (int idx = tid; idx < Hq * kD; idx += kThreads) {
        p.o[(int64_t)bb * Hq * kD + idx] = __float2bfloat16(0.f);
        if (idx < Hq) p.lse[(int64_t)bb * Hq + idx] = -INFINITY;
      }
    }
  }
}

}  // namespace

// Number of CTAs for a launch: one per SM (eight warps each), but never so many that a CTA streams fewer than
// 64 blocks (its fixed ramp + merge cost is worth about that much streaming).
int gqa_pick_ctas(int B, int Hkv, int max_seq_len, int sm_count) {
  const long long blocks = (long long)std::max(B, 1) * Hkv * std::max((max_seq_len + kBlockTok - 1) / kBlockTok, 1);
  long long ctas = std::min<long long>(sm_count, std::max<long long>(blocks / 64, 1));
  return (int)std::min<long long>(ctas, kGqaMaxCtas);
}

void gqa_plan_dynamic(GqaDecodeParams* p, int max_seq_len, int max_helper, int pct_override, int chunk_override,
                      int ahead_override) {
  const int nb = std::max(blocks_of(std::max(max_seq_len, 1)), 1);
  const long long blocks = (long long)std::max(p->B, 1) * p->Hkv * nb;
  p->max_helper = std::min(std::max(max_helper, 0), kGqaMaxHelper);
  p->dyn_min_blocks = 64;
  // a dynamic tail only pays when a CTA's fixed share is long compared with what it keeps drawn ahead
  int pct = (blocks / std::max(p->ctas, 1) >= 256 && p->B <= kGqaSeqTable) ? 30 : 0;
  if (pct_override >= 0) pct = std::min(pct_override, 90);
  const int chunk = chunk_override > 0 ? chunk_override : 8;
  // a global atomic takes about 4 us when HBM is saturated, in which a CTA streams ~24 blocks: stay ~32 ahead
  int ahead = ahead_override > 0 ? ahead_override : (32 + chunk - 1) / chunk;
  ahead = std::min(std::max(ahead, 1), 8);
  if (p->max_helper < p->ctas * kGqaMaxVisits) pct = 0;    // every CTA needs its helper slots
  p->dyn_pct = pct;
  p->dyn_chunk = chunk;
  p->dyn_ahead = ahead;
}

cudaError_t launch_gqa_decode(const GqaDecodeParams& p, bool pdl, cudaStream_t stream) {
  if (p.B <= 0) return cudaSuccess;
  if (p.Hq % p.Hkv != 0 || p.Hq / p.Hkv > 8 || p.page_size % kBlockTok != 0 || p.ctas < 1 || p.ctas > kGqaMaxCtas ||
      p.max_helper < 0 || p.max_helper > kGqaMaxHelper || p.dyn_pct < 0 || p.dyn_pct > 90 ||
      (p.dyn_pct > 0 && (p.dyn_chunk < 1 || p.dyn_ahead < 1 || p.dyn_ahead > 8 || p.max_helper < p.ctas * kGqaMaxVisits)))
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
  cfg.blockDim = dim3(kThreads, 1, 1);
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
