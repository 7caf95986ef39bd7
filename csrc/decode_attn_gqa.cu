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
constexpr int kWarps = 4;
constexpr int kThreads = kWarps * 32;
constexpr int kStages = 3;
constexpr int kTileBytes = kBlockTok * kD * 2;        // 4096: one K (or V) block
constexpr int kStageBytes = 2 * kTileBytes;           // K + V
constexpr int kSmemPipe = kWarps * kStages * kStageBytes;   // 98304
constexpr int kMergeBytes = kWarps * 4 * kD * 4;        // 8192: warps' partial O of four heads / piece list of a fold
constexpr int kSmemBytes = kSmemPipe + kMergeBytes + 1024;   // + alignment slack
constexpr int kMaxList = kMergeBytes / 4;               // pieces one fold can list
constexpr int kMaxPoolChunks = kMaxList - kGqaMaxCtas;   // chunks one pair's pool may hold: a fold lists at most one piece
                                                        // per CTA plus one per chunk of the pair
static_assert(kMaxPoolChunks > 0, "the piece list must hold one piece per CTA");
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
// Warp w folds heads 2w and 2w + 1 together: lanes first share out the pieces' weights, then every lane sums
// four columns of both heads with sixteen independent 16-byte loads in flight.  Kept out of line so that its
// registers do not weigh on the streaming loop.
struct FoldArgs {
  const float* part_o;
  const float* part_lse;
  __nv_bfloat16* o;
  float* lse;
  int Hq, lse_base2;
};
constexpr int kFoldBatch = 8;
__device__ __noinline__ void fold_pieces(FoldArgs p, const int* s_list, int n_pieces, int st_b, int st_kvh, int group,
                                         int warp, int lane) {
  // Warp w folds heads 2w and 2w + 1.  Pieces are taken eight at a time: their LSEs and their rows are requested
  // together (16 + 2 independent loads per lane), so a batch costs ONE round trip to L2; the running maximum is
  // carried from batch to batch as in an online softmax.  (Sixteen at a time needs so many registers that the
  // streaming loop of the kernel around this function starts to spill: measured 30 % slower.)
  const int h0 = warp * 2, h1 = warp * 2 + 1;
  if (h0 >= group) return;
  const bool has1 = h1 < group;
  float M0 = -INFINITY, M1 = -INFINITY, L0 = 0.f, L1 = 0.f;
  float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = 0; c0 < n_pieces; c0 += kFoldBatch) {
    const int nb = min(kFoldBatch, n_pieces - c0);
    const int my_slot = lane < nb ? s_list[c0 + lane] : 0;
    float l0 = -INFINITY, l1 = -INFINITY;
    if (lane < nb) {
      l0 = __ldcg(p.part_lse + (size_t)my_slot * 8 + h0);
      if (has1) l1 = __ldcg(p.part_lse + (size_t)my_slot * 8 + h1);
    }
    float4 v0[kFoldBatch], v1[kFoldBatch];
#pragma unroll
    for (int j = 0; j < kFoldBatch; ++j) {
      if (j < nb) {
        const int sl = __shfl_sync(0xffffffffu, my_slot, j);
        const float4* po = reinterpret_cast<const float4*>(p.part_o + (size_t)sl * 8 * kD);
        v0[j] = __ldcg(po + h0 * (kD / 4) + lane);
        if (has1) v1[j] = __ldcg(po + h1 * (kD / 4) + lane);
      }
    }
    float b0 = l0, b1 = l1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {       // lanes beyond the batch hold -inf
      b0 = fmaxf(b0, __shfl_xor_sync(0xffffffffu, b0, o));
      b1 = fmaxf(b1, __shfl_xor_sync(0xffffffffu, b1, o));
    }
    const float n0 = fmaxf(M0, b0), n1 = fmaxf(M1, b1);
    const float s0 = (M0 == -INFINITY) ? 0.f : fast_exp2(M0 - n0);
    const float s1 = (M1 == -INFINITY) ? 0.f : fast_exp2(M1 - n1);
    const float w0 = (l0 == -INFINITY) ? 0.f : fast_exp2(l0 - n0);
    const float w1 = (l1 == -INFINITY) ? 0.f : fast_exp2(l1 - n1);
    M0 = n0;
    M1 = n1;
    L0 = L0 * s0 + w0;
    L1 = L1 * s1 + w1;
    a0.x *= s0; a0.y *= s0; a0.z *= s0; a0.w *= s0;
    a1.x *= s1; a1.y *= s1; a1.z *= s1; a1.w *= s1;
#pragma unroll
    for (int j = 0; j < kFoldBatch; ++j) {
      if (j < nb) {
        const float x0 = __shfl_sync(0xffffffffu, w0, j);
        const float x1 = __shfl_sync(0xffffffffu, w1, j);
        a0.x += x0 * v0[j].x;
        a0.y += x0 * v0[j].y;
        a0.z += x0 * v0[j].z;
        a0.w += x0 * v0[j].w;
        if (has1) {
          a1.x += x1 * v1[j].x;
          a1.y += x1 * v1[j].y;
          a1.z += x1 * v1[j].z;
          a1.w += x1 * v1[j].w;
        }
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    L0 += __shfl_xor_sync(0xffffffffu, L0, o);
    L1 += __shfl_xor_sync(0xffffffffu, L1, o);
  }
  auto store_head = [&](int hg, float M, float L, const float4& a) {
    const float inv = L > 0.f ? 1.f / L : 0.f;
    const int h = st_kvh * group + hg;
    uint2 packed;
    packed.x = pack_bf16(a.x * inv, a.y * inv);
    packed.y = pack_bf16(a.z * inv, a.w * inv);
    *reinterpret_cast<uint2*>(p.o + ((int64_t)st_b * p.Hq + h) * kD + lane * 4) = packed;
    if (lane == 0) {
      const float lse2 = L > 0.f ? M + log2f(L) : -INFINITY;
      p.lse[(int64_t)st_b * p.Hq + h] = p.lse_base2 ? lse2 : lse2 * kLn2;
    }
  };
  store_head(h0, M0, L0, a0);
  if (has1) store_head(h1, M1, L1, a1);
}

// kTrace: the instance that records time stamps (the stamps cost registers the streaming loop needs)
template <bool kTrace>
__global__ void __launch_bounds__(kThreads, 2) gqa_decode_kernel(const __grid_constant__ GqaDecodeParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t full_bar[kWarps][kStages];
  __shared__ float s_m[kWarps][8], s_l[kWarps][8];
  __shared__ int s_flag;                         // CTA-wide broadcast word (last arrival, scan result, list length)
  __shared__ int s_draw[2];                      // chunk drawn ahead by thread 0 (two slots, used alternately)
  __shared__ int s_scan;                         // chunk drawn while probing the other pools
  __shared__ int s_nb[kGqaSeqTable];             // KV blocks of each sequence
  __shared__ unsigned short s_nc[kGqaSeqTable];  // chunks a pair of the sequence would give to its pool ...
  __shared__ unsigned short s_ncf[kGqaSeqTable]; // ... and what it does give, after the rules below
  __shared__ int s_hb[kGqaSeqTable];             // first helper slot of the sequence's pools

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
  }
  const bool early_kv = p.kv_stable != 0;
  if (!early_kv) asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const unsigned long long t_entry = now_ns();
  const unsigned long long deadline = t_entry + p.timeout_ns;
  unsigned long long t_first = 0, t_static = 0, t_dyn = 0;
  unsigned n_drawn = 0, n_visits = 0;

  // ---- per-sequence tables and totals ------------------------------------------------------------
  const int cd = p.dyn_chunk;
  const bool dyn_cfg = p.dyn_pct > 0 && cd > 0 && p.B <= kGqaSeqTable && p.max_helper > 0;
  bool dyn_on = false;                           // some pair of this launch really has a pool
  const int n_tab = min(p.B, kGqaSeqTable);
  for (int i = tid; i < n_tab; i += kThreads) {
    // (the divisions are done here, one sequence per thread, not in the serial pass below)
    const int nb = blocks_of(p.seq_lens[i]);
    s_nb[i] = nb;
    s_nc[i] = (unsigned short)min(dyn_cfg ? dyn_chunks_of(nb, p.dyn_pct, cd, p.dyn_min_blocks) : 0, 65535);
  }
  __syncthreads();
  long long total_s = 0;                         // blocks in the fixed shares
  {
    long long total = 0;
    for (int b = 0; b < n_tab; ++b) total += s_nb[b];
    for (int b = kGqaSeqTable; b < p.B; ++b) total += blocks_of(p.seq_lens[b]);
    // A pair only gets a pool if what stays in the fixed shares is longer than two shares.  A CTA's share then
    // never holds such a pair from its first block to its last fixed block, so the share's two piece slots
    // (one for a pair it continues, one for a pair it starts) still suffice; some share ends inside the pair, so
    // a CTA is there to take up the pool; and pairs of about a share's length, where nearly every chunk would end
    // up as a parked piece of its own, keep their fixed shares only (measured slower with pools).
    const long long share_max = 2 * ((total * Hkv + G - 1) / G);
    int hb = 0;
    for (int b = 0; b < n_tab; ++b) {
      const int nb = s_nb[b];
      int nc = s_nc[b];
      if (nb - nc * cd <= share_max) nc = 0;
      if (hb + nc * Hkv > p.max_helper || nc > kMaxPoolChunks) nc = 0;    // never more chunks than helper slots
      if (tid == 0) {
        s_ncf[b] = (unsigned short)nc;
        s_hb[b] = hb;
      }
      hb += nc * Hkv;
      total_s += nb - nc * cd;
    }
    for (int b = kGqaSeqTable; b < p.B; ++b) total_s += blocks_of(p.seq_lens[b]);
    total_s *= Hkv;
    dyn_on = hb > 0;
  }
  __syncthreads();
  auto seq_nb = [&](int b) { return b < kGqaSeqTable ? s_nb[b] : blocks_of(p.seq_lens[b]); };
  auto seq_nc = [&](int b) { return (dyn_on && b < kGqaSeqTable) ? (int)s_ncf[b] : 0; };
  auto seq_ns = [&](int b) { return seq_nb(b) - seq_nc(b) * cd; };

  const long long share = max((total_s + G - 1) / (long long)G, 1LL);
  const long long g0 = (long long)blockIdx.x * share;
  const long long g1 = min(total_s, g0 + share);

  int* const done_ctr = p.counters;                      // [P]
  int* const pool_ctr = p.counters + (size_t)p.B * Hkv;   // [P]
  int* const exit_ctr = p.counters + (size_t)2 * p.B * Hkv;
  int* const helper_flag = exit_ctr + 8;                 // [max_helper]
  const int P = p.B * Hkv;

  uint8_t* my_smem = smem + warp * (kStages * kStageBytes);
  const float sl2 = p.scale * kLog2e;
  const int mi = lane >> 3, r8 = lane & 7;
  const uint32_t k_row = (uint32_t)(((mi >> 1) << 3) + r8), k_csel = (uint32_t)(mi & 1);
  const uint32_t v_row = (uint32_t)(((mi & 1) << 3) + r8), v_csel = (uint32_t)(mi >> 1);
  int it_ring = 0;           // TMA iterations issued so far by this warp: fixes stage and parity
  bool ok = true;

  // ---- segments: a run of blocks of one pair that this CTA streams in one go -----------------------
  struct Seg {
    int b, kvh, kb_begin, kb_end, n_blocks, seq_len;
    int slot;                // piece slot, should this segment open a new running state
    bool valid;
  };
  int cur_b = 0;
  long long base = 0;        // share-space index of block 0 of (cur_b, kvh = 0)
  while (cur_b < p.B) {
    const long long span = (long long)seq_ns(cur_b) * Hkv;
    if (g0 < base + span) break;
    base += span;
    ++cur_b;
  }
  long long gcur = g0;
  auto next_static = [&]() {
    Seg sg;
    sg.valid = false;
    while (gcur < g1 && cur_b < p.B) {
      const int ns = seq_ns(cur_b);
      if (ns == 0) {
        ++cur_b;
        continue;
      }
      sg.b = cur_b;
      sg.seq_len = p.seq_lens[cur_b];
      sg.n_blocks = seq_nb(cur_b);
      sg.kvh = (int)((gcur - base) / ns);
      sg.kb_begin = (int)((gcur - base) - (long long)sg.kvh * ns);
      sg.kb_end = (int)min((long long)ns, (long long)sg.kb_begin + (g1 - gcur));
      sg.slot = blockIdx.x * 2 + (sg.kb_begin == 0 ? 1 : 0);   // slot 1: the piece that starts its pair
      sg.valid = true;
      gcur += (sg.kb_end - sg.kb_begin);
      if (sg.kvh == Hkv - 1 && sg.kb_end == ns) {   // the next segment starts the next sequence
        base += (long long)ns * Hkv;
        ++cur_b;
      }
      break;
    }
    return sg;
  };
  auto chunk_seg = [&](int b, int kvh, int c) {
    Seg sg;
    const int nc = seq_nc(b);
    sg.b = b;
    sg.kvh = kvh;
    sg.n_blocks = seq_nb(b);
    sg.seq_len = p.seq_lens[b];
    sg.kb_begin = sg.n_blocks - (nc - c) * cd;
    sg.kb_end = sg.kb_begin + cd;
    sg.slot = 2 * G + s_hb[b] + kvh * nc + c;
    sg.valid = true;
    return sg;
  };
  // Find a pool that still has chunks, starting at pair `start`, and draw one.  Uniform over the CTA.
  // one thread's look at pool start + off + tid; a stale answer is fine, a pool never refills
  auto probe = [&](int start, int off) {
    bool avail = false;
    if (off + tid < P) {
      const int q = (int)(((long long)start + off + tid) % P);
      const int nc = seq_nc(q / Hkv);
      if (nc > 0) avail = ld_relaxed(pool_ctr + q) < nc;
    }
    return avail;
  };
  // `pre`: the first window's look, taken earlier so that its round trip is over by now
  auto scan_pools = [&](int start, bool have_pre, bool pre) {
    Seg sg;
    sg.valid = false;
    int off = 0;
    while (off < P) {
      const bool avail = (have_pre && off == 0) ? pre : probe(start, off);
      have_pre = false;
      if (tid == 0) s_flag = INT_MAX;
      __syncthreads();
      if (avail) atomicMin(&s_flag, off + tid);
      __syncthreads();
      const int f = s_flag;
      if (f == INT_MAX) {
        off += kThreads;
        __syncthreads();
        continue;
      }
      const int q = (int)(((long long)start + f) % P);
      if (tid == 0) s_scan = atomicAdd(pool_ctr + q, 1);
      __syncthreads();
      const int c = s_scan;
      __syncthreads();
      if (c < seq_nc(q / Hkv)) {
        if (kTrace) ++n_visits;
        if (kTrace) ++n_drawn;
        return chunk_seg(q / Hkv, q % Hkv, c);
      }
      // somebody else took the pool's last chunk in between: it shows as empty on the next probe
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
  int* s_list = reinterpret_cast<int*>(smem + kSmemPipe);    // the same bytes list a fold's pieces

  Seg cur = next_static();
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
  bool in_static = cur.valid;
  if (!cur.valid && dyn_on) {          // no fixed share (more CTAs than blocks): go straight to the pools
    cur = scan_pools(blockIdx.x % max(P, 1), false, false);
    if (cur.valid) prologue(cur);
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
    const int kb_begin = cur.kb_begin, kb_end = cur.kb_end;
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
    // What follows this segment?  More of the fixed share, or (when that is done) a chunk of this pair's
    // pool, drawn now so that the atomic's round trip hides behind the streaming below.
    const bool static_more = in_static && gcur < g1;
    const int my_nc = seq_nc(b);
    const bool drew = !static_more && dyn_on && my_nc > 0;
    dpar ^= 1;
    if (drew && tid == 0) s_draw[dpar] = atomicAdd(pool_ctr + (b * Hkv + kvh), 1);
    // ... and a look at the other pools, in case this one turns out to be empty
    const bool look = !static_more && dyn_on;
    const bool pre = look ? probe(b * Hkv + kvh + 1, 0) : false;

    const int32_t* bt = p.block_table + (int64_t)b * p.bt_stride;
    // page ids are looked up one iteration ahead of the TMA that needs them, so the (dependent)
    // block-table load never stalls the warp in front of a copy
    auto page_of = [&](int kb) { return bt[(kb * kBlockTok) / p.page_size]; };
    const int my_first = kb_begin + warp;
    const int my_count = my_first < kb_end ? (kb_end - my_first + kWarps - 1) / kWarps : 0;
    int next_page = kStages < my_count ? page_of(my_first + kStages * kWarps) : 0;

    for (int it = 0; it < my_count; ++it) {
      const int ring = it_ring + it;
      const int stage = ring % kStages;
      const int kb = my_first + it * kWarps;
      if (!mbar_wait(&full_bar[warp][stage], (uint32_t)((ring / kStages) & 1), deadline)) {
        ok = false;
        break;
      }
      if (kTrace && t_first == 0) t_first = now_ns();
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
      // this stage is free again: fetch the block kStages iterations ahead
      __syncwarp();
      if (lane == 0 && it + kStages < my_count) issue(cur, ring + kStages, kb + kStages * kWarps, next_page);
      if (it + 1 + kStages < my_count) next_page = page_of(kb + (kStages + 1) * kWarps);
    }
    it_ring += my_count;
    st_blocks += kb_end - kb_begin;
    // The vote makes a timeout of one warp a decision of the whole CTA, so no warp is ever left
    // alone at a barrier; it also orders the next merge after the reads of the previous one and
    // publishes thread 0's drawn chunk.
    if (!__syncthreads_and(ok ? 1 : 0)) {
      ok = false;
      break;
    }
    if (kTrace) {
      if (in_static) t_static = now_ns();
      else t_dyn = now_ns();
    }
    // ---- pick the next segment and start streaming it before the epilogue of this one ---------------
    Seg nxt;
    nxt.valid = false;
    if (static_more) nxt = next_static();
    if (!nxt.valid) {
      in_static = false;
      if (dyn_on) {
        const int c = drew ? s_draw[dpar] : INT_MAX;
        if (c < my_nc) {
          nxt = chunk_seg(b, kvh, c);
          if (kTrace) ++n_drawn;
        } else {
          nxt = scan_pools(b * Hkv + kvh + 1, look, pre);
        }
      }
    }
    if (nxt.valid) prologue(nxt);

    if (!nxt.valid || nxt.b != st_b || nxt.kvh != st_kvh) {
      // ---- leave the pair: merge the warps' partials, four heads per round --------------------------
      const bool whole = (st_blocks == st_nb);
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
          if (st_slot >= 2 * G) helper_flag[st_slot - 2 * G] = 1;
          const int prev = atom_add_acq_rel(done_ctr + pair, st_blocks);
          s_flag = (prev + st_blocks == st_nb);
        }
        __syncthreads();
        const bool completes = s_flag != 0;
        if (completes) {
          // ---- this piece completed the pair: fold all of its pieces ---------------------------------
          __syncthreads();                    // everybody has read the verdict before s_flag is reused
          // pieces from the fixed shares: one per CTA whose share overlaps the pair's static blocks
          const int nc = seq_nc(st_b), ns = st_nb - nc * cd;
          long long sp0 = 0;
          for (int bb = 0; bb < st_b; ++bb) sp0 += seq_ns(bb);
          sp0 = sp0 * Hkv + (long long)st_kvh * ns;
          const int i0 = (int)(sp0 / share), i1 = (int)((sp0 + ns - 1) / share);
          const int n_fixed = i1 - i0 + 1;
          for (int i = tid; i < n_fixed; i += kThreads) s_list[i] = (i0 + i) * 2 + (i == 0 ? 1 : 0);
          if (tid == 0) s_flag = n_fixed;
          __syncthreads();
          // pieces parked by CTAs that helped out of this pair's pool
          const int hb = nc > 0 ? s_hb[st_b] + st_kvh * nc : 0;
          for (int c = tid; c < nc; c += kThreads) {
            if (ld_relaxed(helper_flag + hb + c) != 0) {
              const int k = atomicAdd(&s_flag, 1);
              if (k < kMaxList) s_list[k] = 2 * G + hb + c;
              helper_flag[hb + c] = 0;                     // ready for the next launch
            }
          }
          __syncthreads();
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
    // the last CTA to leave re-arms the pools for the next launch: nobody draws or probes any more (every warp
    // of this CTA is past the loop above; only this warp waits for the atomic)
    int last = 0;
    if (lane == 0) last = (atom_add_acq_rel(exit_ctr, 1) == G - 1);
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      for (int i = lane; i < P; i += 32) pool_ctr[i] = 0;
      if (lane == 0) *exit_ctr = 0;
    }
  }

  if (kTrace && p.trace != nullptr && tid == 0) {
    unsigned smid;
    asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
    unsigned long long* tr = p.trace + (size_t)blockIdx.x * 8;
    tr[0] = t_entry;
    tr[1] = t_first;
    tr[2] = t_static;
    tr[3] = now_ns();
    tr[4] = t_dyn;
    tr[5] = (unsigned long long)n_drawn | ((unsigned long long)n_visits << 32);
    tr[6] = smid;
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

// Number of CTAs for a launch: two per SM, but never so many that a CTA streams fewer than
// 32 blocks (its fixed ramp + merge cost is worth about that much streaming).
int gqa_pick_ctas(int B, int Hkv, int max_seq_len, int sm_count) {
  const long long blocks = (long long)std::max(B, 1) * Hkv * std::max((max_seq_len + kBlockTok - 1) / kBlockTok, 1);
  long long ctas = std::min<long long>(2LL * sm_count, std::max<long long>(blocks / 32, 1));
  return (int)std::min<long long>(ctas, kGqaMaxCtas);
}

void gqa_plan_dynamic(GqaDecodeParams* p, int max_seq_len, int max_helper, int pct_override, int chunk_override) {
  const int nb = std::max(blocks_of(std::max(max_seq_len, 1)), 1);
  const long long blocks = (long long)std::max(p->B, 1) * p->Hkv * nb;
  p->max_helper = std::min(std::max(max_helper, 0), kGqaMaxHelper);
  p->dyn_min_blocks = 64;
  // a dynamic tail only pays when a CTA's fixed share is long compared with a chunk
  int pct = (blocks / std::max(p->ctas, 1) >= 96 && p->B <= kGqaSeqTable) ? 30 : 0;
  if (pct_override >= 0) pct = std::min(pct_override, 50);
  int chunk = chunk_override > 0 ? chunk_override : 20;   // a chunk has a fixed cost (its first loads only start once it is drawn): 16-24 blocks measured best
  if (pct > 0 && p->max_helper > 0) {
    // never more chunks than helper slots, whatever the sequence lengths turn out to be
    const long long worst = (long long)p->B * p->Hkv * ((long long)nb * pct / 100);
    while ((worst + chunk - 1) / chunk > p->max_helper) chunk += 4;
  } else {
    pct = 0;
  }
  p->dyn_pct = pct;
  p->dyn_chunk = chunk;
}

cudaError_t launch_gqa_decode(const GqaDecodeParams& p, bool pdl, cudaStream_t stream) {
  if (p.B <= 0) return cudaSuccess;
  if (p.Hq % p.Hkv != 0 || p.Hq / p.Hkv > 8 || p.page_size % kBlockTok != 0 || p.ctas < 1 || p.ctas > kGqaMaxCtas ||
      p.max_helper < 0 || p.max_helper > kGqaMaxHelper || p.dyn_pct < 0 || p.dyn_pct > 50)
    return cudaErrorInvalidValue;
  static bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 64 || !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(gqa_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(gqa_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
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
  return p.trace != nullptr ? cudaLaunchKernelEx(&cfg, gqa_decode_kernel<true>, p)
                            : cudaLaunchKernelEx(&cfg, gqa_decode_kernel<false>, p);
}

}  // namespace helix
