// Helix exchange + LSE combine + o_proj in ONE kernel (sm_100a).
// In the reference these are three steps on three code paths: its all-to-all kernel (csrc/helix_alltoall.cu:194-474),
// its Triton combine (patches/dcp_alltoall_helix.py:210-384) behind the hook's layout copies (:511-600), and vLLM's
// cuBLAS o_proj.
//
// With a few rows per call the combined activation never exists in global memory and no CTA waits for another
// CTA of its own GPU; with many rows the slabs of a head group share the receive work (last paragraph):
//   * CTAs [0, S) only SEND: their warps read this rank's attention output in place, frame LL128 lines in
//     registers and post them into the peers' rings over NVLink (plain stores), then leave.
//   * Every other CTA is a GEMM CTA that owns one 128-row slab of W_o and one group of heads (a K-slice of
//     at most 512: `heads_per_split` heads of D dims).  It first requests its whole W slice (<= 128 KB, one
//     bulk copy per 64-wide atom when the weights are pre-packed): the weights do not depend on anything, so
//     they stream while the other GPUs are still computing.  Then its sixteen warps RECEIVE for themselves:
//     for every (token, head of the group) a warp requests this rank's own row and the lines of the N - 1 peers
//     in the local rings together (read-only: any number of CTAs may read the same lines; only sources whose
//     flags are not all there yet are read again), folds them into the
//     online LSE-weighted accumulator in registers and stores the normalised bf16 row straight into shared
//     memory in the swizzled K-major layout the tensor core reads - the B operand of the UMMA.  One
//     fence.proxy.async and a CTA barrier later a single thread issues the UMMAs (D[128, tokens] in TMEM);
//     four warps run the epilogue, and the split-K fold over the head groups is that of the stand-alone GEMM
//     for up to 16 tokens (the slab's last CTA sums the partials).
//   * The rings have many readers now, so nobody acknowledges lines while reading: every GEMM CTA counts
//     itself out when it has read its last line, and the one that counts last publishes the consumed line
//     counts of all rings of the call (locally, and by remote 8-byte stores to the senders).  A call uses a
//     small fraction of a ring, so senders never wait for that.
// Senders depend on ring space only (granted by an EARLIER call), receivers on other GPUs' senders only.
//   * Many rows (more than kFusedShareAbove per GEMM CTA): receiving every row in every slab's CTA would repeat the
//     poll + combine hidden / 128 times, so the slabs of a head group split the group's rows between them, store
//     their combined rows in a global buffer (it stays in L2), count them, wait for the group's count and copy
//     the complete group into their operand buffer with plain 16-byte loads.  The split-K fold is shared the same
//     way (every CTA of a slab sums a share of the tokens once all partials are counted).  These waits are among
//     CTAs of one launch: the launcher only accepts grids that are resident at once.
// Every wait is bounded (%globaltimer); on expiry the status block / error flag is set and the kernel
// returns.  No TMA load uses cluster broadcast; peer memory is only ever written, never read.
#include "fused.h"

#include <algorithm>

#include "exchange_device.cuh"
#include "oproj_device.cuh"

namespace helix {
namespace {

using namespace dev;
using namespace sm100;

constexpr int kReadersDoneOff = 64;   // byte offset inside the status block of the local row
constexpr int kGemmThreads = 128;     // warps 0..3: weight requests, UMMA issue, epilogue
constexpr int kRecvThreads = 512;     // all sixteen warps of a GEMM CTA receive and combine
constexpr int kGemmBarrier = 2;       // named barrier of the 128 GEMM threads
constexpr int kRecvBarrier = 3;       // named barrier of all 512 threads of a GEMM CTA
constexpr int kMaxSources = 8;        // this rank + at most 7 peers per entry (cp <= 8)
constexpr int kMaxAtoms = 8;          // K-slice of a GEMM CTA: at most 8 atoms of 64 = 512
constexpr int kMaxRt0 = kMaxCp * 32;  // consumed-line counts cached per CTA: peers x channels

__device__ __forceinline__ void gemm_sync() { named_barrier(kGemmBarrier, kGemmThreads); }
__device__ __forceinline__ void recv_sync() { named_barrier(kRecvBarrier, kRecvThreads); }

template <bool BF16, int NIT>
__global__ void __launch_bounds__(512, 1) helix_exchange_oproj_kernel(const __grid_constant__ FusedParams fp) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  __shared__ Control ctl;
  __shared__ __align__(8) uint64_t w_bar, acc_bar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_last;
  __shared__ unsigned long long s_rt0[kMaxRt0];

  const ExchangeParams& p = fp.ex;
  const int rank = p.rank_base + blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, tid = threadIdx.x;
  const RankIO& io = p.io[blockIdx.y];
  const int N = p.cp_size, C = p.channels;

  // optional timeline: 8 words per CTA (entry, inputs ready, first / last line posted or receive done / accumulator
  // ready, -, exit, role)
  unsigned long long* tr = p.trace ? p.trace + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 : nullptr;
  if (tr && tid == 0) {
    tr[0] = globaltimer_ns();
    for (int i = 1; i < 8; ++i) tr[i] = 0;
  }
  if ((int)blockIdx.x < fp.exchange_ctas) {
    // ------------------------------------------------------------------------------- send role
    init_control(&ctl);
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    Ctx cx = make_ctx(p, &ctl, rank, blockIdx.x);
    cx.deadline = globaltimer_ns() + p.timeout_ns;
    cx.trace = tr;
    if (tr && tid == 0) tr[1] = globaltimer_ns();
    const int NS = fp.send_warps;
    if (warp < NS) sender_warp<NIT>(p, cx, io, warp, NS, lane);
    if (tr) {
      __syncthreads();
      if (tid == 0) {
        tr[6] = globaltimer_ns();
        tr[7] = 1;
      }
    }
    return;
  }

  // --------------------------------------------------------------------------------- GEMM role
  const OprojParams& gp = fp.gemm[blockIdx.y];
  const int gidx = (int)blockIdx.x - fp.exchange_ctas;
  const int m_tile = gidx / gp.splits, split = gidx % gp.splits;
  const int Hg = fp.heads_per_split;                 // heads of this CTA's K-slice
  const int D = p.o_bytes >> 1;
  const int Kc = Hg * D;
  const int atoms = Kc / 64;
  const int n_pad = gp.n_pad;
  const uint32_t atom_a_bytes = 128 * 64 * 2, atom_b_bytes = (uint32_t)n_pad * 64 * 2;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(dyn_smem) + 1023) & ~uintptr_t(1023));
  uint8_t* smem_w = smem;                                   // [atoms][128 x 128 B]
  uint8_t* smem_x = smem + (size_t)atoms * atom_a_bytes;    // [atoms][n_pad x 128 B]
  uint32_t tmem_cols = 32;
  while ((int)tmem_cols < n_pad) tmem_cols <<= 1;

  if (tid == 0) {
    ctl.abort = 0;
    ctl.done = 0;
    mbar_init(&w_bar, 1);
    mbar_init(&acc_bar, 1);
    mbar_fence_init();
    if (gp.w_packed == nullptr) tma_prefetch_desc(&gp.w_map);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_slot, tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  recv_sync();
  tc_fence_after_sync();
  const uint32_t tmem_d = tmem_slot;

  // the whole W slice of this CTA: nothing it depends on, so it is requested before anything else
  if (tid == 0) {
    mbar_expect_tx(&w_bar, (uint32_t)atoms * atom_a_bytes);
    const int atom0 = split * atoms;
    for (int a = 0; a < atoms; ++a) {
      if (gp.w_packed != nullptr)
        bulk_load_1d(smem_w + (size_t)a * atom_a_bytes,
                     gp.w_packed + ((size_t)m_tile * gp.packed_atoms + (size_t)(atom0 + a)) * atom_a_bytes, atom_a_bytes,
                     &w_bar);
      else
        tma_load_2d(smem_w + (size_t)a * atom_a_bytes, &gp.w_map, &w_bar, (atom0 + a) * 64, m_tile * 128);
    }
  }
  pdl_launch_dependents();
  pdl_wait();             // this rank's attention output, and the counts the previous call published
  Ctx cx = make_ctx(p, &ctl, rank, 0);
  cx.deadline = globaltimer_ns() + p.timeout_ns;
  const unsigned long long deadline = cx.deadline;
  if (tr && tid == 0) tr[1] = globaltimer_ns();

  // consumed-line count of every ring of this row at the start of the call
  for (int idx = tid; idx < N * C; idx += kRecvThreads) {
    const int peer = idx / C, c = idx - peer * C;
    s_rt0[idx] = peer != rank ? ld_volatile_8(cx.my_row + rinfo_slot(cx.lay, peer, c) + kRinfoTailOff) : 0ull;
  }
  recv_sync();

  // ---- receive + combine: the rows of this CTA's head group, straight into the B operand ----------------
  const int payload_words = p.st_words + (p.o_bytes >> 3);
  const int L = ll128::lines_for_words(payload_words);
  const int nchunks = L * kChunksPerLine;
  const int Hl = p.inner;
  bool alive = true;
  const int M = gp.hidden / 128;
  const bool share = fp.share_rows != 0;
  const int total_ent = p.outer * Hg;
  // sharing: slab m takes rows m * 16 + warp, + M * 16, ... of the group; otherwise every CTA takes them all
  const int ent_first = share ? m_tile * (kRecvThreads / 32) + warp : warp;
  const int ent_step = (share ? M : 1) * (kRecvThreads / 32);
  for (int ent = ent_first; ent < total_ent && alive; ent += ent_step) {
    const int b = ent / Hg, hg = ent - b * Hg;
    const int hl = split * Hg + hg;
    const int e = b * Hl + hl;
    const int c = e % C, i = e / C;
    cx.channel = c;
    // All sources of the entry at once: this rank's own row and the message of every peer are requested together
    // (one 16-byte chunk per lane and source: a message fits one warp-wide load), so an entry whose lines have
    // landed costs one round trip to L2 however many ranks there are; only sources whose flags are not all there
    // yet are read again.
    uint64_t lo[kMaxSources], hi[kMaxSources];
    {
      uint64_t l1[1], h1[1];
      load_message<1>(p, msg_src(p, io, e, rank), 0, nchunks, payload_words, lane, l1, h1);
      lo[0] = l1[0];
      hi[0] = h1[0];
    }
    unsigned pending = (1u << (N - 1)) - 1u;          // bit j: peer (rank + N - 1 - j) % N still incomplete
    unsigned spins = 0;
    while (pending != 0u) {
#pragma unroll
      for (int j = 0; j < kMaxSources - 1; ++j) {
        if ((pending >> j) & 1u) {
          const int peer = (rank + N - 1 - j) % N;
          const uint64_t q0 = s_rt0[peer * C + c] + (uint64_t)i * L;
          const uint8_t* ring = cx.my_row + ring_offset(cx.lay, peer, c);
          lo[j + 1] = hi[j + 1] = 0ull;
          if (lane < nchunks) ld_volatile_16(ring + ll128::chunk_ring_offset(q0, lane), lo[j + 1], hi[j + 1]);
        }
      }
#pragma unroll
      for (int j = 0; j < kMaxSources - 1; ++j) {
        if ((pending >> j) & 1u) {
          const int peer = (rank + N - 1 - j) % N;
          const uint64_t q0 = s_rt0[peer * C + c] + (uint64_t)i * L;
          const bool bad = lane < nchunks && (lane & 7) == 7 && hi[j + 1] != ll128::flag_of(q0 + (uint64_t)(lane >> 3));
          if (!__any_sync(kFull, bad)) pending &= ~(1u << j);
        }
      }
      if (pending != 0u && (++spins & 31u) == 0u && __any_sync(kFull, give_up(cx))) {
        if (lane == 0) report(cx, kTimeoutRecv, (rank + N - 1 - (__ffs(pending) - 1)) % N, e);
        alive = false;
        break;
      }
    }
    if (!alive) break;
    Acc<1> acc;
    acc.init();
#pragma unroll
    for (int j = 0; j < kMaxSources; ++j) {
      if (j < N) {
        uint64_t l1[1] = {lo[j]}, h1[1] = {hi[j]};
        acc.template add<BF16>(ingest_lse(__shfl_sync(kFull, lo[j], 0), p.stats_mode, p.base2), l1, h1);
      }
    }
    const float inv = acc.s > 0.f ? 1.0f / acc.s : 0.f;
    uint8_t* xg = (fp.x_out[blockIdx.y] != nullptr && (share || m_tile == 0))
                      ? reinterpret_cast<uint8_t*>(fp.x_out[blockIdx.y]) + ((int64_t)b * Hl + hl) * p.o_bytes
                      : nullptr;
    {
      const int it = 0, ch = lane;
      if (ch < nchunks) {
        const ll128::ChunkMap m = ll128::chunk_map(ch);
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] = acc.v[it][k] * inv;
        const int w0 = m.first, w1 = m.first + 1;
        // payload word w of the row = bytes [8 (w - st_words), +8) of the head's D * 2 bytes
        auto put = [&](int w, const float* v) {
          if (w < p.st_words || w >= payload_words) return;
          const uint64_t packed = pack4<BF16>(v);
          const int byte = hg * p.o_bytes + 8 * (w - p.st_words);       // inside the CTA's K-slice of row b
          const int atom = byte >> 7, inb = byte & 127;
          const uint32_t off = (uint32_t)atom * atom_b_bytes + swz128((uint32_t)b, (uint32_t)(inb >> 4)) + (inb & 15);
          if (!share) *reinterpret_cast<uint64_t*>(smem_x + off) = packed;
          if (xg != nullptr) *reinterpret_cast<uint64_t*>(xg + 8 * (w - p.st_words)) = packed;
        };
        put(w0, f);
        if (!m.has_flag) put(w1, f + 4);
      }
    }
  }
  if (share) {
    // hand the rows over: publish this CTA's share, wait for the whole group, copy it from L2 into the operand
    __threadfence();
    recv_sync();
    int* ready = fp.aux[blockIdx.y] + M + split;
    if (tid == 0) {
      int mine = 0;
      for (int e0 = m_tile * (kRecvThreads / 32); e0 < total_ent; e0 += ent_step) mine += min(kRecvThreads / 32, total_ent - e0);
      atomicAdd(ready, mine);     // also after a failed wait: the call is reported as failed, the counters stay balanced
      unsigned spins = 0;
      while (*reinterpret_cast<volatile int*>(ready) < total_ent) {
        if ((++spins & 63u) == 0u && (*reinterpret_cast<volatile int*>(&ctl.abort) || now_ns() > deadline)) {
          atomicCAS(gp.error_flag, 0, (int)kTimeoutMbarrier);
          *reinterpret_cast<volatile int*>(&ctl.abort) = 1;
          break;
        }
      }
      __threadfence();
    }
    recv_sync();
    if (!*reinterpret_cast<volatile int*>(&ctl.abort)) {
      const int cpr = Kc >> 3;                                      // 16-byte chunks per row of the K-slice
      const size_t row_bytes = (size_t)Hl * p.o_bytes;
      const uint8_t* xs = reinterpret_cast<const uint8_t*>(fp.x_out[blockIdx.y]) + (size_t)split * Kc * 2;
      for (int idx = tid; idx < p.outer * cpr; idx += kRecvThreads) {
        const int b = idx / cpr, ch = idx - b * cpr;
        const int4 v = __ldcg(reinterpret_cast<const int4*>(xs + (size_t)b * row_bytes + (size_t)ch * 16));
        *reinterpret_cast<int4*>(smem_x + (uint32_t)(ch >> 3) * atom_b_bytes + swz128((uint32_t)b, (uint32_t)(ch & 7))) = v;
      }
    }
  }
  // rows written by ordinary stores must be visible to the tensor core's (asynchronous-proxy) reads
  fence_proxy_async_smem();
  recv_sync();
  if (tr && tid == 0) tr[2] = globaltimer_ns();
  const bool bad = *reinterpret_cast<volatile int*>(&ctl.abort) != 0;
  if (tid >= kGemmThreads) return;        // the receive-only warps are done

  // this CTA has read its last line: count it out; the last one of the call publishes the consumed counts
  if (share && tid == 0) {
    // this slab has its copy of the group's rows; the last slab re-arms the group's counters for the next call
    int* ready = fp.aux[blockIdx.y] + M + split;
    int* done = ready + kFusedMaxGroups;
    if (atomicAdd(done, 1) == M - 1) {
      *reinterpret_cast<volatile int*>(ready) = 0;
      *reinterpret_cast<volatile int*>(done) = 0;
    }
  }
  if (warp == 0) {
    unsigned int* readers = reinterpret_cast<unsigned int*>(cx.my_row + cx.lay.status_offset + kReadersDoneOff);
    int last = 0;
    if (lane == 0) {
      __threadfence();
      last = (atomicAdd(readers, 1u) == (unsigned)fp.gemm_ctas - 1u);
    }
    last = __shfl_sync(kFull, last, 0);
    if (last) {
      if (!bad) {
        const int E = p.outer * p.inner;
        for (int idx = lane; idx < N * C; idx += 32) {
          const int peer = idx / C, c = idx - peer * C;
          if (peer == rank) continue;
          const uint64_t t_new = s_rt0[idx] + (uint64_t)entries_of_channel(E, C, c) * L;
          st_volatile_8(cx.my_row + rinfo_slot(cx.lay, peer, c) + kRinfoTailOff, t_new);
          st_volatile_8(cx.ws + (int64_t)peer * cx.stride + sinfo_slot(cx.lay, rank, c) + kSinfoTailOff, t_new);
        }
      }
      __syncwarp();
      if (lane == 0) *reinterpret_cast<volatile unsigned int*>(readers) = 0u;    // re-armed for the next call
    }
  }

  // ---- MMA: D[128, n_pad] = W slab (K-slice) x rows^T ---------------------------------------------------
  bool ok = !bad;
  if (warp == 1 && lane == 0 && ok) {
    if (!mbar_wait(&w_bar, 0, deadline)) {
      atomicCAS(gp.error_flag, 0, (int)kTimeoutMbarrier);
      *reinterpret_cast<volatile int*>(&ctl.abort) = 1;
    } else {
      tc_fence_after_sync();
      const uint32_t idesc = umma_idesc_bf16(128, n_pad);
      const uint32_t a_addr = smem_u32(smem_w), b_addr = smem_u32(smem_x);
      for (int a = 0; a < atoms; ++a) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem_d, umma_desc_k_sw128(a_addr + a * atom_a_bytes + k * 32),
                    umma_desc_k_sw128(b_addr + a * atom_b_bytes + k * 32), idesc, (a | k) != 0);
      }
      umma_commit(&acc_bar);
    }
  }
  // ---- epilogue (all four warps): warp w owns TMEM lanes 32w .. 32w + 31 = rows of the W slab ----------------
  __syncwarp();
  if (ok) {
    int good = 1;
    if (lane == 0) {
      unsigned spins = 0;
      while (!mbar_try_wait(&acc_bar, 0)) {
        if ((++spins & 63u) == 0u && (*reinterpret_cast<volatile int*>(&ctl.abort) || now_ns() > deadline)) {
          good = 0;
          break;
        }
      }
    }
    good = __shfl_sync(kFull, good, 0);
    ok = good != 0;
    if (!ok && lane == 0) atomicCAS(gp.error_flag, 0, (int)kTimeoutMbarrier);
  }
  tc_fence_after_sync();
  if (tr && tid == 0) tr[3] = globaltimer_ns();
  const int row = warp * 32 + lane;
  const int hcol = m_tile * 128 + row;
  float* part = gp.splits > 1 ? gp.partial + ((size_t)(m_tile * gp.splits + split) * n_pad) * 128 : nullptr;
  if (ok) {
    for (int c0 = 0; c0 < n_pad; c0 += 16) {
      uint32_t v[16];
      tmem_ld_32x32b_x16(tmem_d + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int tok = c0 + j;
        if (gp.splits == 1) {
          if (tok < gp.tokens) gp.y[(int64_t)tok * gp.y_stride + hcol] = __float2bfloat16(__uint_as_float(v[j]));
        } else {
          part[(size_t)tok * 128 + row] = __uint_as_float(v[j]);
        }
      }
    }
  }
  tc_fence_before_sync();
  gemm_sync();
  if (warp == 1) tmem_dealloc(tmem_d, tmem_cols);
  if (!ok) {
    // the weight copies may still be on their way into this CTA's shared memory: give them a bounded moment.
    // The CTA still takes part in the fold below (the call is reported as failed; the counters stay balanced).
    if (tid == 0) mbar_wait(&w_bar, 0, now_ns() + 2000000ull);
  }
  if (tr && tid == 0) {
    tr[6] = globaltimer_ns();       // without the fold of the K splits, which only the slab's last CTA runs
    tr[7] = 2;
  }
  if (gp.splits == 1) return;

  // ---- the head groups of a slab are K splits ---------------------------------------------------------------
  __threadfence();
  gemm_sync();
  if (n_pad > 16) {
    // many tokens: every CTA of the slab sums a share of the tokens once all partials are there (the CTAs of a
    // launch are resident together, see the launcher)
    if (tid == 0) {
      atomicAdd(&gp.counters[m_tile], 1);
      int good = 1;
      unsigned spins = 0;
      while (*reinterpret_cast<volatile int*>(&gp.counters[m_tile]) < gp.splits) {
        if ((++spins & 63u) == 0u && now_ns() > deadline) {
          atomicCAS(gp.error_flag, 0, (int)kTimeoutMbarrier);
          good = 0;
          break;
        }
      }
      __threadfence();
      s_last = good;
    }
    gemm_sync();
    if (s_last) {
      const int per = (gp.tokens + gp.splits - 1) / gp.splits;
      const int t0 = split * per, t1 = min(gp.tokens, t0 + per);
      const float* base = gp.partial + (size_t)m_tile * gp.splits * n_pad * 128;
      for (int tok0 = t0; tok0 < t1; tok0 += 8) {
        float accs[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) accs[j] = 0.f;
        for (int s = 0; s < gp.splits; ++s) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (tok0 + j < t1) accs[j] += __ldcg(base + ((size_t)s * n_pad + tok0 + j) * 128 + tid);
        }
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (tok0 + j < t1) gp.y[(int64_t)(tok0 + j) * gp.y_stride + m_tile * 128 + tid] = __float2bfloat16(accs[j]);
      }
    }
    gemm_sync();
    if (tid == 0) {
      int* fold_done = fp.aux[blockIdx.y] + m_tile;
      if (atomicAdd(fold_done, 1) == gp.splits - 1) {
        *reinterpret_cast<volatile int*>(&gp.counters[m_tile]) = 0;
        *reinterpret_cast<volatile int*>(fold_done) = 0;
      }
      if (tr) tr[4] = globaltimer_ns();
    }
    return;
  }
  // few tokens: the last CTA of the slab sums them
  if (tid == 0) s_last = (atomicAdd(&gp.counters[m_tile], 1) == gp.splits - 1);
  gemm_sync();
  if (!s_last) return;
  __threadfence();
  const float* base = gp.partial + (size_t)m_tile * gp.splits * n_pad * 128;
  for (int tok0 = 0; tok0 < gp.tokens; tok0 += 8) {
    float accs[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) accs[j] = 0.f;
    for (int s = 0; s < gp.splits; ++s) {
#pragma unroll
      for (int j = 0; j < 8; ++j)   // rows of the partial are padded to n_pad (a multiple of 16): always in bounds
        accs[j] += __ldcg(base + ((size_t)s * n_pad + tok0 + j) * 128 + tid);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (tok0 + j < gp.tokens) gp.y[(int64_t)(tok0 + j) * gp.y_stride + m_tile * 128 + tid] = __float2bfloat16(accs[j]);
  }
  if (tid == 0) gp.counters[m_tile] = 0;
  if (tr && tid == 0) tr[4] = globaltimer_ns();       // fold done
}

using FusedFn = void (*)(FusedParams);

template <int NIT>
FusedFn pick(bool bf16) {
  return bf16 ? (FusedFn)helix_exchange_oproj_kernel<true, NIT> : (FusedFn)helix_exchange_oproj_kernel<false, NIT>;
}

}  // namespace

int fused_pick_splits(int heads_local, int head_dim) {
  // the smallest number of head groups whose K-slice fits a CTA (512), with equal groups
  for (int s = 1; s <= heads_local; ++s)
    if (heads_local % s == 0 && (heads_local / s) * head_dim <= 64 * kMaxAtoms) return s;
  return 0;
}

size_t fused_smem_bytes(int k_slice, int n_pad) { return (size_t)(k_slice / 64) * (128 + n_pad) * 128 + 1024; }

bool fused_fits(int tokens, int heads_local, int head_dim, int hidden, int cp_size, int sm_count) {
  if (tokens < 1 || cp_size < 2 || cp_size > kMaxSources || hidden % 128 != 0 || (head_dim * 2) % 128 != 0) return false;
  const int splits = fused_pick_splits(heads_local, head_dim);
  if (splits < 1 || splits > kFusedMaxGroups) return false;
  const int n_pad = (tokens + 15) / 16 * 16, Kc = heads_local / splits * head_dim;
  if (n_pad > kFusedMaxTokens || Kc % 64 != 0) return false;
  const int L = ll128::lines_for_words(1 + head_dim / 4);
  if (L > 4) return false;                                             // a message is one warp-wide load
  if (fused_smem_bytes(Kc, n_pad) > 227 * 1024) return false;
  const int gemm_ctas = hidden / 128 * splits, E = tokens * heads_local;
  if (sm_count - gemm_ctas < 1) return false;                          // one CTA per SM, all resident at once
  const int channels = std::max(1, std::min({E, sm_count - gemm_ctas, 32}));
  return (int64_t)ceil_div(E, channels) * L <= kRingLines / 2;
}

cudaError_t launch_exchange_oproj(FusedParams fp, int channel_override, bool pdl, cudaStream_t stream,
                                  LaunchInfo* info_out) {
  ExchangeParams& p = fp.ex;
  const int E = p.outer * p.inner;
  if (E <= 0) return cudaSuccess;
  if (p.mode != kModeCombine || p.ranks_in_launch < 1 || p.ranks_in_launch > kFusedMaxRanks) return cudaErrorInvalidValue;
  const OprojParams& g0 = fp.gemm[0];
  const int D = p.o_bytes / 2;
  if (g0.splits < 1 || p.inner % g0.splits != 0 || (D * 2) % 128 != 0) return cudaErrorInvalidValue;
  const int Hg = p.inner / g0.splits, Kc = Hg * D;
  if (Kc > 64 * kMaxAtoms || Kc % 64 != 0 || g0.n_pad > kFusedMaxTokens || g0.n_pad % 16 != 0) return cudaErrorNotSupported;
  for (int r = 0; r < p.ranks_in_launch; ++r)
    if (fp.gemm[r].splits != g0.splits || (g0.splits > 1 && fp.gemm[r].partial == nullptr)) return cudaErrorInvalidValue;
  fp.heads_per_split = Hg;
  fp.share_rows = fused_shares_rows(p.outer, Hg, g0.hidden) ? 1 : 0;
  if (g0.splits > kFusedMaxGroups) return cudaErrorNotSupported;
  for (int r = 0; r < p.ranks_in_launch; ++r) {
    if (fp.aux[r] == nullptr) return cudaErrorInvalidValue;
    if (fp.share_rows && fp.x_out[r] == nullptr) return cudaErrorInvalidValue;
  }

  LaunchInfo li = plan_launch(p, channel_override);
  // a message must fit one warp-wide load (at most 4 lines: heads of up to 232 dims) and an entry has at most 8 sources
  if (li.iters > 1 || p.cp_size > kMaxSources) return cudaErrorNotSupported;
  FusedFn fn = pick<1>(p.is_bf16);

  const int gemm_ctas = g0.hidden / 128 * g0.splits;
  // few sender CTAs share all entries of the call: every warp of a sender CTA sends (as many per peer as fit)
  {
    const int peers = std::max(1, p.cp_size - 1), warps = kRecvThreads / 32;
    li.send_warps = peers * std::max(1, warps / peers);
  }
  const int threads = kRecvThreads;
  const size_t smem = fused_smem_bytes(Kc, g0.n_pad);
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem);
  if (e != cudaSuccess) return e;
  if (per_sm < 1) return cudaErrorNotSupported;
  const int capacity = per_sm * p.sm_count / p.ranks_in_launch;     // CTAs one rank may have resident
  // Sender CTAs first, then every GEMM CTA resident at once: a GEMM CTA that starts late has not prefetched its
  // weights (and in a launch that plays several ranks it would be waited for by the others).
  if (capacity - gemm_ctas < 1) return cudaErrorNotSupported;
  li.channels = std::max(1, std::min({li.channels, capacity - gemm_ctas, 32}));
  if (p.cp_size * li.channels > kMaxRt0) return cudaErrorNotSupported;
  // the consumed counts are only published at the end of the call: a call must fit well inside a ring
  const int L = li.lines_per_message;
  if ((int64_t)ceil_div(E, li.channels) * L > kRingLines / 2) return cudaErrorNotSupported;

  p.channels = li.channels;
  p.recv_warps = 0;
  p.group_warps = 1;
  p.rounds_per_publish = 0;
  fp.exchange_ctas = li.channels;
  fp.gemm_ctas = gemm_ctas;
  fp.send_warps = li.send_warps;

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(li.channels + gemm_ctas, p.ranks_in_launch, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (pdl && p.ranks_in_launch == 1) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (p.ranks_in_launch > 1) {
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (info_out) *info_out = li;
  return cudaLaunchKernelEx(&cfg, fn, fp);
}

}  // namespace helix
