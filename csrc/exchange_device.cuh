// Device side of the Helix exchange: sender and receiver warp loops.
//
// What the reference does in four shared-memory passes per message (bulk copy to smem,
// frame, register copy to the peer; bulk-copy poll, un-frame, bulk copy out —
// csrc/helix_alltoall.cu:360-473) plus a separate Triton combine
// (patches/dcp_alltoall_helix.py:210-320) happens here in registers:
//
//   sender warp (one per remote peer and channel): reads the message's words straight from
//     the attention output in its native strided layout, builds 128-byte lines in registers
//     (8 lanes x 16 B, flag in the last 8 bytes) and posts them into the ring that lives in
//     the PEER's workspace row (plain stores over NVLink; nothing is ever loaded remotely);
//   receiver warp: polls the ring in its OWN row with 16-byte volatile loads and either
//     writes the row out (exchange mode = the reference's alltoall contract) or folds it
//     into an online LSE-weighted accumulator (combine mode) and writes the final
//     [B, H/N, D] row once every peer's contribution has landed.
//
// Flow control is by line counts: head (sender, local), tail (receiver's consumed count,
// stored remotely into the sender's row).  Every wait is bounded by a %globaltimer deadline;
// when it runs out the warp records a status block in the local row and stops polling, but it
// still walks through every barrier so that no other warp is left waiting for it.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "bounds.cuh"
#include "exchange.h"
#include "fifo.cuh"
#include "ll128.cuh"

namespace helix {
namespace dev {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kAllRecvBarrier = 15;  // named barrier shared by every receiver warp
constexpr int kGroupBarrier0 = 1;    // named barriers 1..14: one per receiver group

// ---- tiny PTX wrappers ---------------------------------------------------------------------
HELIX_D unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
HELIX_D void ld_volatile_16(const void* p, uint64_t& lo, uint64_t& hi) {
  asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(lo), "=l"(hi) : "l"(p) : "memory");
}
HELIX_D void st_volatile_16(void* p, uint64_t lo, uint64_t hi) {
  asm volatile("st.volatile.global.v2.u64 [%0], {%1,%2};" ::"l"(p), "l"(lo), "l"(hi) : "memory");
}
HELIX_D uint64_t ld_volatile_8(const void* p) {
  uint64_t v;
  asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
HELIX_D void st_volatile_8(void* p, uint64_t v) {
  asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
HELIX_D uint64_t ld_8(const void* p) { return *reinterpret_cast<const uint64_t*>(p); }
HELIX_D void st_8(void* p, uint64_t v) { *reinterpret_cast<uint64_t*>(p) = v; }
HELIX_D void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
HELIX_D void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
HELIX_D void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- per-CTA control block (shared memory) and per-warp context -------------------------------
struct Control {
  int abort;
  unsigned done;
  // Sender warps that are done with the ring to a peer (several warps may share one ring: each reads the ring's
  // line count when it starts, and the new count is only stored once all of them have counted themselves in here).
  unsigned sent[kMaxCp];
};

// every thread of the CTA calls this before the first CTA barrier of the kernel
HELIX_D void init_control(Control* ctl) {
  if (threadIdx.x == 0) {
    ctl->abort = 0;
    ctl->done = 0;
  }
  if (threadIdx.x < kMaxCp) ctl->sent[threadIdx.x] = 0u;
}

struct Ctx {
  unsigned long long* trace;   // this CTA's eight time stamps, or null
  uint8_t* ws;
  int64_t stride;
  uint8_t* my_row;
  WorkspaceLayout lay;
  unsigned long long deadline;
  Control* ctl;
  int rank, channel;
};

HELIX_D bool aborted(const Ctx& cx) { return *reinterpret_cast<volatile int*>(&cx.ctl->abort) != 0; }

HELIX_D void report(const Ctx& cx, int code, int peer, int entry) {
  StatusBlock* sb = reinterpret_cast<StatusBlock*>(cx.my_row + cx.lay.status_offset);
  if (atomicCAS(&sb->code, 0ull, (unsigned long long)code) == 0ull) {
    sb->peer = (unsigned long long)peer;
    sb->channel = (unsigned long long)cx.channel;
    sb->entry = (unsigned long long)entry;
  }
  *reinterpret_cast<volatile int*>(&cx.ctl->abort) = 1;
}

// true when a wait should give up: deadline passed, or somebody on this rank already failed
HELIX_D bool give_up(const Ctx& cx) {
  if (aborted(cx)) return true;
  const StatusBlock* sb = reinterpret_cast<const StatusBlock*>(cx.my_row + cx.lay.status_offset);
  if (ld_volatile_8(&sb->code) != 0ull) {
    *reinterpret_cast<volatile int*>(&cx.ctl->abort) = 1;
    return true;
  }
  return globaltimer_ns() > cx.deadline;
}

// ---- message source addressing ---------------------------------------------------------------
struct MsgSrc {
  const uint8_t* o;    // D * es bytes
  const uint8_t* st;   // stats words, or one float when lse_scalar
};

HELIX_D MsgSrc msg_src(const ExchangeParams& p, const RankIO& io, int e, int peer) {
  MsgSrc s;
  s.o = io.o_src + bounds::src_o_off(p, e, peer);
  s.st = io.st_src + bounds::src_st_off(p, e, peer);
  return s;
}

// Debug mode: may message (e, peer) be read / may its row be written?  A span that does not fit the caller's
// tensor is reported once (kBadArgument) and the caller skips the access.
HELIX_D bool check_source(const ExchangeParams& p, const Ctx& cx, int e, int peer, int lane) {
  if (!p.debug_checks || bounds::source_ok(p, e, peer)) return true;
  if (lane == 0) report(cx, kBadArgument, peer, e);
  return false;
}
HELIX_D bool check_dest(const ExchangeParams& p, const Ctx& cx, const RankIO& io, int e, int peer, int lane) {
  if (!p.debug_checks || bounds::dest_ok(p, e, peer, io.st_dst != nullptr)) return true;
  if (lane == 0) report(cx, kBadArgument, peer, e);
  return false;
}

// payload word w of a message, read from the user's tensors
HELIX_D uint64_t load_payload_word(const ExchangeParams& p, const MsgSrc& s, int w, int payload_words) {
  if (w < p.st_words) {
    if (p.lse_scalar) return (uint64_t)__float_as_uint(*reinterpret_cast<const float*>(s.st));
    return ld_8(s.st + 8 * w);
  }
  if (w < payload_words) return ld_8(s.o + 8 * (w - p.st_words));
  return 0ull;
}

template <int NIT>
HELIX_D void load_message(const ExchangeParams& p, const MsgSrc& s, int chunk0, int nchunks, int payload_words,
                          int lane, uint64_t (&lo)[NIT], uint64_t (&hi)[NIT]) {
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    int ch = chunk0 + it * 32 + lane;
    lo[it] = 0ull;
    hi[it] = 0ull;
    if (ch < nchunks) {
      ll128::ChunkMap m = ll128::chunk_map(ch);
      lo[it] = load_payload_word(p, s, m.first, payload_words);
      if (!m.has_flag) hi[it] = load_payload_word(p, s, m.first + 1, payload_words);
    }
  }
}

// ---- element helpers ---------------------------------------------------------------------------
template <bool BF16>
HELIX_D void unpack4(uint64_t w, float (&f)[4]) {
  uint32_t a = (uint32_t)w, b = (uint32_t)(w >> 32);
  if (BF16) {
    f[0] = __uint_as_float(a << 16);
    f[1] = __uint_as_float(a & 0xffff0000u);
    f[2] = __uint_as_float(b << 16);
    f[3] = __uint_as_float(b & 0xffff0000u);
  } else {
    __half2 h0 = *reinterpret_cast<__half2*>(&a);
    __half2 h1 = *reinterpret_cast<__half2*>(&b);
    float2 x = __half22float2(h0), y = __half22float2(h1);
    f[0] = x.x; f[1] = x.y; f[2] = y.x; f[3] = y.y;
  }
}
template <bool BF16>
HELIX_D uint64_t pack4(const float* f) {
  uint32_t a, b;
  if (BF16) {
    __nv_bfloat162 x = __floats2bfloat162_rn(f[0], f[1]);
    __nv_bfloat162 y = __floats2bfloat162_rn(f[2], f[3]);
    a = *reinterpret_cast<uint32_t*>(&x);
    b = *reinterpret_cast<uint32_t*>(&y);
  } else {
    __half2 x = __floats2half2_rn(f[0], f[1]);
    __half2 y = __floats2half2_rn(f[2], f[3]);
    a = *reinterpret_cast<uint32_t*>(&x);
    b = *reinterpret_cast<uint32_t*>(&y);
  }
  return (uint64_t)a | ((uint64_t)b << 32);
}

// LSE of one contribution in the base-2 domain; NaN and +-inf become -inf (the rule of the
// reference's combine, patches/dcp_alltoall_helix.py:174-178,253-257).
HELIX_D float ingest_lse(uint64_t stats_word, int stats_mode, int base2) {
  float s0 = __uint_as_float((uint32_t)stats_word);
  float s1 = __uint_as_float((uint32_t)(stats_word >> 32));
  float l = base2 ? s0 : s0 * kLog2e;
  if (stats_mode == kStatsMaxSumExp) l += log2f(s1);
  if (!(fabsf(l) <= 3.0e38f)) l = -INFINITY;
  return l;
}

// Online LSE-weighted accumulator held by one lane for its chunks of the row.
template <int NIT>
struct Acc {
  float m, s;
  float v[NIT][8];
  HELIX_D void init() {
    m = -INFINITY;
    s = 0.f;
#pragma unroll
    for (int i = 0; i < NIT; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[i][j] = 0.f;
  }
  template <bool BF16>
  HELIX_D void add(float l, const uint64_t (&lo)[NIT], const uint64_t (&hi)[NIT]) {
    if (l == -INFINITY) return;  // warp-uniform
    float mn = fmaxf(m, l);
    float sc = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    float w = exp2f(l - mn);
    s = s * sc + w;
    m = mn;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      float a[4], b[4];
      unpack4<BF16>(lo[it], a);
      unpack4<BF16>(hi[it], b);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        v[it][j] = v[it][j] * sc + w * a[j];
        v[it][4 + j] = v[it][4 + j] * sc + w * b[j];
      }
    }
  }
  // merge a partial accumulator of another warp (same lane mapping), read from shared memory
  HELIX_D void merge(float om, float os, const float* ov, int lane) {
    if (os == 0.f) return;  // warp-uniform
    float mn = fmaxf(m, om);
    float sa = (m == -INFINITY) ? 0.f : exp2f(m - mn);
    float sb = exp2f(om - mn);
    s = s * sa + os * sb;
    m = mn;
#pragma unroll
    for (int it = 0; it < NIT; ++it)
#pragma unroll
      for (int j = 0; j < 8; ++j) v[it][j] = v[it][j] * sa + ov[(it * 8 + j) * 32 + lane] * sb;
  }
};

// floats one warp parks in shared memory when several warps share an entry
template <int NIT>
HELIX_HD int group_slot_floats() { return NIT * 8 * 32 + 4; }

// Poll one message (or one slab of it) until every line carries its flag.  Returns false on
// timeout / abort.  chunk0 is a multiple of 32, so line boundaries align with 8-lane groups.
template <int NIT>
HELIX_D bool poll_message(const Ctx& cx, const uint8_t* ring, uint64_t q0, int chunk0, int nchunks, int lane,
                          uint64_t (&lo)[NIT], uint64_t (&hi)[NIT]) {
  unsigned spins = 0;
#pragma unroll
  for (int it = 0; it < NIT; ++it) lo[it] = hi[it] = 0ull;
  while (true) {
    bool bad = false;
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      int ch = chunk0 + it * 32 + lane;
      if (ch < nchunks) ld_volatile_16(ring + ll128::chunk_ring_offset(q0, ch), lo[it], hi[it]);
    }
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      int ch = chunk0 + it * 32 + lane;
      if (ch < nchunks && (ch & 7) == 7) bad |= (hi[it] != ll128::flag_of(q0 + (uint64_t)(ch >> 3)));
    }
    if (!__any_sync(kFull, bad)) return true;
    if ((++spins & 31u) == 0u) {
      if (__any_sync(kFull, give_up(cx))) return false;
    }
  }
}

// ================================================================================================
// sender: messages of channel c to the peers this warp serves.  With few peers several warps share
// a peer (warp k of K sends messages k, k + K, ...: ring positions are fixed by the message index,
// so they need no coordination); with many peers one warp walks several.  The words of the next
// message are loaded before the current one is stored, so the source latency overlaps the stores.
template <int NIT>
HELIX_D void sender_warp(const ExchangeParams& p, const Ctx& cx, const RankIO& io, int send_warp, int n_send_warps,
                         int lane) {
  const int N = p.cp_size, C = p.channels, c = cx.channel, rank = cx.rank;
  const int E = p.outer * p.inner;
  const int n_mine = entries_of_channel(E, C, c);
  const int payload_words = p.st_words + (p.o_bytes >> 3);
  const int L = ll128::lines_for_words(payload_words);
  const int nchunks = L * kChunksPerLine;
  const int peers = N - 1;
  if (peers <= 0) return;
  const int K = n_send_warps >= peers ? n_send_warps / peers : 1;   // warps per peer
  const int k = n_send_warps >= peers ? send_warp / peers : 0;
  if (k >= K) return;
  const bool single_slab = nchunks <= NIT * 32;

  for (int j = (n_send_warps >= peers ? send_warp % peers : send_warp); j < peers; j += n_send_warps) {
    const int peer = (rank + 1 + j) % N;
    if ((p.skip_peer_mask >> peer) & 1u) continue;
    uint8_t* ring = cx.ws + (int64_t)peer * cx.stride + ring_offset(cx.lay, rank, c);
    uint8_t* sinfo = cx.my_row + sinfo_slot(cx.lay, peer, c);
    // line count of the ring at kernel entry, consumed count, and the first message: one round trip for all three
    const uint64_t head = ld_volatile_8(sinfo + kSinfoHeadOff);
    uint64_t tail = ld_volatile_8(sinfo + kSinfoTailOff);
    bool ok = true;
    if (p.debug_checks) {                      // debug: every message this warp is about to read must fit the tensors
      for (int i = k; i < n_mine && ok; i += K) ok = check_source(p, cx, c + i * C, peer, lane);
      // not ok: reported; nothing is read or sent for this peer (the loops below are skipped)
    }
    if (cx.trace != nullptr && send_warp == 0 && lane == 0 && cx.trace[2] == 0) cx.trace[2] = globaltimer_ns();
    uint64_t lo[NIT], hi[NIT];
    if (ok && single_slab && k < n_mine) load_message<NIT>(p, msg_src(p, io, c + k * C, peer), 0, nchunks, payload_words, lane, lo, hi);
    for (int i = k; i < n_mine && ok; i += K) {
      const int e = c + i * C;
      const uint64_t q0 = head + (uint64_t)i * L;
      // ring space for the whole message (bounded wait on the consumed count the receiver stores here)
      unsigned spins = 0;
      while (!ring_has_room(q0 + (uint64_t)L - 1, tail)) {
        tail = ld_volatile_8(sinfo + kSinfoTailOff);
        if ((++spins & 31u) == 0u && __any_sync(kFull, give_up(cx))) {
          if (lane == 0) report(cx, kTimeoutSendSpace, peer, e);
          ok = false;
          break;
        }
      }
      if (!ok) break;
      if (single_slab) {
        uint64_t nlo[NIT], nhi[NIT];
        const bool more = i + K < n_mine;
        if (more) load_message<NIT>(p, msg_src(p, io, c + (i + K) * C, peer), 0, nchunks, payload_words, lane, nlo, nhi);
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
          int ch = it * 32 + lane;
          if (ch < nchunks) {
            uint64_t h = ((ch & 7) == 7) ? ll128::flag_of(q0 + (uint64_t)(ch >> 3)) : hi[it];
            st_volatile_16(ring + ll128::chunk_ring_offset(q0, ch), lo[it], h);
          }
        }
        if (more) {
#pragma unroll
          for (int it = 0; it < NIT; ++it) {
            lo[it] = nlo[it];
            hi[it] = nhi[it];
          }
        }
      } else {
        const MsgSrc src = msg_src(p, io, e, peer);
        for (int chunk0 = 0; chunk0 < nchunks; chunk0 += NIT * 32) {
          load_message<NIT>(p, src, chunk0, nchunks, payload_words, lane, lo, hi);
#pragma unroll
          for (int it = 0; it < NIT; ++it) {
            int ch = chunk0 + it * 32 + lane;
            if (ch < nchunks) {
              uint64_t h = ((ch & 7) == 7) ? ll128::flag_of(q0 + (uint64_t)(ch >> 3)) : hi[it];
              st_volatile_16(ring + ll128::chunk_ring_offset(q0, ch), lo[it], h);
            }
          }
        }
      }
    }
    // The line count of the call is fixed by its shape, so one warp per ring records it, after every warp that shares
    // the ring has read the old count (each counts itself in when it is done with the ring, whatever happened).
    __syncwarp();
    if (lane == 0) {
      atomicAdd(&cx.ctl->sent[peer], 1u);
      if (ok && k == 0) {
        unsigned spins = 0;
        bool all = true;
        while (*reinterpret_cast<volatile unsigned*>(&cx.ctl->sent[peer]) < (unsigned)K) {
          if ((++spins & 1023u) == 0u && give_up(cx)) {
            all = false;
            break;
          }
        }
        if (all) st_volatile_8(sinfo + kSinfoHeadOff, head + (uint64_t)n_mine * L);
      }
    }
    if (cx.trace != nullptr && send_warp == 0 && lane == 0) cx.trace[3] = globaltimer_ns();
  }
}

// consumed-line counts of ring[lane][c] at kernel entry (lane j < N, j != rank)
HELIX_D uint64_t load_rtail0(const ExchangeParams& p, const Ctx& cx, int lane) {
  if (lane < p.cp_size && lane != cx.rank)
    return ld_volatile_8(cx.my_row + rinfo_slot(cx.lay, lane, cx.channel) + kRinfoTailOff);
  return 0ull;
}

// tell every sender how far its ring has been drained; `entries_done` complete entries
HELIX_D void publish_tails(const ExchangeParams& p, const Ctx& cx, uint64_t rtail0, int entries_done, int L,
                           bool final_, int lane) {
  if (lane < p.cp_size && lane != cx.rank) {
    uint64_t t_new = rtail0 + (uint64_t)entries_done * L;
    if (final_) st_volatile_8(cx.my_row + rinfo_slot(cx.lay, lane, cx.channel) + kRinfoTailOff, t_new);
    st_volatile_8(cx.ws + (int64_t)lane * cx.stride + sinfo_slot(cx.lay, cx.rank, cx.channel) + kSinfoTailOff, t_new);
  }
}

// end of call: the last receiver warp of the CTA publishes the final consumed counts
HELIX_D void finish_receiver(const ExchangeParams& p, const Ctx& cx, uint64_t rtail0, int n_mine, int L, int NR,
                             int lane) {
  __syncwarp();
  unsigned last = 0;
  if (lane == 0) last = (atomicAdd(&cx.ctl->done, 1u) == (unsigned)(NR - 1));
  last = __shfl_sync(kFull, last, 0);
  if (last && !aborted(cx)) publish_tails(p, cx, rtail0, n_mine, L, true, lane);
}

// ---- exchange mode: write every received row (and this rank's own) to the output tensors ------
template <int NIT>
HELIX_D void receiver_exchange_warp(const ExchangeParams& p, const Ctx& cx, const RankIO& io, int r, int NR,
                                    int lane) {
  const int N = p.cp_size, C = p.channels, c = cx.channel, rank = cx.rank;
  const int E = p.outer * p.inner;
  const int n_mine = entries_of_channel(E, C, c);
  const int payload_words = p.st_words + (p.o_bytes >> 3);
  const int L = ll128::lines_for_words(payload_words);
  const int nchunks = L * kChunksPerLine;
  const uint64_t rtail0 = load_rtail0(p, cx, lane);
  bool alive = true;

  // work item t = i * N + j: entry i of this channel, source j (j == N-1: this rank's own row)
  const int items = n_mine * N;
  const int rounds = ceil_div(items, NR);
  for (int k = 0; k < rounds; ++k) {
    const int t = k * NR + r;
    if (t < items && alive) {
      const int i = t / N;
      const int j = t - i * N;
      const int e = c + i * C;
      const int peer = (j == N - 1) ? rank : (rank + N - 1 - j) % N;
      uint8_t* od = io.o_dst + e * p.od_se + peer * p.od_sp;
      uint8_t* sd = io.st_dst + e * p.sd_se + peer * p.sd_sp;
      const uint64_t q0 = __shfl_sync(kFull, rtail0, peer) + (uint64_t)i * L;
      const uint8_t* ring = cx.my_row + ring_offset(cx.lay, peer, c);
      if (!check_dest(p, cx, io, e, peer, lane) || (peer == rank && !check_source(p, cx, e, rank, lane))) {
        alive = false;                         // debug: the row would land outside the caller's tensor
        continue;
      }
      const MsgSrc self = msg_src(p, io, e, rank);
      for (int chunk0 = 0; chunk0 < nchunks; chunk0 += NIT * 32) {
        uint64_t lo[NIT], hi[NIT];
        if (peer == rank) {
          load_message<NIT>(p, self, chunk0, nchunks, payload_words, lane, lo, hi);
        } else if (!poll_message<NIT>(cx, ring, q0, chunk0, nchunks, lane, lo, hi)) {
          if (lane == 0) report(cx, kTimeoutRecv, peer, e);
          alive = false;
          break;
        }
#pragma unroll
        for (int it = 0; it < NIT; ++it) {
          int ch = chunk0 + it * 32 + lane;
          if (ch < nchunks) {
            ll128::ChunkMap m = ll128::chunk_map(ch);
            int w0 = m.first, w1 = m.first + 1;
            if (w0 < p.st_words) st_8(sd + 8 * w0, lo[it]);
            else if (w0 < payload_words) st_8(od + 8 * (w0 - p.st_words), lo[it]);
            if (!m.has_flag) {
              if (w1 < p.st_words) st_8(sd + 8 * w1, hi[it]);
              else if (w1 < payload_words) st_8(od + 8 * (w1 - p.st_words), hi[it]);
            }
          }
        }
      }
    }
    // in-call flow control: every `rounds_per_publish` rounds all receiver warps meet and warp 0
    // tells the senders how far their rings have been drained
    if (p.rounds_per_publish > 0 && (k + 1) % p.rounds_per_publish == 0 && k + 1 < rounds) {
      named_barrier(kAllRecvBarrier, NR * 32);
      if (r == 0 && !aborted(cx)) publish_tails(p, cx, rtail0, ((k + 1) * NR) / N, L, false, lane);
    }
  }
  finish_receiver(p, cx, rtail0, n_mine, L, NR, lane);
}

// Hook run by the finishing warp after it has written the combined row of entry e.
struct NoHook {
  HELIX_D void operator()(int /*e*/, int /*lane*/) const {}
};

// ---- combine mode: G warps share one entry, warp k of a group polls the peers j = k, k+G, ... ---
template <bool BF16, int NIT, class Hook>
HELIX_D void receiver_combine_warp(const ExchangeParams& p, const Ctx& cx, const RankIO& io, int r, int NR,
                                   int lane, float* group_smem, const Hook& hook) {
  const int N = p.cp_size, C = p.channels, c = cx.channel, rank = cx.rank;
  const int E = p.outer * p.inner;
  const int n_mine = entries_of_channel(E, C, c);
  const int payload_words = p.st_words + (p.o_bytes >> 3);  // st_words == 1 here
  const int L = ll128::lines_for_words(payload_words);
  const int nchunks = L * kChunksPerLine;
  const int G = p.group_warps;
  const int NG = NR / G;
  const int g = r / G, k = r - g * G;
  const uint64_t rtail0 = load_rtail0(p, cx, lane);
  bool alive = true;
  const int slot = group_slot_floats<NIT>();

  const int rounds = ceil_div(n_mine, NG);
  for (int rd = 0; rd < rounds; ++rd) {
    const int i = rd * NG + g;
    const bool have = i < n_mine;
    const int e = c + i * C;
    Acc<NIT> acc;
    acc.init();
    if (have && alive && (!check_source(p, cx, e, rank, lane) || !check_dest(p, cx, io, e, 0, lane))) alive = false;
    if (have && alive) {
      uint64_t lo[NIT], hi[NIT];
      if (k == 0) {  // this rank's own contribution comes straight from its attention output
        const MsgSrc self = msg_src(p, io, e, rank);
        load_message<NIT>(p, self, 0, nchunks, payload_words, lane, lo, hi);
        float l = ingest_lse(__shfl_sync(kFull, lo[0], 0), p.stats_mode, p.base2);
        acc.template add<BF16>(l, lo, hi);
      }
      for (int j = k; j < N - 1; j += G) {
        const int peer = (rank + N - 1 - j) % N;
        const uint64_t q0 = __shfl_sync(kFull, rtail0, peer) + (uint64_t)i * L;
        const uint8_t* ring = cx.my_row + ring_offset(cx.lay, peer, c);
        if (!poll_message<NIT>(cx, ring, q0, 0, nchunks, lane, lo, hi)) {
          if (lane == 0) report(cx, kTimeoutRecv, peer, e);
          alive = false;
          break;
        }
        float l = ingest_lse(__shfl_sync(kFull, lo[0], 0), p.stats_mode, p.base2);
        acc.template add<BF16>(l, lo, hi);
        if (cx.trace != nullptr && r == 0 && lane == 0) {
          const unsigned long long now = globaltimer_ns();
          if (cx.trace[4] == 0) cx.trace[4] = now;
          cx.trace[5] = now;
        }
      }
    }
    if (G > 1) {
      // park partial accumulators of warps 1..G-1, double-buffered by round parity
      float* base = group_smem + ((size_t)(g * 2 + (rd & 1)) * (G - 1)) * slot;
      if (k > 0) {
        float* mine = base + (size_t)(k - 1) * slot;
#pragma unroll
        for (int it = 0; it < NIT; ++it)
#pragma unroll
          for (int j = 0; j < 8; ++j) mine[(it * 8 + j) * 32 + lane] = acc.v[it][j];
        if (lane == 0) {
          mine[NIT * 8 * 32] = acc.m;
          mine[NIT * 8 * 32 + 1] = acc.s;
        }
      }
      named_barrier(kGroupBarrier0 + g, G * 32);
      if (k == 0) {
        for (int kk = 1; kk < G; ++kk) {
          const float* other = base + (size_t)(kk - 1) * slot;
          acc.merge(other[NIT * 8 * 32], other[NIT * 8 * 32 + 1], other, lane);
        }
      }
    }
    if (k == 0 && have && !aborted(cx)) {
      const float inv = acc.s > 0.f ? 1.0f / acc.s : 0.f;
      uint8_t* od = io.o_dst + e * p.od_se;
#pragma unroll
      for (int it = 0; it < NIT; ++it) {
        int ch = it * 32 + lane;
        if (ch < nchunks) {
          ll128::ChunkMap m = ll128::chunk_map(ch);
          float f[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = acc.v[it][j] * inv;
          int w0 = m.first, w1 = m.first + 1;
          if (w0 >= p.st_words && w0 < payload_words) st_8(od + 8 * (w0 - p.st_words), pack4<BF16>(f));
          if (!m.has_flag && w1 >= p.st_words && w1 < payload_words)
            st_8(od + 8 * (w1 - p.st_words), pack4<BF16>(f + 4));
        }
      }
      if (io.st_dst != nullptr && lane == 0) {
        float gl = acc.s > 0.f ? (acc.m + log2f(acc.s)) : -INFINITY;
        if (!p.base2) gl *= kLn2;
        reinterpret_cast<float*>(io.st_dst)[e] = gl;
      }
      hook(e, lane);
    } else if (k == 0 && have) {
      // this call gave up on a wait: leave NaN in the row instead of whatever the buffer held, so that a
      // caller who does not read the status block still cannot mistake the row for a result
      const uint64_t nan4 = BF16 ? 0x7FC07FC07FC07FC0ull : 0x7E007E007E007E00ull;
      uint8_t* od = io.o_dst + e * p.od_se;
      for (int w = lane; w < (p.o_bytes >> 3); w += 32) st_8(od + 8 * w, nan4);
      if (io.st_dst != nullptr && lane == 0) reinterpret_cast<float*>(io.st_dst)[e] = __uint_as_float(0x7FC00000u);
    }
    if (p.rounds_per_publish > 0 && (rd + 1) % p.rounds_per_publish == 0 && rd + 1 < rounds) {
      named_barrier(kAllRecvBarrier, NR * 32);
      if (r == 0 && !aborted(cx)) publish_tails(p, cx, rtail0, min((rd + 1) * NG, n_mine), L, false, lane);
    }
  }
  finish_receiver(p, cx, rtail0, n_mine, L, NR, lane);
}

HELIX_D Ctx make_ctx(const ExchangeParams& p, Control* ctl, int rank, int channel) {
  Ctx cx;
  cx.ws = reinterpret_cast<uint8_t*>(p.workspace);
  cx.stride = p.row_stride_bytes;
  cx.my_row = cx.ws + (int64_t)rank * cx.stride;
  cx.lay = make_layout(p.cp_size, p.sm_count);
  cx.ctl = ctl;
  cx.rank = rank;
  cx.channel = channel;
  cx.deadline = 0;
  cx.trace = nullptr;
  return cx;
}

}  // namespace dev
}  // namespace helix
