// Host build of the wire format and FIFO arithmetic, plus a model of the whole protocol.
//
// Compiled with g++ only (no CUDA) into helix_a2a_b200/_ll128_host.so and driven from the CPU
// unit tests through ctypes.  Two parts:
//   1. thin C wrappers around ll128.cuh / fifo.cuh, which are the very functions the device
//      code calls, so framing, ring wrap and layout arithmetic are tested without a GPU;
//   2. `helix_model_run`: a discrete-event model of N ranks exchanging several calls through
//      rings in host memory.  Lines travel through a "network" that delivers them one at a
//      time in random order (so a receiver sees partially arrived messages), senders obey the
//      head/tail flow-control rule and receivers publish consumed counts exactly as the kernel
//      does.  The model checks every delivered payload, that no line is overwritten before it
//      was consumed, and that the run terminates (no deadlock).
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <random>
#include <vector>

#include "fifo.cuh"
#include "bounds.cuh"
#include "ll128.cuh"

using namespace helix;

extern "C" {

int helix_lines_for_words(int w) { return ll128::lines_for_words(w); }
int helix_wire_bytes_for_words(int w) { return ll128::wire_bytes_for_words(w); }
uint64_t helix_flag_of(uint64_t q) { return ll128::flag_of(q); }
uint32_t helix_ring_slot(uint64_t q) { return ll128::ring_slot(q); }
int helix_ring_lines() { return kRingLines; }
uint32_t helix_chunk_ring_offset(uint64_t q0, int ch) { return ll128::chunk_ring_offset(q0, ch); }
void helix_chunk_map(int ch, int* line, int* first, int* has_flag) {
  ll128::ChunkMap m = ll128::chunk_map(ch);
  *line = m.line;
  *first = m.first;
  *has_flag = m.has_flag ? 1 : 0;
}
void helix_pack_message(const uint64_t* payload, int words, uint64_t q0, uint64_t* ring) {
  ll128::pack_message_host(payload, words, q0, ring);
}
void helix_pack_line(const uint64_t* payload, int words, uint64_t q0, int line, uint64_t* ring) {
  ll128::pack_line_host(payload, words, q0, line, ring);
}
int helix_valid_prefix(const uint64_t* ring, int words, uint64_t q0) { return ll128::valid_prefix_host(ring, words, q0); }
int helix_message_ready(const uint64_t* ring, int words, uint64_t q0) {
  return ll128::message_ready_host(ring, words, q0) ? 1 : 0;
}
void helix_unpack_message(const uint64_t* ring, int words, uint64_t q0, uint64_t* payload) {
  ll128::unpack_message_host(ring, words, q0, payload);
}
// chunk-level packing exactly as a sender lane does it: returns the two u64 a lane stores
void helix_chunk_words(const uint64_t* payload, int words, uint64_t q0, int ch, uint64_t* lo, uint64_t* hi) {
  ll128::ChunkMap m = ll128::chunk_map(ch);
  *lo = m.first < words ? payload[m.first] : 0ull;
  if (m.has_flag) *hi = ll128::flag_of(q0 + m.line);
  else *hi = (m.first + 1) < words ? payload[m.first + 1] : 0ull;
}

void helix_layout(int cp, int sm_count, int64_t* out /* 6 */) {
  WorkspaceLayout l = make_layout(cp, sm_count);
  out[0] = l.max_channels;
  out[1] = l.ring_region;
  out[2] = l.sinfo_offset;
  out[3] = l.rinfo_offset;
  out[4] = l.status_offset;
  out[5] = l.row_bytes;
}
int64_t helix_ring_offset(int cp, int sm_count, int sender, int channel) {
  return ring_offset(make_layout(cp, sm_count), sender, channel);
}
int64_t helix_sinfo_slot(int cp, int sm_count, int receiver, int channel) {
  return sinfo_slot(make_layout(cp, sm_count), receiver, channel);
}
int64_t helix_rinfo_slot(int cp, int sm_count, int sender, int channel) {
  return rinfo_slot(make_layout(cp, sm_count), sender, channel);
}
int helix_entries_of_channel(int entries, int channels, int c) { return entries_of_channel(entries, channels, c); }
int helix_ring_has_room(uint64_t q_last, uint64_t tail) { return ring_has_room(q_last, tail) ? 1 : 0; }

// ---------------------------------------------------------------------------------------------
// Protocol model.  Returns 0 on success, otherwise an error code:
//   1 payload mismatch, 2 line overwritten before consumption, 3 no progress (deadlock),
//   4 flag seen on a line that was not the expected one.
// publish_every: receiver publishes its consumed count every this many messages (0 = only at
// the end of a call, as the kernel does for small calls).
// drop_sender: rank whose senders never send (-1 = none); the model must then report 3.
int helix_model_run(int cp, int calls, const int* entries_per_call, int payload_words, int channels,
                    int publish_every, int drop_sender, uint32_t seed, int64_t* lines_moved) {
  const int N = cp, C = channels, L = ll128::lines_for_words(payload_words);
  std::mt19937 rng(seed);
  struct Ring {
    std::vector<uint64_t> mem;        // kRingLines * 16
    std::vector<uint8_t> unread;      // line written and not yet consumed
    uint64_t head = 0;                // sender side (lives in sender's row)
    uint64_t tail_at_sender = 0;      // remote copy the receiver stores into the sender's row
    uint64_t rtail = 0;               // receiver's consumed count
  };
  auto ring_of = [&](std::vector<Ring>& rings, int recv, int send, int c) -> Ring& {
    return rings[((size_t)recv * N + send) * C + c];
  };
  std::vector<Ring> rings((size_t)N * N * C);
  for (auto& r : rings) {
    r.mem.assign((size_t)kRingLines * kLineWords, ~0ull);
    r.unread.assign(kRingLines, 0);
  }
  struct InFlight { int recv, send, c; uint64_t q; uint64_t words[kLineWords]; };
  std::vector<InFlight> net;
  auto payload_word = [&](int call, int send, int recv, int e, int w) -> uint64_t {
    return ((uint64_t)call << 48) ^ ((uint64_t)send << 40) ^ ((uint64_t)recv << 32) ^ ((uint64_t)e << 12) ^ (uint64_t)w ^
           0x9e3779b97f4a7c15ull;
  };
  int64_t moved = 0;
  for (int call = 0; call < calls; ++call) {
    const int E = entries_per_call[call];
    // per (send, recv, c): next message index to send / receive
    std::vector<int> s_next((size_t)N * N * C, 0), r_next((size_t)N * N * C, 0);
    std::vector<uint64_t> head0((size_t)N * N * C), rtail0((size_t)N * N * C);
    for (int recv = 0; recv < N; ++recv)
      for (int send = 0; send < N; ++send)
        for (int c = 0; c < C; ++c) {
          Ring& r = ring_of(rings, recv, send, c);
          head0[((size_t)recv * N + send) * C + c] = r.head;
          rtail0[((size_t)recv * N + send) * C + c] = r.rtail;
        }
    auto done = [&]() {
      for (int recv = 0; recv < N; ++recv)
        for (int send = 0; send < N; ++send) {
          if (send == recv) continue;
          for (int c = 0; c < C; ++c)
            if (r_next[((size_t)recv * N + send) * C + c] < entries_of_channel(E, C, c)) return false;
        }
      return net.empty();
    };
    int idle_rounds = 0;
    while (!done()) {
      bool progress = false;
      // senders
      for (int send = 0; send < N; ++send) {
        if (send == drop_sender) continue;
        for (int recv = 0; recv < N; ++recv) {
          if (recv == send) continue;
          for (int c = 0; c < C; ++c) {
            size_t k = ((size_t)recv * N + send) * C + c;
            int n = entries_of_channel(E, C, c);
            if (s_next[k] >= n || (rng() & 3) == 0) continue;
            Ring& r = ring_of(rings, recv, send, c);
            uint64_t q0 = head0[k] + (uint64_t)s_next[k] * L;
            if (!ring_has_room(q0 + L - 1, r.tail_at_sender)) continue;
            int e = c + s_next[k] * C;
            std::vector<uint64_t> pay(payload_words);
            for (int w = 0; w < payload_words; ++w) pay[w] = payload_word(call, send, recv, e, w);
            for (int j = 0; j < L; ++j) {
              InFlight f;
              f.recv = recv; f.send = send; f.c = c; f.q = q0 + j;
              uint64_t tmp[kLineWords];
              // build the line through the chunk view a warp uses
              for (int kk = 0; kk < kChunksPerLine; ++kk)
                helix_chunk_words(pay.data(), payload_words, q0, j * 8 + kk, &tmp[2 * kk], &tmp[2 * kk + 1]);
              memcpy(f.words, tmp, sizeof(tmp));
              net.push_back(f);
            }
            s_next[k]++;
            if (s_next[k] == n) r.head = head0[k] + (uint64_t)n * L;
            progress = true;
          }
        }
      }
      // network: deliver a random subset of lines, in random order
      std::shuffle(net.begin(), net.end(), rng);
      size_t deliver = net.empty() ? 0 : 1 + rng() % net.size();
      for (size_t i = 0; i < deliver; ++i) {
        InFlight& f = net.back();
        Ring& r = ring_of(rings, f.recv, f.send, f.c);
        uint32_t slot = ll128::ring_slot(f.q);
        if (r.unread[slot]) return 2;
        memcpy(&r.mem[(size_t)slot * kLineWords], f.words, sizeof(f.words));
        r.unread[slot] = 1;
        net.pop_back();
        ++moved;
        progress = true;
      }
      // receivers
      for (int recv = 0; recv < N; ++recv)
        for (int send = 0; send < N; ++send) {
          if (send == recv) continue;
          for (int c = 0; c < C; ++c) {
            size_t k = ((size_t)recv * N + send) * C + c;
            int n = entries_of_channel(E, C, c);
            if (r_next[k] >= n) continue;
            Ring& r = ring_of(rings, recv, send, c);
            uint64_t q0 = rtail0[k] + (uint64_t)r_next[k] * L;
            if (!ll128::message_ready_host(r.mem.data(), payload_words, q0)) continue;
            std::vector<uint64_t> got(payload_words);
            ll128::unpack_message_host(r.mem.data(), payload_words, q0, got.data());
            int e = c + r_next[k] * C;
            for (int w = 0; w < payload_words; ++w)
              if (got[w] != payload_word(call, send, recv, e, w)) return 1;
            for (int j = 0; j < L; ++j) {
              uint32_t slot = ll128::ring_slot(q0 + j);
              if (!r.unread[slot]) return 4;
              r.unread[slot] = 0;
            }
            r_next[k]++;
            bool last = r_next[k] == n;
            if (last || (publish_every > 0 && r_next[k] % publish_every == 0)) {
              uint64_t t = rtail0[k] + (uint64_t)r_next[k] * L;
              r.tail_at_sender = t;
              if (last) r.rtail = t;
            }
            progress = true;
          }
        }
      idle_rounds = progress ? 0 : idle_rounds + 1;
      if (idle_rounds > 64) return 3;
    }
  }
  if (lines_moved) *lines_moved = moved;
  return 0;
}

// Debug bounds checks of the exchange (bounds.cuh): number of messages of a launch whose source or destination
// span leaves the recorded extents.  strides / extents in bytes; mode 0 = exchange, 1 = combine.
int helix_bounds_violations(int cp, int outer, int inner, int mode, int o_bytes, int st_words, int lse_scalar,
                            long long o_sb, long long o_sp, long long o_sh, long long st_sb, long long st_sp,
                            long long st_sh, long long od_se, long long od_sp, long long sd_se, long long sd_sp,
                            long long o_src_bytes, long long st_src_bytes, long long o_dst_bytes,
                            long long st_dst_bytes, int has_st_dst) {
  helix::ExchangeParams p{};
  p.cp_size = cp; p.outer = outer; p.inner = inner; p.mode = mode; p.o_bytes = o_bytes; p.st_words = st_words;
  p.lse_scalar = lse_scalar;
  p.o_sb = o_sb; p.o_sp = o_sp; p.o_sh = o_sh; p.st_sb = st_sb; p.st_sp = st_sp; p.st_sh = st_sh;
  p.od_se = od_se; p.od_sp = od_sp; p.sd_se = sd_se; p.sd_sp = sd_sp;
  p.o_src_bytes = o_src_bytes; p.st_src_bytes = st_src_bytes; p.o_dst_bytes = o_dst_bytes; p.st_dst_bytes = st_dst_bytes;
  return helix::bounds::count_violations(p, has_st_dst != 0);
}

}  // extern "C"
