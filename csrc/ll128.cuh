// LL128-style wire format of the Helix exchange, written for register-to-peer stores.
//
// A message is a payload of Pw 8-byte words (the fp32 softmax stats first, then the
// partial-output row).  On the wire it becomes L = ceil(Pw / 15) lines of 128 bytes.
// Line j carries payload words [15 j, 15 j + 15) in its words 0..14 and a 64-bit flag
// in word 15.  A line is produced by ONE warp-wide store instruction in which 8
// consecutive lanes each write a 16-byte chunk, so data and flag travel over NVLink as
// one 128-byte unit and the receiver needs no separate "ready" write.
//
// Differences from the reference's framing (csrc/ll128_proto.cuh:73-139): the flag
// sits at a fixed slot and the payload is simply cut every 120 bytes, so there are
// no displaced words and no tail lines (9 lines instead of 10 for a 1032-byte MLA
// message, 3 instead of 4 for a 264-byte GQA message), and nothing is staged in
// shared memory.  The flag is the absolute line sequence number of the ring plus one:
// it never repeats, so rings are never cleared or re-armed, and freshly initialised
// memory (all ones) or a line of the previous lap can never look valid.
//
// Every function is host+device so the format is unit-tested on the CPU.
#pragma once

#include "helix_common.cuh"

namespace helix {
namespace ll128 {

// lines needed for a payload of `payload_words` 8-byte words
HELIX_HD int lines_for_words(int payload_words) { return ceil_div(payload_words, kLineDataWords); }

// bytes on the wire for a payload (used by the roofline arithmetic and the tuner)
HELIX_HD int wire_bytes_for_words(int payload_words) { return lines_for_words(payload_words) * kLineBytes; }

// flag carried by the line with absolute sequence number q
HELIX_HD uint64_t flag_of(uint64_t q) { return q + 1ull; }

// position of line q inside its ring
HELIX_HD uint32_t ring_slot(uint64_t q) { return static_cast<uint32_t>(q & (uint64_t)(kRingLines - 1)); }

// A 16-byte chunk `ch` of a message (ch = 8*line + k): which payload words it holds.
// first = payload word index of the low 8 bytes; the high 8 bytes hold word first+1,
// except in the last chunk of a line (k == 7) where they hold the flag.
struct ChunkMap {
  int line;        // line index inside the message
  int first;       // payload word of the low half
  bool has_flag;   // high half is the flag
};

HELIX_HD ChunkMap chunk_map(int ch) {
  ChunkMap m;
  m.line = ch >> 3;
  int k = ch & 7;
  m.first = m.line * kLineDataWords + 2 * k;
  m.has_flag = (k == 7);
  return m;
}

// byte offset of chunk `ch` of the message whose first line has sequence q0, inside the ring
HELIX_HD uint32_t chunk_ring_offset(uint64_t q0, int ch) {
  return ring_slot(q0 + (uint64_t)(ch >> 3)) * kLineBytes + (uint32_t)(ch & 7) * kChunkBytes;
}

// ---- host-side reference implementation (also the oracle for the device code) --------------
// ring: kRingLines * 16 u64 words.

inline void pack_line_host(const uint64_t* payload, int payload_words, uint64_t q0, int line,
                           uint64_t* ring) {
  uint64_t* dst = ring + (size_t)ring_slot(q0 + line) * kLineWords;
  for (int w = 0; w < kLineDataWords; ++w) {
    int pw = line * kLineDataWords + w;
    dst[w] = pw < payload_words ? payload[pw] : 0ull;
  }
  dst[kLineDataWords] = flag_of(q0 + line);
}

inline void pack_message_host(const uint64_t* payload, int payload_words, uint64_t q0, uint64_t* ring) {
  int L = lines_for_words(payload_words);
  for (int j = 0; j < L; ++j) pack_line_host(payload, payload_words, q0, j, ring);
}

// number of lines of the message (in order) whose flag is valid
inline int valid_prefix_host(const uint64_t* ring, int payload_words, uint64_t q0) {
  int L = lines_for_words(payload_words);
  int n = 0;
  for (; n < L; ++n) {
    const uint64_t* src = ring + (size_t)ring_slot(q0 + n) * kLineWords;
    if (src[kLineDataWords] != flag_of(q0 + n)) break;
  }
  return n;
}

inline bool message_ready_host(const uint64_t* ring, int payload_words, uint64_t q0) {
  int L = lines_for_words(payload_words);
  for (int j = 0; j < L; ++j) {
    const uint64_t* src = ring + (size_t)ring_slot(q0 + j) * kLineWords;
    if (src[kLineDataWords] != flag_of(q0 + j)) return false;
  }
  return true;
}

inline void unpack_message_host(const uint64_t* ring, int payload_words, uint64_t q0, uint64_t* payload) {
  int L = lines_for_words(payload_words);
  for (int j = 0; j < L; ++j) {
    const uint64_t* src = ring + (size_t)ring_slot(q0 + j) * kLineWords;
    for (int w = 0; w < kLineDataWords; ++w) {
      int pw = j * kLineDataWords + w;
      if (pw < payload_words) payload[pw] = src[w];
    }
  }
}

}  // namespace ll128
}  // namespace helix
