// Debug bounds checks of the exchange's addressing of USER tensors (ring offsets are modulo by construction).
// The reference validates shapes, dtypes and contiguity on the host only (csrc/torch_binding.cpp:75-113) and its
// kernel takes dense [entries, cp, D] buffers (csrc/helix_alltoall.cu:292-309), so it has no counterpart of these
// checks; here the kernel addresses strided views of the caller's tensors, which is what they cover.
//
// The kernel reads its inputs in their native strided layout and writes its outputs through strides that the
// binding computes; a wrong stride would read or write outside the caller's tensors.  With
// ExchangeParams::debug_checks set (HELIX_A2A_DEBUG=1) every message's source and destination span is checked
// against the byte extents the binding recorded; a span that does not fit is never touched: the warp records
// kBadArgument in the status block and skips the access.  The same functions compile for the host, where the
// unit tests walk every (entry, peer) of a launch.
#pragma once

#include "exchange.h"

namespace helix {
namespace bounds {

// byte offset of message (e, peer) inside the source tensors
HELIX_HD int64_t src_o_off(const ExchangeParams& p, int e, int peer) {
  const int b = e / p.inner, hl = e - b * p.inner;
  return (int64_t)b * p.o_sb + (int64_t)peer * p.o_sp + (int64_t)hl * p.o_sh;
}
HELIX_HD int64_t src_st_off(const ExchangeParams& p, int e, int peer) {
  const int b = e / p.inner, hl = e - b * p.inner;
  return (int64_t)b * p.st_sb + (int64_t)peer * p.st_sp + (int64_t)hl * p.st_sh;
}
HELIX_HD int64_t src_st_len(const ExchangeParams& p) { return p.lse_scalar ? 4 : (int64_t)p.st_words * 8; }
// destinations: exchange mode writes row (e, peer), combine mode row e (and one float of global LSE)
HELIX_HD int64_t dst_o_off(const ExchangeParams& p, int e, int peer) {
  return (int64_t)e * p.od_se + (p.mode == kModeExchange ? (int64_t)peer * p.od_sp : 0);
}
HELIX_HD int64_t dst_st_off(const ExchangeParams& p, int e, int peer) {
  return p.mode == kModeExchange ? (int64_t)e * p.sd_se + (int64_t)peer * p.sd_sp : (int64_t)e * 4;
}
HELIX_HD int64_t dst_st_len(const ExchangeParams& p) { return p.mode == kModeExchange ? (int64_t)p.st_words * 8 : 4; }

// [off, off + len) inside [0, extent); extent <= 0 means "not recorded": nothing to check against
HELIX_HD bool span_ok(int64_t off, int64_t len, int64_t extent) {
  return extent <= 0 || (off >= 0 && len >= 0 && off + len <= extent);
}

HELIX_HD bool source_ok(const ExchangeParams& p, int e, int peer) {
  return span_ok(src_o_off(p, e, peer), p.o_bytes, p.o_src_bytes) &&
         span_ok(src_st_off(p, e, peer), src_st_len(p), p.st_src_bytes);
}
HELIX_HD bool dest_ok(const ExchangeParams& p, int e, int peer, bool has_st_dst) {
  return span_ok(dst_o_off(p, e, peer), p.o_bytes, p.o_dst_bytes) &&
         (!has_st_dst || span_ok(dst_st_off(p, e, peer), dst_st_len(p), p.st_dst_bytes));
}

// host-side walk over a whole launch: number of (entry, peer) messages whose spans do not fit
HELIX_HD int count_violations(const ExchangeParams& p, bool has_st_dst) {
  int bad = 0;
  const int E = p.outer * p.inner;
  for (int e = 0; e < E; ++e)
    for (int peer = 0; peer < p.cp_size; ++peer) {
      if (!source_ok(p, e, peer)) ++bad;
      if (p.mode == kModeExchange ? !dest_ok(p, e, peer, has_st_dst) : (peer == 0 && !dest_ok(p, e, 0, has_st_dst))) ++bad;
    }
  return bad;
}

}  // namespace bounds
}  // namespace helix
