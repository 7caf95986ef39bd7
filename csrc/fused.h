// One kernel for exchange + LSE combine + o_proj: host interface (kernel and design in fused_exchange_oproj.cu).
#pragma once

#include "exchange.h"
#include "oproj.h"

namespace helix {

constexpr int kFusedMaxRanks = 8;     // ranks one launch can play in single-process emulation
constexpr int kFusedMaxTokens = 64;   // tokens per call (padded to 16): W slice + activation rows must fit shared memory

struct FusedParams {
  ExchangeParams ex;                 // combine mode, native layout; o_dst is unused
  // Per emulated rank (index 0 in multi-process use).  `splits` = number of head groups: GEMM CTA (slab, group)
  // owns heads [group * heads_per_split, +heads_per_split); x_map, stages, atoms and ctas are unused.
  OprojParams gemm[kFusedMaxRanks];
  __nv_bfloat16* x_out[kFusedMaxRanks];   // optional [tokens, (H / cp) * D]: the combined activation, for tests
  int exchange_ctas;                 // CTAs [0, exchange_ctas) only send, the rest receive + combine + multiply
  int gemm_ctas;                     // hidden / 128 * splits
  int send_warps;                    // sender warps of a sending CTA
  int heads_per_split;
  // Rows shared between the slabs of a head group (set by the launcher when a call has many rows): the hidden / 128
  // CTAs of a group each receive and combine 1 / (hidden / 128) of the group's rows, store them in x_out (then
  // required), count them in aux and copy the complete group from L2 into their operand buffer.  0: every CTA
  // receives all rows of its group itself (least latency for a few rows).
  int share_rows;
  // Per rank, zero on entry and on exit: [0, hidden / 128) second fold counter, then kFusedMaxGroups "rows ready"
  // and kFusedMaxGroups "slabs done" counters (one per head group).
  int* aux[kFusedMaxRanks];
};

constexpr int kFusedMaxGroups = 64;
inline int fused_aux_ints(int hidden) { return hidden / 128 + 2 * kFusedMaxGroups; }
// rows (token, head) a GEMM CTA would receive by itself above which the slabs of a group share them
constexpr int kFusedShareAbove = 32;
inline bool fused_shares_rows(int tokens, int heads_per_split, int hidden) {
  return hidden / 128 > 1 && tokens * heads_per_split > kFusedShareAbove;
}

// Head groups for a rank that combines `heads_local` heads of `head_dim`: the fewest equal groups whose K-slice is
// at most 512 wide; 0 when even one head is too wide (the fused kernel then does not apply).
int fused_pick_splits(int heads_local, int head_dim);
size_t fused_smem_bytes(int k_slice, int n_pad);
// The launcher's shape rules without a launch: would a call with these sizes run as one kernel on a device with
// `sm_count` SMs (one CTA per SM)?  Callers use it to choose between the one-kernel path and the two-kernel chain.
bool fused_fits(int tokens, int heads_local, int head_dim, int hidden, int cp_size, int sm_count);

// Launches the fused kernel.  cudaErrorNotSupported: the shape does not fit (more than kFusedMaxTokens tokens, a
// head wider than 512, more CTAs than the device holds at once, or a call that would fill half a ring); callers
// then run the exchange and the GEMM as two kernels.
cudaError_t launch_exchange_oproj(FusedParams fp, int channel_override, bool pdl, cudaStream_t stream,
                                  LaunchInfo* info_out);

}  // namespace helix
