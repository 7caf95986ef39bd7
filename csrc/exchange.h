// Public C++ interface of the Helix exchange (+ fused LSE combine) for B200.
//
// Counterpart of the reference's csrc/helix_alltoall.h:16-43, with two additions: the
// sender addresses the attention output in its native [B, H, D] layout through strides
// (so no permute copies are needed), and the receiver can apply the LSE-weighted combine
// while the lines land instead of returning the raw received rows.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "helix_common.cuh"

namespace helix {

enum ExchangeMode : int {
  kModeExchange = 0,   // reference contract: return every received row and its stats
  kModeCombine = 1,    // fused: out[b, hl, :] = sum_p w_p o_p / sum_p w_p
};

enum StatsMode : int {
  kStatsLse = 0,        // stats[0] is the LSE, stats[1] ignored
  kStatsMaxSumExp = 1,  // stats = (running max, sum of exponentials)
};

// Pointers of one rank.  In multi-process use only io[0] is filled; when one process
// plays all ranks (single-GPU emulation, one cooperative launch) io[r] belongs to rank r.
struct RankIO {
  const uint8_t* o_src;    // partial outputs
  const uint8_t* st_src;   // fp32 stats (or one fp32 LSE per entry when lse_scalar)
  uint8_t* o_dst;          // exchange: received rows; combine: combined rows
  uint8_t* st_dst;         // exchange: received stats; combine: optional global LSE (may be null)
};

struct ExchangeParams {
  RankIO io[kMaxEmulatedRanks];
  uint64_t* workspace;          // base of row 0
  int64_t row_stride_bytes;     // distance between rows
  int cp_size;
  int rank_base;                // rank of blockIdx.y == 0
  int ranks_in_launch;          // 1, or cp_size in emulation
  int sm_count;                 // fixes the workspace layout

  // entry e = b * inner + hl,  0 <= b < outer, 0 <= hl < inner
  int outer, inner;
  // message (e, peer p): o bytes at o_src + b*o_sb + p*o_sp + hl*o_sh   (strides in bytes)
  int64_t o_sb, o_sp, o_sh;
  int64_t st_sb, st_sp, st_sh;
  // exchange-mode destination of the row received from peer p for entry e:
  //   o_dst + e*od_se + p*od_sp ; st_dst + e*sd_se + p*sd_sp
  // combine mode: o_dst + e*od_se ; st_dst + e*4
  int64_t od_se, od_sp, sd_se, sd_sp;

  int o_bytes;          // D * element size (multiple of 16)
  int st_words;         // 8-byte words of stats per message (S/2; 1 when lse_scalar)
  int lse_scalar;       // stats source holds ONE float per entry; the wire pads it with 0
  int is_bf16;          // element type of o (else fp16); combine mode only
  int mode;             // ExchangeMode
  int stats_mode;       // StatsMode (combine)
  int base2;            // LSEs are base-2 (combine)
  int channels;         // channels used by this call (<= max channels of the layout)
  int recv_warps;       // receiver warps per CTA
  int group_warps;      // combine: receiver warps that share one entry (each polls a subset of peers)
  int rounds_per_publish;  // 0: publish consumed counts only at the end of the call
  // Optional device timeline (HELIX_A2A_EXCHANGE_TRACE=1): [ranks_in_launch][channels][8] %globaltimer stamps per
  // CTA: kernel entry, after the wait on the previous kernel, first line posted, last line posted, first message
  // complete, last message complete, exit (0: the CTA never got there).  null: no tracing.
  unsigned long long* trace;
  // debug bounds checks (bounds.cuh): byte extents of one rank's tensors, 0 = not recorded
  int64_t o_src_bytes, st_src_bytes, o_dst_bytes, st_dst_bytes;
  int debug_checks;         // check every message's source / destination span against the extents
  uint32_t skip_peer_mask;  // debug / fault tests: sender silently skips these peers
  unsigned long long timeout_ns;
};

struct LaunchInfo {
  int channels;
  int send_warps;
  int recv_warps;
  int group_warps;
  int lines_per_message;
  int iters;            // warp iterations per message (4 lines each)
  int cooperative;
};

int max_channel_count(int cp_size, int sm_count);            // rings per (row, sender)
int64_t workspace_bytes_per_rank(int cp_size, int sm_count);
int device_sm_count();                                       // current device

// Fills the rings of the local row with 0xFF and zeroes info + status (two memsets).
cudaError_t initialize_workspace_row(uint64_t* local_row, int cp_size, int sm_count, cudaStream_t stream);

// Chooses channels / warps for a call (auto-tuner); `channel_override` > 0 pins the channel count.
LaunchInfo plan_launch(const ExchangeParams& p, int channel_override);

// Launches the kernel.  `pdl` adds the programmatic-stream-serialization attribute.
cudaError_t launch_exchange(ExchangeParams p, int channel_override, bool pdl, cudaStream_t stream,
                            LaunchInfo* info_out);

}  // namespace helix
