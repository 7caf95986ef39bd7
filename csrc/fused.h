// One kernel for exchange + LSE combine + o_proj: host interface.
#pragma once

#include "exchange.h"
#include "oproj.h"

namespace helix {

constexpr int kFusedMaxRanks = 4;   // ranks one launch can play in single-process emulation

struct FusedParams {
  ExchangeParams ex;                 // combine mode, native layout; o_dst is the x buffer of the GEMM
  OprojParams gemm[kFusedMaxRanks];  // per emulated rank (index 0 in multi-process use); split-K only without emulation
  int exchange_ctas;                 // CTAs [0, exchange_ctas) exchange, the rest run the GEMM
  int gemm_ctas;                     // hidden / 128 * splits
};

// Launches the fused kernel; returns cudaErrorNotSupported when the GEMM slabs plus at least one
// exchange channel do not fit on the device at once (callers then run the two kernels separately).
cudaError_t launch_exchange_oproj(FusedParams fp, int channel_override, bool pdl, cudaStream_t stream,
                                  LaunchInfo* info_out);

}  // namespace helix
