// Helix exchange kernel for B200 (sm_100a) and its host launcher / auto-tuner.
//
// Kernel: head-scatter all-to-all of split-KV partial attention outputs + fp32 softmax
// stats, with the LSE-weighted combine fused into the receive side (device code in
// exchange_device.cuh).  One CTA per channel; warps [0, NS) are senders (one per remote
// peer), the rest receivers.  One launch may play several ranks (blockIdx.y) when all
// workspace rows live in one process: that is how the multi-rank protocol is exercised on a
// single GPU (cooperative launch, all CTAs co-resident).
//
// Host: workspace sizing / initialisation, channel + warp-count auto-tuner and the launcher
// (counterparts of csrc/helix_alltoall.cu:486-644 in the reference).
#include "exchange.h"

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "exchange_device.cuh"

namespace helix {
namespace {

using namespace dev;

template <bool COMBINE, bool BF16, int NIT>
__global__ void __launch_bounds__(512, 1) helix_exchange_kernel(const __grid_constant__ ExchangeParams p) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  __shared__ Control ctl;

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int NR = p.recv_warps;
  const int NS = (int)(blockDim.x >> 5) - NR;
  const int rank = p.rank_base + blockIdx.y;
  const RankIO& io = p.io[blockIdx.y];

  unsigned long long* tr = p.trace ? p.trace + ((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 : nullptr;
  init_control(&ctl);
  if (threadIdx.x == 0) {
    if (tr) {
      tr[0] = globaltimer_ns();
      for (int i = 1; i < 8; ++i) tr[i] = 0;
    }
  }
  __syncthreads();
  // With programmatic dependent launch the inputs (the attention kernel's outputs) are only
  // guaranteed visible after this wait; without it the instruction is a no-op.
  pdl_wait();
  pdl_launch_dependents();
  Ctx cx = make_ctx(p, &ctl, rank, blockIdx.x);
  cx.deadline = globaltimer_ns() + p.timeout_ns;
  cx.trace = tr;
  if (tr && threadIdx.x == 0) tr[1] = globaltimer_ns();

  if (warp < NS) {
    sender_warp<NIT>(p, cx, io, warp, NS, lane);
  } else if (COMBINE) {
    receiver_combine_warp<BF16, NIT>(p, cx, io, warp - NS, NR, lane, reinterpret_cast<float*>(dyn_smem), NoHook());
  } else {
    receiver_exchange_warp<NIT>(p, cx, io, warp - NS, NR, lane);
  }
  if (tr) {
    __syncthreads();
    if (threadIdx.x == 0) tr[6] = globaltimer_ns();
  }
}

using KernelFn = void (*)(ExchangeParams);

template <int NIT>
KernelFn pick_combine(bool bf16) {
  return bf16 ? (KernelFn)helix_exchange_kernel<true, true, NIT> : (KernelFn)helix_exchange_kernel<true, false, NIT>;
}

// kernel instance + compile-time iteration count for a call
struct Variant {
  KernelFn fn;
  int nit;
};

Variant pick_variant(const ExchangeParams& p, int iters) {
  if (p.mode == kModeCombine) {
    if (iters <= 1) return {pick_combine<1>(p.is_bf16), 1};
    if (iters <= 2) return {pick_combine<2>(p.is_bf16), 2};
    if (iters <= 3) return {pick_combine<3>(p.is_bf16), 3};
    if (iters <= 5) return {pick_combine<5>(p.is_bf16), 5};
    if (iters <= 9) return {pick_combine<9>(p.is_bf16), 9};
    return {nullptr, 0};
  }
  if (iters <= 1) return {(KernelFn)helix_exchange_kernel<false, true, 1>, 1};
  return {(KernelFn)helix_exchange_kernel<false, true, 3>, 3};  // larger messages go in slabs of 3
}

size_t group_smem_bytes(int nit, int recv_warps, int group_warps) {
  if (group_warps <= 1) return 0;
  int groups = recv_warps / group_warps;
  return (size_t)groups * 2 * (group_warps - 1) * (nit * 8 * 32 + 4) * sizeof(float);
}

struct OccKey {
  const void* fn;
  int threads;
  size_t smem;
  int dev;
  bool operator==(const OccKey& o) const { return fn == o.fn && threads == o.threads && smem == o.smem && dev == o.dev; }
};
struct OccHash {
  size_t operator()(const OccKey& k) const {
    return std::hash<const void*>()(k.fn) ^ (size_t)k.threads * 1315423911u ^ k.smem * 2654435761u ^ (size_t)k.dev;
  }
};

// CTAs of `fn` that can be resident on the whole device at once (cached)
int resident_ctas(KernelFn fn, int threads, size_t smem) {
  static std::mutex mu;
  static std::unordered_map<OccKey, int, OccHash> cache;
  int dev = 0;
  cudaGetDevice(&dev);
  OccKey key{(const void*)fn, threads, smem, dev};
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  if (smem > 48 * 1024) cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  int per_sm = 0, sms = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, threads, smem) != cudaSuccess) per_sm = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int total = per_sm * sms;
  cache[key] = total;
  return total;
}

}  // namespace

// ================================================================================================
int device_sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 148;
  if (dev < 64 && cached[dev] > 0) return cached[dev];
  int sms = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  if (dev < 64) cached[dev] = sms;
  return sms;
}

int max_channel_count(int cp_size, int sm_count) { return make_layout(cp_size, sm_count).max_channels; }

int64_t workspace_bytes_per_rank(int cp_size, int sm_count) { return make_layout(cp_size, sm_count).row_bytes; }

cudaError_t initialize_workspace_row(uint64_t* local_row, int cp_size, int sm_count, cudaStream_t stream) {
  WorkspaceLayout lay = make_layout(cp_size, sm_count);
  // Rings all-ones: no valid flag (sequence + 1) ever equals 2^64 - 1.  Counters and status zero.
  cudaError_t err = cudaMemsetAsync(local_row, 0xFF, (size_t)lay.ring_region, stream);
  if (err != cudaSuccess) return err;
  return cudaMemsetAsync(reinterpret_cast<uint8_t*>(local_row) + lay.ring_region, 0,
                         (size_t)(lay.row_bytes - lay.ring_region), stream);
}

// Auto-tuner.  The reference derives the channel count from the SM count alone
// (csrc/helix_alltoall.cu:524-530); for decode the right count depends on how many entries
// a call carries: few entries -> one entry per channel and several warps per entry (latency),
// many entries -> one channel per SM and one warp per entry (bandwidth).
// lines one channel moves per call from which the warps of a CTA are re-balanced towards receiving (measured at
// two ranks: 192, 96, 48 and 24 lines are each at least as good as the next larger value for the calls they add)
constexpr int kBulkLinesPerChannelDefault = 24;
static int bulk_lines_per_channel() {
  if (const char* v = std::getenv("HELIX_A2A_BULK_LINES")) return std::max(1, std::atoi(v));
  return kBulkLinesPerChannelDefault;
}

LaunchInfo plan_launch(const ExchangeParams& p, int channel_override) {
  LaunchInfo li{};
  const int N = p.cp_size;
  const int E = p.outer * p.inner;
  const int payload_words = p.st_words + p.o_bytes / 8;
  const int L = ll128::lines_for_words(payload_words);
  li.lines_per_message = L;
  li.iters = ceil_div(L, 4);
  li.cooperative = p.ranks_in_launch > 1;
  // up to 8 sender warps: with few peers several warps share a peer
  li.send_warps = N <= 1 ? 1 : (N - 1 <= 8 ? (N - 1) * (8 / (N - 1)) : 8);
  const int max_c = max_channel_count(N, p.sm_count);

  int channels = std::min(max_c, std::max(E, 1));
  if (channel_override > 0) channels = std::min(channel_override, max_c);
  const int per_channel = ceil_div(std::max(E, 1), channels);

  int group = 1, recv;
  if (p.mode == kModeCombine) {
    // few entries per channel: let up to 4 warps share an entry, each polling a subset of peers
    if (per_channel <= 2 && N > 2 && li.iters <= 3) group = std::min(4, N - 1);
    int max_recv = kMaxRecvWarps;
    if (N > 1 && (int64_t)per_channel * L >= bulk_lines_per_channel()) {
      // Many lines per channel: the call is bound by throughput, and the receive side (own row, poll, combine,
      // store: one message per warp at a time) is the slower one; the senders keep up with fewer warps.  Of the 16
      // warps of a CTA 4 (two ranks; measured best of 1..7 there: MLA rows, 256 tokens, 35 us against 45 with 6 and
      // 55 with 2) or about 6 (more ranks: at least one per peer) send and the rest receive.
      // HELIX_A2A_BULK_SEND_WARPS / HELIX_A2A_BULK_LINES override the two numbers for experiments.
      int bulk_send = N == 2 ? 4 : 6;
      if (const char* v = std::getenv("HELIX_A2A_BULK_SEND_WARPS")) bulk_send = std::max(1, std::min(12, std::atoi(v)));
      li.send_warps = (N - 1) * std::max(1, bulk_send / (N - 1));
      max_recv = 16 - li.send_warps;
    }
    int groups = std::max(1, std::min(per_channel, max_recv / group));
    if (group > 1) groups = std::min(groups, 2);
    recv = groups * group;
  } else {
    recv = std::max(1, std::min(kMaxRecvWarps, per_channel * N));
  }
  li.group_warps = group;
  li.recv_warps = recv;
  li.channels = channels;
  return li;
}

cudaError_t launch_exchange(ExchangeParams p, int channel_override, bool pdl, cudaStream_t stream,
                            LaunchInfo* info_out) {
  const int E = p.outer * p.inner;
  if (E <= 0) return cudaSuccess;
  if (p.cp_size < 1 || p.cp_size > kMaxCp || p.ranks_in_launch < 1 || p.ranks_in_launch > kMaxEmulatedRanks)
    return cudaErrorInvalidValue;
  LaunchInfo li = plan_launch(p, channel_override);
  Variant var = pick_variant(p, li.iters);
  if (var.fn == nullptr) return cudaErrorInvalidValue;

  int threads = 32 * (li.send_warps + li.recv_warps);
  size_t smem = p.mode == kModeCombine ? group_smem_bytes(var.nit, li.recv_warps, li.group_warps) : 0;
  // every CTA of every rank in the launch must be resident at once
  int capacity = resident_ctas(var.fn, threads, smem);
  if (capacity <= 0) return cudaErrorLaunchOutOfResources;
  int cap_channels = capacity / p.ranks_in_launch;
  if (cap_channels < 1) return cudaErrorLaunchOutOfResources;
  li.channels = std::min(li.channels, cap_channels);

  p.channels = li.channels;
  p.recv_warps = li.recv_warps;
  p.group_warps = li.group_warps;
  // in-call flow control only when one call can fill more than half a ring
  const int L = li.lines_per_message;
  const int per_channel = ceil_div(E, li.channels);
  if ((int64_t)per_channel * L <= kRingLines / 2) {
    p.rounds_per_publish = 0;
  } else {
    // publish whenever about a quarter of a ring has been drained since the last publish.
    // combine: a round consumes recv/group entries; exchange: recv items, i.e. recv/N entries
    if (p.mode == kModeCombine) {
      int entries_per_round = li.recv_warps / li.group_warps;
      p.rounds_per_publish = std::max(1, (kRingLines / 4) / (entries_per_round * L));
    } else {
      p.rounds_per_publish = std::max(1, (kRingLines / 4) * p.cp_size / (li.recv_warps * L));
    }
  }
  if (L > kRingLines / 8) return cudaErrorInvalidValue;  // one message must be a small part of a ring

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(li.channels, p.ranks_in_launch, 1);
  cfg.blockDim = dim3(threads, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (pdl && !li.cooperative) {  // the single-process emulation launch is cooperative and never chained
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  if (li.cooperative) {
    attrs[na].id = cudaLaunchAttributeCooperative;
    attrs[na].val.cooperative = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  if (info_out) *info_out = li;
  return cudaLaunchKernelEx(&cfg, var.fn, p);
}

}  // namespace helix
