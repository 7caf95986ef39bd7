// Helix exchange + LSE combine + o_proj in ONE kernel (sm_100a).
//
// The grid is split by role.  CTAs [0, C) run the exchange: sender warps post LL128 lines of the
// attention output into the peers' rings over NVLink, receiver warps poll the local rings, apply the
// LSE-weighted combine and write the combined activation rows x[B, K] (bf16, L2 resident); after
// each row they bump a "rows ready" counter in the local workspace row.  CTAs [C, C + hidden/128)
// run the o_proj GEMM on tcgen05: each owns one 128-row slab of W_o, starts streaming it with TMA
// right away (the weights do not depend on the exchange), and only then waits for the counter to
// reach the number of rows before it fetches x with TMA and issues the UMMAs.  So the weight stream
// of a layer overlaps the NVLink exchange of the same layer inside one launch, and the combined tile
// goes from the receive warps to the tensor-core operand without a kernel boundary in between.
//
// All CTAs have to be resident at the same time (GEMM CTAs wait for exchange CTAs, which wait for
// other GPUs): the launcher sizes the grid to at most one CTA per SM and refuses shapes that do not
// fit.  Every wait is bounded (%globaltimer); on expiry the status block / error flag is set and the
// kernel returns.  No TMA load uses cluster broadcast; peer memory is only ever written with plain
// stores, never read.
#include "fused.h"

#include <algorithm>

#include "exchange_device.cuh"
#include "oproj_device.cuh"

namespace helix {
namespace {

using namespace dev;

constexpr int kReadyOff = 64;    // byte offsets inside the status block of the local row
constexpr int kGemmSeenOff = 72;
constexpr int kGemmBarrier = 2;  // named barrier of the 128 GEMM threads

struct ReadyHook {
  unsigned int* ready;
  HELIX_D void operator()(int /*e*/, int lane) const {
    __threadfence();          // the row's stores (all lanes) before the counter
    __syncwarp();
    if (lane == 0) atomicAdd(ready, 1u);
  }
};

template <bool BF16, int NIT>
__global__ void __launch_bounds__(512, 1) helix_exchange_oproj_kernel(const __grid_constant__ FusedParams fp) {
  extern __shared__ __align__(16) uint8_t dyn_smem[];
  __shared__ Control ctl;
  const ExchangeParams& p = fp.ex;
  const int rank = p.rank_base + blockIdx.y;
  uint8_t* my_row = reinterpret_cast<uint8_t*>(p.workspace) + (int64_t)rank * p.row_stride_bytes;
  const WorkspaceLayout lay = make_layout(p.cp_size, p.sm_count);
  unsigned int* ready = reinterpret_cast<unsigned int*>(my_row + lay.status_offset + kReadyOff);
  unsigned int* seen = reinterpret_cast<unsigned int*>(my_row + lay.status_offset + kGemmSeenOff);

  if ((int)blockIdx.x < fp.exchange_ctas) {
    // ------------------------------------------------------------------ exchange + combine role
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int NR = p.recv_warps;
    const int NS = (int)(blockDim.x >> 5) - NR;
    const RankIO& io = p.io[blockIdx.y];
    if (threadIdx.x == 0) {
      ctl.abort = 0;
      ctl.done = 0;
    }
    __syncthreads();
    pdl_wait();
    pdl_launch_dependents();
    Ctx cx = make_ctx(p, &ctl, rank, blockIdx.x);
    cx.deadline = globaltimer_ns() + p.timeout_ns;
    load_ring_heads(p, cx);
    if (warp < NS) {
      sender_warp<NIT>(p, cx, io, warp, NS, lane);
    } else {
      receiver_combine_warp<BF16, NIT>(p, cx, io, warp - NS, NR, lane, reinterpret_cast<float*>(dyn_smem),
                                       ReadyHook{ready});
    }
    return;
  }

  // ---------------------------------------------------------------------- o_proj role
  if (threadIdx.x >= oproj_dev::kThreads) return;
  pdl_launch_dependents();
  const OprojParams& gp = fp.gemm[blockIdx.y];
  const unsigned int rows = (unsigned int)(p.outer * p.inner);
  const unsigned int n_gemm = (unsigned int)fp.gemm_ctas;
  const int gidx = (int)blockIdx.x - fp.exchange_ctas;
  oproj_dev::oproj_cta(
      gp, dyn_smem, gidx / gp.splits, gidx % gp.splits, threadIdx.x,
      [] { named_barrier(kGemmBarrier, oproj_dev::kThreads); },
      [&](unsigned long long deadline) {
        // The counters below are shared by all launches and re-armed by the previous one: under programmatic
        // launch this CTA may be resident while that launch still runs, so wait for it first (x depends on the
        // kernel before us anyway; the weight stages were requested above).
        pdl_wait();
        // rows written by the combine warps (generic proxy, other SMs) must be complete before TMA reads them
        unsigned spins = 0;
        while (true) {
          unsigned int v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ready) : "memory");
          if (v >= rows) break;
          if ((++spins & 63u) == 0u) {
            const StatusBlock* sb = reinterpret_cast<const StatusBlock*>(my_row + lay.status_offset);
            if (ld_volatile_8(&sb->code) != 0ull || sm100::now_ns() > deadline) {
              StatusBlock* wsb = reinterpret_cast<StatusBlock*>(my_row + lay.status_offset);
              atomicCAS(&wsb->code, 0ull, (unsigned long long)kTimeoutGemmInput);
              return false;
            }
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        // the last GEMM CTA to get here re-arms both counters for the next launch
        if (atomicAdd(seen, 1u) == n_gemm - 1u) {
          *reinterpret_cast<volatile unsigned int*>(seen) = 0u;
          *reinterpret_cast<volatile unsigned int*>(ready) = 0u;
        }
        return true;
      });
}

using FusedFn = void (*)(FusedParams);

template <int NIT>
FusedFn pick(bool bf16) {
  return bf16 ? (FusedFn)helix_exchange_oproj_kernel<true, NIT> : (FusedFn)helix_exchange_oproj_kernel<false, NIT>;
}

}  // namespace

cudaError_t launch_exchange_oproj(FusedParams fp, int channel_override, bool pdl, cudaStream_t stream,
                                  LaunchInfo* info_out) {
  ExchangeParams& p = fp.ex;
  const int E = p.outer * p.inner;
  if (E <= 0) return cudaSuccess;
  if (p.mode != kModeCombine || p.ranks_in_launch < 1 || p.ranks_in_launch > kFusedMaxRanks) return cudaErrorInvalidValue;
  for (int r = 0; r < p.ranks_in_launch; ++r)
    if (fp.gemm[r].splits < 1 || (fp.gemm[r].splits > 1 && (fp.gemm[r].partial == nullptr || p.ranks_in_launch > 1)))
      return cudaErrorInvalidValue;
  LaunchInfo li = plan_launch(p, channel_override);
  FusedFn fn = nullptr;
  int nit = 0;
  if (li.iters <= 1) { fn = pick<1>(p.is_bf16); nit = 1; }
  else if (li.iters <= 2) { fn = pick<2>(p.is_bf16); nit = 2; }
  else if (li.iters <= 3) { fn = pick<3>(p.is_bf16); nit = 3; }
  else if (li.iters <= 5) { fn = pick<5>(p.is_bf16); nit = 5; }
  else return cudaErrorNotSupported;

  const int threads = 32 * (li.send_warps + li.recv_warps);
  size_t smem_ex = li.group_warps > 1
                       ? (size_t)(li.recv_warps / li.group_warps) * 2 * (li.group_warps - 1) * (nit * 8 * 32 + 4) * sizeof(float)
                       : 0;
  size_t smem = std::max<size_t>(smem_ex, (size_t)oproj_smem_bytes(fp.gemm[0].n_pad, fp.gemm[0].stages));
  cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  int per_sm = 0, sms = p.sm_count;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, std::max(threads, 128), smem);
  if (e != cudaSuccess) return e;
  const int capacity = per_sm * sms / p.ranks_in_launch;     // CTAs one rank may use
  const int gemm_ctas = fp.gemm[0].hidden / 128 * fp.gemm[0].splits;
  if (capacity - gemm_ctas < 1) return cudaErrorNotSupported;
  li.channels = std::min(li.channels, capacity - gemm_ctas);

  p.channels = li.channels;
  p.recv_warps = li.recv_warps;
  p.group_warps = li.group_warps;
  const int L = li.lines_per_message;
  const int per_channel = ceil_div(E, li.channels);
  if ((int64_t)per_channel * L <= kRingLines / 2) p.rounds_per_publish = 0;
  else p.rounds_per_publish = std::max(1, (kRingLines / 4) / ((li.recv_warps / li.group_warps) * L));
  if (L > kRingLines / 8) return cudaErrorInvalidValue;
  fp.exchange_ctas = li.channels;
  fp.gemm_ctas = gemm_ctas;

  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(li.channels + gemm_ctas, p.ranks_in_launch, 1);
  cfg.blockDim = dim3(std::max(threads, 128), 1, 1);
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
