// Stand-alone LSE-weighted combine for B200: [N, rows, D] partial outputs + [N, rows] LSEs -> [rows, D].
//
//   out[r, :] = sum_n w_n o_n[r, :] / sum_n w_n,   w_n = exp(lse_n[r] - max_n lse_n[r])
//
// The fused exchange applies this as the lines land; this kernel is for callers that already hold every
// rank's rows: users of the plain `alltoall`, and the NCCL path of the vLLM hook.  Counterpart of the
// reference's Triton kernel (patches/dcp_alltoall_helix.py:210-384), with its rules: NaN and +-inf LSEs count
// as -inf (no contribution), a row whose LSEs are all -inf comes out as zeros with a global LSE of -inf,
// base e or base 2.  One warp per row, the online accumulator of the exchange's receive side in registers,
// 16-byte loads; a row is read once and never staged.
#include "lse_combine.h"

#include "exchange_device.cuh"

namespace helix {
namespace {

using namespace dev;

constexpr int kWarpsPerCta = 4;

template <bool BF16, int NIT>
__global__ void __launch_bounds__(kWarpsPerCta * 32) lse_combine_kernel(const __grid_constant__ LseCombineParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarpsPerCta + (threadIdx.x >> 5);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (row >= p.rows) return;
  const int nchunks = p.row_bytes >> 4;
  Acc<NIT> acc;
  acc.init();
  for (int n = 0; n < p.n; ++n) {
    const float raw = *reinterpret_cast<const float*>(p.lse + n * p.l_sn + row * p.l_sr);
    float l = p.base2 ? raw : raw * kLog2e;
    if (!(fabsf(l) <= 3.0e38f)) l = -INFINITY;
    if (l == -INFINITY) continue;   // warp-uniform: the row is not even read
    const uint8_t* src = p.o + n * p.o_sn + row * p.o_sr;
    uint64_t lo[NIT], hi[NIT];
#pragma unroll
    for (int it = 0; it < NIT; ++it) {
      const int ch = it * 32 + lane;
      lo[it] = hi[it] = 0ull;
      if (ch < nchunks) {
        const uint4 v = *reinterpret_cast<const uint4*>(src + 16 * ch);
        lo[it] = (uint64_t)v.x | ((uint64_t)v.y << 32);
        hi[it] = (uint64_t)v.z | ((uint64_t)v.w << 32);
      }
    }
    acc.template add<BF16>(l, lo, hi);
  }
  const float inv = acc.s > 0.f ? 1.0f / acc.s : 0.f;
  uint8_t* dst = p.out + row * p.out_sr;
#pragma unroll
  for (int it = 0; it < NIT; ++it) {
    const int ch = it * 32 + lane;
    if (ch < nchunks) {
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = acc.v[it][j] * inv;
      const uint64_t a = pack4<BF16>(f), b = pack4<BF16>(f + 4);
      uint4 v;
      v.x = (uint32_t)a;
      v.y = (uint32_t)(a >> 32);
      v.z = (uint32_t)b;
      v.w = (uint32_t)(b >> 32);
      *reinterpret_cast<uint4*>(dst + 16 * ch) = v;
    }
  }
  if (p.lse_out != nullptr && lane == 0) {
    float gl = acc.s > 0.f ? (acc.m + log2f(acc.s)) : -INFINITY;
    if (!p.base2) gl *= kLn2;
    p.lse_out[row] = gl;
  }
}

using Fn = void (*)(LseCombineParams);
template <int NIT>
Fn pick(bool bf16) {
  return bf16 ? (Fn)lse_combine_kernel<true, NIT> : (Fn)lse_combine_kernel<false, NIT>;
}

}  // namespace

cudaError_t launch_lse_combine(const LseCombineParams& p, bool pdl, cudaStream_t stream) {
  if (p.rows <= 0 || p.n <= 0) return cudaSuccess;
  if (p.row_bytes <= 0 || p.row_bytes % 16 != 0 || p.row_bytes > 4 * 32 * 16) return cudaErrorInvalidValue;
  const int chunks = p.row_bytes / 16;
  Fn fn = chunks <= 32 ? pick<1>(p.is_bf16) : chunks <= 64 ? pick<2>(p.is_bf16) : pick<4>(p.is_bf16);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)((p.rows + kWarpsPerCta - 1) / kWarpsPerCta), 1, 1);
  cfg.blockDim = dim3(kWarpsPerCta * 32, 1, 1);
  cfg.stream = stream;
  cudaLaunchAttribute attrs[1];
  int na = 0;
  if (pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, fn, p);
}

}  // namespace helix
