// Decode o_proj GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulator in TMEM).
//
// Decode batches are small (1..256 tokens) while `hidden` is large, so the product is computed
// transposed ("swap-AB"): the 128-row UMMA M dimension walks `hidden` (rows of W), the token count
// is the UMMA N dimension (padded to a multiple of 16) and D[128, n_pad] fp32 lives in TMEM.  The
// kernel is bound by streaming W once from HBM:
//   grid (hidden / 128, splits); each CTA owns one 128-row slab of W and 1/splits of K;
//   warp 0 (one lane) feeds a ring of shared-memory stages with TMA tiled loads (128-byte swizzle,
//     four [128 x 64] W boxes + four [n_pad x 64] x boxes per stage, no cluster broadcast);
//   warp 1 (one lane) issues sixteen K=16 UMMAs per stage and releases the stage with
//     tcgen05.commit; after the last stage it commits to the accumulator barrier;
//   all four warps then read the accumulator with tcgen05.ld (warp w owns TMEM lanes 32w..32w+31)
//     and write y (bf16) or, with split-K, park an fp32 partial in scratch memory where the last
//     CTA of the slab sums the splits.
// With programmatic dependent launch the W tiles of the first stages are requested BEFORE the
// grid-dependency wait: only the activations depend on the preceding exchange kernel, so the
// weight stream overlaps it.  All mbarrier waits are bounded.
#include "oproj.h"

#include <algorithm>

#include "oproj_device.cuh"

namespace helix {
namespace {

using namespace oproj_dev;

__global__ void __launch_bounds__(kThreads, 1) oproj_kernel(const __grid_constant__ OprojParams p) {
  extern __shared__ uint8_t smem_raw[];
  oproj_cta(
      p, smem_raw, blockIdx.x, blockIdx.y, threadIdx.x, [] { __syncthreads(); },
      [](unsigned long long) {
        // with programmatic dependent launch the activations are valid once the preceding grid is done
        asm volatile("griddepcontrol.wait;" ::: "memory");
        return true;
      });
}

}  // namespace

int oproj_pick_atoms(int n_pad) { return n_pad <= 64 ? 4 : (n_pad <= 128 ? 2 : 1); }

int oproj_pick_splits(int hidden, int K, int sm_count) {
  // split K only when one CTA per 128-row slab would leave SMs idle for long: each CTA should still
  // stream at least 256 KB of W
  const int m_tiles = hidden / kBM;
  int splits = std::max(1, sm_count / std::max(m_tiles, 1));
  const int kb_total = (K + 255) / 256;
  while (splits > 1 && kb_total / splits < 4) --splits;
  return std::min(splits, 8);
}

int oproj_smem_bytes(int n_pad, int stages) {
  return stages * (kBM + n_pad) * kAtomK * oproj_pick_atoms(n_pad) * 2 + 1024;
}

int oproj_pick_stages(int n_pad) {
  const int stage = (kBM + n_pad) * kAtomK * oproj_pick_atoms(n_pad) * 2;
  int s = (222 * 1024) / stage;
  return std::max(2, std::min(s, kMaxStages));
}

cudaError_t launch_oproj(const OprojParams& p, bool pdl, cudaStream_t stream) {
  if (p.tokens <= 0) return cudaSuccess;
  if (p.hidden % kBM != 0 || p.K % kAtomK != 0 || p.n_pad % 16 != 0 || p.n_pad < 16 || p.n_pad > 256 ||
      p.tokens > p.n_pad || (p.atoms != 1 && p.atoms != 2 && p.atoms != 4) || p.stages < 2 || p.stages > kMaxStages || p.splits < 1)
    return cudaErrorInvalidValue;
  const int smem = oproj_smem_bytes(p.n_pad, p.stages);
  cudaError_t e = cudaFuncSetAttribute(oproj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(p.hidden / kBM, p.splits, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = smem;
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
  return cudaLaunchKernelEx(&cfg, oproj_kernel, p);
}

}  // namespace helix
