// o_proj GEMM for decode on B200: y[tokens, hidden] = x[tokens, K] * W[hidden, K]^T  (bf16 in, fp32
// accumulate in TMEM, bf16 out).  In the reference this layer is vLLM's cuBLAS linear; here it is a
// hand-written tcgen05 kernel so that it can chain to the exchange by programmatic dependent launch
// and stream its weights while the exchange is still in flight.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace helix {

struct OprojParams {
  CUtensorMap w_map;     // 2-D (K, hidden), box (64, 128), SWIZZLE_128B
  CUtensorMap x_map;     // 2-D (K, tokens), box (64, n_pad), SWIZZLE_128B
  __nv_bfloat16* y;      // [tokens, hidden]
  int64_t y_stride;      // elements between token rows
  float* partial;        // scratch [m_tiles][splits][n_pad][128] fp32 (splits > 1)
  int* counters;         // scratch [m_tiles], zero on entry and on exit
  int* error_flag;
  int tokens, n_pad, hidden, K, splits, stages, atoms;   // atoms: 64-wide K atoms per stage (1, 2 or 4)
  // Optional pre-packed weights (plain kernel only): per 128-row slab, K / 64 atoms (padded to a multiple of 4)
  // of 16 KB each, every atom already in the 128-byte-swizzled K-major layout the tensor core reads.  A stage
  // is then ONE contiguous bulk copy instead of `atoms` strided tensor copies.  nullptr: use w_map.
  const uint8_t* w_packed;
  int packed_atoms;      // atoms per slab in w_packed (K / 64 rounded up to a multiple of 4)
  int ctas;              // stream-K variant only: CTAs of the launch (splits is ignored there)
  unsigned long long* trace;   // stream-K variant, optional [ctas][8] %globaltimer stamps: entry, set-up done,
                               // first stage landed, last MMA issued, accumulator complete, exit
  unsigned long long timeout_ns;
};

inline size_t oproj_partial_bytes(int hidden, int splits, int n_pad) {
  return (size_t)(hidden / 128) * splits * n_pad * 128 * sizeof(float);
}
int oproj_pick_splits(int hidden, int K, int sm_count);
int oproj_pick_stages(int n_pad);
int oproj_pick_atoms(int n_pad);
int oproj_smem_bytes(int n_pad, int stages);

cudaError_t launch_oproj(const OprojParams& p, bool pdl, cudaStream_t stream);
inline int oproj_packed_atoms(int K) { return ((K + 63) / 64 + 3) / 4 * 4; }
inline size_t oproj_packed_bytes(int hidden, int K) { return (size_t)(hidden / 128) * oproj_packed_atoms(K) * 16384; }

// Stream-K variant: the (slab, k-block) units are dealt evenly to one CTA per SM, so every SM streams the same
// share of W whatever hidden / 128 is.  Scratch: partial [ctas][2][n_pad][128] fp32, counters [hidden / 128].
inline size_t oproj_streamk_partial_floats(int ctas, int n_pad) { return (size_t)ctas * 2 * n_pad * 128; }
bool oproj_streamk_pays(int hidden, int K, int n_pad, int sm_count);
cudaError_t launch_oproj_streamk(const OprojParams& p, bool pdl, cudaStream_t stream);

}  // namespace helix
