// Stand-alone LSE-weighted combine: host interface (kernel in lse_combine.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace helix {

struct LseCombineParams {
  const uint8_t* o;       // partial outputs: row r of rank n at o + n * o_sn + r * o_sr (bytes), row_bytes contiguous
  const uint8_t* lse;     // fp32 LSE of that row at lse + n * l_sn + r * l_sr (bytes)
  uint8_t* out;           // combined rows at out + r * out_sr
  float* lse_out;         // optional global LSE [rows] (null: not wanted)
  int64_t o_sn, o_sr, l_sn, l_sr, out_sr;
  int64_t rows;
  int n;                  // ranks
  int row_bytes;          // D * element size: a multiple of 16, at most 2048
  int is_bf16;            // else fp16
  int base2;              // LSEs are base 2 (else base e); the global LSE comes out in the same base
};

cudaError_t launch_lse_combine(const LseCombineParams& p, bool pdl, cudaStream_t stream);

}  // namespace helix
