// Host helper: build CUtensorMap descriptors for TMA tiled loads (driver entry point resolved at
// run time through the CUDA runtime, so nothing links against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace helix {

enum class TmaSwizzle { kNone, k128B };

// rank <= 4.  dims[0] is the innermost (contiguous) dimension; strides_bytes[i] is the stride of
// dims[i+1] (the innermost stride is the element size).  Returns false on failure (message in *err).
bool encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       TmaSwizzle swizzle, const char** err);

}  // namespace helix
