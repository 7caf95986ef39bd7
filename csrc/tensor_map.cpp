#include "tensor_map.h"

#include <mutex>

namespace helix {
namespace {
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn g_encode = nullptr;
std::once_flag g_once;
}  // namespace

bool encode_tensor_map(CUtensorMap* out, CUtensorMapDataType dtype, int rank, const void* base,
                       const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                       TmaSwizzle swizzle, const char** err) {
  std::call_once(g_once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeFn>(p);
  });
  if (!g_encode) {
    if (err) *err = "cuTensorMapEncodeTiled is not available";
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    if (err) *err = "TMA base address must be 16-byte aligned";
    return false;
  }
  cuuint64_t gdims[4];
  cuuint64_t gstrides[3];
  cuuint32_t gbox[4], estr[4];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) {
      gstrides[i] = strides_bytes[i];
      if (gstrides[i] % 16 != 0) {
        if (err) *err = "TMA strides must be multiples of 16 bytes";
        return false;
      }
    }
  }
  CUresult r = g_encode(out, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle == TmaSwizzle::k128B ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (err) *err = "cuTensorMapEncodeTiled failed";
    return false;
  }
  return true;
}

}  // namespace helix
