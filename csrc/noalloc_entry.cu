// Allocation-free entry point for the GQA decode attention (declaration and rationale in
// helix_noalloc.h).  It reuses the library's attention kernel unchanged; only the scratch memory
// differs: instead of buffers from a caller's allocator it is the file-scope device array below.
#include "helix_noalloc.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "attention.h"
#include "exchange.h"
#include "tensor_map.h"

namespace {

// Layout of the built-in scratch (bytes):
//   [0, kPartO)                    partial outputs   [MAX_CTAS][2][8][128] fp32
//   [kPartO, kPartO + kPartL)      partial LSEs      [MAX_CTAS][2][8]      fp32
//   then                           arrival counters  [MAX_PAIRS]           int32   (must be zero at launch)
//   then                           error word        int32 (+ padding)             (must be zero at launch)
constexpr size_t kPartO = (size_t)HELIX_NOALLOC_MAX_CTAS * 2 * 8 * 128 * sizeof(float);
constexpr size_t kPartL = (size_t)HELIX_NOALLOC_MAX_CTAS * 2 * 8 * sizeof(float);
constexpr size_t kCounters = (size_t)HELIX_NOALLOC_MAX_PAIRS * sizeof(int);
constexpr size_t kErr = 256;
constexpr size_t kScratchBytes = kPartO + kPartL + kCounters + kErr;
static_assert(HELIX_NOALLOC_MAX_CTAS <= helix::kGqaMaxCtas, "the kernel's grid bound sizes the piece slots");
static_assert(kPartO == helix::gqa_part_o_floats(HELIX_NOALLOC_MAX_CTAS, 0) * sizeof(float) &&
                  kPartL == helix::gqa_part_lse_floats(HELIX_NOALLOC_MAX_CTAS, 0) * sizeof(float),
              "scratch layout must match what the kernel indexes");

// The scratch itself.  In host code this name is only a handle for the runtime: its device address
// is obtained with cudaGetSymbolAddress below and that pointer is what the kernel receives.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct DeviceState {
  bool ready = false;
  unsigned char* base = nullptr;
  int sm_count = 0;
};
DeviceState g_state[64];
std::mutex g_mu;
thread_local char g_err[256] = "";

int fail_cuda(cudaError_t e, const char* what) {
  snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
  return kHelixNoAllocCudaError;
}

// One-time set-up for the current device: device address of the scratch array, SM count.
int setup_current_device(DeviceState** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail_cuda(e, "cudaGetDevice");
  if (dev < 0 || dev >= 64) {
    snprintf(g_err, sizeof(g_err), "device index %d out of range", dev);
    return kHelixNoAllocBadArgument;
  }
  std::lock_guard<std::mutex> lk(g_mu);
  DeviceState& st = g_state[dev];
  if (!st.ready) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress(scratch)");
    int sms = 0;
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return fail_cuda(e, "cudaDeviceGetAttribute");
    st.base = static_cast<unsigned char*>(ptr);
    st.sm_count = sms;
    st.ready = true;
  }
  *out = &st;
  return kHelixNoAllocOk;
}

bool make_cache_map(CUtensorMap* m, const void* cache, int64_t pages, int kv_heads, int page_size, int64_t s_page,
                    int64_t s_head, int64_t s_tok) {
  uint64_t dims[4] = {128, (uint64_t)page_size, (uint64_t)kv_heads, (uint64_t)pages};
  uint64_t strides[3] = {(uint64_t)s_tok * 2, (uint64_t)s_head * 2, (uint64_t)s_page * 2};
  uint32_t box[4] = {64, 16, 1, 1};
  const char* err = nullptr;
  if (!helix::encode_tensor_map(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, cache, dims, strides, box,
                                helix::TmaSwizzle::k128B, &err)) {
    snprintf(g_err, sizeof(g_err), "KV cache descriptor: %s", err ? err : "?");
    return false;
  }
  return true;
}

}  // namespace

extern "C" __attribute__((visibility("default"))) int helix_gqa_decode_noalloc(
    const void* q, int64_t q_stride_batch, int64_t q_stride_head, const void* k_cache, const void* v_cache,
    int64_t num_pages, int64_t cache_stride_page, int64_t cache_stride_head, int64_t cache_stride_token,
    const int32_t* block_table, int64_t block_table_stride, const int32_t* seq_lens, void* o, float* lse, int batch,
    int q_heads, int kv_heads, int page_size, int max_seq_len, float scale, int lse_base2, void* stream) {
  g_err[0] = 0;
  if (batch == 0) return kHelixNoAllocOk;
  if (!q || !k_cache || !v_cache || !block_table || !seq_lens || !o || !lse || batch < 0 || kv_heads <= 0 ||
      q_heads <= 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > 8 || page_size <= 0 || page_size % 16 != 0 ||
      num_pages <= 0) {
    snprintf(g_err, sizeof(g_err), "bad argument (null pointer, group > 8 or page size not a multiple of 16)");
    return kHelixNoAllocBadArgument;
  }
  if ((int64_t)batch * kv_heads > HELIX_NOALLOC_MAX_PAIRS) {
    snprintf(g_err, sizeof(g_err), "batch * kv_heads = %lld exceeds the built-in scratch (max %d)",
             (long long)batch * kv_heads, HELIX_NOALLOC_MAX_PAIRS);
    return kHelixNoAllocTooLarge;
  }
  DeviceState* st = nullptr;
  int rc = setup_current_device(&st);
  if (rc != kHelixNoAllocOk) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  helix::GqaDecodeParams p{};
  if (!make_cache_map(&p.k_map, k_cache, num_pages, kv_heads, page_size, cache_stride_page, cache_stride_head,
                      cache_stride_token) ||
      !make_cache_map(&p.v_map, v_cache, num_pages, kv_heads, page_size, cache_stride_page, cache_stride_head,
                      cache_stride_token))
    return kHelixNoAllocBadArgument;
  int ctas = helix::gqa_pick_ctas(batch, kv_heads, max_seq_len > 0 ? max_seq_len : 1, st->sm_count);
  if (ctas > HELIX_NOALLOC_MAX_CTAS) ctas = HELIX_NOALLOC_MAX_CTAS;
  unsigned char* base = st->base;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride_b = q_stride_batch;
  p.q_stride_h = q_stride_head;
  p.block_table = block_table;
  p.bt_stride = block_table_stride;
  p.seq_lens = seq_lens;
  p.o = static_cast<__nv_bfloat16*>(o);
  p.lse = lse;
  p.part_o = reinterpret_cast<float*>(base);
  p.part_lse = reinterpret_cast<float*>(base + kPartO);
  p.counters = reinterpret_cast<int*>(base + kPartO + kPartL);
  p.error_flag = reinterpret_cast<int*>(base + kPartO + kPartL + kCounters);
  p.trace = nullptr;
  p.B = batch;
  p.Hq = q_heads;
  p.Hkv = kv_heads;
  p.page_size = page_size;
  p.ctas = ctas;
  // fixed shares only: the dynamic tail of the kernel needs more scratch than this array has
  p.dyn_pct = 0;
  p.dyn_chunk = 0;
  p.dyn_min_blocks = 0;
  p.max_helper = 0;
  p.scale = scale;
  p.lse_base2 = lse_base2 ? 1 : 0;
  p.timeout_ns = 2000000000ull;
  // the array keeps the previous call's contents: counters and the error word must start at zero
  cudaError_t e = cudaMemsetAsync(p.counters, 0, (size_t)batch * kv_heads * sizeof(int), s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(counters)");
  e = cudaMemsetAsync(p.error_flag, 0, sizeof(int), s);
  if (e != cudaSuccess) return fail_cuda(e, "cudaMemsetAsync(error word)");
  e = helix::launch_gqa_decode(p, false, s);
  if (e != cudaSuccess) return fail_cuda(e, "kernel launch");
  return kHelixNoAllocOk;
}

extern "C" __attribute__((visibility("default"))) int helix_noalloc_read_error(void* stream) {
  DeviceState* st = nullptr;
  if (setup_current_device(&st) != kHelixNoAllocOk) return -1;
  int v = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&v, st->base + kPartO + kPartL + kCounters, sizeof(int), cudaMemcpyDeviceToHost, s) !=
          cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess)
    return -1;
  return v;
}

extern "C" __attribute__((visibility("default"))) const char* helix_noalloc_last_error(void) { return g_err; }
