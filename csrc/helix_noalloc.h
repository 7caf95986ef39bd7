// Allocation-free C entry point for the paged GQA decode attention.
//
// This entry point has no counterpart in the reference (which ships no attention kernel and only
// a torch-bound exchange op, csrc/torch_binding.cpp:177-189).
//
// Who it is for: host programs that may not obtain device memory at the moment they need to run
// attention.  A serving engine typically hands every free byte of HBM to its paged KV cache when it
// starts, so a later cudaMalloc from a library it calls simply fails; an engine that routes all
// device memory through its own pool forbids libraries from calling the CUDA allocator behind its
// back; and a plain C / C++ / Rust host that links this library without PyTorch has no caching
// allocator to lean on at all.  Such callers own the inputs and outputs already.  What they cannot
// supply is the kernel's private scratch (per-CTA partial results and arrival counters of the
// split-KV merge), so here that scratch lives inside the library image.
//
// The scratch is ONE file-scope device array of fixed size (about 5.3 MB, see the limits below).
// Every GPU that loads the library carries it from load until the process ends.  All calls on a
// device share it, and it keeps whatever the previous call left behind: the entry point clears the
// parts that must start at zero (arrival counters, error word) on the caller's stream before each
// launch.  Because the array is shared, two calls whose kernels may overlap on the same GPU (for
// instance on different streams) race on it; callers must order such calls themselves.
//
// The first call on each device performs a one-time set-up (it resolves the device address of the
// array and raises the kernel's shared-memory limit).  Make that first call outside any stream
// capture; later calls only enqueue work on the given stream.
//
// The function never calls cudaMalloc, cudaFree or any allocating library routine.
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Limits of the built-in scratch.  Larger problems are rejected with kHelixNoAllocTooLarge.
#define HELIX_NOALLOC_MAX_PAIRS 4096   /* batch * kv_heads */
#define HELIX_NOALLOC_MAX_CTAS 640     /* CTAs of one launch (the library picks at most 2 per SM) */

enum HelixNoAllocStatus {
  kHelixNoAllocOk = 0,
  kHelixNoAllocBadArgument = 1,   // null pointer, unsupported head_dim / group / page size, misaligned cache
  kHelixNoAllocTooLarge = 2,      // batch * kv_heads exceeds HELIX_NOALLOC_MAX_PAIRS
  kHelixNoAllocCudaError = 3,     // a CUDA call failed; see helix_noalloc_last_error()
};

// Paged split-KV decode attention: q [batch, q_heads, 128] bf16 against each sequence's pages.
//   k_cache / v_cache : bf16, logical shape [num_pages, kv_heads, page_size, 128]; the three strides
//                       (in elements) place page, kv head and token, so both head-major and
//                       token-major page layouts are accepted; the innermost 128 values are contiguous
//   block_table       : int32 [batch, block_table_stride], seq_lens: int32 [batch] (tokens of this shard)
//   o                 : bf16 [batch, q_heads, 128] (normalised), lse: fp32 [batch, q_heads]
//   max_seq_len       : an upper bound of seq_lens (host-side knowledge; the kernel reads the real lengths on
//                       the device).  It only sizes the launch: batch * kv_heads * ceil(max_seq_len / 16) blocks
//                       decide how many CTAs are started (two per SM unless the problem is tiny).  A bound that
//                       is too small costs speed, never correctness; values <= 0 are treated as 1
//   stream            : a cudaStream_t (0 for the default stream)
// Returns a HelixNoAllocStatus.  The call is asynchronous with respect to the host.
int helix_gqa_decode_noalloc(const void* q, int64_t q_stride_batch, int64_t q_stride_head,
                             const void* k_cache, const void* v_cache, int64_t num_pages, int64_t cache_stride_page,
                             int64_t cache_stride_head, int64_t cache_stride_token,
                             const int32_t* block_table, int64_t block_table_stride, const int32_t* seq_lens,
                             void* o, float* lse, int batch, int q_heads, int kv_heads, int page_size,
                             int max_seq_len, float scale, int lse_base2, void* stream);

// Error word of the last launch on the current device (0 = fine); synchronises `stream`.
int helix_noalloc_read_error(void* stream);

// Text of the last CUDA error seen by this entry point on the calling thread ("" if none).
const char* helix_noalloc_last_error(void);

#ifdef __cplusplus
}
#endif
