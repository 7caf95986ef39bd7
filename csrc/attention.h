// Split-KV paged decode attention for B200: host interface.
//
// The reference has no attention kernel (vLLM's FlashInfer / FlashAttention backends produce
// the per-rank partial outputs there, benchmark/sbatch/run_gb200_aiperf_v3.sbatch:95); this
// library supplies it so that the whole decode step attention -> exchange+combine -> o_proj
// runs on hand-written sm_100a kernels.  Outputs are exactly what the exchange consumes:
// normalised partial `o [B, Hq, D]` (bf16) and `lse [B, Hq]` (fp32, base e or base 2).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace helix {

struct GqaDecodeParams {
  const __nv_bfloat16* q;      // [B, Hq, 128]
  int64_t q_stride_b, q_stride_h;   // elements
  CUtensorMap k_map, v_map;    // 4-D (d, token-in-page, kv head, page), box (64, 16, 1, 1), SWIZZLE_128B
  const int32_t* block_table;  // [B, bt_stride]
  int64_t bt_stride;
  const int32_t* seq_lens;     // [B] tokens of the LOCAL KV shard
  __nv_bfloat16* o;            // [B, Hq, 128]
  float* lse;                  // [B, Hq]
  float* part_o;               // scratch [2 * ctas + max_helper][8][128] fp32: piece slots
  float* part_lse;             // scratch [2 * ctas + max_helper][8]
  // scratch, zero on entry and zero again on exit (gqa_counter_ints(B * Hkv, max_helper) ints):
  //   [0, P)          blocks of each (sequence, kv head) pair that have been folded into a piece so far
  //   [P, 2P)         chunks drawn from each pair's dynamic pool          (touched only when dyn_pct > 0)
  //   [2P]            CTAs that have left the launch                      (touched only when dyn_pct > 0)
  //   [2P + 8, ...)   one flag per helper slot: a piece has been parked there
  int* counters;
  int* error_flag;             // set to a helix::Status code when a bounded wait runs out
  unsigned long long* trace;   // optional [ctas][8] stamps (%globaltimer): entry, first data, end of the fixed share,
                               // exit, end of the last drawn chunk, chunks drawn | pools visited << 32, SM id
  int B, Hq, Hkv, page_size, ctas;
  // Dynamic tail: of every pair with at least dyn_min_blocks KV blocks, the last dyn_pct percent (rounded down to
  // whole chunks of dyn_chunk blocks) are not part of any CTA's fixed share; CTAs draw them chunk by chunk when
  // their own share is done, so SMs that stream faster end up streaming more.  dyn_pct = 0: fixed shares only.
  int dyn_pct, dyn_chunk, dyn_min_blocks, max_helper;
  float scale;
  int lse_base2;
  // 1: the kernel before this one in the stream writes at most the newest token of each sequence (the cache
  // append) and q; block_table, seq_lens and all older KV are already final.  Under programmatic launch the
  // first K/V tiles are then requested before the wait on that kernel, except by a CTA whose first segment
  // reaches the end of its sequence.
  int kv_stable;
  unsigned long long timeout_ns;
};

constexpr int kGqaMaxCtas = 640;     // upper bound of the grid
constexpr int kGqaMaxHelper = 1024;  // upper bound of the chunks all dynamic pools hold together
constexpr int kGqaSeqTable = 256;    // batches beyond this run with fixed shares only

// scratch sizes
constexpr size_t gqa_part_o_floats(int ctas, int max_helper) { return ((size_t)ctas * 2 + max_helper) * 8 * 128; }
constexpr size_t gqa_part_lse_floats(int ctas, int max_helper) { return ((size_t)ctas * 2 + max_helper) * 8; }
constexpr size_t gqa_counter_ints(int pairs, int max_helper) { return (size_t)2 * pairs + 8 + max_helper; }

// number of CTAs that fills the device for this batch (two per SM unless the work is tiny)
int gqa_pick_ctas(int B, int Hkv, int max_seq_len, int sm_count);

// Dynamic-tail settings for a launch of `ctas` CTAs: fills dyn_pct / dyn_chunk / dyn_min_blocks / max_helper of *p
// (pct_override / chunk_override < 0: the library's choice; max_helper 0 switches the dynamic tail off).
void gqa_plan_dynamic(GqaDecodeParams* p, int max_seq_len, int max_helper, int pct_override, int chunk_override);

cudaError_t launch_gqa_decode(const GqaDecodeParams& p, bool pdl, cudaStream_t stream);

// ---- MLA (latent) decode attention over a block-scaled fp8 cache ------------------------------------
// Absorbed form: scores = (q_nope . ckv + q_pe . kpe) * scale, values = ckv (the 512-d latent).
struct MlaDecodeParams {
  const __nv_bfloat16* q_nope;   // [B, 128, 512] contiguous (already multiplied by W_uk)
  const __nv_bfloat16* q_pe;     // [B, 128, 64] contiguous
  const uint8_t* ckv;            // [pages * page_size, 512] fp8 e4m3
  const float* scales;           // [pages * page_size, 4]  one scale per 128 latent values
  const __nv_bfloat16* kpe;      // [pages * page_size, 64] rope keys
  const int32_t* block_table;    // [B, bt_stride]
  int64_t bt_stride;
  const int32_t* seq_lens;       // [B]
  __nv_bfloat16* o;              // [B, 128, 512] normalised partial output (latent space)
  float* lse;                    // [B, 128]
  float* part_o;                 // scratch [ctas, 2, 128, 512] fp32
  float* part_lse;               // scratch [ctas, 2, 128]
  int* counters;                 // scratch [B], zero on entry and on exit
  int* error_flag;
  unsigned long long* prof;      // lockstep kernel only, optional [ctas][8] clock64 sums of thread 0: waits, dequantise,
                                 // Q K^T, softmax (+ rescale), P store + P V issue, tiles, all clocks of the tile loop
  int B, page_size, ctas;
  int variant;                   // 0: all warps in lockstep; 1: producer warps + math warps (warp-specialised)
  float scale;
  int lse_base2;
  unsigned long long timeout_ns;
};
constexpr int kMlaMaxCtas = 296;
inline size_t mla_part_o_floats(int ctas) { return (size_t)ctas * 2 * 128 * 512; }
inline size_t mla_part_lse_floats(int ctas) { return (size_t)ctas * 2 * 128; }
int mla_pick_ctas(int B, int max_seq_len, int sm_count);
cudaError_t launch_mla_decode(const MlaDecodeParams& p, bool pdl, cudaStream_t stream);

}  // namespace helix
