// Torch bindings of the compute kernels (decode attention, o_proj GEMM).
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "attention.h"
#include "exchange.h"
#include "fifo.cuh"
#include "fused.h"
#include "oproj.h"
#include "tensor_map.h"

namespace {

unsigned long long env_timeout_ns() {
  const char* v = std::getenv("HELIX_A2A_TIMEOUT_MS");
  int ms = (v && *v) ? std::atoi(v) : 2000;
  if (ms < 1) ms = 1;
  return (unsigned long long)ms * 1000000ull;
}
bool env_pdl() {
  const char* v = std::getenv("HELIX_A2A_ENABLE_PDL");
  return v && std::string(v) == "1";
}

// Per-device scratch owned by the library: error flag, counters, split partials.  One set per device (not per
// stream: calls that may overlap on one GPU must be ordered by the caller).  Grown on demand, never shrunk; a
// buffer that is outgrown is kept alive until the process ends, because a CUDA graph captured earlier may still
// hold its address.  All kernels that use the counters leave them at zero.
struct Scratch {
  torch::Tensor error_flag;    // int32 [1]
  torch::Tensor counters;      // int32 [N]
  torch::Tensor part_a, part_b;  // float32 pools
  torch::Tensor trace;           // int64 [kGqaMaxCtas * 8], only with HELIX_A2A_ATTN_TRACE=1 / HELIX_A2A_OPROJ_TRACE=1
  std::vector<torch::Tensor> retired;
};
std::mutex g_mu;
std::map<int, Scratch> g_scratch;

Scratch& scratch_for(const torch::Device& dev, int64_t counters, int64_t part_a_floats, int64_t part_b_floats) {
  std::lock_guard<std::mutex> lk(g_mu);
  Scratch& s = g_scratch[dev.index()];
  auto iopt = torch::TensorOptions().dtype(torch::kInt32).device(dev);
  auto fopt = torch::TensorOptions().dtype(torch::kFloat32).device(dev);
  auto grow = [&](torch::Tensor& t, int64_t need, int64_t floor, const torch::TensorOptions& opt, bool zero) {
    if (t.defined() && t.numel() >= need) return;
    if (t.defined()) s.retired.push_back(t);
    const int64_t n = std::max<int64_t>(need + need / 4, floor);     // head-room: regrowing is rare
    t = zero ? torch::zeros({n}, opt) : torch::empty({n}, opt);
  };
  if (!s.error_flag.defined()) s.error_flag = torch::zeros({1}, iopt);
  grow(s.counters, counters, 16384, iopt, true);
  grow(s.part_a, part_a_floats, 1, fopt, false);
  grow(s.part_b, part_b_floats, 1, fopt, false);
  return s;
}

int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  return (v && *v) ? std::atoi(v) : dflt;
}

void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "helix: ", what, " failed: ", cudaGetErrorString(e));
}

// ---- tensor-map cache --------------------------------------------------------------------------
using MapKey = std::tuple<const void*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int>;
std::map<MapKey, CUtensorMap> g_maps;

CUtensorMap kv_map(const torch::Tensor& cache, bool hnd) {
  // cache: [pages, Hkv, page, D] (hnd) or [pages, page, Hkv, D]
  const int64_t pages = cache.size(0), D = cache.size(3);
  const int64_t Hkv = hnd ? cache.size(1) : cache.size(2), page = hnd ? cache.size(2) : cache.size(1);
  const int64_t s_page = cache.stride(0), s_head = hnd ? cache.stride(1) : cache.stride(2),
                s_tok = hnd ? cache.stride(2) : cache.stride(1);
  MapKey key{cache.data_ptr(), pages, Hkv, page, D, s_page, s_head, s_tok, 1};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  CUtensorMap m;
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)page, (uint64_t)Hkv, (uint64_t)pages};
  uint64_t strides[3] = {(uint64_t)s_tok * 2, (uint64_t)s_head * 2, (uint64_t)s_page * 2};
  uint32_t box[4] = {64, 16, 1, 1};
  const char* err = nullptr;
  TORCH_CHECK(helix::encode_tensor_map(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, cache.data_ptr(), dims, strides, box,
                                       helix::TmaSwizzle::k128B, &err),
              "helix: KV cache tensor map: ", err ? err : "?");
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  return m;
}

CUtensorMap mat_map(const torch::Tensor& t, int64_t box_rows) {
  // t: [rows, K] bf16, last dim contiguous
  MapKey key{t.data_ptr(), t.size(0), t.size(1), t.stride(0), box_rows, 0, 0, 0, 2};
  std::lock_guard<std::mutex> lk(g_mu);
  auto it = g_maps.find(key);
  if (it != g_maps.end()) return it->second;
  CUtensorMap m;
  uint64_t dims[2] = {(uint64_t)t.size(1), (uint64_t)t.size(0)};
  uint64_t strides[1] = {(uint64_t)t.stride(0) * 2};
  uint32_t box[2] = {64, (uint32_t)box_rows};
  const char* err = nullptr;
  TORCH_CHECK(helix::encode_tensor_map(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, t.data_ptr(), dims, strides, box,
                                       helix::TmaSwizzle::k128B, &err),
              "helix: matrix tensor map: ", err ? err : "?");
  if (g_maps.size() > 4096) g_maps.clear();
  g_maps[key] = m;
  return m;
}

// ---- GQA paged decode attention -----------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor> gqa_decode(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache,
                                                    torch::Tensor block_table, torch::Tensor seq_lens, double scale,
                                                    bool lse_base2, bool hnd, int64_t splits, int64_t max_seq_len, bool kv_stable) {
  TORCH_CHECK(q.is_cuda() && k_cache.is_cuda() && v_cache.is_cuda() && block_table.is_cuda() && seq_lens.is_cuda(),
              "all inputs must be on CUDA");
  TORCH_CHECK(q.scalar_type() == at::ScalarType::BFloat16 && k_cache.scalar_type() == at::ScalarType::BFloat16 &&
                  v_cache.scalar_type() == at::ScalarType::BFloat16,
              "q / k_cache / v_cache must be bfloat16");
  TORCH_CHECK(block_table.scalar_type() == at::ScalarType::Int && seq_lens.scalar_type() == at::ScalarType::Int,
              "block_table / seq_lens must be int32");
  TORCH_CHECK(q.dim() == 3 && q.size(2) == 128 && q.stride(2) == 1, "q must be [B, Hq, 128]");
  TORCH_CHECK(k_cache.dim() == 4 && v_cache.dim() == 4 && k_cache.size(3) == 128 && k_cache.stride(3) == 1 &&
                  v_cache.stride(3) == 1 && k_cache.sizes() == v_cache.sizes(),
              "caches must be 4-D with head_dim 128 innermost");
  TORCH_CHECK(block_table.dim() == 2 && block_table.stride(1) == 1 && block_table.size(0) == q.size(0));
  TORCH_CHECK(seq_lens.dim() == 1 && seq_lens.size(0) == q.size(0) && seq_lens.is_contiguous());
  const int B = (int)q.size(0), Hq = (int)q.size(1);
  const int Hkv = (int)(hnd ? k_cache.size(1) : k_cache.size(2));
  const int page = (int)(hnd ? k_cache.size(2) : k_cache.size(1));
  TORCH_CHECK(Hq % Hkv == 0 && Hq / Hkv <= 8, "query heads per KV head must be <= 8");
  TORCH_CHECK(page % 16 == 0, "page size must be a multiple of 16");
  c10::cuda::CUDAGuard guard(q.device());
  auto stream = at::cuda::getCurrentCUDAStream();

  // splits > 0 asks for about that many CTAs per (sequence, kv head) pair; 0 lets the library choose
  int sp = splits > 0 ? (int)std::min<int64_t>((int64_t)B * Hkv * splits, helix::kGqaMaxCtas)
                      : helix::gqa_pick_ctas(B, Hkv, (int)std::max<int64_t>(max_seq_len, 1), helix::device_sm_count());
  sp = std::max(sp, 1);
  torch::Tensor o = torch::empty({B, Hq, 128}, q.options());
  torch::Tensor lse = torch::empty({B, Hq}, q.options().dtype(torch::kFloat32));
  if (B == 0) return std::make_tuple(o, lse);
  const int max_helper = helix::kGqaMaxHelper;
  // the o_proj counters sit in the last hidden / 128 ints of the same tensor: leave them room
  Scratch& sc = scratch_for(q.device(), (int64_t)helix::gqa_counter_ints(B * Hkv, max_helper) + 2048,
                            (int64_t)helix::gqa_part_o_floats(sp, max_helper),
                            (int64_t)helix::gqa_part_lse_floats(sp, max_helper));
  helix::GqaDecodeParams p{};
  p.q = reinterpret_cast<const __nv_bfloat16*>(q.data_ptr());
  p.q_stride_b = q.stride(0);
  p.q_stride_h = q.stride(1);
  p.k_map = kv_map(k_cache, hnd);
  p.v_map = kv_map(v_cache, hnd);
  p.block_table = block_table.data_ptr<int32_t>();
  p.bt_stride = block_table.stride(0);
  p.seq_lens = seq_lens.data_ptr<int32_t>();
  p.o = reinterpret_cast<__nv_bfloat16*>(o.data_ptr());
  p.lse = lse.data_ptr<float>();
  p.part_o = sc.part_a.data_ptr<float>();
  p.part_lse = sc.part_b.data_ptr<float>();
  p.counters = sc.counters.data_ptr<int32_t>();
  p.error_flag = sc.error_flag.data_ptr<int32_t>();
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.page_size = page; p.ctas = sp;
  // HELIX_A2A_ATTN_DYN_PCT / HELIX_A2A_ATTN_DYN_CHUNK: share of every long pair that is handed out dynamically
  // (0 = fixed shares only) and the chunk size in 16-token blocks; unset = the library's choice
  helix::gqa_plan_dynamic(&p, (int)std::max<int64_t>(max_seq_len, 1), max_helper, env_int("HELIX_A2A_ATTN_DYN_PCT", -1),
                          env_int("HELIX_A2A_ATTN_DYN_CHUNK", -1));
  if (const int mb = env_int("HELIX_A2A_ATTN_DYN_MIN_BLOCKS", -1); mb >= 0) p.dyn_min_blocks = mb;
  p.scale = (float)scale;
  p.lse_base2 = lse_base2 ? 1 : 0;
  p.timeout_ns = env_timeout_ns();
  p.trace = nullptr;
  {
    const char* tr = std::getenv("HELIX_A2A_ATTN_TRACE");
    if (tr && tr[0] == '1') {
      if (!sc.trace.defined()) sc.trace = torch::zeros({helix::kGqaMaxCtas * 8}, q.options().dtype(torch::kInt64));
      p.trace = reinterpret_cast<unsigned long long*>(sc.trace.data_ptr());
    }
  }
  p.kv_stable = kv_stable ? 1 : 0;
  check_cuda(helix::launch_gqa_decode(p, env_pdl(), stream), "gqa decode launch");
  return std::make_tuple(o, lse);
}


constexpr int kMlaDefaultVariant = 1;   // warp-specialised

// ---- MLA fp8 paged decode attention -----------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor> mla_decode(torch::Tensor q_nope, torch::Tensor q_pe, torch::Tensor ckv,
                                                    torch::Tensor scales, torch::Tensor kpe, torch::Tensor block_table,
                                                    torch::Tensor seq_lens, double scale, bool lse_base2, int64_t ctas,
                                                    int64_t max_seq_len) {
  TORCH_CHECK(q_nope.is_cuda() && q_pe.is_cuda() && ckv.is_cuda() && scales.is_cuda() && kpe.is_cuda() &&
                  block_table.is_cuda() && seq_lens.is_cuda(), "all inputs must be on CUDA");
  TORCH_CHECK(q_nope.scalar_type() == at::ScalarType::BFloat16 && q_pe.scalar_type() == at::ScalarType::BFloat16 &&
                  kpe.scalar_type() == at::ScalarType::BFloat16, "q_nope / q_pe / kpe must be bfloat16");
  TORCH_CHECK(ckv.element_size() == 1, "ckv must be fp8 e4m3 (1 byte per element)");
  TORCH_CHECK(scales.scalar_type() == at::ScalarType::Float, "scales must be float32");
  TORCH_CHECK(q_nope.dim() == 3 && q_nope.size(1) == 128 && q_nope.size(2) == 512 && q_nope.is_contiguous(),
              "q_nope must be contiguous [B, 128, 512]");
  TORCH_CHECK(q_pe.dim() == 3 && q_pe.size(0) == q_nope.size(0) && q_pe.size(1) == 128 && q_pe.size(2) == 64 &&
                  q_pe.is_contiguous(), "q_pe must be contiguous [B, 128, 64]");
  TORCH_CHECK(ckv.dim() == 3 && ckv.size(2) == 512 && ckv.is_contiguous(), "ckv must be contiguous [pages, page, 512]");
  TORCH_CHECK(scales.dim() == 3 && scales.size(0) == ckv.size(0) && scales.size(1) == ckv.size(1) && scales.size(2) == 4 &&
                  scales.is_contiguous(), "scales must be contiguous [pages, page, 4]");
  TORCH_CHECK(kpe.dim() == 3 && kpe.size(0) == ckv.size(0) && kpe.size(1) == ckv.size(1) && kpe.size(2) == 64 &&
                  kpe.is_contiguous(), "kpe must be contiguous [pages, page, 64]");
  TORCH_CHECK(block_table.scalar_type() == at::ScalarType::Int && seq_lens.scalar_type() == at::ScalarType::Int &&
                  block_table.dim() == 2 && block_table.stride(1) == 1 && seq_lens.is_contiguous(),
              "block_table [B, n] / seq_lens [B] must be int32");
  const int B = (int)q_nope.size(0), page = (int)ckv.size(1);
  TORCH_CHECK(page % 16 == 0, "page size must be a multiple of 16");
  c10::cuda::CUDAGuard guard(q_nope.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  torch::Tensor o = torch::empty({B, 128, 512}, q_nope.options());
  torch::Tensor lse = torch::empty({B, 128}, q_nope.options().dtype(torch::kFloat32));
  if (B == 0) return std::make_tuple(o, lse);
  int nc = ctas > 0 ? (int)std::min<int64_t>(ctas, helix::kMlaMaxCtas)
                    : helix::mla_pick_ctas(B, (int)std::max<int64_t>(max_seq_len, 1), helix::device_sm_count());
  Scratch& sc = scratch_for(q_nope.device(), (int64_t)B + 1024, (int64_t)helix::mla_part_o_floats(nc),
                            (int64_t)helix::mla_part_lse_floats(nc));
  helix::MlaDecodeParams p{};
  p.q_nope = reinterpret_cast<const __nv_bfloat16*>(q_nope.data_ptr());
  p.q_pe = reinterpret_cast<const __nv_bfloat16*>(q_pe.data_ptr());
  p.ckv = reinterpret_cast<const uint8_t*>(ckv.data_ptr());
  p.scales = scales.data_ptr<float>();
  p.kpe = reinterpret_cast<const __nv_bfloat16*>(kpe.data_ptr());
  p.block_table = block_table.data_ptr<int32_t>();
  p.bt_stride = block_table.stride(0);
  p.seq_lens = seq_lens.data_ptr<int32_t>();
  p.o = reinterpret_cast<__nv_bfloat16*>(o.data_ptr());
  p.lse = lse.data_ptr<float>();
  p.part_o = sc.part_a.data_ptr<float>();
  p.part_lse = sc.part_b.data_ptr<float>();
  p.counters = sc.counters.data_ptr<int32_t>();
  p.error_flag = sc.error_flag.data_ptr<int32_t>();
  p.B = B; p.page_size = page; p.ctas = nc;
  p.scale = (float)scale;
  p.lse_base2 = lse_base2 ? 1 : 0;
  p.timeout_ns = env_timeout_ns();
  {
    // HELIX_A2A_MLA_VARIANT: "ws" = producer warps + math warps, "lockstep" = all warps in lockstep
    const char* v = std::getenv("HELIX_A2A_MLA_VARIANT");
    p.variant = (v && std::string(v) == "lockstep") ? 0 : (v && std::string(v) == "ws") ? 1 : kMlaDefaultVariant;
  }
  p.prof = nullptr;
  {
    static const bool prof_on = [] { const char* v = std::getenv("HELIX_A2A_MLA_PROF"); return v && std::string(v) == "1"; }();
    if (prof_on) {
      if (!sc.trace.defined()) sc.trace = torch::zeros({helix::kGqaMaxCtas * 8}, q_nope.options().dtype(torch::kInt64));
      p.prof = reinterpret_cast<unsigned long long*>(sc.trace.data_ptr());
    }
  }
  check_cuda(helix::launch_mla_decode(p, env_pdl(), stream), "mla decode launch");
  return std::make_tuple(o, lse);
}

// ---- o_proj ----------------------------------------------------------------------------------------
torch::Tensor oproj(torch::Tensor x, torch::Tensor w, int64_t splits) {
  TORCH_CHECK(x.is_cuda() && w.is_cuda(), "inputs must be on CUDA");
  TORCH_CHECK(x.scalar_type() == at::ScalarType::BFloat16 && w.scalar_type() == at::ScalarType::BFloat16,
              "x and w must be bfloat16");
  TORCH_CHECK(x.dim() == 2 && w.dim() == 2 && x.size(1) == w.size(1), "x [tokens, K], w [hidden, K]");
  TORCH_CHECK(x.stride(1) == 1 && w.stride(1) == 1, "innermost dimension must be contiguous");
  TORCH_CHECK(w.size(0) % 128 == 0 && w.size(1) % 64 == 0, "hidden must be a multiple of 128 and K of 64");
  TORCH_CHECK((x.stride(0) * 2) % 16 == 0 && (w.stride(0) * 2) % 16 == 0, "row strides must be multiples of 16 bytes");
  const int tokens = (int)x.size(0), hidden = (int)w.size(0), K = (int)w.size(1);
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  torch::Tensor y = torch::empty({tokens, hidden}, x.options());
  if (tokens == 0) return y;
  // more than 256 tokens: run the kernel per 256-token slice (decode batches are smaller)
  for (int t0 = 0; t0 < tokens; t0 += 256) {
    const int nt = std::min(256, tokens - t0);
    torch::Tensor xs = x.narrow(0, t0, nt);
    const int n_pad = (nt + 15) / 16 * 16;
    int sp = (int)splits;
    const int sms = helix::device_sm_count();
    // splits: 0 = pick (stream-K when it pays), -1 = force stream-K, >= 1 = that many K splits
    bool streamk = sp == -1 || (sp == 0 && helix::oproj_streamk_pays(hidden, K, n_pad, sms));
    if (sp == 0) {
      // HELIX_A2A_OPROJ_STREAMK=1 / 0 overrides the choice for calls that leave it to the library
      if (const char* v = std::getenv("HELIX_A2A_OPROJ_STREAMK")) streamk = std::string(v) == "1";
    }
    const int bk = 64 * helix::oproj_pick_atoms(n_pad);
    const int sk_ctas = (int)std::min<int64_t>(sms, (int64_t)(hidden / 128) * ((K + bk - 1) / bk));
    if (sp <= 0) sp = helix::oproj_pick_splits(hidden, K, sms);
    const int64_t part_floats = streamk ? (int64_t)helix::oproj_streamk_partial_floats(sk_ctas, n_pad)
                                        : (sp > 1 ? (int64_t)helix::oproj_partial_bytes(hidden, sp, n_pad) / 4 : 0);
    Scratch& sc = scratch_for(x.device(), hidden / 128 + 1024, part_floats, 0);
    helix::OprojParams p{};
    p.w_map = mat_map(w, 128);
    p.x_map = mat_map(xs, n_pad);
    p.y = reinterpret_cast<__nv_bfloat16*>(y.data_ptr()) + (int64_t)t0 * y.stride(0);
    p.y_stride = y.stride(0);
    p.partial = sc.part_a.data_ptr<float>();
    // o_proj counters live after the attention counters
    p.counters = sc.counters.data_ptr<int32_t>() + (sc.counters.numel() - hidden / 128);
    p.error_flag = sc.error_flag.data_ptr<int32_t>();
    p.tokens = nt; p.n_pad = n_pad; p.hidden = hidden; p.K = K; p.splits = sp;
    p.stages = helix::oproj_pick_stages(n_pad);
    p.atoms = helix::oproj_pick_atoms(n_pad);
    p.timeout_ns = env_timeout_ns();
    p.ctas = sk_ctas;
    p.trace = nullptr;
    if (streamk) {
      static const bool trace_on = [] { const char* v = std::getenv("HELIX_A2A_OPROJ_TRACE"); return v && std::string(v) == "1"; }();
      if (trace_on) {
        if (!sc.trace.defined()) sc.trace = torch::zeros({helix::kGqaMaxCtas * 8}, x.options().dtype(torch::kInt64));
        p.trace = reinterpret_cast<unsigned long long*>(sc.trace.data_ptr());
      }
    }
    check_cuda(streamk ? helix::launch_oproj_streamk(p, env_pdl(), stream) : helix::launch_oproj(p, env_pdl(), stream),
               "o_proj launch");
  }
  return y;
}

// o_proj on pre-packed weights (see OprojParams::w_packed): `packed` is the uint8 tensor made by
// helix_a2a_b200.ops.oproj.prepack_weight for a [hidden, K] matrix.  Plain split-K kernel only.
torch::Tensor oproj_packed(torch::Tensor x, torch::Tensor packed, int64_t hidden64, int64_t K64, int64_t splits) {
  TORCH_CHECK(x.is_cuda() && packed.is_cuda(), "inputs must be on CUDA");
  TORCH_CHECK(x.scalar_type() == at::ScalarType::BFloat16 && packed.scalar_type() == at::ScalarType::Byte,
              "x must be bfloat16, packed uint8");
  const int hidden = (int)hidden64, K = (int)K64;
  TORCH_CHECK(x.dim() == 2 && x.size(1) == K && x.stride(1) == 1 && (x.stride(0) * 2) % 16 == 0, "x must be [tokens, K]");
  TORCH_CHECK(hidden % 128 == 0 && K % 64 == 0, "hidden must be a multiple of 128 and K of 64");
  TORCH_CHECK(packed.is_contiguous() && (size_t)packed.numel() == helix::oproj_packed_bytes(hidden, K) &&
                  reinterpret_cast<uintptr_t>(packed.data_ptr()) % 128 == 0,
              "packed weight has the wrong size or alignment for [", hidden, ", ", K, "]");
  const int tokens = (int)x.size(0);
  c10::cuda::CUDAGuard guard(x.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  torch::Tensor y = torch::empty({tokens, hidden}, x.options());
  for (int t0 = 0; t0 < tokens; t0 += 256) {
    const int nt = std::min(256, tokens - t0);
    torch::Tensor xs = x.narrow(0, t0, nt);
    const int n_pad = (nt + 15) / 16 * 16;
    int sp = (int)splits;
    if (sp <= 0) sp = helix::oproj_pick_splits(hidden, K, helix::device_sm_count());
    Scratch& sc = scratch_for(x.device(), hidden / 128 + 1024,
                              sp > 1 ? (int64_t)helix::oproj_partial_bytes(hidden, sp, n_pad) / 4 : 0, 0);
    helix::OprojParams p{};
    p.x_map = mat_map(xs, n_pad);
    p.w_map = p.x_map;                       // unused with packed weights; keeps the descriptor prefetch valid
    p.w_packed = packed.data_ptr<uint8_t>();
    p.packed_atoms = helix::oproj_packed_atoms(K);
    p.y = reinterpret_cast<__nv_bfloat16*>(y.data_ptr()) + (int64_t)t0 * y.stride(0);
    p.y_stride = y.stride(0);
    p.partial = sc.part_a.data_ptr<float>();
    p.counters = sc.counters.data_ptr<int32_t>() + (sc.counters.numel() - hidden / 128);
    p.error_flag = sc.error_flag.data_ptr<int32_t>();
    p.tokens = nt; p.n_pad = n_pad; p.hidden = hidden; p.K = K; p.splits = sp;
    p.stages = helix::oproj_pick_stages(n_pad);
    p.atoms = helix::oproj_pick_atoms(n_pad);
    p.timeout_ns = env_timeout_ns();
    check_cuda(helix::launch_oproj(p, env_pdl(), stream), "o_proj (packed) launch");
  }
  return y;
}

torch::Tensor attn_trace(torch::Tensor like) {
  Scratch& sc = scratch_for(like.device(), 1, 0, 0);
  TORCH_CHECK(sc.trace.defined(), "no trace recorded: set HELIX_A2A_ATTN_TRACE=1 (or HELIX_A2A_OPROJ_TRACE=1)");
  return sc.trace.clone();
}


// ---- fused exchange + combine + o_proj --------------------------------------------------------------
// attn_out [B, H, D] bf16, lse [B, H] fp32, w [hidden, (H/cp) * D] bf16 (or the packed form of it) -> y [B, hidden].
// emulate: leading [cp] dim on attn_out, lse, w and y; one cooperative launch plays all ranks, and the combined
// activation x [B, (H/cp) * D] the GEMM consumed is returned as well (it only ever exists in shared memory otherwise).
std::tuple<torch::Tensor, torch::Tensor> fused_impl(torch::Tensor attn_out, torch::Tensor lse, const torch::Tensor* w,
                                                    const torch::Tensor* packed, int64_t hidden, torch::Tensor workspace,
                                                    int64_t cp_rank, int64_t cp_size, bool base2, bool emulate,
                                                    int64_t timeout_ms) {
  TORCH_CHECK(attn_out.is_cuda() && lse.is_cuda() && workspace.is_cuda(), "inputs must be on CUDA");
  TORCH_CHECK(attn_out.scalar_type() == at::ScalarType::BFloat16, "attn_out must be bfloat16");
  TORCH_CHECK(lse.scalar_type() == at::ScalarType::Float, "lse must be float32");
  TORCH_CHECK(attn_out.is_contiguous() && lse.is_contiguous(), "inputs must be contiguous");
  const int lead = emulate ? 1 : 0;
  TORCH_CHECK(attn_out.dim() == 3 + lead && lse.dim() == 2 + lead, "bad input ranks");
  const int64_t B = attn_out.size(lead), H = attn_out.size(lead + 1), D = attn_out.size(lead + 2);
  TORCH_CHECK(H % cp_size == 0, "heads must divide by cp_size");
  const int64_t Hl = H / cp_size, K = Hl * D;
  if (w != nullptr) {
    TORCH_CHECK(w->is_cuda() && w->scalar_type() == at::ScalarType::BFloat16 && w->is_contiguous() && w->dim() == 2 + lead,
                "w must be a contiguous bfloat16 matrix");
    hidden = w->size(lead);
    TORCH_CHECK(w->size(lead + 1) == K, "w must be [hidden, (H/cp) * D]");
  } else {
    TORCH_CHECK(!emulate, "packed weights are not supported when one launch plays all ranks");
    TORCH_CHECK(packed->is_cuda() && packed->scalar_type() == at::ScalarType::Byte && packed->is_contiguous() &&
                    (size_t)packed->numel() == helix::oproj_packed_bytes((int)hidden, (int)K) &&
                    reinterpret_cast<uintptr_t>(packed->data_ptr()) % 128 == 0,
                "packed weight has the wrong size or alignment for [", hidden, ", ", K, "]");
  }
  TORCH_CHECK(hidden % 128 == 0 && K % 64 == 0 && (D * 2) % 128 == 0, "hidden % 128, K % 64, head_dim % 64");
  TORCH_CHECK(B >= 1, "at least one token");
  TORCH_CHECK(workspace.scalar_type() == at::ScalarType::Long && workspace.dim() == 2 && workspace.size(0) == cp_size,
              "workspace must be the [cp_size, elems] int64 tensor");
  const int ranks = emulate ? (int)cp_size : 1;
  TORCH_CHECK(ranks <= helix::kFusedMaxRanks, "at most ", helix::kFusedMaxRanks, " emulated ranks");
  if (emulate) TORCH_CHECK(attn_out.size(0) == cp_size && w->size(0) == cp_size, "leading [cp] dim expected");
  const int splits = helix::fused_pick_splits((int)Hl, (int)D);
  TORCH_CHECK(splits > 0 && B <= helix::kFusedMaxTokens,
              "helix: fused exchange+o_proj does not fit this shape (more than ", helix::kFusedMaxTokens,
              " tokens or a head wider than 512); run alltoall_combine and oproj separately");
  c10::cuda::CUDAGuard guard(attn_out.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  std::vector<int64_t> xs{B, K}, ys{B, hidden};
  if (emulate) { xs.insert(xs.begin(), cp_size); ys.insert(ys.begin(), cp_size); }
  // the combined activation exists in global memory for the tests (emulation) and when the slabs of a head group
  // share its rows
  const bool want_x = emulate || helix::fused_shares_rows((int)B, (int)(Hl / splits), (int)hidden);
  torch::Tensor x = want_x ? torch::empty(xs, attn_out.options()) : torch::empty({0}, attn_out.options());
  torch::Tensor y = torch::empty(ys, attn_out.options());
  const int n_pad = (int)((B + 15) / 16 * 16);
  const int64_t part_floats = splits > 1 ? (int64_t)helix::oproj_partial_bytes((int)hidden, splits, n_pad) / 4 * ranks : 0;
  Scratch& sc = scratch_for(attn_out.device(), (hidden / 128 + helix::fused_aux_ints((int)hidden)) * ranks + 1024, part_floats, 0);

  helix::FusedParams fp{};
  helix::ExchangeParams& p = fp.ex;
  {
    // per-CTA %globaltimer stamps of the one-kernel path (read back with attn_trace)
    static const bool trace_on = [] { const char* v = std::getenv("HELIX_A2A_EXCHANGE_TRACE"); return v && std::string(v) == "1"; }();
    if (trace_on) {
      if (!sc.trace.defined()) sc.trace = torch::zeros({helix::kGqaMaxCtas * 8}, attn_out.options().dtype(torch::kInt64));
      p.trace = reinterpret_cast<unsigned long long*>(sc.trace.data_ptr());
    }
  }
  for (int r = 0; r < ranks; ++r) {
    p.io[r].o_src = reinterpret_cast<const uint8_t*>(attn_out.data_ptr()) + (int64_t)r * B * H * D * 2;
    p.io[r].st_src = reinterpret_cast<const uint8_t*>(lse.data_ptr()) + (int64_t)r * B * H * 4;
    p.io[r].o_dst = nullptr;
    p.io[r].st_dst = nullptr;
    fp.x_out[r] = want_x ? reinterpret_cast<__nv_bfloat16*>(x.data_ptr()) + (int64_t)r * B * K : nullptr;
    helix::OprojParams& g = fp.gemm[r];
    if (w != nullptr) {
      torch::Tensor wr = emulate ? (*w)[r] : *w;
      g.w_map = mat_map(wr, 128);
      g.w_packed = nullptr;
    } else {
      g.w_packed = packed->data_ptr<uint8_t>();
      g.packed_atoms = helix::oproj_packed_atoms((int)K);
    }
    g.y = reinterpret_cast<__nv_bfloat16*>(y.data_ptr()) + (int64_t)r * B * hidden;
    g.y_stride = hidden;
    // every emulated rank needs its own split partials and slab counters
    g.partial = splits > 1 ? sc.part_a.data_ptr<float>() + (int64_t)r * (part_floats / ranks) : nullptr;
    {
      // from the end of the counter buffer: [slab counters | aux] per rank, all zero between calls
      const int64_t per_rank = hidden / 128 + helix::fused_aux_ints((int)hidden);
      g.counters = sc.counters.data_ptr<int32_t>() + (sc.counters.numel() - per_rank * (r + 1));
      fp.aux[r] = g.counters + hidden / 128;
    }
    g.error_flag = sc.error_flag.data_ptr<int32_t>();
    g.tokens = (int)B; g.n_pad = n_pad; g.hidden = (int)hidden; g.K = (int)K; g.splits = splits;
    g.timeout_ns = timeout_ms > 0 ? (unsigned long long)timeout_ms * 1000000ull : env_timeout_ns();
  }
  p.workspace = reinterpret_cast<uint64_t*>(workspace.data_ptr());
  p.row_stride_bytes = workspace.stride(0) * 8;
  p.sm_count = helix::device_sm_count();
  p.cp_size = (int)cp_size;
  p.rank_base = emulate ? 0 : (int)cp_rank;
  p.ranks_in_launch = ranks;
  p.outer = (int)B; p.inner = (int)Hl;
  p.o_sb = H * D * 2; p.o_sp = Hl * D * 2; p.o_sh = D * 2;
  p.st_sb = H * 4; p.st_sp = Hl * 4; p.st_sh = 4;
  p.lse_scalar = 1;
  p.od_se = D * 2;
  p.o_bytes = (int)(D * 2);
  p.st_words = 1;
  p.is_bf16 = 1;
  p.mode = helix::kModeCombine;
  p.stats_mode = 0;
  p.base2 = base2 ? 1 : 0;
  p.timeout_ns = timeout_ms > 0 ? (unsigned long long)timeout_ms * 1000000ull : env_timeout_ns();
  const char* ch = std::getenv("HELIX_A2A_CHANNEL_COUNT");
  cudaError_t e = helix::launch_exchange_oproj(fp, ch ? std::max(std::atoi(ch), 0) : 0, env_pdl(), stream, nullptr);
  TORCH_CHECK(e != cudaErrorNotSupported, "helix: fused exchange+o_proj does not fit this shape on the device; "
              "run alltoall_combine and oproj separately");
  check_cuda(e, "fused exchange+o_proj launch");
  return std::make_tuple(y, x);
}

std::tuple<torch::Tensor, torch::Tensor> alltoall_combine_oproj(torch::Tensor attn_out, torch::Tensor lse,
                                                                torch::Tensor w, torch::Tensor workspace,
                                                                int64_t cp_rank, int64_t cp_size, bool base2,
                                                                bool emulate, int64_t timeout_ms) {
  return fused_impl(attn_out, lse, &w, nullptr, 0, workspace, cp_rank, cp_size, base2, emulate, timeout_ms);
}

torch::Tensor alltoall_combine_oproj_packed(torch::Tensor attn_out, torch::Tensor lse, torch::Tensor packed,
                                            int64_t hidden, torch::Tensor workspace, int64_t cp_rank, int64_t cp_size,
                                            bool base2, int64_t timeout_ms) {
  return std::get<0>(fused_impl(attn_out, lse, nullptr, &packed, hidden, workspace, cp_rank, cp_size, base2, false,
                                timeout_ms));
}

bool fused_oproj_fits(int64_t tokens, int64_t heads_local, int64_t head_dim, int64_t hidden, int64_t cp_size) {
  return helix::fused_fits((int)tokens, (int)heads_local, (int)head_dim, (int)hidden, (int)cp_size, helix::device_sm_count());
}

int64_t read_error_flag(torch::Tensor like) {
  Scratch& sc = scratch_for(like.device(), 1, 0, 0);
  return sc.error_flag.item<int>();
}

void clear_error_flag(torch::Tensor like) {
  Scratch& sc = scratch_for(like.device(), 1, 0, 0);
  sc.error_flag.zero_();
  sc.counters.zero_();
}

}  // namespace

void register_compute_ops(torch::Library& m) {
  m.def(
      "gqa_decode(Tensor q, Tensor k_cache, Tensor v_cache, Tensor block_table, Tensor seq_lens, float scale, bool "
      "lse_base2, bool hnd, int splits, int max_seq_len, bool kv_stable=False) -> (Tensor, Tensor)",
      &gqa_decode);
  m.def(
      "mla_decode(Tensor q_nope, Tensor q_pe, Tensor ckv, Tensor scales, Tensor kpe, Tensor block_table, Tensor seq_lens, "
      "float scale, bool lse_base2, int ctas, int max_seq_len) -> (Tensor, Tensor)",
      &mla_decode);
  m.def("oproj(Tensor x, Tensor w, int splits) -> Tensor", &oproj);
  m.def("oproj_packed(Tensor x, Tensor packed, int hidden, int K, int splits) -> Tensor", &oproj_packed);
  m.def(
      "alltoall_combine_oproj(Tensor attn_out, Tensor lse, Tensor w, Tensor workspace, int cp_rank, int cp_size, bool "
      "base2, bool emulate, int timeout_ms) -> (Tensor, Tensor)",
      &alltoall_combine_oproj);
  m.def(
      "alltoall_combine_oproj_packed(Tensor attn_out, Tensor lse, Tensor packed, int hidden, Tensor workspace, int cp_rank, "
      "int cp_size, bool base2, int timeout_ms) -> Tensor",
      &alltoall_combine_oproj_packed);
  m.def("read_error_flag(Tensor like) -> int", &read_error_flag);
  m.def("attn_trace(Tensor like) -> Tensor", &attn_trace);
  m.def("clear_error_flag(Tensor like) -> ()", &clear_error_flag);
}

void bind_compute(pybind11::module_& m) {
  m.def("gqa_pick_ctas", &helix::gqa_pick_ctas);
  m.def("oproj_pick_splits", &helix::oproj_pick_splits);
  m.def("fused_oproj_fits", &fused_oproj_fits);
}
