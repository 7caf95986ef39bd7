// Torch bindings of the Helix B200 library.
//
// Op library `helix_a2a_b200` keeps the three op names of the reference
// (csrc/torch_binding.cpp:177-189: get_helix_workspace_size_per_rank,
// initialize_helix_workspace, alltoall_helix_native) with the same validation rules
// (csrc/torch_binding.cpp:68-111) and adds the fused ops.  The pybind module `_C` carries the
// VMM allocator and a few host utilities.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <memory>
#include <mutex>

#include <cstdlib>
#include <limits>
#include <string>

#include "exchange.h"
#include "lse_combine.h"
#include "fifo.cuh"
#include "ll128.cuh"
#include "vmm_workspace.h"

namespace {

int env_int(const char* name, int dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  return std::atoi(v);
}
bool env_pdl() {
  const char* v = std::getenv("HELIX_A2A_ENABLE_PDL");
  return v && std::string(v) == "1";
}
int env_channels() { return std::max(env_int("HELIX_A2A_CHANNEL_COUNT", 0), 0); }
unsigned long long timeout_ns(int64_t timeout_ms) {
  int ms = timeout_ms > 0 ? (int)timeout_ms : std::max(env_int("HELIX_A2A_TIMEOUT_MS", 2000), 1);
  return (unsigned long long)ms * 1000000ull;
}

// what the auto-tuner chose for the most recent exchange launch of this process (debug_info); launches may come
// from several threads (one per device), so reads and writes take the lock
std::mutex g_last_launch_mu;
helix::LaunchInfo g_last_launch{};

// HELIX_A2A_DEBUG=1: outputs are pre-filled with NaN so that a row the kernel failed to write shows up
bool env_debug() {
  const char* v = std::getenv("HELIX_A2A_DEBUG");
  return v && v[0] == '1';
}

void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, "helix: ", what, " failed: ", cudaGetErrorString(e));
}

void check_workspace(const torch::Tensor& workspace, int64_t cp_size) {
  TORCH_CHECK(workspace.is_cuda(), "workspace must be on CUDA");
  TORCH_CHECK(workspace.scalar_type() == at::ScalarType::Long, "workspace must be int64 (used as uint64)");
  TORCH_CHECK(workspace.dim() == 2, "workspace must be 2D (strided across ranks)");
  TORCH_CHECK(workspace.size(0) == cp_size, "workspace must have cp_size rows");
  TORCH_CHECK(workspace.stride(1) == 1, "workspace rows must be contiguous");
  int64_t need = helix::workspace_bytes_per_rank((int)cp_size, helix::device_sm_count());
  TORCH_CHECK(workspace.size(1) * 8 >= need, "workspace rows are too small: ", workspace.size(1) * 8, " < ", need);
}

// device timeline of the exchange kernel (HELIX_A2A_EXCHANGE_TRACE=1): one buffer per device, overwritten by every call
std::map<int, torch::Tensor> g_exchange_trace;
constexpr int64_t kTraceWords = (int64_t)helix::kMaxEmulatedRanks * 256 * 8;

unsigned long long* exchange_trace_buffer(const torch::Device& dev) {
  static const bool on = [] { const char* v = std::getenv("HELIX_A2A_EXCHANGE_TRACE"); return v && std::string(v) == "1"; }();
  if (!on) return nullptr;
  torch::Tensor& t = g_exchange_trace[dev.index()];
  if (!t.defined()) t = torch::zeros({kTraceWords}, torch::TensorOptions().dtype(torch::kInt64).device(dev));
  return reinterpret_cast<unsigned long long*>(t.data_ptr());
}

torch::Tensor exchange_trace(torch::Tensor like) {
  auto it = g_exchange_trace.find(like.device().index());
  TORCH_CHECK(it != g_exchange_trace.end() && it->second.defined(), "no exchange trace: set HELIX_A2A_EXCHANGE_TRACE=1");
  return it->second.clone().view({-1, 8});
}

void fill_workspace(helix::ExchangeParams& p, const torch::Tensor& workspace) {
  p.trace = exchange_trace_buffer(workspace.device());
  p.workspace = reinterpret_cast<uint64_t*>(workspace.data_ptr());
  p.row_stride_bytes = workspace.stride(0) * 8;
  p.sm_count = helix::device_sm_count();
}

void launch(helix::ExchangeParams& p, int64_t timeout_ms) {
  p.timeout_ns = timeout_ns(timeout_ms);
  auto stream = at::cuda::getCurrentCUDAStream();
  helix::LaunchInfo li{};
  check_cuda(helix::launch_exchange(p, env_channels(), env_pdl(), stream, &li), "exchange launch");
  {
    std::lock_guard<std::mutex> lk(g_last_launch_mu);
    g_last_launch = li;
  }
}

int64_t get_helix_workspace_size_per_rank(int64_t cp_size) {
  TORCH_CHECK(cp_size >= 1 && cp_size <= helix::kMaxCp, "cp_size must be in [1, ", helix::kMaxCp, "]");
  return helix::workspace_bytes_per_rank((int)cp_size, helix::device_sm_count());
}

void initialize_helix_workspace(torch::Tensor workspace, int64_t cp_rank, int64_t cp_size) {
  check_workspace(workspace, cp_size);
  TORCH_CHECK(cp_rank >= 0 && cp_rank < cp_size, "cp_rank must be in [0, cp_size)");
  c10::cuda::CUDAGuard guard(workspace.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  uint64_t* row = reinterpret_cast<uint64_t*>(workspace.data_ptr()) + cp_rank * workspace.stride(0);
  check_cuda(helix::initialize_workspace_row(row, (int)cp_size, helix::device_sm_count(), stream), "workspace init");
}

// ---- exchange with the reference's contract ---------------------------------------------------
// emulate: tensors carry a leading [cp_size] dim (rank r's inputs at index r) and ONE launch plays
// all ranks against a single-process workspace.
std::tuple<torch::Tensor, torch::Tensor> alltoall_impl(torch::Tensor partial_o, torch::Tensor softmax_stats,
                                                       torch::Tensor workspace, int64_t cp_rank, int64_t cp_size,
                                                       bool emulate, int64_t skip_peer_mask, int64_t timeout_ms) {
  TORCH_CHECK(partial_o.is_cuda(), "partial_o must be on CUDA");
  TORCH_CHECK(softmax_stats.is_cuda(), "softmax_stats must be on CUDA");
  TORCH_CHECK(partial_o.is_contiguous(), "partial_o must be contiguous");
  TORCH_CHECK(softmax_stats.is_contiguous(), "softmax_stats must be contiguous");
  TORCH_CHECK(partial_o.scalar_type() == at::ScalarType::Half || partial_o.scalar_type() == at::ScalarType::BFloat16,
              "partial_o must be half or bfloat16");
  TORCH_CHECK(softmax_stats.scalar_type() == at::ScalarType::Float, "softmax_stats must be float32");
  const int lead = emulate ? 1 : 0;
  TORCH_CHECK(partial_o.dim() >= 2 + lead, "partial_o must have at least 2 dimensions");
  TORCH_CHECK(softmax_stats.dim() >= 2 + lead, "softmax_stats must have at least 2 dimensions");
  TORCH_CHECK(partial_o.dim() == softmax_stats.dim(), "partial_o and softmax_stats must have same number of dimensions");
  TORCH_CHECK(partial_o.size(-2) == cp_size && softmax_stats.size(-2) == cp_size,
              "second-to-last dimension must equal cp_size");
  TORCH_CHECK(softmax_stats.size(-1) % 2 == 0 && softmax_stats.size(-1) >= 2,
              "softmax_stats last dimension must be divisible by 2 (float2)");
  for (int i = 0; i < partial_o.dim() - 2; i++)
    TORCH_CHECK(partial_o.size(i) == softmax_stats.size(i),
                "partial_o and softmax_stats must have matching dimensions except last two");
  const int64_t D = partial_o.size(-1), S = softmax_stats.size(-1), es = partial_o.element_size();
  TORCH_CHECK(D * es % 16 == 0, "partial_o must be aligned to 16 bytes");
  check_workspace(workspace, cp_size);
  TORCH_CHECK(cp_rank >= 0 && cp_rank < cp_size, "cp_rank must be in [0, cp_size)");
  if (emulate) {
    TORCH_CHECK(partial_o.size(0) == cp_size, "emulated exchange needs a leading [cp_size] dimension");
    TORCH_CHECK(cp_size <= helix::kMaxEmulatedRanks, "at most ", helix::kMaxEmulatedRanks, " ranks per launch");
  }
  c10::cuda::CUDAGuard guard(partial_o.device());

  int64_t entries = 1;
  for (int i = lead; i < partial_o.dim() - 2; i++) entries *= partial_o.size(i);
  torch::Tensor o_out = torch::empty_like(partial_o);
  torch::Tensor s_out = torch::empty_like(softmax_stats);
  if (env_debug()) {
    o_out.fill_(std::numeric_limits<float>::quiet_NaN());
    s_out.fill_(std::numeric_limits<float>::quiet_NaN());
  }
  if (entries == 0) return std::make_tuple(o_out, s_out);
  TORCH_CHECK(entries < (int64_t(1) << 30), "too many entries");

  helix::ExchangeParams p{};
  const int ranks = emulate ? (int)cp_size : 1;
  const int64_t o_rank_bytes = entries * cp_size * D * es, s_rank_bytes = entries * cp_size * S * 4;
  for (int r = 0; r < ranks; ++r) {
    p.io[r].o_src = reinterpret_cast<const uint8_t*>(partial_o.data_ptr()) + r * o_rank_bytes;
    p.io[r].st_src = reinterpret_cast<const uint8_t*>(softmax_stats.data_ptr()) + r * s_rank_bytes;
    p.io[r].o_dst = reinterpret_cast<uint8_t*>(o_out.data_ptr()) + r * o_rank_bytes;
    p.io[r].st_dst = reinterpret_cast<uint8_t*>(s_out.data_ptr()) + r * s_rank_bytes;
  }
  fill_workspace(p, workspace);
  p.cp_size = (int)cp_size;
  p.rank_base = emulate ? 0 : (int)cp_rank;
  p.ranks_in_launch = ranks;
  p.outer = (int)entries;
  p.inner = 1;
  p.o_sb = cp_size * D * es;  p.o_sp = D * es;  p.o_sh = 0;
  p.st_sb = cp_size * S * 4;  p.st_sp = S * 4;  p.st_sh = 0;
  p.od_se = cp_size * D * es; p.od_sp = D * es;
  p.sd_se = cp_size * S * 4;  p.sd_sp = S * 4;
  p.o_bytes = (int)(D * es);
  p.st_words = (int)(S / 2);
  p.lse_scalar = 0;
  p.is_bf16 = partial_o.scalar_type() == at::ScalarType::BFloat16;
  p.mode = helix::kModeExchange;
  p.skip_peer_mask = (uint32_t)skip_peer_mask;
  // debug bounds checks: one rank's byte extents; checked per message on the device with HELIX_A2A_DEBUG=1
  p.o_src_bytes = p.o_dst_bytes = o_rank_bytes;
  p.st_src_bytes = p.st_dst_bytes = s_rank_bytes;
  p.debug_checks = env_debug() ? 1 : 0;
  launch(p, timeout_ms);
  return std::make_tuple(o_out, s_out);
}

std::tuple<torch::Tensor, torch::Tensor> alltoall_helix_native(torch::Tensor partial_o, torch::Tensor softmax_stats,
                                                               torch::Tensor workspace, int64_t cp_rank,
                                                               int64_t cp_size) {
  return alltoall_impl(partial_o, softmax_stats, workspace, cp_rank, cp_size, false, 0, 0);
}

// ---- stand-alone LSE combine -------------------------------------------------------------------------
// rank_dim 0: outputs [N, ..., D], lses [N, ...];  rank_dim -2: outputs [..., N, D], lses [..., N] (the layout
// `alltoall` returns; lses may be a strided view such as recv_stats[..., 0]).  Result [..., D] (+ global LSE).
std::tuple<torch::Tensor, torch::Tensor> lse_combine(torch::Tensor outputs, torch::Tensor lses, int64_t rank_dim,
                                                     bool return_lse, bool base2) {
  TORCH_CHECK(outputs.is_cuda() && lses.is_cuda(), "inputs must be on CUDA");
  TORCH_CHECK(outputs.scalar_type() == at::ScalarType::Half || outputs.scalar_type() == at::ScalarType::BFloat16,
              "outputs must be half or bfloat16");
  TORCH_CHECK(lses.scalar_type() == at::ScalarType::Float, "lses must be float32");
  TORCH_CHECK(rank_dim == 0 || rank_dim == -2, "rank_dim must be 0 ([N, ..., D]) or -2 ([..., N, D])");
  TORCH_CHECK(outputs.dim() >= 2 && lses.dim() == outputs.dim() - 1, "outputs [.., D] needs lses with one dim less");
  outputs = outputs.contiguous();
  const int64_t D = outputs.size(-1), es = outputs.element_size();
  TORCH_CHECK(D * es % 16 == 0 && D * es <= 2048, "row size must be a multiple of 16 bytes, at most 2048");
  const int64_t N = rank_dim == 0 ? outputs.size(0) : outputs.size(-2);
  int64_t rows = 1;
  std::vector<int64_t> shape, lshape;
  for (int i = 0; i < outputs.dim() - 1; ++i) {
    const bool is_rank = (rank_dim == 0 && i == 0) || (rank_dim == -2 && i == outputs.dim() - 2);
    TORCH_CHECK(lses.size(i) == outputs.size(i), "lses must match the leading dims of outputs");
    if (is_rank) continue;
    rows *= outputs.size(i);
    shape.push_back(outputs.size(i));
    lshape.push_back(outputs.size(i));
  }
  shape.push_back(D);
  // LSEs as [N, rows] or [rows, N] with arbitrary (uniform) strides: flatten through a contiguous copy only if needed
  torch::Tensor l2 = rank_dim == 0 ? lses.reshape({N, rows}) : lses.reshape({rows, N});
  c10::cuda::CUDAGuard guard(outputs.device());
  torch::Tensor out = torch::empty(shape, outputs.options());
  torch::Tensor lse_out = return_lse ? torch::empty(lshape, lses.options()) : torch::empty({0}, lses.options());
  helix::LseCombineParams p{};
  p.o = reinterpret_cast<const uint8_t*>(outputs.data_ptr());
  p.lse = reinterpret_cast<const uint8_t*>(l2.data_ptr());
  p.out = reinterpret_cast<uint8_t*>(out.data_ptr());
  p.lse_out = return_lse ? lse_out.data_ptr<float>() : nullptr;
  if (rank_dim == 0) {
    p.o_sn = rows * D * es; p.o_sr = D * es;
    p.l_sn = l2.stride(0) * 4; p.l_sr = l2.stride(1) * 4;
  } else {
    p.o_sn = D * es; p.o_sr = N * D * es;
    p.l_sn = l2.stride(1) * 4; p.l_sr = l2.stride(0) * 4;
  }
  p.out_sr = D * es;
  p.rows = rows;
  p.n = (int)N;
  p.row_bytes = (int)(D * es);
  p.is_bf16 = outputs.scalar_type() == at::ScalarType::BFloat16;
  p.base2 = base2 ? 1 : 0;
  cudaError_t e = helix::launch_lse_combine(p, env_pdl(), at::cuda::getCurrentCUDAStream());
  TORCH_CHECK(e == cudaSuccess, "helix: lse_combine launch failed: ", cudaGetErrorString(e));
  return std::make_tuple(out, lse_out);
}

// ---- fused exchange + LSE combine ------------------------------------------------------------------
// layout 0 ("native"): attn_out [B, H, D], stats [B, H] (LSE) or [B, H, 2]; result [B, H/cp, D]
// layout 1 ("entries"): partial_o [..., cp, D], stats [..., cp, 2]; result [..., D]
// emulate: leading [cp] dim on inputs and outputs.
std::tuple<torch::Tensor, torch::Tensor> alltoall_combine(torch::Tensor attn_out, torch::Tensor stats,
                                                          torch::Tensor workspace, int64_t cp_rank, int64_t cp_size,
                                                          int64_t layout, bool return_lse, bool base2,
                                                          int64_t stats_mode, bool emulate, int64_t skip_peer_mask,
                                                          int64_t timeout_ms) {
  TORCH_CHECK(attn_out.is_cuda() && stats.is_cuda(), "inputs must be on CUDA");
  TORCH_CHECK(attn_out.scalar_type() == at::ScalarType::Half || attn_out.scalar_type() == at::ScalarType::BFloat16,
              "attention output must be half or bfloat16");
  TORCH_CHECK(stats.scalar_type() == at::ScalarType::Float, "softmax stats / LSE must be float32");
  TORCH_CHECK(attn_out.is_contiguous() && stats.is_contiguous(), "inputs must be contiguous");
  check_workspace(workspace, cp_size);
  TORCH_CHECK(cp_rank >= 0 && cp_rank < cp_size, "cp_rank must be in [0, cp_size)");
  TORCH_CHECK(stats_mode == 0 || stats_mode == 1, "stats_mode must be 0 (lse) or 1 (max, sum-exp)");
  const int lead = emulate ? 1 : 0;
  if (emulate) {
    TORCH_CHECK(attn_out.size(0) == cp_size && stats.size(0) == cp_size, "emulation needs a leading [cp_size] dim");
    TORCH_CHECK(cp_size <= helix::kMaxEmulatedRanks, "at most ", helix::kMaxEmulatedRanks, " ranks per launch");
  }
  const int64_t es = attn_out.element_size();
  const int64_t D = attn_out.size(-1);
  TORCH_CHECK(D * es % 16 == 0, "row size must be a multiple of 16 bytes");
  c10::cuda::CUDAGuard guard(attn_out.device());
  const int ranks = emulate ? (int)cp_size : 1;
  helix::ExchangeParams p{};
  torch::Tensor out, lse_out;
  int64_t in_o_rank_bytes, in_s_rank_bytes, out_rank_bytes, lse_rank_bytes;

  if (layout == 0) {
    TORCH_CHECK(attn_out.dim() == 3 + lead, "attn_out must be [B, H, D]");
    const int64_t B = attn_out.size(lead), H = attn_out.size(lead + 1);
    TORCH_CHECK(H % cp_size == 0, "number of heads must be divisible by cp_size");
    const int64_t Hl = H / cp_size;
    bool scalar = stats.dim() == 2 + lead;
    TORCH_CHECK(scalar || (stats.dim() == 3 + lead && stats.size(-1) == 2), "stats must be [B, H] or [B, H, 2]");
    TORCH_CHECK(stats.size(lead) == B && stats.size(lead + 1) == H, "stats must match attn_out's [B, H]");
    TORCH_CHECK(!(scalar && stats_mode == 1), "(max, sum-exp) stats need a [B, H, 2] tensor");
    auto shape = std::vector<int64_t>{B, Hl, D};
    auto lshape = std::vector<int64_t>{B, Hl};
    if (emulate) { shape.insert(shape.begin(), cp_size); lshape.insert(lshape.begin(), cp_size); }
    out = torch::empty(shape, attn_out.options());
    lse_out = return_lse ? torch::empty(lshape, stats.options()) : torch::empty({0}, stats.options());
    p.outer = (int)B; p.inner = (int)Hl;
    p.o_sb = H * D * es; p.o_sp = Hl * D * es; p.o_sh = D * es;
    const int64_t sw = scalar ? 4 : 8;
    p.st_sb = H * sw; p.st_sp = Hl * sw; p.st_sh = sw;
    p.lse_scalar = scalar ? 1 : 0;
    in_o_rank_bytes = B * H * D * es; in_s_rank_bytes = B * H * sw;
    out_rank_bytes = B * Hl * D * es; lse_rank_bytes = B * Hl * 4;
  } else {
    TORCH_CHECK(attn_out.dim() >= 2 + lead && attn_out.dim() == stats.dim(), "partial_o / stats rank mismatch");
    TORCH_CHECK(attn_out.size(-2) == cp_size && stats.size(-2) == cp_size, "second-to-last dimension must equal cp_size");
    TORCH_CHECK(stats.size(-1) == 2, "fused combine needs softmax_stats[..., 2]");
    int64_t entries = 1;
    std::vector<int64_t> shape, lshape;
    for (int i = 0; i < attn_out.dim() - 2; i++) {
      TORCH_CHECK(attn_out.size(i) == stats.size(i), "leading dimensions must match");
      if (i >= lead) entries *= attn_out.size(i);
      shape.push_back(attn_out.size(i));
      lshape.push_back(attn_out.size(i));
    }
    shape.push_back(D);
    out = torch::empty(shape, attn_out.options());
    lse_out = return_lse ? torch::empty(lshape, stats.options()) : torch::empty({0}, stats.options());
    p.outer = (int)entries; p.inner = 1;
    p.o_sb = cp_size * D * es; p.o_sp = D * es; p.o_sh = 0;
    p.st_sb = cp_size * 8; p.st_sp = 8; p.st_sh = 0;
    p.lse_scalar = 0;
    in_o_rank_bytes = entries * cp_size * D * es; in_s_rank_bytes = entries * cp_size * 8;
    out_rank_bytes = entries * D * es; lse_rank_bytes = entries * 4;
  }
  if (env_debug()) out.fill_(std::numeric_limits<float>::quiet_NaN());
  if ((int64_t)p.outer * p.inner == 0) return std::make_tuple(out, lse_out);
  for (int r = 0; r < ranks; ++r) {
    p.io[r].o_src = reinterpret_cast<const uint8_t*>(attn_out.data_ptr()) + r * in_o_rank_bytes;
    p.io[r].st_src = reinterpret_cast<const uint8_t*>(stats.data_ptr()) + r * in_s_rank_bytes;
    p.io[r].o_dst = reinterpret_cast<uint8_t*>(out.data_ptr()) + r * out_rank_bytes;
    p.io[r].st_dst = return_lse ? reinterpret_cast<uint8_t*>(lse_out.data_ptr()) + r * lse_rank_bytes : nullptr;
  }
  fill_workspace(p, workspace);
  p.cp_size = (int)cp_size;
  p.rank_base = emulate ? 0 : (int)cp_rank;
  p.ranks_in_launch = ranks;
  p.od_se = D * es;
  p.o_bytes = (int)(D * es);
  p.st_words = 1;
  p.is_bf16 = attn_out.scalar_type() == at::ScalarType::BFloat16;
  p.mode = helix::kModeCombine;
  p.stats_mode = (int)stats_mode;
  p.base2 = base2 ? 1 : 0;
  p.o_src_bytes = in_o_rank_bytes;
  p.st_src_bytes = in_s_rank_bytes;
  p.o_dst_bytes = out_rank_bytes;
  p.st_dst_bytes = lse_rank_bytes;
  p.debug_checks = env_debug() ? 1 : 0;
  p.skip_peer_mask = (uint32_t)skip_peer_mask;
  launch(p, timeout_ms);
  return std::make_tuple(out, lse_out);
}

std::tuple<torch::Tensor, torch::Tensor> alltoall_debug(torch::Tensor partial_o, torch::Tensor softmax_stats,
                                                        torch::Tensor workspace, int64_t cp_rank, int64_t cp_size,
                                                        bool emulate, int64_t skip_peer_mask, int64_t timeout_ms) {
  return alltoall_impl(partial_o, softmax_stats, workspace, cp_rank, cp_size, emulate, skip_peer_mask, timeout_ms);
}

// status block of a row as 8 int64 values on the host (synchronises the current stream)
torch::Tensor read_status(torch::Tensor workspace, int64_t cp_rank, int64_t cp_size) {
  check_workspace(workspace, cp_size);
  helix::WorkspaceLayout lay = helix::make_layout((int)cp_size, helix::device_sm_count());
  c10::cuda::CUDAGuard guard(workspace.device());
  auto stream = at::cuda::getCurrentCUDAStream();
  torch::Tensor host = torch::empty({8}, torch::dtype(torch::kInt64));
  const uint8_t* src = reinterpret_cast<const uint8_t*>(workspace.data_ptr()) + cp_rank * workspace.stride(0) * 8 +
                       lay.status_offset;
  check_cuda(cudaMemcpyAsync(host.data_ptr(), src, 64, cudaMemcpyDeviceToHost, stream), "status read");
  check_cuda(cudaStreamSynchronize(stream), "status sync");
  return host;
}

}  // namespace

// defined in binding_ops.cpp: attention / o_proj / fused ops
void register_compute_ops(torch::Library& m);
void bind_compute(pybind11::module_& m);

TORCH_LIBRARY(helix_a2a_b200, m) {
  m.def("get_helix_workspace_size_per_rank(int cp_size) -> int", &get_helix_workspace_size_per_rank);
  m.def("initialize_helix_workspace(Tensor workspace, int cp_rank, int cp_size) -> ()", &initialize_helix_workspace);
  m.def(
      "alltoall_helix_native(Tensor partial_o, Tensor softmax_stats, Tensor workspace, int cp_rank, int cp_size) -> "
      "(Tensor, Tensor)",
      &alltoall_helix_native);
  m.def(
      "alltoall_debug(Tensor partial_o, Tensor softmax_stats, Tensor workspace, int cp_rank, int cp_size, bool emulate, "
      "int skip_peer_mask, int timeout_ms) -> (Tensor, Tensor)",
      &alltoall_debug);
  m.def(
      "alltoall_combine(Tensor attn_out, Tensor stats, Tensor workspace, int cp_rank, int cp_size, int layout, bool "
      "return_lse, bool base2, int stats_mode, bool emulate, int skip_peer_mask, int timeout_ms) -> (Tensor, Tensor)",
      &alltoall_combine);
  m.def("read_status(Tensor workspace, int cp_rank, int cp_size) -> Tensor", &read_status);
  m.def("exchange_trace(Tensor like) -> Tensor", &exchange_trace);
  m.def("lse_combine(Tensor outputs, Tensor lses, int rank_dim, bool return_lse, bool base2) -> (Tensor, Tensor)",
        &lse_combine);
  register_compute_ops(m);
}

// ---- pybind module: allocator + host utilities ---------------------------------------------------
namespace py = pybind11;

// Allocations are shared between the Python handle and every tensor made from them: the mappings go away when
// the last of these is gone, so an alias of the workspace that outlives the handle object stays valid.
static std::mutex g_vmm_mu;
static std::map<uintptr_t, std::shared_ptr<helix::vmm::Allocation>> g_vmm;

static uintptr_t vmm_register(helix::vmm::Allocation* a) {
  std::lock_guard<std::mutex> lk(g_vmm_mu);
  g_vmm[(uintptr_t)a] = std::shared_ptr<helix::vmm::Allocation>(a, [](helix::vmm::Allocation* p) { helix::vmm::destroy(p); });
  return (uintptr_t)a;
}

static torch::Tensor vmm_as_tensor(uintptr_t handle, int64_t device) {
  std::shared_ptr<helix::vmm::Allocation> owner;
  {
    std::lock_guard<std::mutex> lk(g_vmm_mu);
    auto it = g_vmm.find(handle);
    TORCH_CHECK(it != g_vmm.end(), "helix: unknown or closed workspace handle");
    owner = it->second;
  }
  auto* a = owner.get();
  int64_t cp = helix::vmm::cp_size(a);
  int64_t elems = (int64_t)helix::vmm::mapped_row_bytes(a) / 8;
  int64_t stride = (int64_t)helix::vmm::row_stride(a) / 8;
  // Row 0 may be another GPU's memory, so the pointer's own device is not this rank's device:
  // name the target device explicitly instead of letting ATen query the pointer.
  auto opts = torch::TensorOptions().dtype(torch::kInt64).device(torch::kCUDA);
  return at::for_blob(reinterpret_cast<void*>(helix::vmm::base_address(a)), {cp, elems})
      .strides({stride, 1})
      .deleter([owner](void*) mutable { owner.reset(); })     // the storage holds a share of the allocation
      .options(opts)
      .target_device(c10::Device(c10::kCUDA, (c10::DeviceIndex)device))
      .make_tensor();
}

PYBIND11_MODULE(_C, m) {
  m.doc() = "helix_a2a_b200 native module";
  m.def("vmm_create", [](int cp, int rank, int device, size_t row_bytes, int kind) {
    return vmm_register(helix::vmm::create(cp, rank, device, row_bytes, (helix::vmm::HandleKind)kind));
  });
  m.def("vmm_create_single_process", [](std::vector<int> devices, size_t row_bytes) {
    return vmm_register(helix::vmm::create_single_process(devices, row_bytes));
  });
  m.def("vmm_export_fd", [](uintptr_t h) { return helix::vmm::export_fd((helix::vmm::Allocation*)h); });
  m.def("vmm_export_fabric", [](uintptr_t h) { return py::bytes(helix::vmm::export_fabric((helix::vmm::Allocation*)h)); });
  m.def("vmm_map_local", [](uintptr_t h) { helix::vmm::map_local((helix::vmm::Allocation*)h); });
  m.def("vmm_map_peer_fd", [](uintptr_t h, int peer, int fd) { helix::vmm::map_peer_fd((helix::vmm::Allocation*)h, peer, fd); });
  m.def("vmm_map_peer_fabric", [](uintptr_t h, int peer, std::string blob) {
    helix::vmm::map_peer_fabric((helix::vmm::Allocation*)h, peer, blob);
  });
  m.def("vmm_dup_fd_from_pid", &helix::vmm::dup_fd_from_pid);
  m.def("vmm_send_fd_unix", &helix::vmm::send_fd_unix, py::call_guard<py::gil_scoped_release>());
  m.def("vmm_recv_fd_unix", &helix::vmm::recv_fd_unix, py::call_guard<py::gil_scoped_release>());
  m.def("vmm_fabric_supported", &helix::vmm::fabric_supported);
  m.def("vmm_row_stride", [](uintptr_t h) { return helix::vmm::row_stride((helix::vmm::Allocation*)h); });
  m.def("vmm_row_bytes", [](uintptr_t h) { return helix::vmm::mapped_row_bytes((helix::vmm::Allocation*)h); });
  m.def("vmm_base", [](uintptr_t h) { return helix::vmm::base_address((helix::vmm::Allocation*)h); });
  m.def("vmm_tensor", &vmm_as_tensor);
  // drops the handle's share; the rows are unmapped once no tensor made from the handle is alive either
  m.def("vmm_destroy", [](uintptr_t h) {
    std::shared_ptr<helix::vmm::Allocation> last;
    {
      std::lock_guard<std::mutex> lk(g_vmm_mu);
      auto it = g_vmm.find(h);
      if (it == g_vmm.end()) return;
      last = std::move(it->second);
      g_vmm.erase(it);
    }
  });
  m.def("close_fd", [](int fd) { return ::close(fd); });

  m.def("last_launch_info", []() {
    helix::LaunchInfo li;
    {
      std::lock_guard<std::mutex> lk(g_last_launch_mu);
      li = g_last_launch;
    }
    py::dict d;
    d["channels"] = li.channels;
    d["send_warps"] = li.send_warps;
    d["recv_warps"] = li.recv_warps;
    d["group_warps"] = li.group_warps;
    d["lines_per_message"] = li.lines_per_message;
    d["iters"] = li.iters;
    d["cooperative"] = li.cooperative;
    return d;
  });
  m.def("layout", [](int cp, int sm_count) {
    helix::WorkspaceLayout l = helix::make_layout(cp, sm_count);
    py::dict d;
    d["max_channels"] = l.max_channels;
    d["ring_region"] = l.ring_region;
    d["sinfo_offset"] = l.sinfo_offset;
    d["rinfo_offset"] = l.rinfo_offset;
    d["status_offset"] = l.status_offset;
    d["row_bytes"] = l.row_bytes;
    d["ring_bytes"] = helix::kRingBytes;
    d["ring_lines"] = helix::kRingLines;
    return d;
  });
  m.def("wire_bytes", [](int payload_bytes) { return helix::ll128::wire_bytes_for_words((payload_bytes + 7) / 8); });
  // what the auto-tuner would choose for a call (no launch, no GPU): entries = outer * inner rows of o_bytes + stats
  m.def("plan_info", [](int cp, int sm_count, int outer, int inner, int o_bytes, int st_words, bool combine) {
    helix::ExchangeParams p{};
    p.cp_size = cp; p.sm_count = sm_count; p.outer = outer; p.inner = inner; p.o_bytes = o_bytes; p.st_words = st_words;
    p.mode = combine ? helix::kModeCombine : helix::kModeExchange;
    p.ranks_in_launch = 1;
    helix::LaunchInfo li = helix::plan_launch(p, 0);
    py::dict d;
    d["channels"] = li.channels;
    d["send_warps"] = li.send_warps;
    d["recv_warps"] = li.recv_warps;
    d["group_warps"] = li.group_warps;
    d["lines_per_message"] = li.lines_per_message;
    d["iters"] = li.iters;
    return d;
  });
  bind_compute(m);
}
