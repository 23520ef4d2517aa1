// Python bindings: torch tensors in, raw pointers + current CUDA stream out to
// the C launchers declared in dsb_api.h.  No kernels here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>
#include <vector>

#include "dsb_api.h"
#include "dsb_api_ops.h"

namespace {

using torch::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.scalar_type() == torch::kBFloat16 &&
                  t.stride(1) == 1,
              name, ": expected a 2-D bf16 CUDA tensor with unit inner stride");
  TORCH_CHECK(t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name,
              ": row stride must be a multiple of 8 elements and the base 16-byte aligned");
}
const float* opt_f32(const c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous());
  return t->data_ptr<float>();
}
float* opt_f32_mut(c10::optional<Tensor>& t) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == torch::kFloat32 && t->is_contiguous());
  return t->data_ptr<float>();
}
DsbGate to_gate(const std::vector<double>& g) {
  TORCH_CHECK(g.size() == 8, "gate: expected 8 numbers");
  DsbGate d;
  d.kind = static_cast<int>(g[0]);
  d.sharpness = g[1]; d.act_threshold = g[2]; d.act_cutoff = g[3]; d.epsilon = g[4];
  d.max_intensity = g[5]; d.clip_max = g[6]; d.dead_threshold = g[7];
  return d;
}

// C (=|+=) alpha * row_scale * op(A) . op(B)^T + bias.
//   a_mn == false: A is [M,K];  a_mn == true: A is stored [K,M]
//   b_mn == false: B is [N,K];  b_mn == true: B is stored [K,N]
void gemm(const Tensor& A, bool a_mn, const Tensor& B, bool b_mn, Tensor& C, bool accumulate,
          double alpha, c10::optional<Tensor> row_scale, c10::optional<Tensor> bias,
          int64_t block_n, Tensor& status) {
  check_bf16_2d(A, "A");
  check_bf16_2d(B, "B");
  const c10::cuda::CUDAGuard guard(A.device());
  const int64_t M = a_mn ? A.size(1) : A.size(0);
  const int64_t K = a_mn ? A.size(0) : A.size(1);
  const int64_t N = b_mn ? B.size(1) : B.size(0);
  TORCH_CHECK((b_mn ? B.size(0) : B.size(1)) == K, "gemm: K mismatch");
  TORCH_CHECK(C.is_cuda() && C.dim() == 2 && C.size(0) == M && C.size(1) == N && C.stride(1) == 1,
              "gemm: bad C");
  const bool c_bf16 = C.scalar_type() == torch::kBFloat16;
  TORCH_CHECK(c_bf16 || C.scalar_type() == torch::kFloat32, "gemm: C must be bf16 or fp32");
  TORCH_CHECK(!(accumulate && c_bf16), "gemm: accumulate needs an fp32 C");
  int rc = dsb_gemm_bf16(A.data_ptr(), a_mn, A.stride(0), B.data_ptr(), b_mn, B.stride(0), M, N, K,
                         C.data_ptr(), C.stride(0), c_bf16, accumulate, alpha, opt_f32(row_scale),
                         opt_f32(bias), block_n, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_gemm_bf16 failed with code ", rc);
}

void srw_fwd_gate(const Tensor& h, const Tensor& emb, const Tensor& x, const Tensor& read,
                  Tensor& p_out, const Tensor& tau, const Tensor& inv_sigma, Tensor& den_sum,
                  c10::optional<Tensor> gate_sum, c10::optional<Tensor> alive,
                  c10::optional<Tensor> unit_mask, std::vector<double> gate, Tensor& status) {
  check_bf16_2d(h, "h"); check_bf16_2d(emb, "emb"); check_bf16_2d(x, "x");
  check_bf16_2d(read, "read"); check_bf16_2d(p_out, "p_out");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1), U = emb.size(0), r = emb.size(1);
  TORCH_CHECK(h.size(0) == T && h.size(1) == r && read.size(0) == U && read.size(1) == D);
  TORCH_CHECK(p_out.size(0) == T && p_out.size(1) >= U);
  DsbGate g = to_gate(gate);
  unsigned char* alive_p = nullptr;
  if (alive.has_value() && alive->defined()) {
    TORCH_CHECK(alive->scalar_type() == torch::kUInt8 && alive->numel() >= U);
    alive_p = alive->data_ptr<unsigned char>();
  }
  int rc = dsb_srw_fwd_gate(h.data_ptr(), h.stride(0), emb.data_ptr(), emb.stride(0), x.data_ptr(),
                            x.stride(0), read.data_ptr(), read.stride(0), T, U, r, D,
                            p_out.data_ptr(), p_out.stride(0), tau.data_ptr<float>(),
                            inv_sigma.data_ptr<float>(), den_sum.data_ptr<float>(),
                            opt_f32_mut(gate_sum), alive_p, opt_f32(unit_mask), &g,
                            status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_fwd_gate failed with code ", rc);
}

void srw_bwd_gate(const Tensor& h, const Tensor& emb, const Tensor& x, const Tensor& read,
                  const Tensor& dy, const Tensor& write, Tensor& p_out, Tensor& dxr_out,
                  Tensor& ds_out, const Tensor& tau, const Tensor& inv_sigma, const Tensor& dden,
                  Tensor& dtau_sum, Tensor& dsz_sum, std::vector<double> gate, Tensor& status) {
  check_bf16_2d(h, "h"); check_bf16_2d(emb, "emb"); check_bf16_2d(x, "x");
  check_bf16_2d(read, "read"); check_bf16_2d(dy, "dy"); check_bf16_2d(write, "write");
  check_bf16_2d(p_out, "p_out"); check_bf16_2d(dxr_out, "dxr_out"); check_bf16_2d(ds_out, "ds_out");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1), U = emb.size(0), r = emb.size(1);
  TORCH_CHECK(p_out.stride(0) == dxr_out.stride(0) && p_out.stride(0) == ds_out.stride(0));
  DsbGate g = to_gate(gate);
  int rc = dsb_srw_bwd_gate(h.data_ptr(), h.stride(0), emb.data_ptr(), emb.stride(0), x.data_ptr(),
                            x.stride(0), read.data_ptr(), read.stride(0), dy.data_ptr(),
                            dy.stride(0), write.data_ptr(), write.stride(0), T, U, r, D,
                            p_out.data_ptr(), dxr_out.data_ptr(), ds_out.data_ptr(),
                            p_out.stride(0), tau.data_ptr<float>(), inv_sigma.data_ptr<float>(),
                            dden.data_ptr<float>(), dtau_sum.data_ptr<float>(),
                            dsz_sum.data_ptr<float>(), &g, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_bwd_gate failed with code ", rc);
}

void srw_forward(const Tensor& h, const Tensor& emb, const Tensor& x, const Tensor& read,
                 const Tensor& write, const Tensor& tau, const Tensor& inv_sigma, Tensor& p_scratch,
                 Tensor& raw_out, Tensor& den_sum, c10::optional<Tensor> alive,
                 c10::optional<Tensor> unit_mask, std::vector<double> gate, Tensor& status) {
  check_bf16_2d(h, "h"); check_bf16_2d(emb, "emb"); check_bf16_2d(x, "x");
  check_bf16_2d(read, "read"); check_bf16_2d(write, "write"); check_bf16_2d(p_scratch, "p_scratch");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1), U = emb.size(0), r = emb.size(1);
  TORCH_CHECK(h.size(0) == T && h.size(1) == r && read.size(0) == U && read.size(1) == D &&
              write.size(0) == U && write.size(1) == D);
  TORCH_CHECK(p_scratch.size(0) >= T && p_scratch.stride(0) >= U);
  TORCH_CHECK(raw_out.scalar_type() == torch::kFloat32 && raw_out.size(0) == T &&
              raw_out.size(1) == D && raw_out.stride(1) == 1);
  TORCH_CHECK(den_sum.scalar_type() == torch::kFloat32 && den_sum.numel() >= T);
  DsbGate g = to_gate(gate);
  unsigned char* alive_p = nullptr;
  if (alive.has_value() && alive->defined()) {
    TORCH_CHECK(alive->scalar_type() == torch::kUInt8 && alive->numel() >= U);
    alive_p = alive->data_ptr<unsigned char>();
  }
  int rc = dsb_srw_forward(h.data_ptr(), h.stride(0), emb.data_ptr(), emb.stride(0), x.data_ptr(),
                           x.stride(0), read.data_ptr(), read.stride(0), write.data_ptr(),
                           write.stride(0), T, U, r, D, tau.data_ptr<float>(),
                           inv_sigma.data_ptr<float>(), p_scratch.data_ptr(), p_scratch.stride(0),
                           raw_out.data_ptr<float>(), raw_out.stride(0), den_sum.data_ptr<float>(),
                           alive_p, opt_f32(unit_mask), &g, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_forward failed with code ", rc);
}

struct GatherHolder {
  std::vector<std::vector<const void*>> ptrs;
  std::vector<std::vector<const void*>> stat_ptrs;
  DsbGather g;
};
// stat_lists: for every per-token float4 array, the n_ranks device pointers (as integers)
void fill_gather_stats(GatherHolder& gh, const std::vector<std::vector<int64_t>>& stat_lists) {
  TORCH_CHECK(stat_lists.size() <= 3, "at most three statistics arrays travel with a gather");
  gh.stat_ptrs.resize(stat_lists.size());
  gh.g.n_stats = static_cast<int>(stat_lists.size());
  for (size_t s = 0; s < stat_lists.size(); ++s) {
    TORCH_CHECK(static_cast<int>(stat_lists[s].size()) == gh.g.n_ranks);
    for (auto p : stat_lists[s]) gh.stat_ptrs[s].push_back(reinterpret_cast<const void*>(p));
    gh.g.stats[s] = gh.stat_ptrs[s].data();
  }
}
// tensors: list of (peer pointer list, ld, cols) in the order x, h [, dy]
void fill_gather(GatherHolder& gh, const std::vector<std::vector<int64_t>>& ptr_lists,
                 const std::vector<int64_t>& lds, const std::vector<int64_t>& cols, int64_t my_rank,
                 int64_t rows_per_rank, Tensor& ready, int64_t epoch) {
  memset(&gh.g, 0, sizeof(gh.g));
  gh.ptrs.resize(ptr_lists.size());
  gh.g.n_tensors = static_cast<int>(ptr_lists.size());
  gh.g.n_ranks = static_cast<int>(ptr_lists[0].size());
  gh.g.my_rank = static_cast<int>(my_rank);
  gh.g.rows_per_rank = static_cast<int>(rows_per_rank);
  for (size_t t = 0; t < ptr_lists.size(); ++t) {
    for (auto p : ptr_lists[t]) gh.ptrs[t].push_back(reinterpret_cast<const void*>(p));
    gh.g.bufs[t] = gh.ptrs[t].data();
    gh.g.ld[t] = lds[t];
    gh.g.cols[t] = static_cast<int>(cols[t]);
  }
  TORCH_CHECK(ready.is_cuda() && ready.scalar_type() == torch::kInt32);
  gh.g.ready = reinterpret_cast<unsigned int*>(ready.data_ptr<int>());
  gh.g.epoch = static_cast<unsigned int>(epoch);
}

void srw_fwd_gate_gather(const Tensor& h_full, const Tensor& emb, const Tensor& x_full,
                         const Tensor& read, Tensor& p_out, const Tensor& tau,
                         const Tensor& inv_sigma, Tensor& den_sum, std::vector<double> gate,
                         Tensor& status, std::vector<std::vector<int64_t>> ptr_lists,
                         int64_t my_rank, int64_t rows_per_rank, Tensor& ready, int64_t epoch) {
  check_bf16_2d(h_full, "h_full"); check_bf16_2d(emb, "emb"); check_bf16_2d(x_full, "x_full");
  check_bf16_2d(read, "read"); check_bf16_2d(p_out, "p_out");
  const c10::cuda::CUDAGuard guard(x_full.device());
  const int T = x_full.size(0), D = x_full.size(1), U = emb.size(0), r = emb.size(1);
  DsbGate g = to_gate(gate);
  GatherHolder gh;
  fill_gather(gh, ptr_lists, {x_full.stride(0), h_full.stride(0)}, {D, r}, my_rank, rows_per_rank,
              ready, epoch);
  int rc = dsb_srw_fwd_gate_gather(h_full.data_ptr(), h_full.stride(0), emb.data_ptr(),
                                   emb.stride(0), x_full.data_ptr(), x_full.stride(0),
                                   read.data_ptr(), read.stride(0), T, U, r, D, p_out.data_ptr(),
                                   p_out.stride(0), tau.data_ptr<float>(),
                                   inv_sigma.data_ptr<float>(), den_sum.data_ptr<float>(), nullptr,
                                   nullptr, nullptr, &g, &gh.g, status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_fwd_gate_gather failed with code ", rc);
}

void srw_bwd_gate_gather(const Tensor& h_full, const Tensor& emb, const Tensor& x_full,
                         const Tensor& read, const Tensor& dy_full, const Tensor& write,
                         Tensor& p_out, Tensor& dxr_out, Tensor& ds_out, const Tensor& tau,
                         const Tensor& inv_sigma, const Tensor& dden, Tensor& dtau_sum,
                         Tensor& dsz_sum, std::vector<double> gate, Tensor& status,
                         std::vector<std::vector<int64_t>> ptr_lists, int64_t my_rank,
                         int64_t rows_per_rank, Tensor& ready, int64_t epoch) {
  check_bf16_2d(h_full, "h_full"); check_bf16_2d(x_full, "x_full"); check_bf16_2d(dy_full, "dy_full");
  check_bf16_2d(p_out, "p_out"); check_bf16_2d(dxr_out, "dxr_out"); check_bf16_2d(ds_out, "ds_out");
  const c10::cuda::CUDAGuard guard(x_full.device());
  const int T = x_full.size(0), D = x_full.size(1), U = emb.size(0), r = emb.size(1);
  DsbGate g = to_gate(gate);
  GatherHolder gh;
  fill_gather(gh, ptr_lists, {x_full.stride(0), h_full.stride(0), dy_full.stride(0)}, {D, r, D},
              my_rank, rows_per_rank, ready, epoch);
  int rc = dsb_srw_bwd_gate_gather(
      h_full.data_ptr(), h_full.stride(0), emb.data_ptr(), emb.stride(0), x_full.data_ptr(),
      x_full.stride(0), read.data_ptr(), read.stride(0), dy_full.data_ptr(), dy_full.stride(0),
      write.data_ptr(), write.stride(0), T, U, r, D, p_out.data_ptr(), dxr_out.data_ptr(),
      ds_out.data_ptr(), p_out.stride(0), tau.data_ptr<float>(), inv_sigma.data_ptr<float>(),
      dden.data_ptr<float>(), dtau_sum.data_ptr<float>(), dsz_sum.data_ptr<float>(), &g, &gh.g,
      status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_bwd_gate_gather failed with code ", rc);
}

// Forward gate kernel with optional extras: xr_out keeps the read scalars for
// the backward pass; `stats` (float32 [T, 4]: tau, 1/sigma, -, -) replaces tau /
// inv_sigma; a non-empty ptr_lists fuses the all-gather of the listed bf16 tensors
// (lds / cols per tensor; h and x are then views of this rank's full buffers) and
// of the per-token statistics arrays in stat_lists.
void srw_fwd_gate_xr(const Tensor& h, const Tensor& emb, const Tensor& x, const Tensor& read,
                     Tensor& p_out, c10::optional<Tensor> xr_out, c10::optional<Tensor> tau,
                     c10::optional<Tensor> inv_sigma, c10::optional<Tensor> stats, Tensor& den_sum,
                     c10::optional<Tensor> diag, c10::optional<Tensor> alive,
                     c10::optional<Tensor> unit_mask,
                     std::vector<double> gate, Tensor& status,
                     std::vector<std::vector<int64_t>> ptr_lists, std::vector<int64_t> lds,
                     std::vector<int64_t> cols, std::vector<std::vector<int64_t>> stat_lists,
                     int64_t my_rank, int64_t rows_per_rank, c10::optional<Tensor> ready,
                     int64_t epoch) {
  check_bf16_2d(h, "h"); check_bf16_2d(emb, "emb"); check_bf16_2d(x, "x");
  check_bf16_2d(read, "read"); check_bf16_2d(p_out, "p_out");
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1), U = emb.size(0), r = emb.size(1);
  TORCH_CHECK(h.size(0) == T && h.size(1) == r && read.size(0) == U && read.size(1) == D);
  TORCH_CHECK(p_out.size(0) == T && p_out.size(1) >= U);
  void* xr_p = nullptr;
  long long ldxr = 0;
  if (xr_out.has_value() && xr_out->defined()) {
    check_bf16_2d(*xr_out, "xr_out");
    TORCH_CHECK(xr_out->size(0) == T && xr_out->size(1) >= U);
    xr_p = xr_out->data_ptr();
    ldxr = xr_out->stride(0);
  }
  const void* stats_p = nullptr;
  if (stats.has_value() && stats->defined()) {
    TORCH_CHECK(stats->is_cuda() && stats->scalar_type() == torch::kFloat32 &&
                stats->is_contiguous() && stats->numel() >= static_cast<int64_t>(T) * 4);
    stats_p = stats->data_ptr();
  }
  unsigned char* alive_p = nullptr;
  if (alive.has_value() && alive->defined()) {
    TORCH_CHECK(alive->scalar_type() == torch::kUInt8 && alive->numel() >= U);
    alive_p = alive->data_ptr<unsigned char>();
  }
  float* diag_p = nullptr;
  if (diag.has_value() && diag->defined()) {
    TORCH_CHECK(diag->is_cuda() && diag->scalar_type() == torch::kFloat32 && diag->is_contiguous() &&
                diag->numel() >= static_cast<int64_t>(T) * 12 + 2);
    diag_p = diag->data_ptr<float>();
  }
  DsbGate g = to_gate(gate);
  GatherHolder gh;
  const DsbGather* gp = nullptr;
  if (!ptr_lists.empty()) {
    TORCH_CHECK(ptr_lists.size() == lds.size() && lds.size() == cols.size() && ready.has_value());
    fill_gather(gh, ptr_lists, lds, cols, my_rank, rows_per_rank, *ready, epoch);
    fill_gather_stats(gh, stat_lists);
    gp = &gh.g;
  }
  int rc = dsb_srw_fwd_gate_xr(h.data_ptr(), h.stride(0), emb.data_ptr(), emb.stride(0),
                               x.data_ptr(), x.stride(0), read.data_ptr(), read.stride(0), T, U, r,
                               D, p_out.data_ptr(), p_out.stride(0), xr_p, ldxr, opt_f32(tau),
                               opt_f32(inv_sigma), stats_p, den_sum.data_ptr<float>(), nullptr,
                               diag_p, alive_p, opt_f32(unit_mask), &g, gp, status.data_ptr<int>(),
                               cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_fwd_gate_xr failed with code ", rc);
}

// Backward gate step from saved read scalars.  `stats` (float32 [T, 4]: tau,
// 1/sigma, dden, -) replaces the three per-token arrays.  Gathered tensors
// (optional): any bf16 full buffers (h, dy, and x for the GEMMs that follow).
void srw_bwd_gate_xr(const Tensor& h, const Tensor& emb, const Tensor& dy, const Tensor& write,
                     const Tensor& xr, Tensor& p_out, Tensor& dxr_out, Tensor& ds_out,
                     c10::optional<Tensor> tau, c10::optional<Tensor> inv_sigma,
                     c10::optional<Tensor> dden, c10::optional<Tensor> stats, Tensor& dtau_sum,
                     std::vector<double> gate, Tensor& status,
                     std::vector<std::vector<int64_t>> ptr_lists, std::vector<int64_t> lds,
                     std::vector<int64_t> cols, std::vector<std::vector<int64_t>> stat_lists,
                     int64_t my_rank, int64_t rows_per_rank, c10::optional<Tensor> ready,
                     int64_t epoch) {
  check_bf16_2d(h, "h"); check_bf16_2d(emb, "emb"); check_bf16_2d(dy, "dy");
  check_bf16_2d(write, "write"); check_bf16_2d(xr, "xr");
  check_bf16_2d(p_out, "p_out"); check_bf16_2d(dxr_out, "dxr_out"); check_bf16_2d(ds_out, "ds_out");
  const c10::cuda::CUDAGuard guard(h.device());
  const int T = h.size(0), D = dy.size(1), U = emb.size(0), r = emb.size(1);
  TORCH_CHECK(dy.size(0) == T && write.size(0) == U && write.size(1) == D && h.size(1) == r);
  TORCH_CHECK(xr.size(0) == T && xr.size(1) >= U && p_out.size(0) == T && p_out.size(1) >= U);
  TORCH_CHECK(p_out.stride(0) == dxr_out.stride(0) && p_out.stride(0) == ds_out.stride(0));
  const void* stats_p = nullptr;
  if (stats.has_value() && stats->defined()) {
    TORCH_CHECK(stats->is_cuda() && stats->scalar_type() == torch::kFloat32 &&
                stats->is_contiguous() && stats->numel() >= static_cast<int64_t>(T) * 4);
    stats_p = stats->data_ptr();
  }
  DsbGate g = to_gate(gate);
  GatherHolder gh;
  const DsbGather* gp = nullptr;
  if (!ptr_lists.empty()) {
    TORCH_CHECK(ptr_lists.size() == lds.size() && lds.size() == cols.size() && ready.has_value());
    fill_gather(gh, ptr_lists, lds, cols, my_rank, rows_per_rank, *ready, epoch);
    fill_gather_stats(gh, stat_lists);
    gp = &gh.g;
  }
  int rc = dsb_srw_bwd_gate_xr(h.data_ptr(), h.stride(0), emb.data_ptr(), emb.stride(0),
                               dy.data_ptr(), dy.stride(0), write.data_ptr(), write.stride(0),
                               xr.data_ptr(), xr.stride(0), T, U, r, D, p_out.data_ptr(),
                               dxr_out.data_ptr(), ds_out.data_ptr(), p_out.stride(0),
                               opt_f32(tau), opt_f32(inv_sigma), opt_f32(dden), stats_p,
                               dtau_sum.data_ptr<float>(), &g, gp, status.data_ptr<int>(),
                               cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_bwd_gate_xr failed with code ", rc);
}

bool srw_wide_tiles(int64_t U) { return dsb_srw_wide_tiles(static_cast<int>(U)) != 0; }

// Fused GEMM -> reduce-scatter.  `out_ptrs`: data pointers of every rank's
// [rows_per_rank, N] fp32 buffer (index = rank), as integers.
void gemm_scatter(const Tensor& A, bool a_mn, const Tensor& B, bool b_mn,
                  std::vector<int64_t> out_ptrs, int64_t my_rank, int64_t rows_per_rank,
                  int64_t ldc, bool out_bf16, double alpha, c10::optional<Tensor> row_scale,
                  Tensor& status, c10::optional<Tensor> aux_src, std::vector<int64_t> aux_ptrs) {
  check_bf16_2d(A, "A");
  check_bf16_2d(B, "B");
  const c10::cuda::CUDAGuard guard(A.device());
  const int64_t M = a_mn ? A.size(1) : A.size(0);
  const int64_t K = a_mn ? A.size(0) : A.size(1);
  const int64_t N = b_mn ? B.size(1) : B.size(0);
  std::vector<void*> outs;
  for (auto p : out_ptrs) outs.push_back(reinterpret_cast<void*>(p));
  std::vector<float*> auxd;
  for (auto p : aux_ptrs) auxd.push_back(reinterpret_cast<float*>(p));
  const float* aux = opt_f32(aux_src);
  TORCH_CHECK(aux == nullptr || (auxd.size() == outs.size() && aux_src->numel() >= M));
  int rc = dsb_gemm_bf16_scatter_aux(A.data_ptr(), a_mn, A.stride(0), B.data_ptr(), b_mn,
                                     B.stride(0), M, N, K, outs.data(),
                                     static_cast<int>(outs.size()), my_rank, rows_per_rank, ldc,
                                     out_bf16 ? 1 : 0, alpha, opt_f32(row_scale), aux,
                                     aux != nullptr ? auxd.data() : nullptr,
                                     status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_gemm_bf16_scatter failed with code ", rc);
}

// [n_slabs * rows, cols] (bf16 / fp32, contiguous) -> [rows, cols] sum over slabs
Tensor sum_slabs(const Tensor& in, int64_t n_slabs, bool out_bf16) {
  TORCH_CHECK(in.is_cuda() && in.dim() == 2 && in.is_contiguous() && in.size(0) % n_slabs == 0 &&
              (in.scalar_type() == torch::kBFloat16 || in.scalar_type() == torch::kFloat32));
  const c10::cuda::CUDAGuard guard(in.device());
  const int64_t rows = in.size(0) / n_slabs, cols = in.size(1);
  auto out = torch::empty({rows, cols}, in.options().dtype(out_bf16 ? torch::kBFloat16 : torch::kFloat32));
  int rc = dsb_sum_slabs(in.data_ptr(), in.scalar_type() == torch::kBFloat16 ? 1 : 0, n_slabs,
                         rows * cols, out.data_ptr(), out_bf16 ? 1 : 0, cur_stream());
  TORCH_CHECK(rc == 0, "dsb_sum_slabs failed with code ", rc);
  return out;
}

// Owner side of a route's fused reduce-scatter: [n_slabs * rows, cols] bf16 partial
// outputs and [n_slabs * rows] fp32 partial denominators -> (scale * sum / max(den, 1), den).
std::vector<Tensor> sum_slabs_div(const Tensor& in, int64_t n_slabs, const Tensor& den_in,
                                  const Tensor& scale) {
  TORCH_CHECK(in.is_cuda() && in.dim() == 2 && in.is_contiguous() && in.size(0) % n_slabs == 0 &&
              in.scalar_type() == torch::kBFloat16);
  const int64_t rows = in.size(0) / n_slabs, cols = in.size(1);
  TORCH_CHECK(den_in.scalar_type() == torch::kFloat32 && den_in.is_contiguous() &&
              den_in.numel() >= n_slabs * rows && scale.scalar_type() == torch::kFloat32 &&
              scale.numel() == 1 && scale.is_cuda());
  const c10::cuda::CUDAGuard guard(in.device());
  auto out = torch::empty({rows, cols}, in.options().dtype(torch::kFloat32));
  auto den = torch::empty({rows}, in.options().dtype(torch::kFloat32));
  int rc = dsb_sum_slabs_div(in.data_ptr(), n_slabs, rows, cols, den_in.data_ptr<float>(),
                             scale.data_ptr<float>(), out.data_ptr<float>(), den.data_ptr<float>(),
                             cur_stream());
  TORCH_CHECK(rc == 0, "dsb_sum_slabs_div failed with code ", rc);
  return {out, den};
}

void peer_barrier(const Tensor& pads_dev, int64_t rank, int64_t world, int64_t epoch,
                  int64_t slot_base, Tensor& status, int64_t wait_cycles) {
  TORCH_CHECK(pads_dev.is_cuda() && pads_dev.scalar_type() == torch::kInt64);
  const c10::cuda::CUDAGuard guard(pads_dev.device());
  int rc = dsb_peer_barrier(reinterpret_cast<unsigned int* const*>(pads_dev.data_ptr<int64_t>()),
                            rank, world, static_cast<unsigned int>(epoch), slot_base,
                            status.data_ptr<int>(), wait_cycles, cur_stream());
  TORCH_CHECK(rc == 0, "dsb_peer_barrier failed with code ", rc);
}

void small_allreduce(const Tensor& stage_dev, const Tensor& pads_dev, int64_t rank, int64_t world,
                     int64_t epoch, int64_t slot_base, const Tensor& in, Tensor& out, int64_t cap,
                     Tensor& status, int64_t wait_cycles) {
  TORCH_CHECK(in.is_cuda() && in.scalar_type() == torch::kFloat32 && in.is_contiguous() &&
              out.scalar_type() == torch::kFloat32 && out.is_contiguous() &&
              out.numel() == in.numel());
  const c10::cuda::CUDAGuard guard(in.device());
  int rc = dsb_small_allreduce(reinterpret_cast<float* const*>(stage_dev.data_ptr<int64_t>()),
                               reinterpret_cast<unsigned int* const*>(pads_dev.data_ptr<int64_t>()),
                               rank, world, static_cast<unsigned int>(epoch), slot_base,
                               in.data_ptr<float>(), out.data_ptr<float>(), in.numel(), cap,
                               status.data_ptr<int>(), wait_cycles, cur_stream());
  TORCH_CHECK(rc == 0, "dsb_small_allreduce failed with code ", rc);
}

void zero_reduce(const Tensor& grads_dev, int64_t world, int64_t lo, int64_t n, double scale,
                 Tensor& g_own, Tensor& sq) {
  TORCH_CHECK(g_own.is_cuda() && g_own.scalar_type() == torch::kFloat32 && g_own.is_contiguous() &&
              g_own.numel() >= n && sq.scalar_type() == torch::kFloat32);
  const c10::cuda::CUDAGuard guard(g_own.device());
  int rc = dsb_zero_reduce(reinterpret_cast<const float* const*>(grads_dev.data_ptr<int64_t>()),
                           world, lo, n, scale, g_own.data_ptr<float>(), sq.data_ptr<float>(),
                           cur_stream());
  TORCH_CHECK(rc == 0, "dsb_zero_reduce failed with code ", rc);
}

void zero_adam_scatter(const Tensor& params_dev, int64_t world, int64_t rank, int64_t lo, int64_t n,
                       const Tensor& g, Tensor& m, Tensor& v, const Tensor& clip_scale, double lr,
                       double b1, double b2, double eps, double wd, double bc1, double bc2) {
  TORCH_CHECK(g.is_cuda() && g.scalar_type() == torch::kFloat32 && m.numel() >= n &&
              v.numel() >= n && g.numel() >= n && m.is_contiguous() && v.is_contiguous());
  const c10::cuda::CUDAGuard guard(g.device());
  int rc = dsb_zero_adam_scatter(reinterpret_cast<float* const*>(params_dev.data_ptr<int64_t>()),
                                 world, rank, lo, n, g.data_ptr<float>(), m.data_ptr<float>(),
                                 v.data_ptr<float>(), clip_scale.data_ptr<float>(), lr, b1, b2, eps,
                                 wd, bc1, bc2, cur_stream());
  TORCH_CHECK(rc == 0, "dsb_zero_adam_scatter failed with code ", rc);
}

std::vector<Tensor> layernorm_fwd(const Tensor& x, const Tensor& w, const Tensor& b, double eps) {
  TORCH_CHECK(x.is_cuda() && x.dim() == 2 && x.scalar_type() == torch::kFloat32 && x.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1);
  auto y = torch::empty({T, D}, x.options().dtype(torch::kBFloat16));
  auto mean = torch::empty({T}, x.options());
  auto rstd = torch::empty({T}, x.options());
  TORCH_CHECK(dsb_layernorm_fwd(x.data_ptr<float>(), w.data_ptr<float>(), b.data_ptr<float>(),
                                y.data_ptr(), mean.data_ptr<float>(), rstd.data_ptr<float>(), T, D,
                                eps, cur_stream()) == 0);
  return {y, mean, rstd};
}

std::vector<Tensor> layernorm_bwd(const Tensor& dy, const Tensor& x, const Tensor& w,
                                  const Tensor& mean, const Tensor& rstd) {
  TORCH_CHECK(dy.scalar_type() == torch::kBFloat16 && dy.is_contiguous() && x.is_contiguous());
  const c10::cuda::CUDAGuard guard(x.device());
  const int T = x.size(0), D = x.size(1);
  auto dx = torch::empty_like(x);
  auto dw = torch::zeros({D}, x.options());
  auto db = torch::zeros({D}, x.options());
  TORCH_CHECK(dsb_layernorm_bwd(dy.data_ptr(), x.data_ptr<float>(), w.data_ptr<float>(),
                                mean.data_ptr<float>(), rstd.data_ptr<float>(),
                                dx.data_ptr<float>(), dw.data_ptr<float>(), db.data_ptr<float>(), T,
                                D, cur_stream()) == 0);
  return {dx, dw, db};
}

void ce_fwd(const Tensor& logits, const Tensor& labels, int64_t V, Tensor& lse, Tensor& lab,
            Tensor& pred) {
  TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.stride(1) == 1 &&
              labels.scalar_type() == torch::kInt64 && labels.is_contiguous());
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(dsb_ce_fwd(logits.data_ptr<float>(), logits.stride(0),
                         reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                         logits.size(0), V, lse.data_ptr<float>(), lab.data_ptr<float>(),
                         reinterpret_cast<long long*>(pred.data_ptr<int64_t>()), cur_stream()) == 0);
}

void ce_bwd(const Tensor& logits, const Tensor& labels, const Tensor& lse, const Tensor& scale,
            int64_t V, Tensor& dl) {
  TORCH_CHECK(logits.scalar_type() == torch::kFloat32 && logits.stride(1) == 1 &&
              dl.scalar_type() == torch::kBFloat16 && dl.stride(1) == 1);
  const c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(dsb_ce_bwd(logits.data_ptr<float>(), logits.stride(0),
                         reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                         lse.data_ptr<float>(), scale.data_ptr<float>(), logits.size(0), V,
                         dl.data_ptr(), dl.stride(0), cur_stream()) == 0);
}

// Fused tied LM head + cross-entropy statistics: returns (logits bf16 [T, V] view of a padded
// buffer, lse, label_logit, argmax).
std::vector<Tensor> lm_head_ce_fwd(const Tensor& x, const Tensor& emb, const Tensor& labels,
                                   Tensor& status) {
  check_bf16_2d(x, "x"); check_bf16_2d(emb, "emb");
  TORCH_CHECK(labels.is_cuda() && labels.scalar_type() == torch::kInt64 && labels.is_contiguous() &&
              labels.numel() == x.size(0) && x.size(1) == emb.size(1));
  const c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0), V = emb.size(0), K = x.size(1);
  const int64_t ldl = (V + 7) / 8 * 8, n_tiles = (V + 255) / 256;
  auto logits = torch::empty({T, ldl}, x.options());
  auto partial = torch::empty({T, n_tiles, 4}, x.options().dtype(torch::kFloat32));
  auto lse = torch::empty({T}, x.options().dtype(torch::kFloat32));
  auto lab = torch::empty({T}, x.options().dtype(torch::kFloat32));
  auto pred = torch::empty({T}, x.options().dtype(torch::kInt64));
  int rc = dsb_lm_head_ce_fwd(x.data_ptr(), x.stride(0), emb.data_ptr(), emb.stride(0), T, V, K,
                              reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                              logits.data_ptr(), ldl, partial.data_ptr(), lse.data_ptr<float>(),
                              lab.data_ptr<float>(),
                              reinterpret_cast<long long*>(pred.data_ptr<int64_t>()),
                              status.data_ptr<int>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_lm_head_ce_fwd failed with code ", rc);
  return {logits, lse, lab, pred};
}

void lm_head_ce_bwd_inplace(Tensor& logits, int64_t V, const Tensor& labels, const Tensor& lse,
                            const Tensor& scale) {
  TORCH_CHECK(logits.is_cuda() && logits.scalar_type() == torch::kBFloat16 && logits.dim() == 2 &&
              logits.is_contiguous() && labels.is_contiguous() && lse.is_contiguous() &&
              scale.scalar_type() == torch::kFloat32 && scale.is_contiguous() &&
              scale.numel() == logits.size(0));
  const c10::cuda::CUDAGuard guard(logits.device());
  int rc = dsb_lm_head_ce_bwd_inplace(logits.data_ptr(), logits.size(1), logits.size(0), V,
                                      reinterpret_cast<const long long*>(labels.data_ptr<int64_t>()),
                                      lse.data_ptr<float>(), scale.data_ptr<float>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_lm_head_ce_bwd_inplace failed with code ", rc);
}

std::vector<Tensor> attention_fwd(const Tensor& q, const Tensor& k, const Tensor& v, int64_t H,
                                  double p_drop, int64_t seed, Tensor& status) {
  TORCH_CHECK(q.is_cuda() && q.dim() == 3 && q.scalar_type() == torch::kBFloat16 &&
              q.is_contiguous() && k.is_contiguous() && v.is_contiguous() &&
              k.scalar_type() == torch::kBFloat16 && v.scalar_type() == torch::kBFloat16 &&
              k.sizes() == q.sizes() && v.sizes() == q.sizes());
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), S = q.size(1), D = q.size(2);
  TORCH_CHECK(H > 0 && D % H == 0, "d_model must be a multiple of the head count");
  auto out = torch::empty_like(q);
  auto lse = torch::empty({B, H, S}, q.options().dtype(torch::kFloat32));
  int rc = dsb_attention_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                             lse.data_ptr<float>(), B, H, S, D / H, p_drop,
                             static_cast<unsigned long long>(seed), status.data_ptr<int>(),
                             cur_stream());
  TORCH_CHECK(rc == 0, "dsb_attention_fwd failed with code ", rc);
  return {out, lse};
}

std::vector<Tensor> attention_bwd(const Tensor& q, const Tensor& k, const Tensor& v,
                                  const Tensor& out, const Tensor& d_out, const Tensor& lse,
                                  int64_t H, double p_drop, int64_t seed, Tensor& status) {
  TORCH_CHECK(d_out.is_cuda() && d_out.scalar_type() == torch::kBFloat16 && d_out.is_contiguous() &&
              d_out.sizes() == q.sizes() && out.is_contiguous() && q.is_contiguous() &&
              k.is_contiguous() && v.is_contiguous() && lse.is_contiguous());
  const c10::cuda::CUDAGuard guard(q.device());
  const int B = q.size(0), S = q.size(1), D = q.size(2);
  auto dq = torch::zeros({B, S, D}, q.options().dtype(torch::kFloat32));
  auto dk = torch::empty_like(q);
  auto dv = torch::empty_like(q);
  auto delta = torch::empty_like(lse);
  int rc = dsb_attention_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(),
                             d_out.data_ptr(), lse.data_ptr<float>(), delta.data_ptr<float>(),
                             dq.data_ptr<float>(), dk.data_ptr(), dv.data_ptr(), B, H, S, D / H,
                             p_drop, static_cast<unsigned long long>(seed), status.data_ptr<int>(),
                             cur_stream());
  TORCH_CHECK(rc == 0, "dsb_attention_bwd failed with code ", rc);
  return {dq, dk, dv};
}

Tensor embed_fwd(const Tensor& ids, const Tensor& tok, const Tensor& pos) {
  TORCH_CHECK(ids.is_cuda() && ids.dim() == 2 && ids.scalar_type() == torch::kInt64 &&
              ids.is_contiguous() && tok.scalar_type() == torch::kFloat32 && tok.is_contiguous() &&
              pos.scalar_type() == torch::kFloat32 && pos.is_contiguous());
  const c10::cuda::CUDAGuard guard(ids.device());
  const int B = ids.size(0), S = ids.size(1), D = tok.size(1);
  TORCH_CHECK(pos.size(0) >= S && pos.size(1) == D);
  auto out = torch::empty({B, S, D}, tok.options());
  TORCH_CHECK(dsb_embed_fwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                            tok.data_ptr<float>(), pos.data_ptr<float>(), out.data_ptr<float>(),
                            B * S, S, D, tok.size(0), cur_stream()) == 0);
  return out;
}

std::vector<Tensor> embed_bwd(const Tensor& ids, const Tensor& dy, int64_t V, int64_t P) {
  TORCH_CHECK(dy.is_cuda() && dy.dim() == 3 && dy.scalar_type() == torch::kFloat32 &&
              dy.is_contiguous() && ids.is_contiguous());
  const c10::cuda::CUDAGuard guard(dy.device());
  const int B = dy.size(0), S = dy.size(1), D = dy.size(2);
  auto dtok = torch::zeros({V, D}, dy.options());
  auto dpos = torch::zeros({P, D}, dy.options());
  TORCH_CHECK(dsb_embed_bwd(reinterpret_cast<const long long*>(ids.data_ptr<int64_t>()),
                            dy.data_ptr<float>(), dtok.data_ptr<float>(), dpos.data_ptr<float>(),
                            B, S, D, V, cur_stream()) == 0);
  return {dtok, dpos};
}

std::vector<Tensor> offdiag_abs(const Tensor& sim) {
  TORCH_CHECK(sim.is_cuda() && sim.dim() == 2 && sim.scalar_type() == torch::kFloat32 &&
              sim.stride(1) == 1 && sim.size(0) == sim.size(1));
  const c10::cuda::CUDAGuard guard(sim.device());
  const int m = sim.size(0);
  const int64_t ld_s = (m + 7) / 8 * 8;
  auto sgn = torch::empty({m, ld_s}, sim.options().dtype(torch::kBFloat16));
  auto total = torch::zeros({}, sim.options());
  TORCH_CHECK(dsb_offdiag_abs(sim.data_ptr<float>(), sim.stride(0), m, sgn.data_ptr(), ld_s,
                              total.data_ptr<float>(), cur_stream()) == 0);
  return {total, sgn.slice(1, 0, m)};
}

std::vector<Tensor> route_bwd_prologue(const Tensor& dy, const Tensor& y, const Tensor& row_scale) {
  TORCH_CHECK(dy.is_cuda() && dy.dim() == 2 && dy.scalar_type() == torch::kFloat32 &&
              dy.is_contiguous() && y.scalar_type() == torch::kFloat32 && y.is_contiguous() &&
              y.sizes() == dy.sizes() && row_scale.scalar_type() == torch::kFloat32 &&
              row_scale.is_contiguous() && row_scale.numel() == dy.size(0));
  const c10::cuda::CUDAGuard guard(dy.device());
  const int T = dy.size(0), D = dy.size(1);
  auto dyb = torch::empty({T, D}, dy.options().dtype(torch::kBFloat16));
  auto rowdot = torch::empty({T}, dy.options());
  TORCH_CHECK(dsb_route_bwd_prologue(dy.data_ptr<float>(), y.data_ptr<float>(), row_scale.data_ptr<float>(),
                                     dyb.data_ptr(), rowdot.data_ptr<float>(), T, D,
                                     cur_stream()) == 0);
  return {dyb, rowdot};
}

// tau, isd, mu, sd [N] and the column sums of h [r] from hg = h . G.
std::vector<Tensor> score_stats_fwd(const Tensor& hg, const Tensor& h, const Tensor& esum,
                                    const Tensor& off, double inv_u) {
  check_bf16_2d(h, "h");
  TORCH_CHECK(hg.is_cuda() && hg.dim() == 2 && hg.scalar_type() == torch::kFloat32 &&
              hg.is_contiguous() && hg.size(0) == h.size(0) && hg.size(1) == h.size(1));
  TORCH_CHECK(esum.scalar_type() == torch::kFloat32 && esum.is_contiguous() &&
              esum.numel() == h.size(1) && off.scalar_type() == torch::kFloat32 &&
              off.is_contiguous() && off.numel() == h.size(0));
  const c10::cuda::CUDAGuard guard(h.device());
  const int N = h.size(0), r = h.size(1);
  auto o = hg.options();
  auto tau = torch::empty({N}, o), isd = torch::empty({N}, o), mu = torch::empty({N}, o),
       sd = torch::empty({N}, o), hsum = torch::zeros({r}, o);
  int rc = dsb_score_stats_fwd(hg.data_ptr<float>(), h.data_ptr(), h.stride(0),
                               esum.data_ptr<float>(), off.data_ptr<float>(), inv_u, N, r,
                               tau.data_ptr<float>(), isd.data_ptr<float>(), mu.data_ptr<float>(),
                               sd.data_ptr<float>(), hsum.data_ptr<float>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_score_stats_fwd failed with code ", rc);
  return {tau, isd, mu, sd, hsum};
}

// SRW pool op for up to four token rows in one streaming pass (decoding).
// -> out fp32 [N, D] (normalised and scaled), den fp32 [N]
std::vector<Tensor> srw_rows(const Tensor& h, const Tensor& x, const Tensor& tau, const Tensor& isd,
                             const Tensor& emb, const Tensor& read, const Tensor& write,
                             c10::optional<Tensor> unit_mask, std::vector<double> gate, double scale,
                             c10::optional<Tensor> scale_t) {
  check_bf16_2d(h, "h"); check_bf16_2d(x, "x"); check_bf16_2d(emb, "emb");
  check_bf16_2d(read, "read"); check_bf16_2d(write, "write");
  const int N = h.size(0), r = h.size(1), D = x.size(1), U = emb.size(0);
  TORCH_CHECK(h.is_contiguous() && x.is_contiguous() && x.size(0) == N && emb.size(1) == r &&
              read.size(0) == U && read.size(1) == D && write.size(0) == U && write.size(1) == D);
  TORCH_CHECK(N >= 1 && N <= dsb_srw_rows_max(D), "srw_rows: too many rows for this d_model");
  TORCH_CHECK(tau.scalar_type() == torch::kFloat32 && tau.is_contiguous() && tau.numel() == N &&
              isd.scalar_type() == torch::kFloat32 && isd.is_contiguous() && isd.numel() == N);
  const c10::cuda::CUDAGuard guard(x.device());
  const int NR = N <= 1 ? 1 : N <= 2 ? 2 : 4;
  const int blocks = dsb_srw_rows_blocks(N, D);
  auto o = tau.options();
  auto part = torch::empty({static_cast<int64_t>(blocks) * NR * (D + 1)}, o);
  auto out = torch::empty({N, D}, o), den = torch::empty({N}, o);
  DsbGate g = to_gate(gate);
  const float* sp = nullptr;
  if (scale_t.has_value() && scale_t->defined()) {
    TORCH_CHECK(scale_t->is_cuda() && scale_t->scalar_type() == torch::kFloat32 && scale_t->numel() == 1);
    sp = scale_t->data_ptr<float>();
  }
  float* part_p = part.data_ptr<float>();
  int rc = dsb_srw_rows(h.data_ptr(), x.data_ptr(), tau.data_ptr<float>(), isd.data_ptr<float>(),
                        emb.data_ptr(), emb.stride(0), read.data_ptr(), read.stride(0),
                        write.data_ptr(), write.stride(0), opt_f32(unit_mask), N, U, r, D, &g,
                        static_cast<float>(scale), sp, part_p,
                        part_p + static_cast<size_t>(blocks) * NR * D, out.data_ptr<float>(),
                        den.data_ptr<float>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_srw_rows failed with code ", rc);
  return {out, den};
}

// res + dropout(x) (res optional) with a counter-based mask; see dsb_dropout.
Tensor dropout(c10::optional<Tensor> res, const Tensor& x, int64_t seed, double p) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == torch::kFloat32 && x.is_contiguous() &&
              x.numel() % 4 == 0, "dropout: fp32 contiguous tensor with a multiple of 4 elements");
  const float* rp = nullptr;
  if (res.has_value() && res->defined()) {
    TORCH_CHECK(res->is_cuda() && res->scalar_type() == torch::kFloat32 && res->is_contiguous() &&
                res->numel() == x.numel());
    rp = res->data_ptr<float>();
  }
  const c10::cuda::CUDAGuard guard(x.device());
  auto y = torch::empty_like(x);
  int rc = dsb_dropout(rp, x.data_ptr<float>(), y.data_ptr<float>(), x.numel(),
                       static_cast<unsigned long long>(seed), static_cast<float>(p), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_dropout failed with code ", rc);
  return y;
}

// y = x . W^T + bias for up to four rows (SIMT, one pass over W).
void gemv_rows(const Tensor& x, const Tensor& w, c10::optional<Tensor> bias, Tensor& y) {
  check_bf16_2d(x, "x"); check_bf16_2d(w, "w");
  TORCH_CHECK(x.is_contiguous() && x.size(1) == w.size(1) && y.is_cuda() && y.dim() == 2 &&
              y.scalar_type() == torch::kFloat32 && y.stride(1) == 1 && y.size(0) == x.size(0) &&
              y.size(1) == w.size(0));
  const c10::cuda::CUDAGuard guard(x.device());
  int rc = dsb_gemv_rows(x.data_ptr(), w.data_ptr(), w.stride(0), opt_f32(bias), y.data_ptr<float>(),
                         y.stride(0), x.size(0), w.size(0), x.size(1), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_gemv_rows failed with code ", rc);
}

// Decode-time attention of one new token per sequence over the KV cache (which it extends).
Tensor kv_decode_attention(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& cache_k,
                           Tensor& cache_v, const Tensor& pos, int64_t H) {
  auto ok = [](const Tensor& t) { return t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(); };
  TORCH_CHECK(ok(q) && ok(k) && ok(v) && ok(cache_k) && ok(cache_v) && q.dim() == 2);
  const int B = q.size(0), D = q.size(1);
  TORCH_CHECK(D % H == 0 && k.sizes() == q.sizes() && v.sizes() == q.sizes());
  const int dh = D / H;
  TORCH_CHECK(cache_k.dim() == 4 && cache_k.size(0) == B && cache_k.size(1) == H &&
              cache_k.size(3) == dh && cache_v.sizes() == cache_k.sizes());
  TORCH_CHECK(pos.is_cuda() && pos.scalar_type() == torch::kInt64 && pos.numel() == 1);
  const c10::cuda::CUDAGuard guard(q.device());
  auto out = torch::empty_like(q);
  int rc = dsb_kv_decode_attention(q.data_ptr<float>(), k.data_ptr<float>(), v.data_ptr<float>(),
                                   cache_k.data_ptr<float>(), cache_v.data_ptr<float>(),
                                   reinterpret_cast<const long long*>(pos.data_ptr<int64_t>()), B, H, dh,
                                   cache_k.size(2), out.data_ptr<float>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_kv_decode_attention failed with code ", rc);
  return out;
}

// Route-major tau, isd [R*T] and bf16(h) [R*T, r] for a handful of rows (one launch).
std::vector<Tensor> score_stats_rows(const Tensor& h, const Tensor& off, const Tensor& gram,
                                     const Tensor& esum, double inv_u) {
  TORCH_CHECK(h.is_cuda() && h.dim() == 3 && h.scalar_type() == torch::kFloat32 && h.stride(2) == 1);
  const int T = h.size(0), R = h.size(1), r = h.size(2);
  TORCH_CHECK(off.is_cuda() && off.dim() == 2 && off.scalar_type() == torch::kFloat32 &&
              off.size(0) == T && off.size(1) == R);
  TORCH_CHECK(gram.scalar_type() == torch::kFloat32 && gram.is_contiguous() && gram.dim() == 2 &&
              gram.size(0) == r && gram.size(1) == r && esum.scalar_type() == torch::kFloat32 &&
              esum.is_contiguous() && esum.numel() == r);
  const c10::cuda::CUDAGuard guard(h.device());
  auto o = gram.options();
  auto tau = torch::empty({R * T}, o), isd = torch::empty({R * T}, o);
  auto hb = torch::empty({R * T, r}, o.dtype(torch::kBFloat16));
  int rc = dsb_score_stats_rows(h.data_ptr<float>(), h.stride(0), h.stride(1), off.data_ptr<float>(),
                                off.stride(0), off.stride(1), gram.data_ptr<float>(),
                                esum.data_ptr<float>(), inv_u, T, R, r, tau.data_ptr<float>(),
                                isd.data_ptr<float>(), hb.data_ptr(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_score_stats_rows failed with code ", rc);
  return {tau, isd, hb};
}

// dh fp32 [N, r], w bf16 [N, r] (row stride padded to 8), d_off [N], d_esum [r].
std::vector<Tensor> score_stats_bwd(c10::optional<Tensor> d_tau, c10::optional<Tensor> d_isd,
                                    c10::optional<Tensor> d_hsum, c10::optional<Tensor> d_hb,
                                    const Tensor& off, const Tensor& mu, const Tensor& sd,
                                    const Tensor& hg, const Tensor& h, const Tensor& esum,
                                    double inv_u) {
  check_bf16_2d(h, "h");
  const c10::cuda::CUDAGuard guard(h.device());
  const int N = h.size(0), r = h.size(1);
  const void* dhb = nullptr;
  if (d_hb.has_value() && d_hb->defined()) {
    TORCH_CHECK(d_hb->scalar_type() == torch::kBFloat16 && d_hb->is_contiguous() &&
                d_hb->numel() == static_cast<int64_t>(N) * r);
    dhb = d_hb->data_ptr();
  }
  auto o = hg.options();
  const int64_t ldw = (r + 7) / 8 * 8;
  auto dh = torch::empty({N, r}, o);
  auto w = torch::empty({N, ldw}, o.dtype(torch::kBFloat16));
  auto d_off = torch::empty({N}, o), d_esum = torch::zeros({r}, o);
  int rc = dsb_score_stats_bwd(opt_f32(d_tau), opt_f32(d_isd), opt_f32(d_hsum), dhb,
                               off.data_ptr<float>(), mu.data_ptr<float>(), sd.data_ptr<float>(),
                               hg.data_ptr<float>(), h.data_ptr(), h.stride(0),
                               esum.data_ptr<float>(), inv_u, N, r, dh.data_ptr<float>(),
                               w.data_ptr(), ldw, d_off.data_ptr<float>(),
                               d_esum.data_ptr<float>(), cur_stream());
  TORCH_CHECK(rc == 0, "dsb_score_stats_bwd failed with code ", rc);
  return {dh, w.slice(1, 0, r), d_off, d_esum};
}

void adamw_multi(std::vector<Tensor> params, std::vector<Tensor> grads, std::vector<Tensor> exp_avg,
                 std::vector<Tensor> exp_avg_sq, const Tensor& clip_scale, double lr, double b1,
                 double b2, double eps, double wd, double bc1, double bc2) {
  if (params.empty()) return;
  const size_t k = params.size();
  TORCH_CHECK(grads.size() == k && exp_avg.size() == k && exp_avg_sq.size() == k);
  std::vector<float*> p(k), m(k), v(k);
  std::vector<const float*> g(k);
  std::vector<long long> n(k);
  for (size_t i = 0; i < k; ++i) {
    auto ok = [](const Tensor& t) { return t.is_cuda() && t.scalar_type() == torch::kFloat32 && t.is_contiguous(); };
    TORCH_CHECK(ok(params[i]) && ok(grads[i]) && ok(exp_avg[i]) && ok(exp_avg_sq[i]) &&
                grads[i].numel() == params[i].numel() && exp_avg[i].numel() == params[i].numel() &&
                exp_avg_sq[i].numel() == params[i].numel() && params[i].device() == params[0].device());
    p[i] = params[i].data_ptr<float>();
    g[i] = grads[i].data_ptr<float>();
    m[i] = exp_avg[i].data_ptr<float>();
    v[i] = exp_avg_sq[i].data_ptr<float>();
    n[i] = params[i].numel();
  }
  const c10::cuda::CUDAGuard guard(params[0].device());
  TORCH_CHECK(dsb_adamw_multi(p.data(), g.data(), m.data(), v.data(), n.data(), static_cast<int>(k),
                              clip_scale.data_ptr<float>(), lr, b1, b2, eps, wd, bc1, bc2,
                              cur_stream()) == 0);
}

Tensor grad_sq_norm(std::vector<Tensor> grads) {
  TORCH_CHECK(!grads.empty());
  const c10::cuda::CUDAGuard guard(grads[0].device());
  auto out = torch::zeros({}, grads[0].options().dtype(torch::kFloat32));
  std::vector<const float*> g(grads.size());
  std::vector<long long> n(grads.size());
  for (size_t i = 0; i < grads.size(); ++i) {
    TORCH_CHECK(grads[i].is_cuda() && grads[i].scalar_type() == torch::kFloat32 &&
                grads[i].is_contiguous() && grads[i].device() == grads[0].device());
    g[i] = grads[i].data_ptr<float>();
    n[i] = grads[i].numel();
  }
  TORCH_CHECK(dsb_sqnorm_multi(g.data(), n.data(), static_cast<int>(grads.size()),
                               out.data_ptr<float>(), cur_stream()) == 0);
  return out;
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemm", &gemm);
  m.def("srw_fwd_gate", &srw_fwd_gate);
  m.def("srw_bwd_gate", &srw_bwd_gate);
  m.def("srw_forward", &srw_forward);
  m.def("srw_fwd_gate_xr", &srw_fwd_gate_xr);
  m.def("srw_bwd_gate_xr", &srw_bwd_gate_xr);
  m.def("srw_wide_tiles", &srw_wide_tiles);
  m.def("gemm_scatter", &gemm_scatter);
  m.def("sum_slabs", &sum_slabs);
  m.def("sum_slabs_div", &sum_slabs_div);
  m.def("layernorm_fwd", &layernorm_fwd);
  m.def("layernorm_bwd", &layernorm_bwd);
  m.def("ce_fwd", &ce_fwd);
  m.def("lm_head_ce_fwd", &lm_head_ce_fwd);
  m.def("lm_head_ce_bwd_inplace", &lm_head_ce_bwd_inplace);
  m.def("ce_bwd", &ce_bwd);
  m.def("adamw_multi", &adamw_multi);
  m.def("embed_fwd", &embed_fwd);
  m.def("embed_bwd", &embed_bwd);
  m.def("offdiag_abs", &offdiag_abs);
  m.def("route_bwd_prologue", &route_bwd_prologue);
  m.def("attention_fwd", &attention_fwd);
  m.def("attention_bwd", &attention_bwd);
  m.def("grad_sq_norm", &grad_sq_norm);
  m.def("score_stats_fwd", &score_stats_fwd);
  m.def("score_stats_bwd", &score_stats_bwd);
  m.def("score_stats_rows", &score_stats_rows);
  m.def("srw_rows", &srw_rows);
  m.def("gemv_rows", &gemv_rows);
  m.def("dropout", &dropout);
  m.def("kv_decode_attention", &kv_decode_attention);
  m.def("srw_rows_max", [](int64_t D) { return dsb_srw_rows_max(static_cast<int>(D)); });
  m.def("srw_fwd_gate_gather", &srw_fwd_gate_gather);
  m.def("srw_bwd_gate_gather", &srw_bwd_gate_gather);
  m.def("peer_barrier", &peer_barrier);
  m.def("small_allreduce", &small_allreduce);
  m.def("zero_reduce", &zero_reduce);
  m.def("zero_adam_scatter", &zero_adam_scatter);
}
