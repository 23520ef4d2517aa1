// Per-token score statistics of the SRW pool op without a pass over the scores.
//
// With s_u = <h, e_u> over a pool of U units,
//   mean_U s   = <h, sum_u e_u> / U               (esum, [r])
//   mean_U s^2 = h (E^T E) h^T / U                (Gram matrix G, [r, r])
// so mu, sigma, the threshold tau = mu + tau_off * sigma and 1 / sigma of every
// token follow from hg = h . G (a [N, r] x [r, r] GEMM on the tensor engine, G
// split into two bf16 terms so that the product is fp32-accurate) and one row
// kernel.  The reference sweeps all [T, U] scores for the same numbers
// (models/dawn_spatial_v41_exp.py:433-464).  The kernels here are the row parts,
// forward and backward; the column sums of h (the per-unit mean score used by the
// load-balance and dead-unit terms is emb . mean_t h) ride along.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "dsb_api_ops.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr float kVarFloor = 1e-12f;   // variance floor under the square root
constexpr float kSdEps = 1e-8f;       // sigma = sqrt(var) + eps, as in the reference
constexpr int kMaxR = 512;            // d_route of every supported model is <= 384

// One warp per row, grid-stride; a block adds its column sums of h into hsum
// once at the end (shared-memory partials first).
__global__ void score_stats_fwd_kernel(const float* __restrict__ hg, const __nv_bfloat16* __restrict__ h,
                                       long long ldh, const float* __restrict__ esum,
                                       const float* __restrict__ off, float inv_u, int N, int r,
                                       float* __restrict__ tau, float* __restrict__ isd,
                                       float* __restrict__ mu_out, float* __restrict__ sd_out,
                                       float* __restrict__ hsum) {
  __shared__ float s_sum[kMaxR];
  for (int j = threadIdx.x; j < r; j += blockDim.x) s_sum[j] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  float csum[kMaxR / 32];
#pragma unroll
  for (int k = 0; k < kMaxR / 32; ++k) csum[k] = 0.f;
  for (int row = blockIdx.x * warps + (threadIdx.x >> 5); row < N; row += gridDim.x * warps) {
    const float* g = hg + static_cast<size_t>(row) * r;
    const __nv_bfloat16* hr = h + static_cast<size_t>(row) * ldh;
    float m2 = 0.f, m1 = 0.f;
#pragma unroll
    for (int k = 0; k < kMaxR / 32; ++k) {
      const int j = lane + 32 * k;
      if (j < r) {
        const float hv = __bfloat162float(hr[j]);
        m2 = fmaf(g[j], hv, m2);
        m1 = fmaf(esum[j], hv, m1);
        csum[k] += hv;
      }
    }
    m2 = warp_sum(m2) * inv_u;
    const float mu = warp_sum(m1) * inv_u;
    if (lane == 0) {
      const float sd = sqrtf(fmaxf(m2 - mu * mu, kVarFloor)) + kSdEps;
      tau[row] = fmaf(off[row], sd, mu);
      isd[row] = 1.f / sd;
      mu_out[row] = mu;
      sd_out[row] = sd;
    }
  }
  if (hsum != nullptr) {
#pragma unroll
    for (int k = 0; k < kMaxR / 32; ++k) {
      const int j = lane + 32 * k;
      if (j < r) atomicAdd(&s_sum[j], csum[k]);
    }
    __syncthreads();
    for (int j = threadIdx.x; j < r; j += blockDim.x) atomicAdd(hsum + j, s_sum[j]);
  }
}

// Backward of the row part.  Given the cotangents of tau, 1/sigma and of the
// column sums of h:
//   d_sd = d_tau * off - d_isd / sd^2,   d_off = d_tau * sd
//   d_var = d_sd / (2 sqrt(var))  (0 where the variance floor is active)
//   d_mu  = d_tau - 2 mu d_var
//   dh    = (2 d_var / U) hg + (d_mu / U) esum + d_hsum + d_hb   (d_hb: cotangent that
//           reached the bf16 copy of h from the gate kernels)
//   w     = bf16(d_var * h)      operand of  dG = w^T h / U  (engine GEMM)
//   d_esum += (d_mu / U) h       (shared-memory partials, one atomic per column and block)
__global__ void score_stats_bwd_kernel(const float* __restrict__ d_tau, const float* __restrict__ d_isd,
                                       const float* __restrict__ d_hsum,
                                       const __nv_bfloat16* __restrict__ d_hb,
                                       const float* __restrict__ off,
                                       const float* __restrict__ mu_in, const float* __restrict__ sd_in,
                                       const float* __restrict__ hg, const __nv_bfloat16* __restrict__ h,
                                       long long ldh, const float* __restrict__ esum, float inv_u, int N,
                                       int r, float* __restrict__ dh, __nv_bfloat16* __restrict__ w,
                                       long long ldw, float* __restrict__ d_off,
                                       float* __restrict__ d_esum) {
  __shared__ float s_sum[kMaxR];
  for (int j = threadIdx.x; j < r; j += blockDim.x) s_sum[j] = 0.f;
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  float csum[kMaxR / 32];
#pragma unroll
  for (int k = 0; k < kMaxR / 32; ++k) csum[k] = 0.f;
  for (int row = blockIdx.x * warps + (threadIdx.x >> 5); row < N; row += gridDim.x * warps) {
    const float sd = sd_in[row], mu = mu_in[row];
    const float dt = d_tau != nullptr ? d_tau[row] : 0.f;
    const float di = d_isd != nullptr ? d_isd[row] : 0.f;
    const float d_sd = dt * off[row] - di / (sd * sd);
    const float sq = sd - kSdEps;
    const float d_var = sq > 1.5e-6f ? d_sd / (2.f * sq) : 0.f;   // sqrt(floor) = 1e-6
    const float d_mu = dt - 2.f * mu * d_var;
    if (lane == 0) d_off[row] = dt * sd;
    const float a = 2.f * d_var * inv_u, b = d_mu * inv_u;
    const float* g = hg + static_cast<size_t>(row) * r;
    const __nv_bfloat16* hr = h + static_cast<size_t>(row) * ldh;
    float* dr = dh + static_cast<size_t>(row) * r;
    __nv_bfloat16* wr = w + static_cast<size_t>(row) * ldw;
#pragma unroll
    for (int k = 0; k < kMaxR / 32; ++k) {
      const int j = lane + 32 * k;
      if (j < r) {
        const float hv = __bfloat162float(hr[j]);
        float acc = fmaf(a, g[j], fmaf(b, esum[j], d_hsum != nullptr ? d_hsum[j] : 0.f));
        if (d_hb != nullptr) acc += __bfloat162float(d_hb[static_cast<size_t>(row) * r + j]);
        dr[j] = acc;
        wr[j] = __float2bfloat16(d_var * hv);
        csum[k] = fmaf(b, hv, csum[k]);
      }
    }
  }
#pragma unroll
  for (int k = 0; k < kMaxR / 32; ++k) {
    const int j = lane + 32 * k;
    if (j < r) atomicAdd(&s_sum[j], csum[k]);
  }
  __syncthreads();
  for (int j = threadIdx.x; j < r; j += blockDim.x) atomicAdd(d_esum + j, s_sum[j]);
}

constexpr int kRowGroups = 8;      // thread groups that share the rows of G
constexpr int kRowThreads = 128;   // threads of a group: one column of G each (strided)

// A handful of rows (decoding): the whole statistic in one launch, fp32 throughout.
// Block n handles token t = n % T of route ri = n / T (route-major output rows, the
// order in which the routes of one pool are stacked into one gate-kernel call).
// Thread j owns column j of the symmetric G: consecutive threads read consecutive
// addresses of every row of G.
__global__ void score_stats_rows_kernel(const float* __restrict__ h, long long h_st, long long h_sr,
                                        const float* __restrict__ off, long long o_st, long long o_sr,
                                        const float* __restrict__ gram, const float* __restrict__ esum,
                                        float inv_u, int T, int r, float* __restrict__ tau,
                                        float* __restrict__ isd, __nv_bfloat16* __restrict__ hb) {
  __shared__ float s_h[kMaxR];
  __shared__ float s_part[kRowGroups][kMaxR];
  __shared__ float s_red[2][32];
  const int n = blockIdx.x, t = n % T, ri = n / T;
  const float* hr = h + t * h_st + ri * h_sr;
  for (int j = threadIdx.x; j < r; j += blockDim.x) {
    const __nv_bfloat16 q = __float2bfloat16(hr[j]);     // the gate kernels see bf16(h)
    hb[static_cast<size_t>(n) * r + j] = q;
    s_h[j] = __bfloat162float(q);
  }
  __syncthreads();
  // (G h)_j: the rows of G are dealt to kRowGroups thread groups, eight independent
  // accumulators per thread keep the loads in flight
  const int grp = threadIdx.x / kRowThreads, tj = threadIdx.x % kRowThreads;
  const int rows_per = (r + kRowGroups - 1) / kRowGroups;
  const int i0 = grp * rows_per, i1 = min(r, i0 + rows_per);
  for (int j = tj; j < r; j += kRowThreads) {
    float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    int i = i0;
    for (; i + 8 <= i1; i += 8) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        a[k] = fmaf(gram[static_cast<size_t>(i + k) * r + j], s_h[i + k], a[k]);
    }
    for (; i < i1; ++i) a[0] = fmaf(gram[static_cast<size_t>(i) * r + j], s_h[i], a[0]);
    s_part[grp][j] = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
  }
  __syncthreads();
  float m2 = 0.f, m1 = 0.f;
  for (int j = threadIdx.x; j < r; j += blockDim.x) {
    float acc = 0.f;
#pragma unroll
    for (int g = 0; g < kRowGroups; ++g) acc += s_part[g][j];
    m2 = fmaf(acc, s_h[j], m2);
    m1 = fmaf(esum[j], s_h[j], m1);
  }
  m2 = warp_sum(m2);
  m1 = warp_sum(m1);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { s_red[0][warp] = m2; s_red[1][warp] = m1; }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    m2 = warp_sum(lane < nw ? s_red[0][lane] : 0.f) * inv_u;
    const float mu = warp_sum(lane < nw ? s_red[1][lane] : 0.f) * inv_u;
    if (lane == 0) {
      const float sd = sqrtf(fmaxf(m2 - mu * mu, kVarFloor)) + kSdEps;
      tau[n] = fmaf(off[t * o_st + ri * o_sr], sd, mu);
      isd[n] = 1.f / sd;
    }
  }
}

int stats_grid(int N) {
  const int blocks = (N + 7) / 8;
  return blocks < 148 * 4 ? (blocks < 1 ? 1 : blocks) : 148 * 4;
}

}  // namespace

extern "C" int dsb_score_stats_fwd(const float* hg, const void* h_bf16, long long ldh,
                                   const float* esum, const float* off, float inv_u, int N, int r,
                                   float* tau, float* isd, float* mu, float* sd, float* hsum,
                                   cudaStream_t stream) {
  if (N <= 0) return 0;
  if (r <= 0 || r > kMaxR) return 801;
  score_stats_fwd_kernel<<<stats_grid(N), 256, 0, stream>>>(
      hg, static_cast<const __nv_bfloat16*>(h_bf16), ldh, esum, off, inv_u, N, r, tau, isd, mu, sd,
      hsum);
  return cudaGetLastError() == cudaSuccess ? 0 : 802;
}

extern "C" int dsb_score_stats_bwd(const float* d_tau, const float* d_isd, const float* d_hsum,
                                   const void* d_hb_bf16, const float* off, const float* mu,
                                   const float* sd,
                                   const float* hg, const void* h_bf16, long long ldh,
                                   const float* esum, float inv_u, int N, int r, float* dh,
                                   void* w_bf16, long long ldw, float* d_off, float* d_esum,
                                   cudaStream_t stream) {
  if (N <= 0) return 0;
  if (r <= 0 || r > kMaxR) return 801;
  score_stats_bwd_kernel<<<stats_grid(N), 256, 0, stream>>>(
      d_tau, d_isd, d_hsum, static_cast<const __nv_bfloat16*>(d_hb_bf16), off, mu, sd, hg,
      static_cast<const __nv_bfloat16*>(h_bf16), ldh, esum,
      inv_u, N, r, dh, static_cast<__nv_bfloat16*>(w_bf16), ldw, d_off, d_esum);
  return cudaGetLastError() == cudaSuccess ? 0 : 802;
}

extern "C" int dsb_score_stats_rows(const float* h, long long h_st, long long h_sr, const float* off,
                                    long long o_st, long long o_sr, const float* gram,
                                    const float* esum, float inv_u, int T, int R, int r, float* tau,
                                    float* isd, void* hb_bf16, cudaStream_t stream) {
  if (T <= 0 || R <= 0) return 0;
  if (r <= 0 || r > kMaxR) return 801;
  score_stats_rows_kernel<<<T * R, kRowGroups * kRowThreads, 0, stream>>>(h, h_st, h_sr, off, o_st, o_sr, gram, esum, inv_u,
                                                     T, r, tau, isd,
                                                     static_cast<__nv_bfloat16*>(hb_bf16));
  return cudaGetLastError() == cudaSuccess ? 0 : 802;
}
