// Memory-bound kernels around the GEMMs: LayerNorm forward/backward (bf16 out),
// row-wise softmax cross-entropy statistics and gradient for the chunked tied
// LM head, and the AdamW update with the clip factor read from device memory.
// Reference math: LayerNorm eps 1e-6, population variance
// (models/dawn_spatial_v41_exp.py:321-324); CE on shifted labels (:1642-1668);
// optimizer chain (scripts/train_jax.py:2083-2089).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <float.h>
#include <stdint.h>

#include "dsb_api_ops.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row.  x fp32 [T, D]; y bf16 [T, D]; mean/rstd fp32 [T].
// kRegs > 0: the row (D <= 32 * kRegs) is read once and kept in registers, all
// loads in flight together; kRegs == 0: three passes over the row for any D.
template <int kRegs>
__global__ void ln_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                              const float* __restrict__ b, __nv_bfloat16* __restrict__ y,
                              float* __restrict__ mean, float* __restrict__ rstd, int T, int D,
                              float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const float* xr = x + static_cast<size_t>(row) * D;
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * D;
  if constexpr (kRegs > 0) {
    float v[kRegs];
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kRegs; ++k) {
      const int i = lane + 32 * k;
      v[k] = i < D ? xr[i] : 0.f;
      s += v[k];
    }
    const float mu = warp_sum(s) / D;
    float q = 0.f;
#pragma unroll
    for (int k = 0; k < kRegs; ++k) {
      const float d = lane + 32 * k < D ? v[k] - mu : 0.f;
      q += d * d;
    }
    const float rs = rsqrtf(warp_sum(q) / D + eps);
#pragma unroll
    for (int k = 0; k < kRegs; ++k) {
      const int i = lane + 32 * k;
      if (i < D) yr[i] = __float2bfloat16((v[k] - mu) * rs * w[i] + b[i]);
    }
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  } else {
    float s = 0.f;
    for (int i = lane; i < D; i += 32) s += xr[i];
    const float mu = warp_sum(s) / D;
    float q = 0.f;
    for (int i = lane; i < D; i += 32) { const float d = xr[i] - mu; q += d * d; }
    const float rs = rsqrtf(warp_sum(q) / D + eps);
    for (int i = lane; i < D; i += 32) yr[i] = __float2bfloat16((xr[i] - mu) * rs * w[i] + b[i]);
    if (lane == 0) { mean[row] = mu; rstd[row] = rs; }
  }
}

// A few rows only (decoding): one block of 256 threads per row, the row in
// registers (D <= 256 * 8), two block reductions.
__global__ void __launch_bounds__(256) ln_fwd_block_kernel(
    const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
    __nv_bfloat16* __restrict__ y, float* __restrict__ mean, float* __restrict__ rstd, int D,
    float eps) {
  __shared__ float s_red[2][8];
  const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* xr = x + static_cast<size_t>(row) * D;
  float v[8];
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = tid + 256 * k;
    v[k] = i < D ? xr[i] : 0.f;
    s += v[k];
  }
  s = warp_sum(s);
  if (lane == 0) s_red[0][warp] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += s_red[0][k];
  const float mu = tot / D;
  float q = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const float d = tid + 256 * k < D ? v[k] - mu : 0.f;
    q += d * d;
  }
  q = warp_sum(q);
  if (lane == 0) s_red[1][warp] = q;
  __syncthreads();
  tot = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) tot += s_red[1][k];
  const float rs = rsqrtf(tot / D + eps);
  __nv_bfloat16* yr = y + static_cast<size_t>(row) * D;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int i = tid + 256 * k;
    if (i < D) yr[i] = __float2bfloat16((v[k] - mu) * rs * w[i] + b[i]);
  }
  if (tid == 0) { mean[row] = mu; rstd[row] = rs; }
}

// LayerNorm backward in two kernels.  (1) dx: one warp per row, two passes over
// the row (row sums, then dx).  (2) dw, db: a block covers 32 columns x 256
// rows (a warp reads 32 consecutive columns of one row, so loads are
// coalesced), reduces over its rows in shared memory and adds one partial per
// column to dw / db.
__global__ void ln_bwd_dx_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                                 const float* __restrict__ w, const float* __restrict__ mean,
                                 const float* __restrict__ rstd, float* __restrict__ dx, int T,
                                 int D) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= T) return;
  const float mu = mean[row], rs = rstd[row];
  const float* xr = x + static_cast<size_t>(row) * D;
  const __nv_bfloat16* dyr = dy + static_cast<size_t>(row) * D;
  float s1 = 0.f, s2 = 0.f;
  for (int i = lane; i < D; i += 32) {
    const float g = __bfloat162float(dyr[i]) * w[i];
    s1 += g;
    s2 += g * (xr[i] - mu) * rs;
  }
  s1 = warp_sum(s1) / D;
  s2 = warp_sum(s2) / D;
  float* dxr = dx + static_cast<size_t>(row) * D;
  for (int i = lane; i < D; i += 32) {
    const float xh = (xr[i] - mu) * rs;
    dxr[i] = rs * (__bfloat162float(dyr[i]) * w[i] - s1 - xh * s2);
  }
}

constexpr int kLnRowsPerBlock = 256;
__global__ void ln_bwd_dwdb_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                                   const float* __restrict__ mean, const float* __restrict__ rstd,
                                   float* __restrict__ dw, float* __restrict__ db, int T, int D) {
  __shared__ float sw[8][33], sb[8][33];
  const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;      // 32 columns x 8 row lanes
  const int col = blockIdx.x * 32 + cx;
  const int row_lo = blockIdx.y * kLnRowsPerBlock;
  const int row_hi = min(T, row_lo + kLnRowsPerBlock);
  float aw = 0.f, ab = 0.f;
  if (col < D) {
    for (int row = row_lo + ry; row < row_hi; row += 8) {
      const float d = __bfloat162float(dy[static_cast<size_t>(row) * D + col]);
      const float xh = (x[static_cast<size_t>(row) * D + col] - mean[row]) * rstd[row];
      aw += d * xh;
      ab += d;
    }
  }
  sw[ry][cx] = aw;
  sb[ry][cx] = ab;
  __syncthreads();
  if (ry == 0 && col < D) {
    float tw = 0.f, tb = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { tw += sw[k][cx]; tb += sb[k][cx]; }
    atomicAdd(dw + col, tw);
    atomicAdd(db + col, tb);
  }
}

// One block per row of logits [R, ld] (fp32, V valid columns).
__global__ void ce_fwd_kernel(const float* __restrict__ logits, long long ld,
                              const long long* __restrict__ labels, int V, float* __restrict__ lse,
                              float* __restrict__ label_logit, long long* __restrict__ argmax) {
  const int row = blockIdx.x;
  const float* lr = logits + row * ld;
  float m = -FLT_MAX;
  int mi = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    const float v = lr[i];
    if (v > m) { m = v; mi = i; }
  }
  __shared__ float sm[32];
  __shared__ int si[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
    if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
  }
  if (lane == 0) { sm[warp] = m; si[warp] = mi; }
  __syncthreads();
  if (warp == 0) {
    m = lane < nwarp ? sm[lane] : -FLT_MAX;
    mi = lane < nwarp ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, m, o);
      const int oi = __shfl_xor_sync(0xffffffffu, mi, o);
      if (om > m || (om == m && oi < mi)) { m = om; mi = oi; }
    }
    if (lane == 0) { sm[0] = m; si[0] = mi; }
  }
  __syncthreads();
  m = sm[0];
  float s = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) s += __expf(lr[i] - m);
  s = warp_sum(s);
  __shared__ float ss[32];
  if (lane == 0) ss[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < nwarp; ++k) t += ss[k];
    lse[row] = m + logf(t);
    long long lab = labels[row];
    if (lab < 0) lab = 0;
    label_logit[row] = lr[lab];
    argmax[row] = si[0];
  }
}

// dl[row, i] = scale[row] * (softmax(logits[row])[i] - [i == label]) as bf16 [R, ldo].
__global__ void ce_bwd_kernel(const float* __restrict__ logits, long long ld,
                              const long long* __restrict__ labels, const float* __restrict__ lse,
                              const float* __restrict__ scale, int V, __nv_bfloat16* __restrict__ dl,
                              long long ldo) {
  const int row = blockIdx.x;
  const float* lr = logits + row * ld;
  __nv_bfloat16* dr = dl + row * ldo;
  const float l = lse[row], sc = scale[row];
  long long lab = labels[row];
  if (lab < 0) lab = 0;
  for (int i = threadIdx.x; i < V; i += blockDim.x) {
    float v = __expf(lr[i] - l);
    if (i == lab) v -= 1.f;
    dr[i] = __float2bfloat16(v * sc);
  }
  for (long long i = V + threadIdx.x; i < ldo; i += blockDim.x) dr[i] = __float2bfloat16(0.f);
}

__global__ void adamw_kernel(float* __restrict__ p, const float* __restrict__ g,
                             float* __restrict__ m, float* __restrict__ v, long long n,
                             const float* __restrict__ clip_scale, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2) {
  const float cs = *clip_scale;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const float gi = g[i] * cs;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float pi = p[i];
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi;
    p[i] = pi - lr * upd;
  }
}

// out[0] += sum(g^2)
__global__ void sqnorm_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  float s = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += stride) {
    const float v = g[i];
    s += v * v;
  }
  s = warp_sum(s);
  __shared__ float sh[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) t += sh[k];
    atomicAdd(out, t);
  }
}


// ---------------------------------------------------------------------------
// Token + position embedding.  out[t, :] = tok[ids[t], :] + pos[t % S, :]
// (models/dawn_spatial_v41_exp.py:1504-1507).  One warp per token, float4 lanes.
__global__ void embed_fwd_kernel(const long long* __restrict__ ids, const float* __restrict__ tok,
                                 const float* __restrict__ pos, float* __restrict__ out, int T,
                                 int S, int D, int V) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  long long id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const float4* a = reinterpret_cast<const float4*>(tok + static_cast<size_t>(id) * D);
  const float4* b = reinterpret_cast<const float4*>(pos + static_cast<size_t>(t % S) * D);
  float4* o = reinterpret_cast<float4*>(out + static_cast<size_t>(t) * D);
  for (int i = lane; i < (D >> 2); i += 32) {
    const float4 x = a[i], y = b[i];
    o[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  }
}

// dtok[ids[t], :] += dy[t, :] (atomic: a token may repeat), one warp per token.
__global__ void embed_bwd_tok_kernel(const long long* __restrict__ ids, const float* __restrict__ dy,
                                     float* __restrict__ dtok, int T, int D, int V) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  long long id = ids[t];
  id = id < 0 ? 0 : (id >= V ? V - 1 : id);
  const float* g = dy + static_cast<size_t>(t) * D;
  float* d = dtok + static_cast<size_t>(id) * D;
  for (int i = lane; i < D; i += 32) atomicAdd(d + i, g[i]);
}

// dpos[s, :] = sum_b dy[b*S + s, :]; one thread per (s, column), fixed order.
__global__ void embed_bwd_pos_kernel(const float* __restrict__ dy, float* __restrict__ dpos, int B,
                                     int S, int D) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(S) * D) return;
  float acc = 0.f;
  for (int b = 0; b < B; ++b) acc += dy[static_cast<size_t>(b) * S * D + idx];
  dpos[idx] = acc;
}

// ---------------------------------------------------------------------------
// Off-diagonal |cos| statistics of a similarity matrix sim [m, m] (fp32, row
// stride ld): total[0] += sum_{i != j} |sim_ij|, and sgn[i, j] = sign(sim_ij)
// (0 on the diagonal) as bf16 for the backward GEMM.
__global__ void offdiag_abs_kernel(const float* __restrict__ sim, long long ld, int m,
                                   __nv_bfloat16* __restrict__ sgn, long long ld_s,
                                   float* __restrict__ total) {
  float acc = 0.f;
  const long long n = static_cast<long long>(m) * m;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long k = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; k < n;
       k += stride) {
    const int i = static_cast<int>(k / m), j = static_cast<int>(k % m);
    const float v = sim[i * ld + j];
    float sg = 0.f;
    if (i != j) {
      acc += fabsf(v);
      sg = v > 0.f ? 1.f : (v < 0.f ? -1.f : 0.f);
    }
    sgn[i * ld_s + j] = __float2bfloat16(sg);
  }
  acc = warp_sum(acc);
  __shared__ float sh[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) t += sh[k];
    atomicAdd(total, t);
  }
}

// ---------------------------------------------------------------------------
// Backward prologue of a scaled, sum-normalised SRW route y = s * raw / den:
//   dy_bf[t, :] = bf16(dy[t, :] * row_scale[t])        (row_scale = s / max(den, 1))
//   rowdot[t]   = sum_d dy[t, d] * y[t, d]             (feeds d_den and d_s)
// One warp per row; dy and y fp32.
__global__ void route_bwd_prologue_kernel(const float* __restrict__ dy, const float* __restrict__ y,
                                          const float* __restrict__ row_scale,
                                          __nv_bfloat16* __restrict__ dy_bf,
                                          float* __restrict__ rowdot, int T, int D) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float rs = row_scale[t];
  const float4* g = reinterpret_cast<const float4*>(dy + static_cast<size_t>(t) * D);
  const float4* yy = reinterpret_cast<const float4*>(y + static_cast<size_t>(t) * D);
  uint2* o = reinterpret_cast<uint2*>(dy_bf + static_cast<size_t>(t) * D);
  float acc = 0.f;
  for (int i = lane; i < (D >> 2); i += 32) {
    const float4 a = g[i], b = yy[i];
    acc += a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w;
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x * rs, a.y * rs);
    __nv_bfloat162 hi = __floats2bfloat162_rn(a.z * rs, a.w * rs);
    uint2 w;
    w.x = *reinterpret_cast<uint32_t*>(&lo);
    w.y = *reinterpret_cast<uint32_t*>(&hi);
    o[i] = w;
  }
  acc = warp_sum(acc);
  if (lane == 0) rowdot[t] = acc;
}

inline int grid_for(long long n, int block, int cap) {
  long long g = (n + block - 1) / block;
  return static_cast<int>(g < cap ? (g < 1 ? 1 : g) : cap);
}

}  // namespace

extern "C" int dsb_layernorm_fwd(const float* x, const float* w, const float* b, void* y_bf16,
                                 float* mean, float* rstd, int T, int D, float eps,
                                 cudaStream_t stream) {
  if (T <= 0) return 0;
  __nv_bfloat16* y = reinterpret_cast<__nv_bfloat16*>(y_bf16);
  if (T <= 296 && D <= 2048) {   // few rows: a block per row instead of a warp per row
    ln_fwd_block_kernel<<<T, 256, 0, stream>>>(x, w, b, y, mean, rstd, D, eps);
    return cudaGetLastError() == cudaSuccess ? 0 : 1;
  }
  const int warps = 8;
  const dim3 grid((T + warps - 1) / warps), block(warps * 32);
  if (D <= 32 * 16) ln_fwd_kernel<16><<<grid, block, 0, stream>>>(x, w, b, y, mean, rstd, T, D, eps);
  else if (D <= 32 * 40) ln_fwd_kernel<40><<<grid, block, 0, stream>>>(x, w, b, y, mean, rstd, T, D, eps);
  else if (D <= 32 * 64) ln_fwd_kernel<64><<<grid, block, 0, stream>>>(x, w, b, y, mean, rstd, T, D, eps);
  else ln_fwd_kernel<0><<<grid, block, 0, stream>>>(x, w, b, y, mean, rstd, T, D, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_layernorm_bwd(const void* dy_bf16, const float* x, const float* w,
                                 const float* mean, const float* rstd, float* dx, float* dw,
                                 float* db, int T, int D, cudaStream_t stream) {
  if (T <= 0) return 0;
  const __nv_bfloat16* dy = reinterpret_cast<const __nv_bfloat16*>(dy_bf16);
  ln_bwd_dx_kernel<<<(T + 7) / 8, 256, 0, stream>>>(dy, x, w, mean, rstd, dx, T, D);
  const dim3 grid((D + 31) / 32, (T + kLnRowsPerBlock - 1) / kLnRowsPerBlock);
  ln_bwd_dwdb_kernel<<<grid, 256, 0, stream>>>(dy, x, mean, rstd, dw, db, T, D);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_ce_fwd(const float* logits, long long ld, const long long* labels, int R, int V,
                          float* lse, float* label_logit, long long* argmax, cudaStream_t stream) {
  if (R <= 0) return 0;
  ce_fwd_kernel<<<R, 256, 0, stream>>>(logits, ld, labels, V, lse, label_logit, argmax);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_ce_bwd(const float* logits, long long ld, const long long* labels,
                          const float* lse, const float* scale, int R, int V, void* dl_bf16,
                          long long ldo, cudaStream_t stream) {
  if (R <= 0) return 0;
  ce_bwd_kernel<<<R, 256, 0, stream>>>(logits, ld, labels, lse, scale, V,
                                       reinterpret_cast<__nv_bfloat16*>(dl_bf16), ldo);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_adamw(float* p, const float* g, float* m, float* v, long long n,
                         const float* clip_scale, float lr, float b1, float b2, float eps, float wd,
                         float bc1, float bc2, cudaStream_t stream) {
  if (n <= 0) return 0;
  adamw_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, stream>>>(p, g, m, v, n, clip_scale, lr, b1,
                                                               b2, eps, wd, bc1, bc2);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_sqnorm_accumulate(const float* g, long long n, float* out,
                                     cudaStream_t stream) {
  if (n <= 0) return 0;
  sqnorm_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, stream>>>(g, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_embed_fwd(const long long* ids, const float* tok, const float* pos, float* out,
                             int T, int S, int D, int V, cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D & 3) return 2;
  embed_fwd_kernel<<<(T + 7) / 8, 256, 0, stream>>>(ids, tok, pos, out, T, S, D, V);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_embed_bwd(const long long* ids, const float* dy, float* dtok, float* dpos, int B,
                             int S, int D, int V, cudaStream_t stream) {
  const int T = B * S;
  if (T <= 0) return 0;
  embed_bwd_tok_kernel<<<(T + 7) / 8, 256, 0, stream>>>(ids, dy, dtok, T, D, V);
  const long long n = static_cast<long long>(S) * D;
  embed_bwd_pos_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(dy, dpos, B, S, D);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_offdiag_abs(const float* sim, long long ld, int m, void* sgn_bf16,
                               long long ld_s, float* total, cudaStream_t stream) {
  if (m <= 0) return 0;
  const long long n = static_cast<long long>(m) * m;
  offdiag_abs_kernel<<<grid_for(n, 256, 148 * 8), 256, 0, stream>>>(
      sim, ld, m, reinterpret_cast<__nv_bfloat16*>(sgn_bf16), ld_s, total);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

extern "C" int dsb_route_bwd_prologue(const float* dy, const float* y, const float* row_scale,
                                      void* dy_bf16, float* rowdot, int T, int D,
                                      cudaStream_t stream) {
  if (T <= 0) return 0;
  if (D & 3) return 2;
  route_bwd_prologue_kernel<<<(T + 7) / 8, 256, 0, stream>>>(
      dy, y, row_scale, reinterpret_cast<__nv_bfloat16*>(dy_bf16), rowdot, T, D);
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// ------------------------------------------------------------------ dropout
// Keep-mask dropout scaled by 1 / keep, optionally fused with the residual add
// that follows it (y = res + dropout(x)).  The mask is a counter-based hash of
// (seed, element index): nothing is stored, the backward kernel regenerates it.
// (The reference draws from the JAX key stream, models/dawn_spatial_v41_exp.py:
// 308-318; same distribution, different bits.)
namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}

// element 4*i4 + k of the tensor is kept iff its 32 hash bits are >= thresh
__device__ __forceinline__ void keep4(uint64_t seed, long long i4, uint32_t thresh, float scale,
                                      float (&m)[4]) {
  const uint64_t a = mix64(seed + static_cast<uint64_t>(2 * i4) * 0x9E3779B97F4A7C15ull);
  const uint64_t b = mix64(seed + static_cast<uint64_t>(2 * i4 + 1) * 0x9E3779B97F4A7C15ull);
  m[0] = static_cast<uint32_t>(a) >= thresh ? scale : 0.f;
  m[1] = static_cast<uint32_t>(a >> 32) >= thresh ? scale : 0.f;
  m[2] = static_cast<uint32_t>(b) >= thresh ? scale : 0.f;
  m[3] = static_cast<uint32_t>(b >> 32) >= thresh ? scale : 0.f;
}

__global__ void dropout_kernel(const float4* __restrict__ res, const float4* __restrict__ x,
                               float4* __restrict__ y, long long n4, uint64_t seed, uint32_t thresh,
                               float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n4;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    float m[4];
    keep4(seed, i, thresh, scale, m);
    const float4 v = x[i];
    float4 o = make_float4(v.x * m[0], v.y * m[1], v.z * m[2], v.w * m[3]);
    if (res != nullptr) {
      const float4 r = res[i];
      o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
    }
    y[i] = o;
  }
}

}  // namespace

extern "C" int dsb_dropout(const float* res, const float* x, float* y, long long n,
                           unsigned long long seed, float p, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 3) || !(p >= 0.f && p < 1.f)) return 2;
  const long long n4 = n >> 2;
  const uint32_t thresh = static_cast<uint32_t>(static_cast<double>(p) * 4294967296.0);
  long long blocks = (n4 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  dropout_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      reinterpret_cast<const float4*>(res), reinterpret_cast<const float4*>(x),
      reinterpret_cast<float4*>(y), n4, seed, thresh, 1.f / (1.f - p));
  return cudaGetLastError() == cudaSuccess ? 0 : 1;
}

// ----------------------------------------------------- multi-tensor launches
// AdamW and the squared gradient norm over a whole list of tensors in one launch
// each: a block takes one 64 K-element chunk of one tensor; the chunk -> tensor
// map is a prefix table in the kernel parameters (binary search, 8 steps).
namespace {

constexpr int kMultiMax = 160;                 // tensors per launch
constexpr long long kMultiChunk = 1 << 16;     // elements per block

struct MultiTable {
  const float* g[kMultiMax];
  float* p[kMultiMax];
  float* m[kMultiMax];
  float* v[kMultiMax];
  long long n[kMultiMax];
  int first_chunk[kMultiMax + 1];
  int count;
};

__device__ __forceinline__ int chunk_owner(const MultiTable& t, int chunk) {
  int lo = 0, hi = t.count - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (t.first_chunk[mid] <= chunk) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

__global__ void __launch_bounds__(256) adamw_multi_kernel(const __grid_constant__ MultiTable t,
                                                          const float* __restrict__ clip_scale,
                                                          float lr, float b1, float b2, float eps,
                                                          float wd, float bc1, float bc2) {
  const int ti = chunk_owner(t, blockIdx.x);
  const long long off = static_cast<long long>(blockIdx.x - t.first_chunk[ti]) * kMultiChunk;
  const long long n = min(kMultiChunk, t.n[ti] - off);
  float* __restrict__ p = t.p[ti] + off;
  const float* __restrict__ g = t.g[ti] + off;
  float* __restrict__ m = t.m[ti] + off;
  float* __restrict__ v = t.v[ti] + off;
  const float cs = *clip_scale;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const float gi = g[i] * cs;
    const float mi = b1 * m[i] + (1.f - b1) * gi;
    const float vi = b2 * v[i] + (1.f - b2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float pi = p[i];
    const float upd = (mi / bc1) / (sqrtf(vi / bc2) + eps) + wd * pi;
    p[i] = pi - lr * upd;
  }
}

__global__ void __launch_bounds__(256) sqnorm_multi_kernel(const __grid_constant__ MultiTable t,
                                                           float* __restrict__ out) {
  const int ti = chunk_owner(t, blockIdx.x);
  const long long off = static_cast<long long>(blockIdx.x - t.first_chunk[ti]) * kMultiChunk;
  const long long n = min(kMultiChunk, t.n[ti] - off);
  const float* __restrict__ g = t.g[ti] + off;
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) {
    const float x = g[i];
    s = fmaf(x, x, s);
  }
  s = warp_sum(s);
  __shared__ float sh[8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += sh[k];
    atomicAdd(out, tot);
  }
}

// Fills `t` with tensors [i0, i0 + cnt) of the lists; returns the number of chunks.
int fill_table(MultiTable& t, const float* const* g, float* const* p, float* const* m, float* const* v,
               const long long* n, int i0, int cnt) {
  int chunks = 0, k = 0;
  for (int i = i0; i < i0 + cnt; ++i) {
    if (n[i] <= 0) continue;
    t.g[k] = g[i];
    t.p[k] = p != nullptr ? p[i] : nullptr;
    t.m[k] = m != nullptr ? m[i] : nullptr;
    t.v[k] = v != nullptr ? v[i] : nullptr;
    t.n[k] = n[i];
    t.first_chunk[k] = chunks;
    chunks += static_cast<int>((n[i] + kMultiChunk - 1) / kMultiChunk);
    ++k;
  }
  t.first_chunk[k] = chunks;
  t.count = k;
  return chunks;
}

}  // namespace

extern "C" int dsb_adamw_multi(float* const* p, const float* const* g, float* const* m, float* const* v,
                               const long long* n, int count, const float* clip_scale, float lr,
                               float b1, float b2, float eps, float wd, float bc1, float bc2,
                               cudaStream_t stream) {
  for (int i0 = 0; i0 < count; i0 += kMultiMax) {
    MultiTable t;
    const int cnt = count - i0 < kMultiMax ? count - i0 : kMultiMax;
    const int chunks = fill_table(t, g, p, m, v, n, i0, cnt);
    if (chunks == 0) continue;
    adamw_multi_kernel<<<chunks, 256, 0, stream>>>(t, clip_scale, lr, b1, b2, eps, wd, bc1, bc2);
    if (cudaGetLastError() != cudaSuccess) return 1;
  }
  return 0;
}

extern "C" int dsb_sqnorm_multi(const float* const* g, const long long* n, int count, float* out,
                                cudaStream_t stream) {
  for (int i0 = 0; i0 < count; i0 += kMultiMax) {
    MultiTable t;
    const int cnt = count - i0 < kMultiMax ? count - i0 : kMultiMax;
    const int chunks = fill_table(t, g, nullptr, nullptr, nullptr, n, i0, cnt);
    if (chunks == 0) continue;
    sqnorm_multi_kernel<<<chunks, 256, 0, stream>>>(t, out);
    if (cudaGetLastError() != cudaSuccess) return 1;
  }
  return 0;
}
