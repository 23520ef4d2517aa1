// SRW pool op for a handful of token rows (KV-cache decoding at batch 1..4).
//
// With one to four rows the op is a stream over the pool: per unit u it needs
// e_u (r values), r_u and w_u (d_model values each), about 5.6 KB at the 400M
// shapes, and a few hundred FMAs.  A tensor-core tile would spend a 128-row MMA on
// those rows, so this path is plain SIMT and bound by HBM: one warp per unit,
//   s_t  = <h_t, e_u>           (warp reduction)
//   g_t  = gate(s_t; tau_t, 1/sigma_t),   den_t += den_term
//   xr_t = <x_t, r_u>           (only if some g_t != 0: the relu-type gates of
//                                v3.9.4 / v4.0.1 are exactly zero below the
//                                threshold, and then r_u and w_u are not read)
//   acc_t += bf16(g_t * xr_t) * w_u
// Each block keeps its partial outputs; a second kernel adds the blocks' partials
// and applies scale / max(sum den, 1).  The reference runs the generic chunked
// kernels for decoding (models/dawn_spatial_v41_exp.py:1713-1739, 1913-1957).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "common/gate_math.cuh"
#include "dsb_api.h"
#include "dsb_api_ops.h"

namespace dsb {
namespace {

constexpr int kRowWarps = 8;        // warps per block
constexpr int kMaxRouteDim = 512;   // d_route <= 384 in every supported model

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// 8 bf16 -> 8 floats
__device__ __forceinline__ void unpack8(const uint4& q, float* f) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&q);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 v = __bfloat1622float2(p[i]);
    f[2 * i] = v.x;
    f[2 * i + 1] = v.y;
  }
}

__device__ __forceinline__ uint4 ldg_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

struct RowsParams {
  const __nv_bfloat16* h;       // [N, r]   contiguous
  const __nv_bfloat16* x;       // [N, D]   contiguous
  const float* tau;             // [N]
  const float* isd;             // [N]
  const __nv_bfloat16* emb;     // [U, lde]
  const __nv_bfloat16* read;    // [U, ldr]
  const __nv_bfloat16* write;   // [U, ldw]
  const float* unit_mask;       // [U] or null
  long long lde, ldr, ldw;
  int N, U, r, D;
  float* part;                  // [blocks, NR, D] partial outputs
  float* den_part;              // [blocks, NR]
  GateConsts gc;
};

// NR: rows handled (N <= NR); KC: 16-byte chunks of a d_model row per lane.
template <int KIND, int NR, int KC>
__global__ void __launch_bounds__(kRowWarps * 32, (NR == 1 && KC == 5) ? 2 : 1) srw_rows_kernel(const RowsParams p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);                  // [NR][D]
  __nv_bfloat16* s_h = s_x + NR * p.D;                                              // [NR][r]
  float* s_acc = reinterpret_cast<float*>(s_h + NR * p.r);                          // [NR][D]
  float* s_den = s_acc + NR * p.D;                                                  // [NR]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < NR * p.D; i += blockDim.x) {
    const int t = i / p.D;
    s_x[i] = t < p.N ? p.x[i] : __float2bfloat16(0.f);
    s_acc[i] = 0.f;
  }
  for (int i = tid; i < NR * p.r; i += blockDim.x) {
    const int t = i / p.r;
    s_h[i] = t < p.N ? p.h[i] : __float2bfloat16(0.f);
  }
  if (tid < NR) s_den[tid] = 0.f;
  __syncthreads();
  RowGate rg[NR];
#pragma unroll
  for (int t = 0; t < NR; ++t)
    rg[t] = row_gate<KIND>(p.gc, t < p.N ? p.tau[t] : 0.f, t < p.N ? p.isd[t] : 1.f);

  const int d_chunks = p.D >> 3, r_chunks = p.r >> 3;
  float acc[NR][KC * 8];
  float den[NR];
#pragma unroll
  for (int t = 0; t < NR; ++t) {
    den[t] = 0.f;
#pragma unroll
    for (int j = 0; j < KC * 8; ++j) acc[t][j] = 0.f;
  }
  const int warps_total = gridDim.x * kRowWarps;
  constexpr int kEC = kMaxRouteDim / 256;      // 16-byte chunks of an embedding row per lane
  auto load_emb = [&](int u, uint4 (&eq)[kEC]) {
#pragma unroll
    for (int k = 0; k < kEC; ++k) {
      const int c = lane + 32 * k;
      eq[k] = (u < p.U && c < r_chunks) ? ldg_stream(p.emb + static_cast<size_t>(u) * p.lde + 8 * c)
                                        : make_uint4(0u, 0u, 0u, 0u);
    }
  };
  uint4 e_next[kEC];
  load_emb(blockIdx.x * kRowWarps + warp, e_next);
  for (int u = blockIdx.x * kRowWarps + warp; u < p.U; u += warps_total) {
    // ---- scores of this unit for all rows; the next unit's embedding row is already on its way
    uint4 e_cur[kEC];
#pragma unroll
    for (int k = 0; k < kEC; ++k) e_cur[k] = e_next[k];
    load_emb(u + warps_total, e_next);
    float s[NR];
#pragma unroll
    for (int t = 0; t < NR; ++t) s[t] = 0.f;
#pragma unroll
    for (int k = 0; k < kEC; ++k) {
      const int c = lane + 32 * k;
      if (c < r_chunks) {
        float e[8];
        unpack8(e_cur[k], e);
#pragma unroll
        for (int t = 0; t < NR; ++t) {
          float hv[8];
          unpack8(*reinterpret_cast<const uint4*>(s_h + t * p.r + 8 * c), hv);
#pragma unroll
          for (int j = 0; j < 8; ++j) s[t] = fmaf(e[j], hv[j], s[t]);
        }
      }
    }
    float g[NR];
    bool any = false;
    const float um = p.unit_mask != nullptr ? p.unit_mask[u] : 1.f;
#pragma unroll
    for (int t = 0; t < NR; ++t) {
      const float st = warp_sum(s[t]);
      float dt;
      gate_fwd_shifted<KIND>(p.gc, fmaf(st, rg[t].a, rg[t].b), g[t], dt);
      g[t] *= um;
      dt *= um;
      if (t < p.N) {
        den[t] += dt;
        any = any || g[t] != 0.f;
      }
    }
    if (!any) continue;                                   // warp-uniform: nothing to read or write
    // ---- read scalars and the gated write, both rows of the unit in flight together
    uint4 rq[KC], wq[KC];
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = lane + 32 * k;
      if (c < d_chunks) {
        rq[k] = ldg_stream(p.read + static_cast<size_t>(u) * p.ldr + 8 * c);
        wq[k] = ldg_stream(p.write + static_cast<size_t>(u) * p.ldw + 8 * c);
      } else {
        rq[k] = make_uint4(0u, 0u, 0u, 0u);
        wq[k] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    float xr[NR];
#pragma unroll
    for (int t = 0; t < NR; ++t) xr[t] = 0.f;
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = lane + 32 * k;
      if (c < d_chunks) {
        float rv[8];
        unpack8(rq[k], rv);
#pragma unroll
        for (int t = 0; t < NR; ++t) {
          float xv[8];
          unpack8(*reinterpret_cast<const uint4*>(s_x + t * p.D + 8 * c), xv);
#pragma unroll
          for (int j = 0; j < 8; ++j) xr[t] = fmaf(rv[j], xv[j], xr[t]);
        }
      }
    }
    float pv[NR];
#pragma unroll
    for (int t = 0; t < NR; ++t)   // p is rounded to bf16, as the tile kernels store it
      pv[t] = __bfloat162float(__float2bfloat16(g[t] * warp_sum(xr[t])));
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      float wv[8];
      unpack8(wq[k], wv);
#pragma unroll
      for (int t = 0; t < NR; ++t)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[t][8 * k + j] = fmaf(pv[t], wv[j], acc[t][8 * k + j]);
    }
  }
  // ---- block partials: warps add into shared memory, the block writes one slab
#pragma unroll
  for (int t = 0; t < NR; ++t) {
#pragma unroll
    for (int k = 0; k < KC; ++k) {
      const int c = lane + 32 * k;
      if (c < d_chunks) {
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(&s_acc[t * p.D + 8 * c + j], acc[t][8 * k + j]);
      }
    }
    if (lane == 0) atomicAdd(&s_den[t], den[t]);
  }
  __syncthreads();
  float* out = p.part + static_cast<size_t>(blockIdx.x) * NR * p.D;
  for (int i = tid; i < NR * p.D; i += blockDim.x) out[i] = s_acc[i];
  if (tid < NR) p.den_part[blockIdx.x * NR + tid] = s_den[tid];
}

// out[t, :] = (sum_b part[b, t, :]) * scale / max(sum_b den_part[b, t], 1).
// A block covers 32 columns of one row: 8 groups of 32 threads share the blocks'
// partials (coalesced 128-byte reads), then meet in shared memory.
__global__ void __launch_bounds__(256) srw_rows_finish_kernel(
    const float* __restrict__ part, const float* __restrict__ den_part, int blocks, int NR, int N,
    int D, float scale, const float* __restrict__ scale_ptr, float* __restrict__ out,
    float* __restrict__ den_out) {
  __shared__ float s_col[8][32];
  __shared__ float s_den[8];
  const int t = blockIdx.y, tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  const int j = blockIdx.x * 32 + lane;
  float d = 0.f;
  for (int b = tid; b < blocks; b += 256) d += den_part[b * NR + t];
  d = warp_sum(d);
  if (lane == 0) s_den[grp] = d;
  float a0 = 0.f, a1 = 0.f;
  if (j < D) {
    int b = grp;
    for (; b + 8 < blocks; b += 16) {
      a0 += part[(static_cast<size_t>(b) * NR + t) * D + j];
      a1 += part[(static_cast<size_t>(b + 8) * NR + t) * D + j];
    }
    if (b < blocks) a0 += part[(static_cast<size_t>(b) * NR + t) * D + j];
  }
  s_col[grp][lane] = a0 + a1;
  __syncthreads();
  if (grp == 0) {
    float den = 0.f, a = 0.f;
#pragma unroll
    for (int g = 0; g < 8; ++g) { den += s_den[g]; a += s_col[g][lane]; }
    const float sc = (scale_ptr != nullptr ? scale_ptr[0] : scale) / fmaxf(den, 1.f);
    if (j < D) out[static_cast<size_t>(t) * D + j] = a * sc;
    if (den_out != nullptr && blockIdx.x == 0 && lane == 0) den_out[t] = den;
  }
}

// One decoded token of one (batch, head): append k, v to the cache at position
// pos[0], then softmax(q . K[0..pos]^T / sqrt(dh)) . V[0..pos].  q, k, v, out are
// token-major fp32 [B, H * dh]; the caches are fp32 [B, H, S_max, dh].  The position
// is a device scalar so that the launch can sit in a captured graph.
__global__ void __launch_bounds__(128) kv_decode_attention_kernel(
    const float* __restrict__ q, const float* __restrict__ k, const float* __restrict__ v,
    float* __restrict__ cache_k, float* __restrict__ cache_v, const long long* __restrict__ pos_ptr,
    int H, int dh, int s_max, float inv_sqrt_dh, float* __restrict__ out) {
  extern __shared__ float s_p[];                 // [s_max] scores, then probabilities
  __shared__ float s_red[4];
  __shared__ float s_q[128];
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  long long pos = pos_ptr[0];
  if (pos < 0) pos = 0;
  if (pos >= s_max) pos = s_max - 1;
  const int n = static_cast<int>(pos) + 1;
  const size_t row = static_cast<size_t>(b) * H * dh + static_cast<size_t>(h) * dh;
  float* ck = cache_k + (static_cast<size_t>(b) * H + h) * s_max * dh;
  float* cv = cache_v + (static_cast<size_t>(b) * H + h) * s_max * dh;
  if (tid < dh) {
    ck[pos * dh + tid] = k[row + tid];
    cv[pos * dh + tid] = v[row + tid];
    s_q[tid] = q[row + tid] * inv_sqrt_dh;
  }
  __syncthreads();
  // scores: one warp per cache position
  float mx = -3.0e38f;
  for (int j = warp; j < n; j += 4) {
    float a = 0.f;
    for (int t = lane; t < dh; t += 32) a = fmaf(s_q[t], ck[static_cast<size_t>(j) * dh + t], a);
    a = warp_sum(a);
    if (lane == 0) s_p[j] = a;
    mx = fmaxf(mx, a);
  }
  if (lane == 0) s_red[warp] = mx;
  __syncthreads();
  mx = fmaxf(fmaxf(s_red[0], s_red[1]), fmaxf(s_red[2], s_red[3]));
  __syncthreads();
  float sum = 0.f;
  for (int j = tid; j < n; j += 128) {
    const float e = __expf(s_p[j] - mx);
    s_p[j] = e;
    sum += e;
  }
  sum = warp_sum(sum);
  if (lane == 0) s_red[warp] = sum;
  __syncthreads();
  const float inv = 1.f / (s_red[0] + s_red[1] + s_red[2] + s_red[3]);
  if (tid < dh) {
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    int j = 0;
    for (; j + 4 <= n; j += 4) {
      a0 = fmaf(s_p[j], cv[static_cast<size_t>(j) * dh + tid], a0);
      a1 = fmaf(s_p[j + 1], cv[static_cast<size_t>(j + 1) * dh + tid], a1);
      a2 = fmaf(s_p[j + 2], cv[static_cast<size_t>(j + 2) * dh + tid], a2);
      a3 = fmaf(s_p[j + 3], cv[static_cast<size_t>(j + 3) * dh + tid], a3);
    }
    for (; j < n; ++j) a0 = fmaf(s_p[j], cv[static_cast<size_t>(j) * dh + tid], a0);
    out[row + tid] = ((a0 + a1) + (a2 + a3)) * inv;
  }
}

// y[t, n] = <x_t, W_n> + bias[n] for up to four rows x_t: one warp per output column, the
// weight matrix streamed once with 16-byte loads, x in shared memory.  x bf16 [N, K]
// contiguous, W bf16 [n_out, ldw], y fp32 [N, ldy]; K % 8 == 0.
template <int NR>
__global__ void __launch_bounds__(256) gemv_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                                        const __nv_bfloat16* __restrict__ w, long long ldw,
                                                        const float* __restrict__ bias,
                                                        float* __restrict__ y, long long ldy, int N,
                                                        int n_out, int K) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* s_x = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  for (int i = threadIdx.x; i < NR * K; i += blockDim.x)
    s_x[i] = i / K < N ? x[i] : __float2bfloat16(0.f);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, chunks = K >> 3;
  for (int n = blockIdx.x * 8 + warp; n < n_out; n += gridDim.x * 8) {
    float acc[NR];
#pragma unroll
    for (int t = 0; t < NR; ++t) acc[t] = 0.f;
    const __nv_bfloat16* wr = w + static_cast<size_t>(n) * ldw;
    for (int c = lane; c < chunks; c += 32) {
      float wv[8];
      unpack8(ldg_stream(wr + 8 * c), wv);
#pragma unroll
      for (int t = 0; t < NR; ++t) {
        float xv[8];
        unpack8(*reinterpret_cast<const uint4*>(s_x + t * K + 8 * c), xv);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[t] = fmaf(wv[j], xv[j], acc[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < NR; ++t) {
      const float a = warp_sum(acc[t]);
      if (lane == 0 && t < N) y[static_cast<size_t>(t) * ldy + n] = a + (bias != nullptr ? bias[n] : 0.f);
    }
  }
}

template <int KIND, int NR, int KC>
int launch_rows(const RowsParams& p, int blocks, cudaStream_t stream) {
  const size_t smem = static_cast<size_t>(NR) * (p.D + p.r) * 2 + static_cast<size_t>(NR) * p.D * 4 + NR * 4 + 16;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(srw_rows_kernel<KIND, NR, KC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             96 * 1024) != cudaSuccess)
      return 902;
    attr_set = true;
  }
  if (smem > 96 * 1024) return 903;
  srw_rows_kernel<KIND, NR, KC><<<blocks, kRowWarps * 32, smem, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : 904;
}

template <int KIND>
int dispatch_rows(const RowsParams& p, int NR, int KC, int blocks, cudaStream_t stream) {
  if (KC == 5) {
    if (NR == 1) return launch_rows<KIND, 1, 5>(p, blocks, stream);
    if (NR == 2) return launch_rows<KIND, 2, 5>(p, blocks, stream);
    return launch_rows<KIND, 4, 5>(p, blocks, stream);
  }
  if (NR == 1) return launch_rows<KIND, 1, 8>(p, blocks, stream);
  if (NR == 2) return launch_rows<KIND, 2, 8>(p, blocks, stream);
  return 905;
}

}  // namespace
}  // namespace dsb

using namespace dsb;

extern "C" int dsb_srw_rows_max(int D) {
  if (D % 8 != 0 || D > 2048) return 0;
  return D <= 1280 ? 4 : 2;
}

extern "C" int dsb_srw_rows_blocks(int N, int D) {
  int dev = 0, n = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
  if (n <= 0) n = 148;
  return (N <= 1 && D <= 1280) ? 2 * n : n;   // one row needs 128 registers: two blocks per SM
}

extern "C" int dsb_srw_rows(const void* h, const void* x, const float* tau, const float* isd,
                            const void* emb, long long lde, const void* read, long long ldr,
                            const void* write, long long ldw, const float* unit_mask, int N, int U,
                            int r, int D, const DsbGate* gate, float scale, const float* scale_ptr,
                            float* part, float* den_part, float* out, float* den_out,
                            cudaStream_t stream) {
  if (N <= 0 || U <= 0) return 0;
  const int max_rows = dsb_srw_rows_max(D);
  if (N > max_rows || r % 8 != 0 || r > kMaxRouteDim || lde % 8 != 0 || ldr % 8 != 0 || ldw % 8 != 0)
    return 901;
  const int NR = N <= 1 ? 1 : N <= 2 ? 2 : 4;
  const int KC = D <= 1280 ? 5 : 8;
  const int blocks = dsb_srw_rows_blocks(N, D);
  RowsParams p;
  p.h = static_cast<const __nv_bfloat16*>(h);
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.tau = tau;
  p.isd = isd;
  p.emb = static_cast<const __nv_bfloat16*>(emb);
  p.read = static_cast<const __nv_bfloat16*>(read);
  p.write = static_cast<const __nv_bfloat16*>(write);
  p.unit_mask = unit_mask;
  p.lde = lde; p.ldr = ldr; p.ldw = ldw;
  p.N = N; p.U = U; p.r = r; p.D = D;
  p.part = part;
  p.den_part = den_part;
  p.gc = {gate->kind, gate->sharpness, gate->act_threshold, gate->act_cutoff, gate->epsilon,
          gate->max_intensity, gate->clip_max, gate->dead_threshold};
  int rc;
  if (gate->kind == 0) rc = dispatch_rows<0>(p, NR, KC, blocks, stream);
  else if (gate->kind == 1) rc = dispatch_rows<1>(p, NR, KC, blocks, stream);
  else rc = dispatch_rows<2>(p, NR, KC, blocks, stream);
  if (rc) return rc;
  const dim3 grid((D + 31) / 32, N);
  srw_rows_finish_kernel<<<grid, 256, 0, stream>>>(part, den_part, blocks, NR, N, D, scale, scale_ptr,
                                                   out, den_out);
  return cudaGetLastError() == cudaSuccess ? 0 : 906;
}

extern "C" int dsb_kv_decode_attention(const float* q, const float* k, const float* v, float* cache_k,
                                       float* cache_v, const long long* pos, int B, int H, int dh,
                                       int s_max, float* out, cudaStream_t stream) {
  if (B <= 0 || H <= 0) return 0;
  if (dh <= 0 || dh > 128 || s_max <= 0 || s_max > 8192) return 911;
  const dim3 grid(H, B);
  kv_decode_attention_kernel<<<grid, 128, static_cast<size_t>(s_max) * sizeof(float), stream>>>(
      q, k, v, cache_k, cache_v, pos, H, dh, s_max, rsqrtf(static_cast<float>(dh)), out);
  return cudaGetLastError() == cudaSuccess ? 0 : 912;
}

extern "C" int dsb_gemv_rows(const void* x, const void* w, long long ldw, const float* bias, float* y,
                             long long ldy, int N, int n_out, int K, cudaStream_t stream) {
  if (N <= 0 || n_out <= 0) return 0;
  if (N > 4 || K % 8 != 0 || K > 8192 || ldw % 8 != 0) return 921;
  const int NR = N <= 1 ? 1 : N <= 2 ? 2 : 4;
  int blocks = (n_out + 7) / 8;
  const int cap = 8 * dsb_srw_rows_blocks(4, 2048);
  if (blocks > cap) blocks = cap;
  const size_t smem = static_cast<size_t>(NR) * K * 2;
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(gemv_rows_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    cudaFuncSetAttribute(gemv_rows_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    cudaFuncSetAttribute(gemv_rows_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    attr_set = true;
  }
  const __nv_bfloat16* xb = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wb = static_cast<const __nv_bfloat16*>(w);
  if (NR == 1) gemv_rows_kernel<1><<<blocks, 256, smem, stream>>>(xb, wb, ldw, bias, y, ldy, N, n_out, K);
  else if (NR == 2) gemv_rows_kernel<2><<<blocks, 256, smem, stream>>>(xb, wb, ldw, bias, y, ldy, N, n_out, K);
  else gemv_rows_kernel<4><<<blocks, 256, smem, stream>>>(xb, wb, ldw, bias, y, ldy, N, n_out, K);
  return cudaGetLastError() == cudaSuccess ? 0 : 922;
}
