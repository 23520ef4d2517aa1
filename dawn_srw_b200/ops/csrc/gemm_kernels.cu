// tcgen05 GEMM kernels built on the engine: a plain GEMM with a fused
// scale/bias/accumulate epilogue, and the two SRW "gate" kernels whose
// epilogues turn score / read / grad accumulators into the gated operand
// tiles the following GEMMs consume.
//
// SRW forward gate kernel (per 128-token x 128-unit tile):
//   S  = h . emb^T   (K = d_route)      -> TMEM accumulator 0
//   XR = x . read^T  (K = d_model)      -> TMEM accumulator 1
//   epilogue: g = gate(S, tau, 1/sigma); p = g * XR -> bf16 [T, U];
//             sum_U den_term -> den_sum[T] (atomic); per-unit "alive" flags.
// SRW backward gate kernel adds DP = dy . write^T (accumulator 2) and emits
//   p, dxr = DP*g, ds = d(loss)/dS through the gate, plus the per-token sums
//   that flow to tau and sigma.
// The reference computes the same quantities chunk by chunk in XLA
// (models/dawn_spatial_v41_exp.py:485-586) and derives the backward by autodiff.
#include <stdlib.h>
#include <string.h>

#include <cuda_fp16.h>

#include "common/gate_math.cuh"
#include "common/gemm_engine.cuh"
#include "common/host_utils.cuh"
#include "dsb_api.h"

namespace dsb {

// Returns g; ds = d loss / d s through the gate given dg (grad on the gate
// value) and dden (grad on the denominator term); dsz = ds * z (v4.0.1 only).
template <int KIND>
__device__ __forceinline__ float gate_bwd(const GateConsts& gc, float s, float tau, float isg,
                                          float dg, float dden, float& ds, float& dsz) {
  float g;
  dsz = 0.f;
  if constexpr (KIND == 0) {
    const float raw = s - tau;
    g = fminf(fmaxf(raw, 0.f), gc.clip_max);
    ds = (raw > 0.f && raw < gc.clip_max) ? (dg + dden) : 0.f;
  } else if constexpr (KIND == 1) {
    const float zr = (s - tau) * isg;
    const float z = fmaxf(zr, 0.f);
    float phi, pdf;
    phi_pdf(z, phi, pdf);
    g = z * phi;
    ds = zr > 0.f ? (dg + dden) * fmaf(z, pdf, phi) * isg : 0.f;
    dsz = ds * z;
  } else {
    const float m = s - tau - gc.thr;
    const float act = rcp_approx(1.f + __expf(-gc.sharp * m));
    const float amr = m - gc.cut;
    const float inten = gc.eps + fminf(fmaxf(amr, 0.f), gc.max_int);
    g = act * inten;
    const float lin = (amr > 0.f && amr < gc.max_int) ? 1.f : 0.f;
    ds = dg * inten * gc.sharp * act * (1.f - act) + (dg * act + dden) * lin;
  }
  return g;
}

// Stage 32 fp32 values of this thread's row as bf16 into chunks
// [chunk0, chunk0+4) of a 64-column bf16 slab.
__device__ __forceinline__ void stage_bf16_32(const WarpStager& st, uint32_t buf, int chunk0,
                                              const float* v) {
#pragma unroll
  for (int q = 0; q < 4; ++q)
    st.put(buf, chunk0 + q, pack_bf16x2(v[8 * q], v[8 * q + 1]),
           pack_bf16x2(v[8 * q + 2], v[8 * q + 3]), pack_bf16x2(v[8 * q + 4], v[8 * q + 5]),
           pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
}
__device__ __forceinline__ void stage_bf16_16(const WarpStager& st, uint32_t buf, int chunk0,
                                              const float* v) {
#pragma unroll
  for (int q = 0; q < 2; ++q)
    st.put(buf, chunk0 + q, pack_bf16x2(v[8 * q], v[8 * q + 1]),
           pack_bf16x2(v[8 * q + 2], v[8 * q + 3]), pack_bf16x2(v[8 * q + 4], v[8 * q + 5]),
           pack_bf16x2(v[8 * q + 6], v[8 * q + 7]));
}

// --------------------------------------------------------- plain epilogue
struct PlainEpi {
  static constexpr int kNumAcc = 1;
  static constexpr int kNumOut = 1;   // (kMaxOut maps when scattering; they are not prefetched)
  static constexpr int kOutBufs = 2;
  static constexpr int kEpiWarps = 4;
  __host__ __device__ static constexpr int acc_bufs(int) { return 2; }
  struct Params {
    float alpha;
    const float* row_scale;  // optional [M]
    const float* bias;       // optional [N]
    int out_bf16;            // 1: bf16 output, 0: fp32
    int accumulate;          // 1: out += result (fp32 output only; TMA reduce-add)
    // Fused reduce-scatter, first half: when > 0, global row R of the result
    // belongs to rank R / scatter_rows and is stored into slot `scatter_rank` of
    // that rank's receive buffer [n_ranks * scatter_rows, N] (tensor map index =
    // owner rank; peer memory for the other ranks).  Plain TMA stores: every
    // (owner, slot) row is written by exactly one rank, the owner sums its
    // slots afterwards (dsb_sum_slabs).  Stores cross NVLink at write bandwidth,
    // which remote reduce-adds (atomics) do not.
    int scatter_rows;
    int scatter_rank;
    // With a scatter: an fp32 value per row of the result (a partial per-token sum such as
    // the denominator) that goes to the row's owner too: aux_dst[owner][scatter_rank *
    // scatter_rows + local row] = aux_src[row], written by the tiles of the first column block.
    const float* aux_src;
    float* aux_dst[kMaxOut];
  };
  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    const int r0 = m0 + warp * 32;
    if (r0 >= M) { ctl.skip(); return; }  // whole 32-row slab is outside the matrix (warp-uniform)
    const uint32_t acc0 = ctl.wait(0);
    const int row = r0 + lane;
    const float scale = p.alpha * ((row < M && p.row_scale) ? p.row_scale[row] : 1.f);
    if (p.scatter_rows > 0 && p.aux_src != nullptr && n0 == 0 && row < M) {
      const int owner = r0 / p.scatter_rows;
      p.aux_dst[owner][p.scatter_rank * p.scatter_rows + (row - owner * p.scatter_rows)] =
          p.aux_src[row];
    }
    int slab = 0;
    if (p.out_bf16) {
#pragma unroll 1
      for (int c = 0; c < BN; c += 64, ++slab) {
        const int col0 = n0 + c;
        if (col0 >= N) break;
        st.wait_free<1>();
        const uint32_t buf = st.buf(slab & 1);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float v[32];
          tmem_ld32(acc0 + c + 32 * half, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] *= scale;
          if (p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int col = col0 + 32 * half + j;
              if (col < N) v[j] += p.bias[col];
            }
          }
          stage_bf16_32(st, buf, 4 * half, v);
        }
        if (p.scatter_rows > 0) {
          const int owner = r0 / p.scatter_rows;
          st.flush(&maps[owner], buf, col0,
                   p.scatter_rank * p.scatter_rows + (r0 - owner * p.scatter_rows), false, true);
        } else {
          st.flush(&maps[0], buf, col0, r0, false, true);
        }
      }
    } else {
#pragma unroll 1
      for (int c = 0; c < BN; c += 32, ++slab) {
        const int col0 = n0 + c;
        if (col0 >= N) break;
        st.wait_free<1>();
        const uint32_t buf = st.buf(slab & 1);
        float v[32];
        tmem_ld32(acc0 + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] *= scale;
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int col = col0 + j;
            if (col < N) v[j] += p.bias[col];
          }
        }
#pragma unroll
        for (int q = 0; q < 8; ++q)
          st.put(buf, q, __float_as_uint(v[4 * q]), __float_as_uint(v[4 * q + 1]),
                 __float_as_uint(v[4 * q + 2]), __float_as_uint(v[4 * q + 3]));
        if (p.scatter_rows > 0) {
          const int owner = r0 / p.scatter_rows;
          st.flush(&maps[owner], buf, col0,
                   p.scatter_rank * p.scatter_rows + (r0 - owner * p.scatter_rows), false, true);
        } else {
          st.flush(&maps[0], buf, col0, r0, p.accumulate != 0, true);
        }
      }
    }
    ctl.release(0);
  }
};

// ------------------------------------------------- LM-head cross-entropy epilogue
// Tied-embedding logits L = x . E^T (T x V, V = vocabulary) with the softmax
// statistics taken while the tile is still in TMEM: per row and per 256-column
// tile the epilogue emits (max, sum exp(l - max), arg-max, label logit) as one
// float4 and stores the logits as bf16, so no fp32 [T, V] tensor ever exists (the
// reference keeps the full fp32 logits, models/dawn_spatial_v41_exp.py:1642-1668).
// A row kernel merges the per-tile partials into logsumexp / label logit / arg-max;
// the backward pass turns the stored bf16 logits into d(loss)/d(logits) in place.
struct CeFwdEpi {
  static constexpr int kNumAcc = 1;
  static constexpr int kNumOut = 1;
  static constexpr int kOutBufs = 2;
  static constexpr int kEpiWarps = 4;
  __host__ __device__ static constexpr int acc_bufs(int) { return 2; }
  struct Params {
    const long long* labels;   // [M] label per row (< 0: no label)
    float4* partial;           // [M, n_tiles]
    int n_tiles;
  };
  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    const int r0 = m0 + warp * 32;
    if (r0 >= M) { ctl.skip(); return; }
    const uint32_t acc0 = ctl.wait(0);
    const int row = r0 + lane;
    const bool row_ok = row < M;
    const int label = row_ok ? static_cast<int>(p.labels[row]) : -1;
    float mx = -3.0e38f, sum = 0.f, lab_logit = 0.f;
    int amax = n0;
    int slab = 0;
#pragma unroll 1
    for (int c = 0; c < BN; c += 64, ++slab) {
      const int col0 = n0 + c;
      if (col0 >= N) break;
      st.wait_free<1>();
      const uint32_t buf = st.buf(slab & 1);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float v[32];
        tmem_ld32(acc0 + c + 32 * half, v);
        tmem_ld_wait();
        const int cb = col0 + 32 * half;
        // chunk maximum first, then one rescale of the running sum per chunk
        float cm = -3.0e38f;
        int ci = cb;
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const bool in = cb + j < N;
          if (in && v[j] > cm) { cm = v[j]; ci = cb + j; }
          if (cb + j == label) lab_logit = v[j];
        }
        if (cm > mx) {
          sum *= __expf(mx - cm);
          mx = cm;
          amax = ci;
        }
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (cb + j < N) sum += __expf(v[j] - mx);
        stage_bf16_32(st, buf, 4 * half, v);
      }
      st.flush(&maps[0], buf, col0, r0, false, true);
    }
    ctl.release(0);
    if (row_ok)
      p.partial[static_cast<size_t>(row) * p.n_tiles + n0 / BN] =
          make_float4(mx, sum, __int_as_float(amax), lab_logit);
  }
};

// One warp per row: merge the per-tile partials.
__global__ void ce_merge_kernel(const float4* __restrict__ partial, int n_tiles, int M,
                                const long long* __restrict__ labels, float* __restrict__ lse,
                                float* __restrict__ label_logit, long long* __restrict__ argmax) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  float mx = -3.0e38f, sum = 0.f, lab = 0.f;
  int am = 0x7fffffff;
  for (int t = lane; t < n_tiles; t += 32) {
    const float4 v = partial[static_cast<size_t>(row) * n_tiles + t];
    const int ai = __float_as_int(v.z);
    if (v.x > mx || (v.x == mx && ai < am)) {
      sum = sum * __expf(mx - v.x) + v.y;
      mx = v.x;
      am = ai;
    } else {
      sum += v.y * __expf(v.x - mx);
    }
    lab += v.w;      // exactly one tile holds the label's column, the others contribute 0
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float omx = __shfl_xor_sync(0xffffffffu, mx, o);
    const float osum = __shfl_xor_sync(0xffffffffu, sum, o);
    const int oam = __shfl_xor_sync(0xffffffffu, am, o);
    lab += __shfl_xor_sync(0xffffffffu, lab, o);
    if (omx > mx || (omx == mx && oam < am)) {
      sum = sum * __expf(mx - omx) + osum;
      mx = omx;
      am = oam;
    } else {
      sum += osum * __expf(omx - mx);
    }
  }
  if (lane == 0) {
    lse[row] = mx + __logf(sum);
    label_logit[row] = labels[row] >= 0 ? lab : 0.f;
    argmax[row] = am;
  }
}

// In place on the stored bf16 logits: dl = scale[row] * (exp(l - lse) - [col == label]);
// columns V.. of the padded row are zeroed.  One block per row.
__global__ void ce_bwd_inplace_kernel(__nv_bfloat16* __restrict__ logits, long long ld, int V,
                                      const long long* __restrict__ labels,
                                      const float* __restrict__ lse,
                                      const float* __restrict__ scale) {
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + static_cast<size_t>(row) * ld;
  const float l = lse[row], sc = scale[row];
  const int lab = static_cast<int>(labels[row]);
  for (int i = threadIdx.x * 8; i < ld; i += blockDim.x * 8) {
    uint4 u = *reinterpret_cast<const uint4*>(lr + i);
    __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 f = __bfloat1622float2(h2[e]);
      const int c0 = i + 2 * e;
      f.x = c0 < V ? sc * (__expf(f.x - l) - (c0 == lab ? 1.f : 0.f)) : 0.f;
      f.y = c0 + 1 < V ? sc * (__expf(f.y - l) - (c0 + 1 == lab ? 1.f : 0.f)) : 0.f;
      h2[e] = __floats2bfloat162_rn(f.x, f.y);
    }
    *reinterpret_cast<uint4*>(lr + i) = u;
  }
}

// ------------------------------------------------------ forward gate epilogue
// Eight epilogue warps: warp w handles rows 32(w%4).. of the tile and the
// (w/4)-th 64-column half, i.e. exactly one staged slab per tile.
struct FwdGateParams {
  // Per-token constants: either two arrays, or (wide kernels with a fused gather) one
  // float4 per token (tau, 1/sigma, -, -) that the gather warps bring in with the rows.
  const float4* stats;     // optional [T]
  const float* tau;        // [T]
  const float* inv_sigma;  // [T]
  float* den_sum;          // [T] += sum_U den_term
  float* gate_sum;         // optional [T] += sum_U g
  unsigned char* alive;    // optional [U]: 1 if any token gates the unit >= dead_thr
  const float* unit_mask;  // optional [U] multiplier on the gate (ablation)
  // Optional routing diagnostics (log steps; wide kernels only): per token kDiagCols fp32
  // accumulators over the units, see DiagCol, and two scalars (max intensity, count of
  // intensities at the cap) for the two-stage gate.  Zeroed by the caller.
  float* diag;             // [T, kDiagCols]
  float* diag_scalars;     // [2]
  GateConsts gc;
};
constexpr int kDiagCols = 12;
enum DiagCol : int {
  kDgGateSum = 0,   // sum_U g
  kDgActive = 1,    // units counted active (g > 0; act > 0.5 for the two-stage gate)
  kDgStrong = 2,    // g > 0.5 (act > 0.9)
  kDgBand = 3,      // Phi(z) outside [0.05, 0.95]  (act inside (0.1, 0.9))
  kDgZSum = 4,      // sum of positive z (sum of intensities)
  kDgB075 = 5,      // 0 < z < 0.75  (act inside (0.05, 0.95))
  kDgB030 = 6,      // 0 < z < 0.30  (act inside (0.2, 0.8))
  kDgGLogG = 7,     // sum g log(g + 1e-8)
  kDgS3 = 8,        // sum s^3
  kDgS4 = 9,        // sum s^4
  kDgGateMax = 10,  // max_U g (atomicMax on the bit pattern; g >= 0)
};

// Per-element contribution to the diagnostics.  `s` is the raw score, `zt` the shifted score
// (see RowGate), `g` the gate value (after any unit mask), `dt` its denominator term.
template <int KIND>
__device__ __forceinline__ void diag_accumulate(const GateConsts& gc, float s, float zt, float g,
                                                float dt, float (&d)[kDiagCols], float& int_max,
                                                float& int_cap) {
  d[kDgGateSum] += g;
  d[kDgGLogG] = fmaf(g, __logf(g + 1e-8f), d[kDgGLogG]);
  const float s2 = s * s;
  d[kDgS3] = fmaf(s2, s, d[kDgS3]);
  d[kDgS4] = fmaf(s2, s2, d[kDgS4]);
  d[kDgGateMax] = fmaxf(d[kDgGateMax], g);
  if constexpr (KIND == 0) {
    d[kDgActive] += zt > 0.f ? 1.f : 0.f;
  } else if constexpr (KIND == 1) {
    d[kDgActive] += g > 0.f ? 1.f : 0.f;
    d[kDgStrong] += g > 0.5f ? 1.f : 0.f;
    d[kDgBand] += fabsf(zt) > 1.6448536f ? 1.f : 0.f;      // Phi(z) > 0.95 or < 0.05
    d[kDgZSum] += fmaxf(zt, 0.f);
    d[kDgB075] += (zt > 0.f && zt < 0.75f) ? 1.f : 0.f;
    d[kDgB030] += (zt > 0.f && zt < 0.30f) ? 1.f : 0.f;
  } else {
    // act = sigmoid(sharp * zt): act > a  <=>  sharp * zt > log(a / (1 - a))
    const float a = gc.sharp * zt;
    d[kDgActive] += a > 0.f ? 1.f : 0.f;
    d[kDgStrong] += a > 2.1972246f ? 1.f : 0.f;                 // 0.9
    d[kDgBand] += fabsf(a) < 2.1972246f ? 1.f : 0.f;            // (0.1, 0.9)
    d[kDgZSum] += dt;                                           // intensity
    d[kDgB075] += fabsf(a) < 2.9444390f ? 1.f : 0.f;            // (0.05, 0.95)
    d[kDgB030] += fabsf(a) < 1.3862944f ? 1.f : 0.f;            // (0.2, 0.8)
    int_max = fmaxf(int_max, dt);
    int_cap += dt >= gc.eps + gc.max_int - 1e-3f ? 1.f : 0.f;
  }
}
template <int KIND>
struct FwdGateEpi {
  static constexpr int kNumAcc = 2;
  static constexpr int kNumOut = 1;
  static constexpr int kOutBufs = 1;
  static constexpr int kEpiWarps = 8;
  __host__ __device__ static constexpr int acc_bufs(int) { return 2; }   // S and XR, two tiles in flight
  using Params = FwdGateParams;

  // kGeneral: column tail, unit mask or alive flags are in play for this slab.
  template <int BN, bool kGeneral>
  __device__ static __forceinline__ void slab(const Params& p, uint32_t buf, const WarpStager& st,
                                              uint32_t acc_s, uint32_t acc_xr, int col0, int N,
                                              bool row_ok, float tau, float isg, float& den_acc,
                                              float& g_acc, int lane) {
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      float s[32], xr[32];
      tmem_ld32(acc_s + 32 * half, s);
      tmem_ld32(acc_xr + 32 * half, xr);
      tmem_ld_wait();
      const int cbase = col0 + 32 * half;
      unsigned alive_bits = 0u;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float g, dt;
        gate_fwd<KIND>(p.gc, s[j], tau, isg, g, dt);
        if (kGeneral) {
          if (cbase + j >= N) { g = 0.f; dt = 0.f; }
          if (p.unit_mask != nullptr && cbase + j < N) {
            const float um = p.unit_mask[cbase + j];
            g *= um;
            dt *= um;
          }
          if (row_ok && g >= p.gc.dead_thr) alive_bits |= 1u << j;
        }
        den_acc += dt;
        g_acc += g;
        s[j] = g * xr[j];
      }
      if (kGeneral && p.alive != nullptr) {
        const unsigned any = __reduce_or_sync(0xffffffffu, alive_bits);  // OR over the 32 rows
        if (((any >> lane) & 1u) && cbase + lane < N) p.alive[cbase + lane] = 1;
      }
      stage_bf16_32(st, buf, 4 * half, s);
    }
  }

  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    static_assert(BN == 128, "one 64-column slab per warp");
    const int r0 = m0 + (warp & 3) * 32;
    const int c = (warp >> 2) * 64;
    const int col0 = n0 + c;
    if (r0 >= M || col0 >= N) { ctl.skip(); return; }  // warp-uniform
    const int row = r0 + lane;
    const bool row_ok = row < M;
    // rows past M hold zero accumulators; their results are clipped by the
    // store and never reach den_sum, so they need no masking
    const float tau = row_ok ? p.tau[row] : 0.f;
    const float isg = row_ok ? p.inv_sigma[row] : 1.f;
    float den_acc = 0.f, g_acc = 0.f;
    st.wait_free<0>();
    const uint32_t buf = st.buf(0);
    const uint32_t acc_s = ctl.wait(0) + c, acc_xr = ctl.wait(1) + c;
    const bool general = (col0 + 64 > N) || p.unit_mask != nullptr || p.alive != nullptr;
    if (general) slab<BN, true>(p, buf, st, acc_s, acc_xr, col0, N, row_ok, tau, isg, den_acc, g_acc, lane);
    else slab<BN, false>(p, buf, st, acc_s, acc_xr, col0, N, row_ok, tau, isg, den_acc, g_acc, lane);
    ctl.release(0);
    ctl.release(1);
    st.flush(&maps[0], buf, col0, r0, false, true);
    if (row_ok) {
      atomicAdd(p.den_sum + row, den_acc);
      if (p.gate_sum != nullptr) atomicAdd(p.gate_sum + row, g_acc);
    }
  }
};

template <int KIND>
__device__ __forceinline__ float gate_shifted(const GateConsts& gc, float s, float tau, float isg) {
  if constexpr (KIND == 0) return s - tau;
  else if constexpr (KIND == 1) return (s - tau) * isg;
  else return s - tau - gc.thr;
}
// (g, A1, A2) from the shifted score; ds = A1 * (dp * xr) + A2 * dden.
template <int KIND>
__device__ __forceinline__ float gate_coeffs_shifted(const GateConsts& gc, float zt, float isg,
                                                     float& a1, float& a2) {
  float g;
  if constexpr (KIND == 0) {
    g = fminf(fmaxf(zt, 0.f), gc.clip_max);
    a1 = (zt > 0.f && zt < gc.clip_max) ? 1.f : 0.f;
    a2 = a1;
  } else if constexpr (KIND == 1) {
    const float z = fmaxf(zt, 0.f);
    float phi, pdf;
    phi_pdf(z, phi, pdf);
    g = z * phi;
    a1 = zt > 0.f ? fmaf(z, pdf, phi) * isg : 0.f;
    a2 = a1;
  } else {
    const float act = rcp_approx(1.f + __expf(-gc.sharp * zt));
    const float amr = zt - gc.cut;
    const float inten = gc.eps + fminf(fmaxf(amr, 0.f), gc.max_int);
    g = act * inten;
    a2 = (amr > 0.f && amr < gc.max_int) ? 1.f : 0.f;
    a1 = inten * gc.sharp * act * (1.f - act) + act * a2;
  }
  return g;
}
// 16-byte asynchronous copy global -> shared; src_bytes == 0 writes zeros.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.wait_all;" ::: "memory");
}
__device__ __forceinline__ uint4 ld_shared_v4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_half2(uint32_t w) {
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// Wide variant: 256-column tiles on CTA pairs.  S and XR take 256 TMEM columns
// each (all 512), one buffer per accumulator, so nothing may sit between an
// accumulator becoming complete and its release: the epilogue drains each
// accumulator into registers in compact form and releases it at once.
//   phase 1 (while the five-times-longer XR MMAs of the tile still run): S ->
//            gate values, kept as bf16 pairs (64 registers for the thread's 128
//            columns); S released.
//   drain:   XR -> bf16 pairs (64 registers); XR released.  From here on the
//            tensor core is free to run the next tile.
//   phase 2: p = g * xr from registers, staged and stored (and xr itself when
//            it is kept), overlapping the next tile's MMAs.
// The gate arithmetic is one exponential and ~10 FP32 instructions per element
// for the z * Phi(z) gate; TMEM loads are software-pipelined (the load of chunk
// q+1 is in flight while chunk q is processed).  256-wide tiles halve the
// shared-memory bytes per FLOP of the 128-wide variant, whose tensor-pipe
// utilisation is capped by shared-memory bandwidth.
// Warp w: rows 32(w%4).., columns 128(w/4).. of the CTA's 128 x 256 tile.
// kSaveXr: the read scalars xr = x . read^T are written out as bf16 next to p,
// so that the backward pass need not recompute them (BwdGateEpiXr).
template <int KIND, bool kSaveXr>
struct FwdGateEpiWide {
  static constexpr int kNumAcc = 2;
  static constexpr int kNumOut = kSaveXr ? 2 : 1;
  static constexpr int kOutBufs = 2;
  static constexpr int kEpiWarps = 8;
  __host__ __device__ static constexpr int acc_bufs(int) { return 1; }
  using Params = FwdGateParams;

  // kGeneral: column tail, unit mask or alive flags in play; kDiag: routing diagnostics wanted
  // (then kGeneral too, so that padded columns are left out of the counts).
  template <bool kGeneral, bool kDiag = false>
  __device__ static __forceinline__ void phase1(const Params& p, uint32_t acc_s, int col0, int N,
                                                bool row_ok, RowGate rg, uint32_t (&gp)[64],
                                                float& den_acc, float& g_acc, int lane, int row) {
    float sb[2][32];
    float dg[kDiagCols];
    float int_max = 0.f, int_cap = 0.f;
    if constexpr (kDiag) {
#pragma unroll
      for (int k = 0; k < kDiagCols; ++k) dg[k] = 0.f;
    }
    tmem_ld32(acc_s, sb[0]);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float* s = sb[q & 1];
      tmem_ld_wait_dep32(s);
      if (q < 3) tmem_ld32(acc_s + 32 * (q + 1), sb[(q + 1) & 1]);
      const int cbase = col0 + 32 * q;
      unsigned alive_bits = 0u;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float g, dt;
        const float zt = fmaf(s[j], rg.a, rg.b);
        gate_fwd_shifted<KIND>(p.gc, zt, g, dt);
        if constexpr (kGeneral) {
          if (cbase + j >= N) { g = 0.f; dt = 0.f; }
          if (p.unit_mask != nullptr && cbase + j < N) {
            const float um = p.unit_mask[cbase + j];
            g *= um;
            dt *= um;
          }
          if (row_ok && g >= p.gc.dead_thr) alive_bits |= 1u << j;
        }
        if constexpr (kDiag) {
          if (cbase + j < N) diag_accumulate<KIND>(p.gc, s[j], zt, g, dt, dg, int_max, int_cap);
        }
        den_acc += dt;
        if constexpr (KIND == 2) g_acc += g;
        s[j] = g;
      }
      if constexpr (kGeneral) {
        if (p.alive != nullptr) {
          const unsigned any = __reduce_or_sync(0xffffffffu, alive_bits);
          if (((any >> lane) & 1u) && cbase + lane < N) p.alive[cbase + lane] = 1;
        }
      }
#pragma unroll
      for (int j = 0; j < 16; ++j) gp[16 * q + j] = pack_bf16x2(s[2 * j], s[2 * j + 1]);
    }
    if constexpr (kDiag) {
      if (row_ok) {
        float* dst = p.diag + static_cast<size_t>(row) * kDiagCols;
#pragma unroll
        for (int k = 0; k < kDiagCols; ++k) {
          if (k == kDgGateMax) atomicMax(reinterpret_cast<int*>(dst + k), __float_as_int(dg[k]));
          else if (k < kDgGateMax) atomicAdd(dst + k, dg[k]);
        }
        if constexpr (KIND == 2) {
          atomicMax(reinterpret_cast<int*>(p.diag_scalars), __float_as_int(int_max));
          atomicAdd(p.diag_scalars + 1, int_cap);
        }
      }
    }
  }

  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    static_assert(BN == 256, "two 64-column slabs per warp");
    const int r0 = m0 + (warp & 3) * 32;
    const int c = (warp >> 2) * 128;
    const int col0 = n0 + c;
    if (r0 >= M || col0 >= N) { ctl.skip(); return; }  // warp-uniform
    const int row = r0 + lane;
    const bool row_ok = row < M;
    float den_acc = 0.f, g_acc = 0.f;
    const bool general = (col0 + 128 > N) || p.unit_mask != nullptr || p.alive != nullptr;
    // ---- phase 1: scores -> gate values (bf16 pairs in registers)
    uint32_t gp[64];
    const uint32_t acc_s = ctl.wait(0) + c;
    // The row constants are read only now: with a fused gather they arrive together with
    // the rows, which the completed score MMAs of this tile have consumed.
    float tau = 0.f, isg = 1.f;
    if (row_ok) {
      if (p.stats != nullptr) {
        const float4 sv = __ldcg(p.stats + row);
        tau = sv.x;
        isg = sv.y;
      } else {
        tau = p.tau[row];
        isg = p.inv_sigma[row];
      }
    }
    const RowGate rg = row_gate<KIND>(p.gc, tau, isg);
    if (p.diag != nullptr) phase1<true, true>(p, acc_s, col0, N, row_ok, rg, gp, den_acc, g_acc, lane, row);
    else if (general) phase1<true>(p, acc_s, col0, N, row_ok, rg, gp, den_acc, g_acc, lane, row);
    else phase1<false>(p, acc_s, col0, N, row_ok, rg, gp, den_acc, g_acc, lane, row);
    ctl.release(0);   // the next tile's score MMAs may start
    if constexpr (KIND != 2) g_acc = den_acc;
    // ---- drain XR into bf16 pairs and release it
    uint32_t xp[64];
    {
      const uint32_t acc_xr = ctl.wait(1) + c;
      float xb[2][32];
      tmem_ld32(acc_xr, xb[0]);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float* xr = xb[i & 1];
        tmem_ld_wait_dep32(xr);
        if (i < 3) tmem_ld32(acc_xr + 32 * (i + 1), xb[(i + 1) & 1]);
#pragma unroll
        for (int j = 0; j < 16; ++j) xp[16 * i + j] = pack_bf16x2(xr[2 * j], xr[2 * j + 1]);
      }
      ctl.release(1);   // the next tile's read MMAs may start
    }
    // ---- phase 2: p = g * xr from registers; nothing here holds the tensor core up
    auto put_p = [&](int sl, uint32_t b) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {               // 16-byte chunk k of the slab: 8 columns
        uint32_t pw[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int idx = 32 * sl + 4 * k + e;
          const float2 gf =
              __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gp[idx]));
          const float2 xf =
              __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xp[idx]));
          pw[e] = pack_bf16x2(gf.x * xf.x, gf.y * xf.y);
        }
        st.put(b, k, pw[0], pw[1], pw[2], pw[3]);
      }
    };
    auto put_x = [&](int sl, uint32_t b) {
#pragma unroll
      for (int k = 0; k < 8; ++k)
        st.put(b, k, xp[32 * sl + 4 * k], xp[32 * sl + 4 * k + 1], xp[32 * sl + 4 * k + 2],
               xp[32 * sl + 4 * k + 3]);
    };
    const bool in0 = col0 < N, in1 = col0 + 64 < N;   // warp-uniform
    if constexpr (!kSaveXr) {
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        st.wait_free<1>();
        put_p(sl, st.buf(sl));
        st.flush(&maps[0], st.buf(sl), col0 + 64 * sl, r0, false, sl == 0 ? in0 : in1);
      }
    } else {
      // Two fences per tile: both read-scalar slabs behind one, both p slabs
      // behind the other.
      st.wait_free<0>();
      put_x(0, st.buf(0));
      put_x(1, st.buf(1));
      st.publish();
      st.store(&maps[1], st.buf(0), col0, r0, false, in0);
      st.store(&maps[1], st.buf(1), col0 + 64, r0, false, in1);
      st.wait_free<1>();
      put_p(0, st.buf(0));
      st.wait_free<0>();
      put_p(1, st.buf(1));
      st.publish();
      st.store(&maps[0], st.buf(0), col0, r0, false, in0);
      st.store(&maps[0], st.buf(1), col0 + 64, r0, false, in1);
    }
    if (row_ok) {
      atomicAdd(p.den_sum + row, den_acc);
      if (p.gate_sum != nullptr) atomicAdd(p.gate_sum + row, g_acc);
    }
  }
};

// ----------------------------------------------------- backward gate epilogue
struct BwdGateParams {
  const float* tau;        // [T]
  const float* inv_sigma;  // [T]
  const float* dden;       // [T] grad on sum_U den_term
  float* dtau_sum;         // [T] += -sum_U ds
  float* dsz_sum;          // [T] += sum_U ds * z     (v4.0.1)
  GateConsts gc;
};
// Backward gate coefficients from one score: returns g and writes A1, A2 with
//   ds = A1 * (dp * xr) + A2 * dden        (dg = dp * xr)
template <int KIND>
__device__ __forceinline__ float gate_bwd_coeffs(const GateConsts& gc, float s, float tau,
                                                 float isg, float& a1, float& a2) {
  float g;
  if constexpr (KIND == 0) {
    const float raw = s - tau;
    g = fminf(fmaxf(raw, 0.f), gc.clip_max);
    a1 = (raw > 0.f && raw < gc.clip_max) ? 1.f : 0.f;
    a2 = a1;
  } else if constexpr (KIND == 1) {
    const float zr = (s - tau) * isg;
    const float z = fmaxf(zr, 0.f);
    float phi, pdf;
    phi_pdf(z, phi, pdf);
    g = z * phi;
    a1 = zr > 0.f ? fmaf(z, pdf, phi) * isg : 0.f;
    a2 = a1;
  } else {
    const float m = s - tau - gc.thr;
    const float act = rcp_approx(1.f + __expf(-gc.sharp * m));
    const float amr = m - gc.cut;
    const float inten = gc.eps + fminf(fmaxf(amr, 0.f), gc.max_int);
    g = act * inten;
    a2 = (amr > 0.f && amr < gc.max_int) ? 1.f : 0.f;
    a1 = inten * gc.sharp * act * (1.f - act) + act * a2;
  }
  return g;
}

// Three accumulators per tile: S (one buffer), XR (two), DP (one) = 512 TMEM
// columns.  Phase 1 turns S into per-element (g, A1[, A2]) held in registers as
// bf16 and frees S; phase 2 combines them with XR and DP.  Because XR has two
// buffers and S is freed early, the tensor core computes the next tile's S and
// XR while this tile's phase 2 runs; only DP of the next tile waits for it.
template <int KIND>
struct BwdGateEpi {
  static constexpr int kNumAcc = 3;
  static constexpr int kNumOut = 3;   // p, dxr, ds
  static constexpr int kOutBufs = 3;  // one staged slab per output per warp per tile
  static constexpr int kEpiWarps = 8;
  __host__ __device__ static constexpr int acc_bufs(int a) { return a == 1 ? 2 : 1; }
  using Params = BwdGateParams;
  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    static_assert(BN == 128, "one 64-column slab per warp");
    const int r0 = m0 + (warp & 3) * 32;
    const int c = (warp >> 2) * 64;
    const int col0 = n0 + c;
    if (r0 >= M || col0 >= N) { ctl.skip(); return; }
    const int row = r0 + lane;
    const bool row_ok = row < M;
    const float tau = row_ok ? p.tau[row] : 0.f;
    const float isg = row_ok ? p.inv_sigma[row] : 1.f;
    const float dden = row_ok ? p.dden[row] : 0.f;
    const bool tail = col0 + 64 > N;

    // ---- phase 1: S -> (g, A1), two bf16 per register.  For the two-stage gate
    // A2 (0 or 1) rides in the sign of g, which is never negative itself.
    uint32_t st_g[32], st_a[32];
    {
      const uint32_t acc_s = ctl.wait(0) + c;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float s[16];
        tmem_ld16(acc_s + 16 * q, s);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          float a1x, a2x, a1y, a2y;
          float gx = gate_bwd_coeffs<KIND>(p.gc, s[j], tau, isg, a1x, a2x);
          float gy = gate_bwd_coeffs<KIND>(p.gc, s[j + 1], tau, isg, a1y, a2y);
          if (tail) {
            const int col = col0 + 16 * q + j;
            if (col >= N) { gx = 0.f; a1x = 0.f; a2x = 0.f; }
            if (col + 1 >= N) { gy = 0.f; a1y = 0.f; a2y = 0.f; }
          }
          if constexpr (KIND == 2) {
            if (a2x != 0.f) gx = -gx;
            if (a2y != 0.f) gy = -gy;
          }
          st_g[8 * q + j / 2] = pack_bf16x2(gx, gy);
          st_a[8 * q + j / 2] = pack_bf16x2(a1x, a1y);
        }
      }
      ctl.release(0);
    }

    // ---- phase 2: XR and DP
    float dtau_acc = 0.f;
    st.wait_free<0>();
    const uint32_t b_p = st.buf(0), b_dxr = st.buf(1), b_ds = st.buf(2);
    const uint32_t acc_xr = ctl.wait(1) + c, acc_dp = ctl.wait(2) + c;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float xr[16], dp[16], ds[16];
      tmem_ld16(acc_xr + 16 * q, xr);
      tmem_ld16(acc_dp + 16 * q, dp);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const uint32_t wg = st_g[8 * q + j / 2], wa = st_a[8 * q + j / 2];
        // bf16 -> fp32: the value sits in the upper half of the fp32 word
        float g = __uint_as_float((j & 1) ? (wg & 0xffff0000u) : (wg << 16));
        const float a1 = __uint_as_float((j & 1) ? (wa & 0xffff0000u) : (wa << 16));
        float a2 = a1;
        if constexpr (KIND == 2) {
          a2 = g < 0.f ? 1.f : 0.f;
          g = fabsf(g);
        }
        const float d = fmaf(a1, dp[j] * xr[j], a2 * dden);
        dtau_acc -= d;
        ds[j] = d;
        const float pv = g * xr[j];
        dp[j] = dp[j] * g;  // dxr
        xr[j] = pv;         // p
      }
      stage_bf16_16(st, b_p, 2 * q, xr);
      stage_bf16_16(st, b_dxr, 2 * q, dp);
      stage_bf16_16(st, b_ds, 2 * q, ds);
    }
    ctl.release(1);
    ctl.release(2);
    st.flush(&maps[0], b_p, col0, r0, false, true);
    st.flush(&maps[1], b_dxr, col0, r0, false, true);
    st.flush(&maps[2], b_ds, col0, r0, false, true);
    if (row_ok) atomicAdd(p.dtau_sum + row, dtau_acc);
  }
};

// ------------------------------------------- wide backward gate kernel pair
// With three accumulators (S, XR, DP) the backward gate kernel cannot use
// 256-column tiles (768 TMEM columns).  The wide variant is two launches of two
// accumulators each, both with the two-phase epilogue of FwdGateEpiWide:
//   A: S, XR -> p = g * xr and c1 = A1 * xr                     (bf16 [T, U] each)
//   B: S, DP -> dxr = dp * g,  ds = dp * c1 + A2 * dden,  dtau  (reads c1 back)
// S (K = d_route) is computed twice, +9 % MMA work, in exchange for tiles that
// run ~1.5x faster.  Between the phases a thread keeps the shifted score of
// its 128 columns as fp16 pairs (64 registers) and re-evaluates the gate
// coefficients from it in phase 2.  c1 lives in the ds output buffer: B reads
// a slab's c1 values before it stores ds over them.
struct BwdWideParams {
  const float* tau;        // [T]
  const float* inv_sigma;  // [T]
  const float* dden;       // [T]   (kernel B)
  float* dtau_sum;         // [T] += -sum_U ds   (kernel B)
  const __nv_bfloat16* c1; // [T, ldc1] written by kernel A, read by kernel B
  long long ldc1;
  GateConsts gc;
};

// kStage: 0 = kernel A (accumulators S, XR), 1 = kernel B (accumulators S, DP).
template <int KIND, int kStage>
struct BwdGateEpiWide {
  static constexpr int kNumAcc = 2;
  static constexpr int kNumOut = 2;
  static constexpr int kOutBufs = kStage == 1 ? 3 : 2;   // B: dxr, and one c1/ds buffer per slab
  static constexpr int kEpiWarps = 8;
  __host__ __device__ static constexpr int acc_bufs(int) { return 1; }
  using Params = BwdWideParams;

  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    static_assert(BN == 256, "two 64-column slabs per warp");
    const int r0 = m0 + (warp & 3) * 32;
    const int c = (warp >> 2) * 128;
    const int col0 = n0 + c;
    if (r0 >= M || col0 >= N) { ctl.skip(); return; }  // warp-uniform
    const int row = r0 + lane;
    const bool row_ok = row < M;
    const float tau = row_ok ? p.tau[row] : 0.f;
    const float isg = row_ok ? p.inv_sigma[row] : 1.f;
    // ---- phase 1: shifted scores, fp16 pairs in registers
    uint32_t zp[64];
    const uint32_t acc_s = ctl.wait(0) + c;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float s[32];
      tmem_ld32(acc_s + 32 * q, s);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 16; ++j)
        zp[16 * q + j] = pack_half2(gate_shifted<KIND>(p.gc, s[2 * j], tau, isg),
                                    gate_shifted<KIND>(p.gc, s[2 * j + 1], tau, isg));
    }
    ctl.release(0);   // the next tile's score MMAs may start
    // ---- phase 2
    const float dden = (kStage == 1 && row_ok) ? p.dden[row] : 0.f;
    float dtau_acc = 0.f;
    if (kStage == 1) {
      // Fetch this warp's two 32 x 64 c1 slabs while the DP MMAs still run: asynchronous
      // 16-byte copies straight into shared memory (8 lanes per row, coalesced), in the
      // swizzled layout of the staging buffers.  Slab sl lands in buffer 1 + sl, the buffer
      // that later stages ds of the same slab, so a thread reads its c1 chunk before it
      // overwrites it.
      st.wait_free<0>();                          // the previous tile's stores have read them
      const int ch = lane & 7;
#pragma unroll
      for (int sl = 0; sl < 2; ++sl) {
        const int colS = col0 + 64 * sl + ch * 8;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
          const int rr = it * 4 + (lane >> 3);
          const bool ok = r0 + rr < M && colS < p.ldc1;
          const __nv_bfloat16* src = ok ? p.c1 + static_cast<size_t>(r0 + rr) * p.ldc1 + colS : p.c1;
          cp_async_16(st.buf(1 + sl) + rr * 128 + ((ch ^ (rr & 7)) << 4), src, ok ? 16 : 0);
        }
      }
    }
    const uint32_t acc_v = ctl.wait(1) + c;       // XR (A) or DP (B)
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      if (col0 + 64 * sl < N) {                   // warp-uniform
        if (kStage == 0 || sl == 1) st.wait_free<0>();
        const uint32_t b0 = st.buf(0), b1 = st.buf(kStage == 1 ? 1 + sl : 1);
        if (kStage == 1 && sl == 0) {
          cp_async_wait_all();          // both c1 slabs of this tile are in shared memory
          __syncwarp();
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          float v[32], w[32];
          tmem_ld32(acc_v + 64 * sl + 32 * half, v);
          const int cb = col0 + 64 * sl + 32 * half;
          if (kStage == 1) {
            // this row's c1 values of the 32 columns, from the slab the warp just staged
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint4 u = ld_shared_v4(b1 + lane * 128 + (((4 * half + k) ^ (lane & 7)) << 4));
              const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(h2[e]);
                w[8 * k + 2 * e] = f.x;
                w[8 * k + 2 * e + 1] = f.y;
              }
            }
          }
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float2 zt = unpack_half2(zp[32 * sl + 16 * half + j]);
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int jj = 2 * j + e;
              float a1, a2;
              const float g = gate_coeffs_shifted<KIND>(p.gc, e == 0 ? zt.x : zt.y, isg, a1, a2);
              if (kStage == 0) {
                w[jj] = a1 * v[jj];     // c1
                v[jj] = g * v[jj];      // p
              } else {
                float d = fmaf(v[jj], w[jj], a2 * dden);
                if (cb + jj >= N) d = 0.f;
                dtau_acc -= d;
                w[jj] = d;              // ds
                v[jj] = v[jj] * g;      // dxr
              }
            }
          }
          stage_bf16_32(st, b0, 4 * half, v);
          stage_bf16_32(st, b1, 4 * half, w);
        }
        if (sl == 1 || col0 + 64 >= N) ctl.release(1);   // last TMEM read of this tile
        st.flush(&maps[0], b0, col0 + 64 * sl, r0, false, true);
        st.flush(&maps[1], b1, col0 + 64 * sl, r0, false, true);
      }
    }
    if (kStage == 1 && row_ok) atomicAdd(p.dtau_sum + row, dtau_acc);
  }
};

// ------------------------------------- backward gate kernel on saved read scalars
// When the forward pass kept xr = x . read^T (bf16 [T, U], FwdGateEpiWide with
// kSaveXr), the backward gate step is ONE 256-wide launch with two accumulators:
//   S = h . emb^T (K = d_route)  and  DP = dy . write^T (K = d_model),
// i.e. neither the XR product nor a second pass over S is recomputed.  Both
// accumulators are single-buffered, so the epilogue drains each into registers
// the moment it completes and releases it:
//   S  -> shifted scores as fp16 pairs (64 registers), while the DP MMAs run;
//   DP -> bf16 pairs (64 registers).
// Everything after that works from registers and overlaps the next tile's MMAs:
// gate coefficients (g, A1, A2) from the shifted score, then
//   p = g * xr,   dxr = DP * g,   ds = A1 * (DP * xr) + A2 * dden,   dtau -= ds.
// The xr rows of a slab are fetched into a staging buffer with 16-byte asynchronous
// copies (8 lanes per row, i.e. full lines; a thread reading its own row straight
// from global memory measured 1.7x slower for the whole kernel) and p is staged over
// them chunk by chunk (a thread reads its chunk first), so p may also be written
// over xr in place in global memory.  The first slab's fetch is issued before the
// drains and is long complete when it is needed; the second slab's fetch waits for
// the first slab's p store to leave the buffer and is the one exposed latency.
struct BwdXrParams {
  const float4* stats;     // optional [T]: (tau, 1/sigma, dden, -) per token, see FwdGateParams
  const float* tau;        // [T]
  const float* inv_sigma;  // [T]
  const float* dden;       // [T]
  float* dtau_sum;         // [T] += -sum_U ds
  const __nv_bfloat16* xr; // [T, ldxr] read scalars saved by the forward pass
  long long ldxr;
  GateConsts gc;
};

template <int KIND>
struct BwdGateEpiXr {
  static constexpr int kNumAcc = 2;
  static constexpr int kNumOut = 3;    // p, dxr, ds
  static constexpr int kOutBufs = 3;   // 0: xr in, p out (in place); 1: dxr; 2: ds
  static constexpr int kEpiWarps = 8;
  __host__ __device__ static constexpr int acc_bufs(int) { return 1; }
  using Params = BwdXrParams;

  // Asynchronous fetch of one 32-row x 64-column xr slab into a staging buffer, in the
  // swizzled layout of the TMA boxes: 8 lanes cover the 128 bytes of a row, so every
  // request is a full line (a thread reading its own row would touch 32 lines per load).
  __device__ static __forceinline__ void fetch_xr(const Params& p, uint32_t buf, int r0, int colS0,
                                                  int M, int lane) {
    const int ch = lane & 7;
    const int colS = colS0 + ch * 8;
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rr = it * 4 + (lane >> 3);
      const bool ok = r0 + rr < M && colS < p.ldxr;
      const __nv_bfloat16* src = ok ? p.xr + static_cast<size_t>(r0 + rr) * p.ldxr + colS : p.xr;
      cp_async_16(buf + rr * 128 + ((ch ^ (rr & 7)) << 4), src, ok ? 16 : 0);
    }
  }

  template <int BN, class Ctl>
  __device__ static void run(const Params& p, const CUtensorMap* maps, WarpStager& st, Ctl& ctl,
                             int m0, int n0, int M, int N, int warp, int lane) {
    static_assert(BN == 256, "two 64-column slabs per warp");
    const int r0 = m0 + (warp & 3) * 32;
    const int c = (warp >> 2) * 128;
    const int col0 = n0 + c;
    if (r0 >= M || col0 >= N) { ctl.skip(); return; }  // warp-uniform
    const int row = r0 + lane;
    const bool row_ok = row < M;
    const bool tail = col0 + 128 > N;
    const uint32_t b_x = st.buf(0), b_dxr = st.buf(1), b_ds = st.buf(2);

    // xr of slab 0 starts moving now; it is needed only after both drains
    st.wait_free<0>();                            // the previous tile's stores have read the buffers
    fetch_xr(p, b_x, r0, col0, M, lane);

    // ---- drain S: shifted scores as fp16 pairs
    uint32_t zp[64];
    float isg = 1.f, dden = 0.f;
    {
      const uint32_t acc_s = ctl.wait(0) + c;
      // row constants, read once the tile's rows (and the statistics that travel with them
      // under a fused gather) are known to be in place
      float tau = 0.f;
      if (row_ok) {
        if (p.stats != nullptr) {
          const float4 sv = __ldcg(p.stats + row);
          tau = sv.x;
          isg = sv.y;
          dden = sv.z;
        } else {
          tau = p.tau[row];
          isg = p.inv_sigma[row];
          dden = p.dden[row];
        }
      }
      const RowGate rg = row_gate<KIND>(p.gc, tau, isg);
      float sb[2][16];
      tmem_ld16(acc_s, sb[0]);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float* s = sb[q & 1];
        tmem_ld_wait_dep16(s);
        if (q < 7) tmem_ld16(acc_s + 16 * (q + 1), sb[(q + 1) & 1]);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          zp[8 * q + j] = pack_half2(fmaf(s[2 * j], rg.a, rg.b), fmaf(s[2 * j + 1], rg.a, rg.b));
      }
      ctl.release(0);   // the next tile's score MMAs may start
    }
    // ---- drain DP: bf16 pairs
    uint32_t dpp[64];
    {
      const uint32_t acc_dp = ctl.wait(1) + c;
      float db[2][16];
      tmem_ld16(acc_dp, db[0]);
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        float* d = db[q & 1];
        tmem_ld_wait_dep16(d);
        if (q < 7) tmem_ld16(acc_dp + 16 * (q + 1), db[(q + 1) & 1]);
#pragma unroll
        for (int j = 0; j < 8; ++j) dpp[8 * q + j] = pack_bf16x2(d[2 * j], d[2 * j + 1]);
      }
      ctl.release(1);   // the next tile's MMAs may start
    }

    // ---- outputs, from registers and the staged xr slab; nothing here holds the tensor core up
    float dtau_acc = 0.f;
#pragma unroll
    for (int sl = 0; sl < 2; ++sl) {
      cp_async_wait_all();                        // this slab's xr is in shared memory
      __syncwarp();
      if (sl == 1) st.wait_free<0>();             // slab 0's dxr / ds stores have read their buffers
#pragma unroll
      for (int qq = 0; qq < 4; ++qq) {
        const int q = 4 * sl + qq, k0 = 2 * qq;
        const uint4 u0 = ld_shared_v4(b_x + lane * 128 + ((k0 ^ (lane & 7)) << 4));
        const uint4 u1 = ld_shared_v4(b_x + lane * 128 + (((k0 + 1) ^ (lane & 7)) << 4));
        const uint32_t xw[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
        uint32_t pw[8], dxw[8], dsw[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 zt = unpack_half2(zp[8 * q + j]);
          const float2 dp =
              __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dpp[8 * q + j]));
          const float2 xr = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xw[j]));
          float a1x, a2x, a1y, a2y;
          const float gx = gate_coeffs_shifted<KIND>(p.gc, zt.x, isg, a1x, a2x);
          const float gy = gate_coeffs_shifted<KIND>(p.gc, zt.y, isg, a1y, a2y);
          float dsx, dsy;
          if constexpr (KIND == 2) {
            dsx = fmaf(a1x, dp.x * xr.x, a2x * dden);
            dsy = fmaf(a1y, dp.y * xr.y, a2y * dden);
          } else {
            dsx = a1x * fmaf(dp.x, xr.x, dden);
            dsy = a1y * fmaf(dp.y, xr.y, dden);
          }
          if (tail) {
            const int col = col0 + 16 * q + 2 * j;
            if (col >= N) dsx = 0.f;
            if (col + 1 >= N) dsy = 0.f;
          }
          dtau_acc -= dsx + dsy;
          pw[j] = pack_bf16x2(gx * xr.x, gy * xr.y);
          dxw[j] = pack_bf16x2(dp.x * gx, dp.y * gy);
          dsw[j] = pack_bf16x2(dsx, dsy);
        }
        // p goes over the xr chunk this thread has just read
        st.put(b_x, k0, pw[0], pw[1], pw[2], pw[3]);
        st.put(b_x, k0 + 1, pw[4], pw[5], pw[6], pw[7]);
        st.put(b_dxr, k0, dxw[0], dxw[1], dxw[2], dxw[3]);
        st.put(b_dxr, k0 + 1, dxw[4], dxw[5], dxw[6], dxw[7]);
        st.put(b_ds, k0, dsw[0], dsw[1], dsw[2], dsw[3]);
        st.put(b_ds, k0 + 1, dsw[4], dsw[5], dsw[6], dsw[7]);
      }
      const bool in_range = col0 + 64 * sl < N;
      st.publish();                               // one proxy fence for the three slabs
      st.store(&maps[0], b_x, col0 + 64 * sl, r0, false, in_range);      // p first: its buffer
      st.store(&maps[1], b_dxr, col0 + 64 * sl, r0, false, in_range);    // is wanted back soonest
      st.store(&maps[2], b_ds, col0 + 64 * sl, r0, false, in_range);
      if (sl == 0) {
        st.wait_free<2>();                        // the p store has read the buffer ...
        fetch_xr(p, b_x, r0, col0 + 64, M, lane); // ... which takes the second slab's xr
      }
    }
    if (row_ok) atomicAdd(p.dtau_sum + row, dtau_acc);
  }
};

// ----------------------------------------------------------- host launchers
struct OperandDesc {
  const void* ptr;
  int mn_major;    // 0: stored [rows][K]; 1: stored [K][rows]
  long long ld;    // elements between stored rows
};

static bool use_cta_pairs();
static bool use_wide_gate();
static int fill_operand(CUtensorMap* map, const OperandDesc& o, long long rows, long long K,
                        int box_rows) {
  if (o.mn_major) return make_tmap_bf16(map, o.ptr, rows, K, o.ld, 64, 64);
  return make_tmap_bf16(map, o.ptr, K, rows, o.ld, 64, box_rows);
}

// kCtas == 2 launches 2-CTA clusters (one SM pair per 256-row tile).
template <int BN, class Epi, int kCtas, int kGather = 0>
static int launch_engine_impl(GemmParams<typename Epi::Params>& gp, cudaStream_t stream) {
  using Smem = EngineSmem<BN / kCtas, Epi::kOutBufs, Epi::kEpiWarps, kGather>;
  auto kern = gemm_engine_kernel<BN, Epi, kCtas, kGather>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Smem::kTotalBytes) != cudaSuccess)
      return 10;
    attr_set = true;
  }
  gp.m_tiles = (gp.M + kBlockM * kCtas - 1) / (kBlockM * kCtas);
  gp.n_tiles = (gp.N + BN - 1) / BN;
  gp.n_fastest = gp.n_tiles <= gp.m_tiles ? 1 : 0;
  gp.m_first = 0;
  if (kGather != 0 && gp.gather.n_ranks > 1 && !gp.n_fastest)
    gp.m_first = gp.gather.rows_per_rank / (kBlockM * kCtas);   // own rows first, then the peers'
  // work items of the persistent loop: output tiles times the K splits of each
  const long long total =
      static_cast<long long>(gp.m_tiles) * gp.n_tiles * (gp.k_splits > 1 ? gp.k_splits : 1);
  if (total <= 0) return 0;
  const int units = sm_count() / kCtas;
  const int grid = kCtas * static_cast<int>(total < units ? total : units);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(engine_threads<Epi, kGather>());
  cfg.dynamicSmemBytes = Smem::kTotalBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = kCtas;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, gp) == cudaSuccess ? 0 : 11;
}

// Environment switch DSB_WIDE_GATE=0 keeps the forward gate kernel on 128-wide tiles (profiling).
static bool use_wide_gate() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DSB_WIDE_GATE");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

// Environment switch DSB_CTA_PAIRS=0 falls back to single-CTA tiles (profiling).
static bool use_cta_pairs() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DSB_CTA_PAIRS");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int BN, class Epi>
static int launch_engine(GemmParams<typename Epi::Params>& gp, cudaStream_t stream) {
  if (use_cta_pairs()) return launch_engine_impl<BN, Epi, 2>(gp, stream);
  return launch_engine_impl<BN, Epi, 1>(gp, stream);
}

// Gate kernels with the all-gather of their token operands fused in (CTA pairs only).
// `regs`: copy through registers (no shared-memory bounce buffers, the operand ring keeps all
// its stages) - for launches that run long enough to hide the lower copy rate.
template <int BN, class Epi>
static int launch_engine_gather(GemmParams<typename Epi::Params>& gp, cudaStream_t stream,
                                bool regs = false) {
  if (regs) return launch_engine_impl<BN, Epi, 2, kGatherRegs>(gp, stream);
  return launch_engine_impl<BN, Epi, 2, kGatherBounce>(gp, stream);
}

// Local units from which a gate kernel's own run time hides a register-copy gather.
static bool gather_through_registers(int units, const GatherParams& g) {
  static int thr = -1;
  if (thr < 0) {
    const char* e = getenv("DSB_GATHER_REGS_MIN_UNITS");
    thr = e ? atoi(e) : 4096;
  }
  // ... or little to copy (one route's h rows): not worth a stage of the operand ring
  int cols = 0;
  for (int t = 0; t < g.n_tensors; ++t) cols += g.cols[t];
  return units >= thr || cols <= 512;
}

static int fill_gather(GatherParams* g, const DsbGather* d, int total_rows, int* m_rot) {
  memset(g, 0, sizeof(*g));
  *m_rot = 0;
  if (d == nullptr || d->n_ranks <= 1) return 0;
  if (d->n_ranks > kMaxRanks || d->n_tensors < 1 || d->n_tensors > kMaxGatherTensors ||
      d->rows_per_rank % 256 != 0 || d->n_ranks * d->rows_per_rank != total_rows ||
      d->ready == nullptr)
    return 700;
  g->n_tensors = d->n_tensors;
  g->n_ranks = d->n_ranks;
  g->my_rank = d->my_rank;
  g->rows_per_rank = d->rows_per_rank;
  g->ready = d->ready;
  g->epoch = d->epoch;
  for (int t = 0; t < d->n_tensors; ++t) {
    if (d->cols[t] % 64 != 0) return 701;
    g->cols[t] = d->cols[t];
    for (int j = 0; j < d->n_ranks; ++j) {
      int rc = make_tmap_bf16(&g->src[t][j], d->bufs[t][j], d->cols[t], total_rows, d->ld[t], 64, 64);
      if (rc) return 710 + rc;
    }
    g->dst[t] = g->src[t][d->my_rank];
    if (d->ld[t] % 8 != 0) return 702;
    g->ld16[t] = d->ld[t] / 8;
    for (int j = 0; j < d->n_ranks; ++j) {
      if (reinterpret_cast<uintptr_t>(d->bufs[t][j]) & 15) return 703;
      g->src_ptr[t][j] = static_cast<const uint4*>(d->bufs[t][j]);
    }
    g->dst_ptr[t] = const_cast<uint4*>(g->src_ptr[t][d->my_rank]);
  }
  if (d->n_stats < 0 || d->n_stats > kMaxGatherTensors) return 704;
  g->n_stats = d->n_stats;
  for (int sidx = 0; sidx < d->n_stats; ++sidx) {
    for (int j = 0; j < d->n_ranks; ++j) {
      if (reinterpret_cast<uintptr_t>(d->stats[sidx][j]) & 15) return 705;
      g->stat_src[sidx][j] = static_cast<const float4*>(d->stats[sidx][j]);
    }
    g->stat_dst[sidx] = const_cast<float4*>(g->stat_src[sidx][d->my_rank]);
  }
  *m_rot = d->my_rank * d->rows_per_rank / (2 * kBlockM);
  return 0;
}

static GateConsts gate_consts_of(const DsbGate* g) {
  return {g->kind, g->sharpness, g->act_threshold, g->act_cutoff, g->epsilon, g->max_intensity,
          g->clip_max, g->dead_threshold};
}

// Environment switch DSB_WIDE_BWD=0 keeps the backward gate kernel on 128-wide tiles.
static bool use_wide_bwd() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("DSB_WIDE_BWD");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int kStage>
static int launch_bwd_wide(GemmParams<BwdWideParams>& gp, int kind, bool fused, cudaStream_t stream) {
  if (fused) {
    if (kind == 0) return launch_engine_gather<256, BwdGateEpiWide<0, kStage>>(gp, stream);
    if (kind == 1) return launch_engine_gather<256, BwdGateEpiWide<1, kStage>>(gp, stream);
    return launch_engine_gather<256, BwdGateEpiWide<2, kStage>>(gp, stream);
  }
  if (kind == 0) return launch_engine_impl<256, BwdGateEpiWide<0, kStage>, 2>(gp, stream);
  if (kind == 1) return launch_engine_impl<256, BwdGateEpiWide<1, kStage>, 2>(gp, stream);
  return launch_engine_impl<256, BwdGateEpiWide<2, kStage>, 2>(gp, stream);
}

// The backward gate step as two 256-wide launches (see BwdGateEpiWide).  With a
// gather, launch A pulls the peers' x and h rows (tensors 0 and 1 of the
// descriptor, epoch e) and launch B the dy rows (tensor 2, epoch e + 1): the
// caller must not reuse e + 1.
static int bwd_gate_wide(const void* h, long long ldh, const void* emb, long long lde, const void* x,
                         long long ldx, const void* read, long long ldr, const void* dy,
                         long long lddy, const void* write, long long ldw, int T, int U, int r,
                         int D, void* p_out, void* dxr_out, void* ds_out, long long ld_out,
                         const float* tau, const float* inv_sigma, const float* dden,
                         float* dtau_sum, const DsbGate* gate, const DsbGather* gather, int* status,
                         cudaStream_t stream) {
  const bool fused = gather != nullptr && gather->n_ranks > 1;
  if (fused && gather->n_tensors != 3) return 703;
  const int brows = 128;
  for (int stage = 0; stage < 2; ++stage) {
    GemmParams<BwdWideParams> gp;
    memset(&gp, 0, sizeof(gp));
    int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
    rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, brows);
    if (stage == 0) {
      rc |= fill_operand(&gp.tma_a[1], {x, 0, ldx}, T, D, kBlockM);
      rc |= fill_operand(&gp.tma_b[1], {read, 0, ldr}, U, D, brows);
    } else {
      rc |= fill_operand(&gp.tma_a[1], {dy, 0, lddy}, T, D, kBlockM);
      rc |= fill_operand(&gp.tma_b[1], {write, 0, ldw}, U, D, brows);
    }
    if (rc) return 100 + rc;
    gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
    gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
    gp.n_seg = 2;
    gp.M = T;
    gp.N = U;
    gp.status = status;
    rc = make_out_tmap(&gp.tma_out[0], stage == 0 ? p_out : dxr_out, T, U, ld_out, 2);
    rc |= make_out_tmap(&gp.tma_out[1], ds_out, T, U, ld_out, 2);
    if (rc) return 300 + rc;
    gp.epi = {tau, inv_sigma, dden, dtau_sum, reinterpret_cast<const __nv_bfloat16*>(ds_out), ld_out,
              gate_consts_of(gate)};
    if (fused) {
      DsbGather sub = *gather;
      if (stage == 0) {
        sub.n_tensors = 2;                       // x, h
      } else {
        sub.n_tensors = 1;                       // dy
        sub.bufs[0] = gather->bufs[2];
        sub.ld[0] = gather->ld[2];
        sub.cols[0] = gather->cols[2];
        sub.epoch = gather->epoch + 1;
      }
      rc = fill_gather(&gp.gather, &sub, T, &gp.m_rot);
      if (rc) return rc;
    }
    rc = stage == 0 ? launch_bwd_wide<0>(gp, gate->kind, fused, stream)
                    : launch_bwd_wide<1>(gp, gate->kind, fused, stream);
    if (rc) return rc;
  }
  return 0;
}

}  // namespace dsb

using namespace dsb;

extern "C" int dsb_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                             long long ldb, int M, int N, int K, void* C, long long ldc,
                             int c_is_bf16, int accumulate, float alpha, const float* row_scale,
                             const float* bias, int block_n, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  GemmParams<PlainEpi::Params> gp;
  memset(&gp, 0, sizeof(gp));
  const int BN = (block_n & 0xffff) == 128 ? 128 : 256;
  // up to 128 rows fit one CTA's tile: no pairs, so twice as many workers share N and K
  const bool pairs = use_cta_pairs() && M > kBlockM;
  int rc = fill_operand(&gp.tma_a[0], {A, a_mn, lda}, M, K, kBlockM);
  if (rc) return 100 + rc;
  rc = fill_operand(&gp.tma_b[0], {B, b_mn, ldb}, N, K, pairs ? BN / 2 : BN);
  if (rc) return 200 + rc;
  gp.seg[0] = {(K + kBlockK - 1) / kBlockK, 0, a_mn, b_mn};
  gp.n_seg = 1;
  gp.M = M;
  gp.N = N;
  gp.status = status;
  rc = make_out_tmap(&gp.tma_out[0], C, M, N, ldc, c_is_bf16 ? 2 : 4);
  if (rc) return 300 + rc;
  gp.epi = {alpha, row_scale, bias, c_is_bf16, accumulate, 0, 0, nullptr, {}};
  if (accumulate && !c_is_bf16 && bias == nullptr) {
    // few output tiles but a long K (pool gradients of a small unit shard): cut K so
    // that every SM pair has work; the splits meet in the fp32 reduce-add epilogue
    const int tm = pairs ? 2 * kBlockM : kBlockM;
    const long long tiles = static_cast<long long>((M + tm - 1) / tm) * ((N + BN - 1) / BN);
    const int units = sm_count() / (pairs ? 2 : 1);
    const int k_tiles = gp.seg[0].k_tiles;
    if (tiles < 2 * units && k_tiles >= 64) {
      // tiles * splits should fill a whole number of waves (1..3) of SM pairs; a
      // longer wave count is taken only if it fills the machine 5 % better
      // every split reduce-adds a whole output tile: long splits unless the output is a few rows
      const int max_by_k = k_tiles / (M <= tm ? 8 : 32);
      int want = 1;
      double best = static_cast<double>(tiles) / ((tiles + units - 1) / units * units);
      for (int w = 1; w <= 3; ++w) {
        int s = static_cast<int>(static_cast<long long>(w) * units / tiles);
        if (s > max_by_k) s = max_by_k;
        if (s < 2) continue;
        const long long items = tiles * s;
        const double fill = static_cast<double>(items) / ((items + units - 1) / units * units);
        if (fill > best + 0.05) { best = fill; want = s; }
      }
      if (want > 1) gp.k_splits = want;
    }
  }
  if (!pairs)
    return BN == 128 ? launch_engine_impl<128, PlainEpi, 1>(gp, stream)
                     : launch_engine_impl<256, PlainEpi, 1>(gp, stream);
  return BN == 128 ? launch_engine_impl<128, PlainEpi, 2>(gp, stream)
                   : launch_engine_impl<256, PlainEpi, 2>(gp, stream);
}

static GateConsts make_gc(const DsbGate* g) {
  return {g->kind, g->sharpness, g->act_threshold, g->act_cutoff, g->epsilon, g->max_intensity,
          g->clip_max, g->dead_threshold};
}

extern "C" int dsb_srw_fwd_gate(const void* h, long long ldh, const void* emb, long long lde,
                                const void* x, long long ldx, const void* read, long long ldr,
                                int T, int U, int r, int D, void* p_out, long long ldp,
                                const float* tau, const float* inv_sigma, float* den_sum,
                                float* gate_sum, unsigned char* alive, const float* unit_mask,
                                const DsbGate* gate, int* status, cudaStream_t stream) {
  return dsb_srw_fwd_gate_xr(h, ldh, emb, lde, x, ldx, read, ldr, T, U, r, D, p_out, ldp, nullptr, 0,
                             tau, inv_sigma, nullptr, den_sum, gate_sum, nullptr, alive, unit_mask,
                             gate, nullptr, status, stream);
}

extern "C" int dsb_srw_fwd_gate_gather(const void* h, long long ldh, const void* emb,
                                       long long lde, const void* x, long long ldx,
                                       const void* read, long long ldr, int T, int U, int r, int D,
                                       void* p_out, long long ldp, const float* tau,
                                       const float* inv_sigma, float* den_sum, float* gate_sum,
                                       unsigned char* alive, const float* unit_mask,
                                       const DsbGate* gate, const DsbGather* gather, int* status,
                                       cudaStream_t stream) {
  return dsb_srw_fwd_gate_xr(h, ldh, emb, lde, x, ldx, read, ldr, T, U, r, D, p_out, ldp, nullptr, 0,
                             tau, inv_sigma, nullptr, den_sum, gate_sum, nullptr, alive, unit_mask,
                             gate, gather, status, stream);
}

extern "C" int dsb_srw_wide_tiles(int U) {
  return (use_cta_pairs() && use_wide_gate() && U >= 512) ? 1 : 0;
}

namespace dsb {
template <bool kSaveXr>
static int launch_fwd_wide(GemmParams<FwdGateParams>& gp, int kind, bool fused, cudaStream_t stream) {
  if (fused) {
    const bool regs = gather_through_registers(gp.N, gp.gather);
    if (kind == 0) return launch_engine_gather<256, FwdGateEpiWide<0, kSaveXr>>(gp, stream, regs);
    if (kind == 1) return launch_engine_gather<256, FwdGateEpiWide<1, kSaveXr>>(gp, stream, regs);
    return launch_engine_gather<256, FwdGateEpiWide<2, kSaveXr>>(gp, stream, regs);
  }
  if (kind == 0) return launch_engine_impl<256, FwdGateEpiWide<0, kSaveXr>, 2>(gp, stream);
  if (kind == 1) return launch_engine_impl<256, FwdGateEpiWide<1, kSaveXr>, 2>(gp, stream);
  return launch_engine_impl<256, FwdGateEpiWide<2, kSaveXr>, 2>(gp, stream);
}
}  // namespace dsb

extern "C" int dsb_srw_fwd_gate_xr(const void* h, long long ldh, const void* emb, long long lde,
                                   const void* x, long long ldx, const void* read, long long ldr,
                                   int T, int U, int r, int D, void* p_out, long long ldp,
                                   void* xr_out, long long ldxr, const float* tau,
                                   const float* inv_sigma, const void* stats, float* den_sum,
                                   float* gate_sum, float* diag, unsigned char* alive,
                                   const float* unit_mask, const DsbGate* gate,
                                   const DsbGather* gather, int* status, cudaStream_t stream) {
  if (T <= 0 || U <= 0) return 0;
  constexpr int BN = 128;
  GemmParams<FwdGateParams> gp;
  memset(&gp, 0, sizeof(gp));
  // 256-wide tiles (CTA pairs only) once the pool is wide enough to fill the machine with them
  // A caller that asks for what only the wide kernel does (read scalars out, per-token float4
  // statistics in, routing diagnostics) gets it for any unit count: in a sharded group every
  // rank must take the same path although the last rank may hold fewer than 512 units.
  const bool wide_only = xr_out != nullptr || stats != nullptr || diag != nullptr;
  const bool wide = dsb_srw_wide_tiles(U) != 0 ||
                    (wide_only && use_cta_pairs() && use_wide_gate());
  if (wide_only && !wide) return 704;
  if (stats == nullptr && (tau == nullptr || inv_sigma == nullptr)) return 707;
  // A handful of token rows (decoding): a CTA pair would spend a 256-row tile on them, so
  // single CTAs take 128 x 256 tiles and twice as many of them stream the pool.
  const bool solo = wide && T <= kBlockM && xr_out == nullptr && diag == nullptr &&
                    !(gather != nullptr && gather->n_ranks > 1);
  const int brows = solo ? 256 : wide ? 128 : (use_cta_pairs() ? BN / 2 : BN);
  int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
  rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, brows);
  rc |= fill_operand(&gp.tma_a[1], {x, 0, ldx}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[1], {read, 0, ldr}, U, D, brows);
  if (rc) return 100 + rc;
  gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
  gp.n_seg = 2;
  gp.M = T;
  gp.N = U;
  gp.status = status;
  rc = make_out_tmap(&gp.tma_out[0], p_out, T, U, ldp, 2);
  if (xr_out != nullptr) rc |= make_out_tmap(&gp.tma_out[1], xr_out, T, U, ldxr, 2);
  if (rc) return 300 + rc;
  gp.epi = {static_cast<const float4*>(stats), tau, inv_sigma, den_sum, gate_sum, alive, unit_mask,
            diag, diag != nullptr ? diag + static_cast<size_t>(T) * kDiagCols : nullptr,
            make_gc(gate)};
  const bool fused = gather != nullptr && gather->n_ranks > 1;
  if (fused) {
    if (!use_cta_pairs()) return 702;
    rc = fill_gather(&gp.gather, gather, T, &gp.m_rot);
    if (rc) return rc;
  }
  if (solo) {
    if (gate->kind == 0) return launch_engine_impl<256, FwdGateEpiWide<0, false>, 1>(gp, stream);
    if (gate->kind == 1) return launch_engine_impl<256, FwdGateEpiWide<1, false>, 1>(gp, stream);
    return launch_engine_impl<256, FwdGateEpiWide<2, false>, 1>(gp, stream);
  }
  if (wide) {
    return xr_out != nullptr ? launch_fwd_wide<true>(gp, gate->kind, fused, stream)
                             : launch_fwd_wide<false>(gp, gate->kind, fused, stream);
  }
  if (fused) {
    if (gate->kind == 0) return launch_engine_gather<BN, FwdGateEpi<0>>(gp, stream);
    if (gate->kind == 1) return launch_engine_gather<BN, FwdGateEpi<1>>(gp, stream);
    return launch_engine_gather<BN, FwdGateEpi<2>>(gp, stream);
  }
  if (gate->kind == 0) return launch_engine<BN, FwdGateEpi<0>>(gp, stream);
  if (gate->kind == 1) return launch_engine<BN, FwdGateEpi<1>>(gp, stream);
  return launch_engine<BN, FwdGateEpi<2>>(gp, stream);
}

// Backward gate step from saved read scalars (see BwdGateEpiXr): one launch,
// S = h.emb^T and DP = dy.write^T.  With a gather, the kernel pulls the peers'
// rows of every listed tensor (the caller lists h, dy and, for the GEMMs that
// follow, x) under one epoch.
extern "C" int dsb_srw_bwd_gate_xr(const void* h, long long ldh, const void* emb, long long lde,
                                   const void* dy, long long lddy, const void* write,
                                   long long ldw, const void* xr, long long ldxr, int T, int U,
                                   int r, int D, void* p_out, void* dxr_out, void* ds_out,
                                   long long ld_out, const float* tau, const float* inv_sigma,
                                   const float* dden, const void* stats, float* dtau_sum,
                                   const DsbGate* gate, const DsbGather* gather, int* status,
                                   cudaStream_t stream) {
  if (T <= 0 || U <= 0) return 0;
  if (!(use_cta_pairs() && use_wide_gate())) return 704;   // any unit count: see the forward entry
  if (stats == nullptr && (tau == nullptr || inv_sigma == nullptr || dden == nullptr)) return 707;
  if (xr == nullptr || ldxr < U || (ldxr & 7) != 0 || (reinterpret_cast<uintptr_t>(xr) & 15) != 0)
    return 705;
  GemmParams<BwdXrParams> gp;
  memset(&gp, 0, sizeof(gp));
  const int brows = 128;
  int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
  rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, brows);
  rc |= fill_operand(&gp.tma_a[1], {dy, 0, lddy}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[1], {write, 0, ldw}, U, D, brows);
  if (rc) return 100 + rc;
  gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
  gp.n_seg = 2;
  gp.M = T;
  gp.N = U;
  gp.status = status;
  rc = make_out_tmap(&gp.tma_out[0], p_out, T, U, ld_out, 2);
  rc |= make_out_tmap(&gp.tma_out[1], dxr_out, T, U, ld_out, 2);
  rc |= make_out_tmap(&gp.tma_out[2], ds_out, T, U, ld_out, 2);
  if (rc) return 300 + rc;
  gp.epi = {static_cast<const float4*>(stats), tau, inv_sigma, dden, dtau_sum,
            reinterpret_cast<const __nv_bfloat16*>(xr), ldxr, make_gc(gate)};
  const bool fused = gather != nullptr && gather->n_ranks > 1;
  if (fused) {
    rc = fill_gather(&gp.gather, gather, T, &gp.m_rot);
    if (rc) return rc;
    const bool regs = gather_through_registers(U, gp.gather);
    if (gate->kind == 0) return launch_engine_gather<256, BwdGateEpiXr<0>>(gp, stream, regs);
    if (gate->kind == 1) return launch_engine_gather<256, BwdGateEpiXr<1>>(gp, stream, regs);
    return launch_engine_gather<256, BwdGateEpiXr<2>>(gp, stream, regs);
  }
  if (gate->kind == 0) return launch_engine_impl<256, BwdGateEpiXr<0>, 2>(gp, stream);
  if (gate->kind == 1) return launch_engine_impl<256, BwdGateEpiXr<1>, 2>(gp, stream);
  return launch_engine_impl<256, BwdGateEpiXr<2>, 2>(gp, stream);
}

extern "C" int dsb_srw_bwd_gate(const void* h, long long ldh, const void* emb, long long lde,
                                const void* x, long long ldx, const void* read, long long ldr,
                                const void* dy, long long lddy, const void* write, long long ldw,
                                int T, int U, int r, int D, void* p_out, void* dxr_out,
                                void* ds_out, long long ld_out, const float* tau,
                                const float* inv_sigma, const float* dden, float* dtau_sum,
                                float* dsz_sum, const DsbGate* gate, int* status,
                                cudaStream_t stream) {
  return dsb_srw_bwd_gate_gather(h, ldh, emb, lde, x, ldx, read, ldr, dy, lddy, write, ldw, T, U, r,
                                 D, p_out, dxr_out, ds_out, ld_out, tau, inv_sigma, dden, dtau_sum,
                                 dsz_sum, gate, nullptr, status, stream);
}

extern "C" int dsb_srw_bwd_gate_gather(const void* h, long long ldh, const void* emb,
                                       long long lde, const void* x, long long ldx,
                                       const void* read, long long ldr, const void* dy,
                                       long long lddy, const void* write, long long ldw, int T,
                                       int U, int r, int D, void* p_out, void* dxr_out,
                                       void* ds_out, long long ld_out, const float* tau,
                                       const float* inv_sigma, const float* dden, float* dtau_sum,
                                       float* dsz_sum, const DsbGate* gate,
                                       const DsbGather* gather, int* status, cudaStream_t stream) {
  if (T <= 0 || U <= 0) return 0;
  if (use_cta_pairs() && use_wide_bwd() && U >= 512)
    return bwd_gate_wide(h, ldh, emb, lde, x, ldx, read, ldr, dy, lddy, write, ldw, T, U, r, D, p_out,
                         dxr_out, ds_out, ld_out, tau, inv_sigma, dden, dtau_sum, gate, gather,
                         status, stream);
  constexpr int BN = 128;
  GemmParams<BwdGateParams> gp;
  memset(&gp, 0, sizeof(gp));
  const int brows = use_cta_pairs() ? BN / 2 : BN;
  int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
  rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, brows);
  rc |= fill_operand(&gp.tma_a[1], {x, 0, ldx}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[1], {read, 0, ldr}, U, D, brows);
  rc |= fill_operand(&gp.tma_a[2], {dy, 0, lddy}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[2], {write, 0, ldw}, U, D, brows);
  if (rc) return 100 + rc;
  gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
  gp.seg[2] = {(D + kBlockK - 1) / kBlockK, 2, 0, 0};
  gp.n_seg = 3;
  gp.M = T;
  gp.N = U;
  gp.status = status;
  rc = make_out_tmap(&gp.tma_out[0], p_out, T, U, ld_out, 2);
  rc |= make_out_tmap(&gp.tma_out[1], dxr_out, T, U, ld_out, 2);
  rc |= make_out_tmap(&gp.tma_out[2], ds_out, T, U, ld_out, 2);
  if (rc) return 300 + rc;
  gp.epi = {tau, inv_sigma, dden, dtau_sum, dsz_sum, make_gc(gate)};
  if (gather != nullptr && gather->n_ranks > 1) {
    if (!use_cta_pairs()) return 702;
    rc = fill_gather(&gp.gather, gather, T, &gp.m_rot);
    if (rc) return rc;
    if (gate->kind == 0) return launch_engine_gather<BN, BwdGateEpi<0>>(gp, stream);
    if (gate->kind == 1) return launch_engine_gather<BN, BwdGateEpi<1>>(gp, stream);
    return launch_engine_gather<BN, BwdGateEpi<2>>(gp, stream);
  }
  if (gate->kind == 0) return launch_engine<BN, BwdGateEpi<0>>(gp, stream);
  if (gate->kind == 1) return launch_engine<BN, BwdGateEpi<1>>(gp, stream);
  return launch_engine<BN, BwdGateEpi<2>>(gp, stream);
}

// One route of the SRW forward op: p = gate(h.emb^T) * (x.read^T) into the
// caller's scratch buffer, then raw_out = p . write.  den_sum is cleared here
// and receives sum_U den_term.
extern "C" int dsb_srw_forward(const void* h, long long ldh, const void* emb, long long lde,
                               const void* x, long long ldx, const void* read, long long ldr,
                               const void* write, long long ldw, int T, int U, int r, int D,
                               const float* tau, const float* inv_sigma, void* p_scratch,
                               long long ldp, float* raw_out, long long ldo, float* den_sum,
                               unsigned char* alive, const float* unit_mask, const DsbGate* gate,
                               int* status, cudaStream_t stream) {
  if (T <= 0 || U <= 0) return 0;
  if (ldp < U || (ldp & 7) != 0) return 400;
  if (cudaMemsetAsync(den_sum, 0, sizeof(float) * T, stream) != cudaSuccess) return 401;
  int rc = dsb_srw_fwd_gate(h, ldh, emb, lde, x, ldx, read, ldr, T, U, r, D, p_scratch, ldp, tau,
                            inv_sigma, den_sum, nullptr, alive, unit_mask, gate, status, stream);
  if (rc) return rc;
  // raw_out[T,D] = p[T,U] . write[U,D]   (write is the MN-major B operand)
  return dsb_gemm_bf16(p_scratch, 0, ldp, write, 1, ldw, T, D, U, raw_out, ldo, 0, 0, 1.0f,
                       nullptr, nullptr, 256, status, stream);
}

// GEMM whose output rows are scattered to their owner ranks (first half of a
// fused reduce-scatter): C = alpha * row_scale * A.B^T over M = n_ranks *
// rows_per_rank rows; row block j goes to rank j.  `outs[j]` is rank j's
// receive buffer [n_ranks * rows_per_rank, ldc] (bf16 or fp32, peer memory for
// j != my_rank); this rank writes slot `my_rank` of each.  The owner reads its
// buffer only after every rank's kernel has finished (a barrier) and sums the
// n_ranks slots with dsb_sum_slabs.
extern "C" int dsb_gemm_bf16_scatter(const void* A, int a_mn, long long lda, const void* B,
                                     int b_mn, long long ldb, int M, int N, int K,
                                     void* const* outs, int n_ranks, int my_rank,
                                     int rows_per_rank, long long ldc, int out_is_bf16,
                                     float alpha, const float* row_scale, int* status,
                                     cudaStream_t stream) {
  return dsb_gemm_bf16_scatter_aux(A, a_mn, lda, B, b_mn, ldb, M, N, K, outs, n_ranks, my_rank,
                                   rows_per_rank, ldc, out_is_bf16, alpha, row_scale, nullptr,
                                   nullptr, status, stream);
}

extern "C" int dsb_gemm_bf16_scatter_aux(const void* A, int a_mn, long long lda, const void* B,
                                         int b_mn, long long ldb, int M, int N, int K,
                                         void* const* outs, int n_ranks, int my_rank,
                                         int rows_per_rank, long long ldc, int out_is_bf16,
                                         float alpha, const float* row_scale,
                                         const float* aux_src, float* const* aux_dsts,
                                         int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (n_ranks < 1 || n_ranks > kMaxOut || rows_per_rank % 32 != 0 || my_rank < 0 ||
      my_rank >= n_ranks || static_cast<long long>(n_ranks) * rows_per_rank != M)
    return 500;
  GemmParams<PlainEpi::Params> gp;
  memset(&gp, 0, sizeof(gp));
  constexpr int BN = 256;
  int rc = fill_operand(&gp.tma_a[0], {A, a_mn, lda}, M, K, kBlockM);
  if (rc) return 100 + rc;
  rc = fill_operand(&gp.tma_b[0], {B, b_mn, ldb}, N, K, use_cta_pairs() ? BN / 2 : BN);
  if (rc) return 200 + rc;
  for (int j = 0; j < n_ranks; ++j) {
    rc = make_out_tmap(&gp.tma_out[j], outs[j], static_cast<uint64_t>(n_ranks) * rows_per_rank, N,
                       ldc, out_is_bf16 ? 2 : 4);
    if (rc) return 300 + rc;
  }
  gp.seg[0] = {(K + kBlockK - 1) / kBlockK, 0, a_mn, b_mn};
  gp.n_seg = 1;
  gp.M = M;
  gp.N = N;
  gp.status = status;
  gp.epi = {alpha, row_scale, nullptr, out_is_bf16 ? 1 : 0, 0, rows_per_rank, my_rank, nullptr, {}};
  if (aux_src != nullptr && aux_dsts != nullptr) {
    gp.epi.aux_src = aux_src;
    for (int j = 0; j < n_ranks; ++j) gp.epi.aux_dst[j] = aux_dsts[j];
  }
  // Every rank starts with the rows of a different owner (rank+1, rank+2, ..., itself last), so
  // at any moment the ranks store to distinct peers instead of all converging on one GPU.
  const int tile_m = (use_cta_pairs() ? 2 : 1) * kBlockM;
  if (rows_per_rank % tile_m == 0)
    gp.m_rot = ((my_rank + 1) % n_ranks) * (rows_per_rank / tile_m);
  return launch_engine<BN, PlainEpi>(gp, stream);
}

// Tied LM head + cross-entropy statistics in one pass: logits_bf16 [M, ldl] = x . E^T as bf16
// (ldl >= V, a multiple of 8), lse / label_logit fp32 [M], argmax int64 [M].  `partial` is
// scratch of M * ceil(V / 256) float4.
extern "C" int dsb_lm_head_ce_fwd(const void* x, long long ldx, const void* emb, long long lde,
                                  int M, int V, int K, const long long* labels, void* logits_bf16,
                                  long long ldl, void* partial, float* lse, float* label_logit,
                                  long long* argmax, int* status, cudaStream_t stream) {
  if (M <= 0 || V <= 0 || K <= 0) return 0;
  constexpr int BN = 256;
  GemmParams<CeFwdEpi::Params> gp;
  memset(&gp, 0, sizeof(gp));
  int rc = fill_operand(&gp.tma_a[0], {x, 0, ldx}, M, K, kBlockM);
  if (rc) return 100 + rc;
  rc = fill_operand(&gp.tma_b[0], {emb, 0, lde}, V, K, use_cta_pairs() ? BN / 2 : BN);
  if (rc) return 200 + rc;
  gp.seg[0] = {(K + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.n_seg = 1;
  gp.M = M;
  gp.N = V;
  gp.status = status;
  rc = make_out_tmap(&gp.tma_out[0], logits_bf16, M, V, ldl, 2);
  if (rc) return 300 + rc;
  const int n_tiles = (V + BN - 1) / BN;
  gp.epi = {labels, static_cast<float4*>(partial), n_tiles};
  rc = launch_engine<BN, CeFwdEpi>(gp, stream);
  if (rc) return rc;
  ce_merge_kernel<<<(M + 7) / 8, 256, 0, stream>>>(static_cast<const float4*>(partial), n_tiles, M,
                                                   labels, lse, label_logit, argmax);
  return cudaGetLastError() == cudaSuccess ? 0 : 12;
}

extern "C" int dsb_lm_head_ce_bwd_inplace(void* logits_bf16, long long ldl, int M, int V,
                                          const long long* labels, const float* lse,
                                          const float* scale, cudaStream_t stream) {
  if (M <= 0) return 0;
  if ((ldl & 7) != 0 || (reinterpret_cast<uintptr_t>(logits_bf16) & 15) != 0) return 13;
  ce_bwd_inplace_kernel<<<M, 256, 0, stream>>>(static_cast<__nv_bfloat16*>(logits_bf16), ldl, V,
                                               labels, lse, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : 12;
}
