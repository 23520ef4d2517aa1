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
#include "common/gemm_engine.cuh"
#include "common/host_utils.cuh"
#include "dsb_api.h"

namespace dsb {

// ------------------------------------------------------------------ gates
struct GateConsts {
  int kind;  // 0 relu-clip (v3.9.4), 1 z*Phi(z) (v4.0.1), 2 two-stage (v4.1)
  float sharp, thr, cut, eps, max_int, clip_max, dead_thr;
};

__device__ __forceinline__ void gate_fwd(const GateConsts& gc, float s, float tau, float isg,
                                         float& g, float& dterm) {
  if (gc.kind == 0) {
    g = fminf(fmaxf(s - tau, 0.f), gc.clip_max);
    dterm = g;
  } else if (gc.kind == 1) {
    const float z = (s - tau) * isg;
    g = z > 0.f ? z * 0.5f * (1.f + erff(z * 0.70710678f)) : 0.f;
    dterm = g;
  } else {
    const float m = s - tau - gc.thr;
    const float act = 1.f / (1.f + __expf(-gc.sharp * m));
    const float inten = gc.eps + fminf(fmaxf(m - gc.cut, 0.f), gc.max_int);
    g = act * inten;
    dterm = inten;
  }
}

// Returns g; ds = d loss / d s through the gate given dg (grad on the gate
// value) and dden (grad on the denominator term); dsz = ds * z (v4.0.1 only).
__device__ __forceinline__ float gate_bwd(const GateConsts& gc, float s, float tau, float isg,
                                          float dg, float dden, float& ds, float& dsz) {
  float g;
  dsz = 0.f;
  if (gc.kind == 0) {
    const float raw = s - tau;
    g = fminf(fmaxf(raw, 0.f), gc.clip_max);
    ds = (raw > 0.f && raw < gc.clip_max) ? (dg + dden) : 0.f;
  } else if (gc.kind == 1) {
    const float z = (s - tau) * isg;
    if (z > 0.f) {
      const float phi = 0.5f * (1.f + erff(z * 0.70710678f));
      const float pdf = 0.39894228f * __expf(-0.5f * z * z);
      g = z * phi;
      ds = (dg + dden) * (phi + z * pdf) * isg;
      dsz = ds * z;
    } else {
      g = 0.f;
      ds = 0.f;
    }
  } else {
    const float m = s - tau - gc.thr;
    const float act = 1.f / (1.f + __expf(-gc.sharp * m));
    const float amr = m - gc.cut;
    const float inten = gc.eps + fminf(fmaxf(amr, 0.f), gc.max_int);
    g = act * inten;
    const float lin = (amr > 0.f && amr < gc.max_int) ? 1.f : 0.f;
    ds = dg * inten * gc.sharp * act * (1.f - act) + (dg * act + dden) * lin;
  }
  return g;
}

__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* dst, const float* v, int n_valid,
                                               int n) {
  // dst: start of this thread's n-element run; n_valid of them are in range.
  if (n_valid >= n && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
    for (int j = 0; j < n; j += 8)
      st_global_v4(dst + j, pack_bf16x2(v[j], v[j + 1]), pack_bf16x2(v[j + 2], v[j + 3]),
                   pack_bf16x2(v[j + 4], v[j + 5]), pack_bf16x2(v[j + 6], v[j + 7]));
  } else {
    for (int j = 0; j < n; ++j)
      if (j < n_valid) dst[j] = __float2bfloat16(v[j]);
  }
}

// --------------------------------------------------------- plain epilogue
struct PlainEpi {
  static constexpr int kNumAcc = 1;
  struct Params {
    void* out;
    long long ldc;
    float alpha;
    const float* row_scale;  // optional [M]
    const float* bias;       // optional [N]
    int out_bf16;            // 1: bf16 output, 0: fp32
    int accumulate;          // 1: out += result (fp32 output only)
  };
  template <int BN>
  __device__ static void run(const Params& p, int m0, int n0, int M, int N, uint32_t acc0,
                             int warp, int lane) {
    const int row = m0 + warp * 32 + lane;
    const bool row_ok = row < M;
    const float scale = p.alpha * ((row_ok && p.row_scale) ? p.row_scale[row] : 1.f);
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      const int col0 = n0 + c;
      if (col0 >= N) break;
      float v[32];
      tmem_ld32(acc0 + c, v);
      tmem_ld_wait();
      if (!row_ok) continue;
      const int nv = min(32, N - col0);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        v[j] *= scale;
        if (p.bias != nullptr && j < nv) v[j] += p.bias[col0 + j];
      }
      if (p.out_bf16) {
        store_bf16_row(reinterpret_cast<__nv_bfloat16*>(p.out) + row * p.ldc + col0, v, nv, 32);
      } else {
        float* o = reinterpret_cast<float*>(p.out) + row * p.ldc + col0;
        if (nv == 32 && (reinterpret_cast<uintptr_t>(o) & 15) == 0) {
          float4* o4 = reinterpret_cast<float4*>(o);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float4 t = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            if (p.accumulate) {
              const float4 old = o4[j];
              t.x += old.x; t.y += old.y; t.z += old.z; t.w += old.w;
            }
            o4[j] = t;
          }
        } else {
          for (int j = 0; j < nv; ++j) o[j] = p.accumulate ? o[j] + v[j] : v[j];
        }
      }
    }
  }
};

// ------------------------------------------------------ forward gate epilogue
struct FwdGateEpi {
  static constexpr int kNumAcc = 2;
  struct Params {
    __nv_bfloat16* p_out;  // [T, ldp]
    long long ldp;
    const float* tau;        // [T]
    const float* inv_sigma;  // [T]
    float* den_sum;          // [T] += sum_U den_term
    float* gate_sum;         // optional [T] += sum_U g
    unsigned char* alive;    // optional [U]: 1 if any token gates the unit >= dead_thr
    const float* unit_mask;  // optional [U] multiplier on the gate (ablation)
    GateConsts gc;
  };
  template <int BN>
  __device__ static void run(const Params& p, int m0, int n0, int M, int N, uint32_t acc0,
                             int warp, int lane) {
    const int row = m0 + warp * 32 + lane;
    const bool row_ok = row < M;
    const float tau = row_ok ? p.tau[row] : 0.f;
    const float isg = row_ok ? p.inv_sigma[row] : 1.f;
    float den_acc = 0.f, g_acc = 0.f;
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      const int col0 = n0 + c;
      if (col0 >= N) break;
      float s[32], xr[32];
      tmem_ld32(acc0 + c, s);
      tmem_ld32(acc0 + BN + c, xr);
      tmem_ld_wait();
      const int nv = min(32, N - col0);
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float g, dt;
        gate_fwd(p.gc, s[j], tau, isg, g, dt);
        if (j >= nv || !row_ok) { g = 0.f; dt = 0.f; }
        if (p.unit_mask != nullptr && j < nv) { const float um = p.unit_mask[col0 + j]; g *= um; dt *= um; }
        den_acc += dt;
        g_acc += g;
        if (p.alive != nullptr) {
          const unsigned b = __ballot_sync(0xffffffffu, g >= p.gc.dead_thr);
          if (lane == 0 && b != 0u && j < nv) p.alive[col0 + j] = 1;
        }
        s[j] = g * xr[j];
      }
      if (row_ok) store_bf16_row(p.p_out + row * p.ldp + col0, s, nv, 32);
    }
    if (row_ok) {
      atomicAdd(p.den_sum + row, den_acc);
      if (p.gate_sum != nullptr) atomicAdd(p.gate_sum + row, g_acc);
    }
  }
};

// ----------------------------------------------------- backward gate epilogue
struct BwdGateEpi {
  static constexpr int kNumAcc = 3;
  struct Params {
    __nv_bfloat16* p_out;    // [T, ld]  g * xr
    __nv_bfloat16* dxr_out;  // [T, ld]  dp * g
    __nv_bfloat16* ds_out;   // [T, ld]  d loss / d score through the gate
    long long ld;
    const float* tau;        // [T]
    const float* inv_sigma;  // [T]
    const float* dden;       // [T] grad on sum_U den_term
    float* dtau_sum;         // [T] += -sum_U ds
    float* dsz_sum;          // [T] += sum_U ds * z     (v4.0.1)
    GateConsts gc;
  };
  template <int BN>
  __device__ static void run(const Params& p, int m0, int n0, int M, int N, uint32_t acc0,
                             int warp, int lane) {
    const int row = m0 + warp * 32 + lane;
    const bool row_ok = row < M;
    const float tau = row_ok ? p.tau[row] : 0.f;
    const float isg = row_ok ? p.inv_sigma[row] : 1.f;
    const float dden = row_ok ? p.dden[row] : 0.f;
    float dtau_acc = 0.f, dsz_acc = 0.f;
#pragma unroll 1
    for (int c = 0; c < BN; c += 16) {
      const int col0 = n0 + c;
      if (col0 >= N) break;
      float s[16], xr[16], dp[16];
      tmem_ld16(acc0 + c, s);
      tmem_ld16(acc0 + BN + c, xr);
      tmem_ld16(acc0 + 2 * BN + c, dp);
      tmem_ld_wait();
      const int nv = min(16, N - col0);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        float ds, dsz;
        const float g = gate_bwd(p.gc, s[j], tau, isg, dp[j] * xr[j], dden, ds, dsz);
        if (j >= nv || !row_ok) { ds = 0.f; dsz = 0.f; }
        dtau_acc -= ds;
        dsz_acc += dsz;
        s[j] = ds;
        const float pv = g * xr[j];
        dp[j] = dp[j] * g;  // dxr
        xr[j] = pv;         // p
      }
      if (row_ok) {
        const long long off = row * p.ld + col0;
        store_bf16_row(p.p_out + off, xr, nv, 16);
        store_bf16_row(p.dxr_out + off, dp, nv, 16);
        store_bf16_row(p.ds_out + off, s, nv, 16);
      }
    }
    if (row_ok) {
      atomicAdd(p.dtau_sum + row, dtau_acc);
      if (p.gc.kind == 1) atomicAdd(p.dsz_sum + row, dsz_acc);
    }
  }
};

// ----------------------------------------------------------- host launchers
struct OperandDesc {
  const void* ptr;
  int mn_major;    // 0: stored [rows][K]; 1: stored [K][rows]
  long long ld;    // elements between stored rows
};

static int fill_operand(CUtensorMap* map, const OperandDesc& o, long long rows, long long K,
                        int box_rows) {
  if (o.mn_major) return make_tmap_bf16(map, o.ptr, rows, K, o.ld, 64, 64);
  return make_tmap_bf16(map, o.ptr, K, rows, o.ld, 64, box_rows);
}

template <int BN, class Epi>
static int launch_engine(GemmParams<typename Epi::Params>& gp, cudaStream_t stream) {
  using Smem = EngineSmem<BN>;
  auto kern = gemm_engine_kernel<BN, Epi>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Smem::kTotalBytes) != cudaSuccess)
      return 10;
    attr_set = true;
  }
  gp.m_tiles = (gp.M + kBlockM - 1) / kBlockM;
  gp.n_tiles = (gp.N + BN - 1) / BN;
  gp.n_fastest = gp.n_tiles <= gp.m_tiles ? 1 : 0;
  const long long total = static_cast<long long>(gp.m_tiles) * gp.n_tiles;
  if (total <= 0) return 0;
  const int grid = static_cast<int>(total < sm_count() ? total : sm_count());
  kern<<<grid, kNumThreads, Smem::kTotalBytes, stream>>>(gp);
  return cudaGetLastError() == cudaSuccess ? 0 : 11;
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
  const int BN = block_n == 128 ? 128 : 256;
  int rc = fill_operand(&gp.tma_a[0], {A, a_mn, lda}, M, K, kBlockM);
  if (rc) return 100 + rc;
  rc = fill_operand(&gp.tma_b[0], {B, b_mn, ldb}, N, K, BN);
  if (rc) return 200 + rc;
  gp.seg[0] = {(K + kBlockK - 1) / kBlockK, 0, a_mn, b_mn};
  gp.n_seg = 1;
  gp.M = M;
  gp.N = N;
  gp.status = status;
  gp.epi = {C, ldc, alpha, row_scale, bias, c_is_bf16, accumulate};
  return BN == 128 ? launch_engine<128, PlainEpi>(gp, stream)
                   : launch_engine<256, PlainEpi>(gp, stream);
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
  if (T <= 0 || U <= 0) return 0;
  constexpr int BN = 128;
  GemmParams<FwdGateEpi::Params> gp;
  memset(&gp, 0, sizeof(gp));
  int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
  rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, BN);
  rc |= fill_operand(&gp.tma_a[1], {x, 0, ldx}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[1], {read, 0, ldr}, U, D, BN);
  if (rc) return 100 + rc;
  gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
  gp.n_seg = 2;
  gp.M = T;
  gp.N = U;
  gp.status = status;
  gp.epi = {reinterpret_cast<__nv_bfloat16*>(p_out), ldp, tau, inv_sigma, den_sum, gate_sum,
            alive, unit_mask, make_gc(gate)};
  return launch_engine<BN, FwdGateEpi>(gp, stream);
}

extern "C" int dsb_srw_bwd_gate(const void* h, long long ldh, const void* emb, long long lde,
                                const void* x, long long ldx, const void* read, long long ldr,
                                const void* dy, long long lddy, const void* write, long long ldw,
                                int T, int U, int r, int D, void* p_out, void* dxr_out,
                                void* ds_out, long long ld_out, const float* tau,
                                const float* inv_sigma, const float* dden, float* dtau_sum,
                                float* dsz_sum, const DsbGate* gate, int* status,
                                cudaStream_t stream) {
  if (T <= 0 || U <= 0) return 0;
  constexpr int BN = 128;
  GemmParams<BwdGateEpi::Params> gp;
  memset(&gp, 0, sizeof(gp));
  int rc = fill_operand(&gp.tma_a[0], {h, 0, ldh}, T, r, kBlockM);
  rc |= fill_operand(&gp.tma_b[0], {emb, 0, lde}, U, r, BN);
  rc |= fill_operand(&gp.tma_a[1], {x, 0, ldx}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[1], {read, 0, ldr}, U, D, BN);
  rc |= fill_operand(&gp.tma_a[2], {dy, 0, lddy}, T, D, kBlockM);
  rc |= fill_operand(&gp.tma_b[2], {write, 0, ldw}, U, D, BN);
  if (rc) return 100 + rc;
  gp.seg[0] = {(r + kBlockK - 1) / kBlockK, 0, 0, 0};
  gp.seg[1] = {(D + kBlockK - 1) / kBlockK, 1, 0, 0};
  gp.seg[2] = {(D + kBlockK - 1) / kBlockK, 2, 0, 0};
  gp.n_seg = 3;
  gp.M = T;
  gp.N = U;
  gp.status = status;
  gp.epi = {reinterpret_cast<__nv_bfloat16*>(p_out), reinterpret_cast<__nv_bfloat16*>(dxr_out),
            reinterpret_cast<__nv_bfloat16*>(ds_out), ld_out, tau, inv_sigma, dden, dtau_sum,
            dsz_sum, make_gc(gate)};
  return launch_engine<BN, BwdGateEpi>(gp, stream);
}
