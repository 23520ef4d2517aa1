// Gate arithmetic of the SRW pool op shared by the tensor-engine epilogues and
// the row kernels of the generation path (reference gate definitions:
// models/dawn_spatial_v41_exp.py:485-586 and the v3.9.4 / v4.0.1 model files).
#pragma once

namespace dsb {

// ------------------------------------------------------------------ gates
struct GateConsts {
  int kind;  // 0 relu-clip (v3.9.4), 1 z*Phi(z) (v4.0.1), 2 two-stage (v4.1)
  float sharp, thr, cut, eps, max_int, clip_max, dead_thr;
};

__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;  // rcp(+inf) = 0, no slow path
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 1 - Phi(z) for z >= 0, Phi the standard normal CDF, as 2^P(z) with P a
// degree-5 polynomial fitted to log2(0.5 erfc(z / sqrt 2)): absolute error
// below 5e-7 for all z >= 0 (P decreases without bound, so large z give 0).
// One exponential and five FMAs; no reciprocal, no branch.
__device__ __forceinline__ float phi_tail(float z) {
  float p = fmaf(z, -0.0005216513f, 0.0073997346f);
  p = fmaf(p, z, -0.052554633f);
  p = fmaf(p, z, -0.45927137f);
  p = fmaf(p, z, -1.1510814f);
  p = fmaf(p, z, -1.0000014f);
  return ex2_approx(p);
}
// Phi(z) and the N(0,1) density for z >= 0.
__device__ __forceinline__ void phi_pdf(float z, float& phi, float& pdf) {
  phi = 1.f - phi_tail(z);
  pdf = 0.39894228f * ex2_approx(-0.72134752f * z * z);
}

template <int KIND>
__device__ __forceinline__ void gate_fwd(const GateConsts& gc, float s, float tau, float isg,
                                         float& g, float& dterm) {
  if constexpr (KIND == 0) {
    g = fminf(fmaxf(s - tau, 0.f), gc.clip_max);
    dterm = g;
  } else if constexpr (KIND == 1) {
    const float z = fmaxf((s - tau) * isg, 0.f);
    g = fmaf(-z, phi_tail(z), z);  // z * Phi(z); z == 0 gives exactly 0
    dterm = g;
  } else {
    const float m = s - tau - gc.thr;
    const float act = rcp_approx(1.f + __expf(-gc.sharp * m));
    const float inten = gc.eps + fminf(fmaxf(m - gc.cut, 0.f), gc.max_int);
    g = act * inten;
    dterm = inten;
  }
}

// ------------------------------------------------ shifted-score gate helpers
// The wide epilogues work on the shifted score zt = a * s + b with per-row
// constants (a, b), so the per-element cost of the shift is one FMA:
//   v3.9.4: zt = s - tau;  v4.0.1: zt = (s - tau) / sigma;  v4.1: zt = s - tau - threshold.
struct RowGate {
  float a, b;
};
template <int KIND>
__device__ __forceinline__ RowGate row_gate(const GateConsts& gc, float tau, float isg) {
  if constexpr (KIND == 0) return {1.f, -tau};
  else if constexpr (KIND == 1) return {isg, -tau * isg};
  else return {1.f, -tau - gc.thr};
}
// Forward gate value and denominator term from the shifted score.
template <int KIND>
__device__ __forceinline__ void gate_fwd_shifted(const GateConsts& gc, float zt, float& g,
                                                 float& dterm) {
  if constexpr (KIND == 0) {
    g = fminf(fmaxf(zt, 0.f), gc.clip_max);
    dterm = g;
  } else if constexpr (KIND == 1) {
    const float z = fmaxf(zt, 0.f);
    g = fmaf(-z, phi_tail(z), z);
    dterm = g;
  } else {
    const float act = rcp_approx(1.f + __expf(-gc.sharp * zt));
    const float inten = gc.eps + fminf(fmaxf(zt - gc.cut, 0.f), gc.max_int);
    g = act * inten;
    dterm = inten;
  }
}

}  // namespace dsb
