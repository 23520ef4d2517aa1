// Causal self-attention for sm_100a: tcgen05 MMAs with TMEM accumulators, TMA
// tile loads, softmax by one thread per query row (= one TMEM lane).
//
// Tensors are token-major: Q, K, V, O, dO are bf16 [B, S, H*dh]; head h owns
// columns [h*dh, (h+1)*dh).  dh is a multiple of 16, at most 128.  Tiles are
// 128 query rows x 128 keys; a head's columns are staged as one or two
// 64-column, 128-byte-swizzled atoms (NA), so the same shared-memory bytes
// serve as a K-major operand (contraction over dh) and as an MN-major operand
// (contraction over rows).  Rows past the end of a sequence are zero-filled by
// TMA and excluded by the causal mask.
//
// Forward, per CTA = (batch, head, 128-query tile), keys in blocks of 128:
//   sweep 1: S = Q K^T per key block -> row max m and l = sum exp(s - m);
//   sweep 2: S again, P = exp(s - m) / l (dropout applied) as bf16 into shared
//            memory, O += P V accumulated in TMEM; no rescaling of O is needed.
//   S is double-buffered in TMEM so the MMAs of block j+1 overlap the softmax
//   of block j.  Saves LSE = m*scale + log(l) per row for the backward pass.
//
// Backward, per CTA = (batch, head, 128-key block j), loop over query tiles
// i >= j:  S = Q_i K_j^T, dP = dO_i V_j^T (TMEM) -> P = exp(s*scale - LSE),
// dS = P o (dP - delta) * scale as bf16 in shared memory ->
//   dV_j += P^T dO_i,  dK_j += dS^T Q_i   (accumulated in TMEM over i)
//   dQ_i  = dS K_j  -> staged in shared memory, TMA reduce-add into fp32 dQ.
//
// The reference computes attention as a dense softmax(QK^T/sqrt(dh) + mask) V
// with dropout on the weights (models/dawn_spatial_v41_exp.py:1194-1219).
// Dropout here uses a counter-based hash of (seed, batch*head, query, key), so
// the backward pass regenerates the forward mask.
#include "common/host_utils.cuh"
#include "common/ptx.cuh"
#include "dsb_api_ops.h"

namespace dsb {
namespace attn {

constexpr int kTile = 128;
constexpr int kAtomBytes = kTile * 128;  // 128 rows x 64 bf16
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_reduce_add_3d(const CUtensorMap* map, uint32_t src_smem,
                                                  int c0, int c1, int c2) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group "
      "[%0, {%2, %3, %4}], [%1];" ::"l"(reinterpret_cast<uint64_t>(map)),
      "r"(src_smem), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Keep-mask of attention dropout: a 64-bit mix of the element's global index.
__device__ __forceinline__ bool drop_keep(uint64_t seed, uint64_t idx, uint32_t thresh) {
  uint64_t x = seed + idx * 0x9E3779B97F4A7C15ULL;
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ULL;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBULL;
  x ^= x >> 31;
  return static_cast<uint32_t>(x) >= thresh;
}

// K-major descriptor of k16-step `kk` inside a tile made of 64-column atoms.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_addr, int kk) {
  return umma_desc(tile_addr + (kk >> 2) * kAtomBytes + (kk & 3) * 32, 16, 1024);
}
// MN-major descriptor of k16-step `kk` (16 rows = 2048 bytes further down).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_addr, int kk) {
  return umma_desc(tile_addr + kk * 2048, kAtomBytes, 1024);
}
// Address of the 16-byte chunk holding columns [8*c8, 8*c8+8) of `row` in a
// [128 rows][128 columns] bf16 tile stored as two swizzled atoms.
__device__ __forceinline__ uint32_t swz_chunk(uint32_t tile_addr, int row, int c8) {
  return tile_addr + (c8 >> 3) * kAtomBytes + row * 128 + (((c8 & 7) ^ (row & 7)) << 4);
}

struct FwdParams {
  CUtensorMap q, k, v;
  __nv_bfloat16* out;
  float* lse;            // [B, H, S]
  int B, H, S, dh;
  float scale;           // 1 / sqrt(dh)
  uint32_t drop_thresh;  // keep iff hash >= thresh; 0 = no dropout
  float drop_scale;      // 1 / (1 - p)
  uint64_t seed;
  int* status;
};

template <int NA>
struct FwdSmem {
  static constexpr int kQ = 0;
  static constexpr int kK = NA * kAtomBytes;
  static constexpr int kV = kK + 2 * NA * kAtomBytes;
  static constexpr int kP = kV + 2 * NA * kAtomBytes;
  static constexpr int kBar = kP + 2 * kAtomBytes;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int NA>
__global__ void __launch_bounds__(160, 1) attn_fwd_kernel(const __grid_constant__ FwdParams p) {
  using L = FwdSmem<NA>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* q_full = bars;          // 1
  uint64_t* kv_full = bars + 1;     // [2]
  uint64_t* kv_empty = bars + 3;    // [2]
  uint64_t* s_full = bars + 5;      // [2]
  uint64_t* s_empty = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* p_empty = bars + 10;
  uint64_t* o_full = bars + 11;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;   // long tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int nkb = qt + 1, nj = 2 * nkb;
  const int dh = p.dh, ksteps = dh >> 4;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&kv_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(p_empty, 1);
    mbar_init(o_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q);
    tma_prefetch_desc(&p.k);
    tma_prefetch_desc(&p.v);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t q_addr = smem_u32(smem + L::kQ), k_addr = smem_u32(smem + L::kK),
                 v_addr = smem_u32(smem + L::kV), p_addr = smem_u32(smem + L::kP);

  if (warp == 4) {
    // ------------------------------------------- TMA producer + MMA issuer
    if (lane == 0) {
      bool ok = true;
      const int x0 = h * dh;
      const uint32_t idesc_s = umma_idesc_bf16(kTile, kTile, 0, 0);
      const uint32_t idesc_pv = umma_idesc_bf16(kTile, dh, 0, 1);
      auto load_kv = [&](int j) {
        const int st = j & 1, kb = j < nkb ? j : j - nkb;
        const bool second = j >= nkb;
        if (!mbar_wait(&kv_empty[st], ((j >> 1) & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(&kv_full[st], NA * kAtomBytes * (second ? 2 : 1));
        for (int a = 0; a < NA; ++a)
          tma_load_3d(smem + L::kK + (st * NA + a) * kAtomBytes, &p.k, &kv_full[st], x0 + 64 * a,
                      kb * kTile, b);
        if (second)
          for (int a = 0; a < NA; ++a)
            tma_load_3d(smem + L::kV + (st * NA + a) * kAtomBytes, &p.v, &kv_full[st],
                        x0 + 64 * a, kb * kTile, b);
      };
      auto issue_s = [&](int j) {
        const int st = j & 1;
        const uint32_t par = (j >> 1) & 1;
        if (!mbar_wait(&kv_full[st], par, abort_flag)) { ok = false; return; }
        if (!mbar_wait(&s_empty[st], par ^ 1, abort_flag)) { ok = false; return; }
        tc_fence_after();
        const uint32_t kst = k_addr + st * NA * kAtomBytes;
        for (int kk = 0; kk < ksteps; ++kk)
          mma_bf16_ss(tmem_base + st * kTile, desc_kmajor(q_addr, kk), desc_kmajor(kst, kk),
                      idesc_s, kk > 0);
        mma_commit(&s_full[st]);
        if (j < nkb) mma_commit(&kv_empty[st]);
      };
      mbar_expect_tx(q_full, NA * kAtomBytes);
      for (int a = 0; a < NA; ++a)
        tma_load_3d(smem + L::kQ + a * kAtomBytes, &p.q, q_full, x0 + 64 * a, qt * kTile, b);
      load_kv(0);
      if (ok && !mbar_wait(q_full, 0, abort_flag)) ok = false;
      if (ok) issue_s(0);
      for (int j = 0; j < nj && ok; ++j) {
        if (j + 1 < nj) {
          load_kv(j + 1);
          if (ok) issue_s(j + 1);
        }
        if (ok && j >= nkb) {
          const int i = j - nkb, st = j & 1;
          if (!mbar_wait(p_full, i & 1, abort_flag)) { ok = false; break; }
          tc_fence_after();
          const uint32_t vst = v_addr + st * NA * kAtomBytes;
          for (int kk = 0; kk < kTile / 16; ++kk)
            mma_bf16_ss(tmem_base + 2 * kTile, desc_kmajor(p_addr, kk), desc_mnmajor(vst, kk),
                        idesc_pv, (i > 0 || kk > 0) ? 1u : 0u);
          mma_commit(p_empty);
          mma_commit(&kv_empty[st]);
        }
      }
      if (ok) mma_commit(o_full);
    }
  } else {
    // ------------------------------------------------ softmax / epilogue
    const int row = threadIdx.x;
    const int qi = qt * kTile + row;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    const uint64_t bh = static_cast<uint64_t>(b) * p.H + h;
    const uint64_t drop_row = (bh * p.S + static_cast<uint64_t>(qi)) * p.S;
    float m = -INFINITY, l = 0.f, inv_l = 0.f, msl = 0.f;
    bool ok = true;
    for (int j = 0; j < nj && ok; ++j) {
      const int buf = j & 1, kb = j < nkb ? j : j - nkb;
      ok = __all_sync(0xffffffffu, mbar_wait(&s_full[buf], (j >> 1) & 1, abort_flag));
      if (!ok) break;
      tc_fence_after();
      const bool diag = kb == qt;
      const uint32_t s_addr = lane_addr + buf * kTile;
      if (j < nkb) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float v[32];
          tmem_ld32(s_addr + c * 32, v);
          tmem_ld_wait();
          if (diag) {
            const int k0 = kb * kTile + c * 32;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (k0 + e > qi) v[e] = -INFINITY;
          }
          float bm = v[0];
#pragma unroll
          for (int e = 1; e < 32; ++e) bm = fmaxf(bm, v[e]);
          const float m_new = fmaxf(m, bm);
          if (m_new > -INFINITY) {
            float acc = 0.f;
            const float mo = m_new * sl2;
#pragma unroll
            for (int e = 0; e < 32; ++e) acc += exp2f(v[e] * sl2 - mo);
            l = l * exp2f((m - m_new) * sl2) + acc;
            m = m_new;
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_empty[buf]);
      } else {
        const int i = j - nkb;
        if (i == 0) {
          inv_l = l > 0.f ? 1.f / l : 0.f;
          msl = m * sl2;
        }
        ok = __all_sync(0xffffffffu, mbar_wait(p_empty, (i & 1) ^ 1, abort_flag));
        if (!ok) break;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float v[32];
          tmem_ld32(s_addr + c * 32, v);
          tmem_ld_wait();
          const int k0 = kb * kTile + c * 32;
#pragma unroll
          for (int e = 0; e < 32; ++e) {
            float pv = exp2f(v[e] * sl2 - msl) * inv_l;
            if (diag && k0 + e > qi) pv = 0.f;
            if (p.drop_thresh != 0u)
              pv = drop_keep(p.seed, drop_row + static_cast<uint64_t>(k0 + e), p.drop_thresh)
                       ? pv * p.drop_scale : 0.f;
            v[e] = pv;
          }
#pragma unroll
          for (int g = 0; g < 4; ++g)
            st_shared_v4(swz_chunk(p_addr, row, c * 4 + g), pack_bf16x2(v[8 * g], v[8 * g + 1]),
                         pack_bf16x2(v[8 * g + 2], v[8 * g + 3]),
                         pack_bf16x2(v[8 * g + 4], v[8 * g + 5]),
                         pack_bf16x2(v[8 * g + 6], v[8 * g + 7]));
        }
        tc_fence_before();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&s_empty[buf]);
          mbar_arrive(p_full);
        }
      }
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(o_full, 0, abort_flag));
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* orow = p.out + (static_cast<size_t>(b) * p.S + qi) * (static_cast<size_t>(p.H) * dh) +
                            static_cast<size_t>(h) * dh;
      for (int c = 0; c < ksteps; ++c) {
        float v[16];
        tmem_ld16(lane_addr + 2 * kTile + c * 16, v);
        tmem_ld_wait();
        if (qi < p.S) {
          st_global_v4(orow + c * 16, pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                       pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
          st_global_v4(orow + c * 16 + 8, pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]),
                       pack_bf16x2(v[12], v[13]), pack_bf16x2(v[14], v[15]));
        }
      }
      if (qi < p.S && p.lse != nullptr)
        p.lse[(bh * p.S) + qi] = m * p.scale + logf(l);
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusWaitTimeout);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------------------
struct BwdParams {
  CUtensorMap q, k, v, d_o;   // bf16 [B, S, D]
  CUtensorMap dq;             // fp32 [B, S, D], box 16 x 32 x 1, no swizzle
  __nv_bfloat16* dk;
  __nv_bfloat16* dv;
  const float* lse;           // [B, H, S]
  const float* delta;         // [B, H, S]
  int B, H, S, dh;
  float scale;
  uint32_t drop_thresh;
  float drop_scale;
  uint64_t seed;
  int* status;
};

template <int NA>
struct BwdSmem {
  static constexpr int kK = 0;
  static constexpr int kV = NA * kAtomBytes;
  static constexpr int kQ = 2 * NA * kAtomBytes;
  static constexpr int kDO = 3 * NA * kAtomBytes;
  static constexpr int kP = 4 * NA * kAtomBytes;        // P, then dS; dQ staging aliases both
  static constexpr int kDS = kP + 2 * kAtomBytes;
  static constexpr int kBar = kDS + 2 * kAtomBytes;
  static constexpr int kTotal = kBar + 256 + 1024;
};

template <int NA>
__global__ void __launch_bounds__(160, 1) attn_bwd_kernel(const __grid_constant__ BwdParams p) {
  using L = BwdSmem<NA>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBar);
  uint64_t* kv_full = bars;        // K_j and V_j landed
  uint64_t* qdo_full = bars + 1;   // Q_i and dO_i landed
  uint64_t* qdo_empty = bars + 2;  // the MMAs of iteration i have consumed them
  uint64_t* sdp_full = bars + 3;   // S and dP are in TMEM
  uint64_t* pds_full = bars + 4;   // P and dS are in shared memory (4 warps)
  uint64_t* dq_full = bars + 5;    // dV, dK updated and dQ_i in TMEM
  uint64_t* acc_free = bars + 6;   // the S/dQ and dP columns have been read (4 warps)
  uint64_t* stage_free = bars + 7; // every warp's dQ reduce has read its staging boxes (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int nq = (p.S + kTile - 1) / kTile;
  const int dh = p.dh, ksteps = dh >> 4;
  const int n_it = nq - jb;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(qdo_full, 1);
    mbar_init(qdo_empty, 1);
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, 4);
    mbar_init(dq_full, 1);
    mbar_init(acc_free, 4);
    mbar_init(stage_free, 4);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&p.q);
    tma_prefetch_desc(&p.k);
    tma_prefetch_desc(&p.v);
    tma_prefetch_desc(&p.d_o);
    tma_prefetch_desc(&p.dq);
  }
  if (warp == 4) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV),
                 q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDO),
                 p_addr = smem_u32(smem + L::kP), ds_addr = smem_u32(smem + L::kDS);
  constexpr uint32_t kColS = 0, kColDP = 128, kColDV = 256, kColDK = 384;

  if (warp == 4) {
    if (lane == 0) {
      bool ok = true;
      const int x0 = h * dh;
      const uint32_t idesc_s = umma_idesc_bf16(kTile, kTile, 0, 0);      // Q K^T, dO V^T
      const uint32_t idesc_tn = umma_idesc_bf16(kTile, dh, 1, 1);        // P^T dO, dS^T Q
      const uint32_t idesc_dq = umma_idesc_bf16(kTile, dh, 0, 1);        // dS K
      mbar_expect_tx(kv_full, 2 * NA * kAtomBytes);
      for (int a = 0; a < NA; ++a) {
        tma_load_3d(smem + L::kK + a * kAtomBytes, &p.k, kv_full, x0 + 64 * a, jb * kTile, b);
        tma_load_3d(smem + L::kV + a * kAtomBytes, &p.v, kv_full, x0 + 64 * a, jb * kTile, b);
      }
      auto load_qdo = [&](int it) {
        if (!mbar_wait(qdo_empty, (it & 1) ^ 1, abort_flag)) { ok = false; return; }
        mbar_expect_tx(qdo_full, 2 * NA * kAtomBytes);
        const int q0 = (jb + it) * kTile;
        for (int a = 0; a < NA; ++a) {
          tma_load_3d(smem + L::kQ + a * kAtomBytes, &p.q, qdo_full, x0 + 64 * a, q0, b);
          tma_load_3d(smem + L::kDO + a * kAtomBytes, &p.d_o, qdo_full, x0 + 64 * a, q0, b);
        }
      };
      load_qdo(0);
      if (ok && !mbar_wait(kv_full, 0, abort_flag)) ok = false;
      for (int it = 0; it < n_it && ok; ++it) {
        const uint32_t par = it & 1;
        if (!mbar_wait(qdo_full, par, abort_flag)) { ok = false; break; }
        if (!mbar_wait(acc_free, par ^ 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int kk = 0; kk < ksteps; ++kk)
          mma_bf16_ss(tmem_base + kColS, desc_kmajor(q_addr, kk), desc_kmajor(k_addr, kk), idesc_s,
                      kk > 0);
        for (int kk = 0; kk < ksteps; ++kk)
          mma_bf16_ss(tmem_base + kColDP, desc_kmajor(do_addr, kk), desc_kmajor(v_addr, kk),
                      idesc_s, kk > 0);
        mma_commit(sdp_full);
        if (!mbar_wait(pds_full, par, abort_flag)) { ok = false; break; }
        tc_fence_after();
        for (int kk = 0; kk < kTile / 16; ++kk)       // dV += P^T dO   (contraction over queries)
          mma_bf16_ss(tmem_base + kColDV, desc_mnmajor(p_addr, kk), desc_mnmajor(do_addr, kk),
                      idesc_tn, (it > 0 || kk > 0) ? 1u : 0u);
        for (int kk = 0; kk < kTile / 16; ++kk)       // dK += dS^T Q
          mma_bf16_ss(tmem_base + kColDK, desc_mnmajor(ds_addr, kk), desc_mnmajor(q_addr, kk),
                      idesc_tn, (it > 0 || kk > 0) ? 1u : 0u);
        for (int kk = 0; kk < kTile / 16; ++kk)       // dQ = dS K      (contraction over keys)
          mma_bf16_ss(tmem_base + kColS, desc_kmajor(ds_addr, kk), desc_mnmajor(k_addr, kk),
                      idesc_dq, kk > 0);
        mma_commit(dq_full);
        mma_commit(qdo_empty);
        if (it + 1 < n_it) load_qdo(it + 1);
      }
    }
  } else {
    const int row = threadIdx.x;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
    const float sl2 = p.scale * kLog2e;
    const uint64_t bh = static_cast<uint64_t>(b) * p.H + h;
    const uint32_t stage_addr = p_addr + warp * (32 * kTile * 4);   // this warp's dQ staging
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const uint32_t par = it & 1;
      const int qtile = jb + it;
      const int qi = qtile * kTile + row;
      const bool qvalid = qi < p.S;
      const float lse2 = qvalid ? p.lse[bh * p.S + qi] * kLog2e : 0.f;
      const float dlt = qvalid ? p.delta[bh * p.S + qi] : 0.f;
      const uint64_t drop_row = (bh * p.S + static_cast<uint64_t>(qi)) * p.S;
      const bool diag = it == 0;
      ok = __all_sync(0xffffffffu, mbar_wait(sdp_full, par, abort_flag));
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        float s[32], dp[32];
        tmem_ld32(lane_addr + kColS + c * 32, s);
        tmem_ld32(lane_addr + kColDP + c * 32, dp);
        tmem_ld_wait();
        const int k0 = jb * kTile + c * 32;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float pv = exp2f(s[e] * sl2 - lse2);
          if (!qvalid || (diag && k0 + e > qi)) pv = 0.f;
          float pd = pv, dpe = dp[e];
          if (p.drop_thresh != 0u) {
            const bool keep = drop_keep(p.seed, drop_row + static_cast<uint64_t>(k0 + e), p.drop_thresh);
            pd = keep ? pv * p.drop_scale : 0.f;
            dpe = keep ? dpe * p.drop_scale : 0.f;
          }
          s[e] = pd;                                 // weights that multiplied V in the forward
          dp[e] = pv * (dpe - dlt) * p.scale;        // dS
        }
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          st_shared_v4(swz_chunk(p_addr, row, c * 4 + g), pack_bf16x2(s[8 * g], s[8 * g + 1]),
                       pack_bf16x2(s[8 * g + 2], s[8 * g + 3]),
                       pack_bf16x2(s[8 * g + 4], s[8 * g + 5]),
                       pack_bf16x2(s[8 * g + 6], s[8 * g + 7]));
          st_shared_v4(swz_chunk(ds_addr, row, c * 4 + g), pack_bf16x2(dp[8 * g], dp[8 * g + 1]),
                       pack_bf16x2(dp[8 * g + 2], dp[8 * g + 3]),
                       pack_bf16x2(dp[8 * g + 4], dp[8 * g + 5]),
                       pack_bf16x2(dp[8 * g + 6], dp[8 * g + 7]));
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
      ok = __all_sync(0xffffffffu, mbar_wait(dq_full, par, abort_flag));
      if (!ok) break;
      tc_fence_after();
      // dQ_i: TMEM -> this warp's staging boxes ([32 rows][16 fp32]) -> reduce-add
      for (int c = 0; c < ksteps; ++c) {
        float v[16];
        tmem_ld16(lane_addr + kColS + c * 16, v);
        tmem_ld_wait();
        const uint32_t dst = stage_addr + c * 2048 + lane * 64;
        const uint32_t* u = reinterpret_cast<const uint32_t*>(v);
#pragma unroll
        for (int g = 0; g < 4; ++g)
          st_shared_v4(dst + g * 16, u[4 * g], u[4 * g + 1], u[4 * g + 2], u[4 * g + 3]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(acc_free);
        const int r0 = qtile * kTile + warp * 32;
        if (r0 < p.S) {
          for (int c = 0; c < ksteps; ++c)
            tma_reduce_add_3d(&p.dq, stage_addr + c * 2048, h * dh + c * 16, r0, b);
          bulk_commit();
          bulk_wait_read<0>();
        }
        mbar_arrive(stage_free);
      }
      // the staging boxes alias P / dS rows of other warps: nobody refills P / dS
      // before every warp's reduce has finished reading shared memory (a bounded
      // wait, so an aborting CTA cannot strand a warp here)
      ok = __all_sync(0xffffffffu, mbar_wait(stage_free, par, abort_flag));
    }
    if (ok) {
      // after the last iteration's dq_full every MMA into dV / dK has retired
      tc_fence_after();
      const int kj = jb * kTile + row;
      const size_t D = static_cast<size_t>(p.H) * dh;
      const size_t off = (static_cast<size_t>(b) * p.S + kj) * D + static_cast<size_t>(h) * dh;
      for (int which = 0; which < 2; ++which) {
        __nv_bfloat16* dst = (which == 0 ? p.dv : p.dk) + off;
        const uint32_t col = which == 0 ? kColDV : kColDK;
        for (int c = 0; c < ksteps; ++c) {
          float v[16];
          tmem_ld16(lane_addr + col + c * 16, v);
          tmem_ld_wait();
          if (kj < p.S) {
            st_global_v4(dst + c * 16, pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                         pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
            st_global_v4(dst + c * 16 + 8, pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]),
                         pack_bf16x2(v[12], v[13]), pack_bf16x2(v[14], v[15]));
          }
        }
      }
    }
    if (lane == 0) bulk_wait<0>();
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicExch(p.status, kStatusWaitTimeout);
    const long long t0 = clock64();
    while (clock64() - t0 < 2000000LL) { }
    __syncthreads();
  }
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// delta[b, h, s] = sum_d dO[b, s, h*dh + d] * O[b, s, h*dh + d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o,
                                  const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                  int B, int H, int S, int dh) {
  const long long n = static_cast<long long>(B) * S * H;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= n) return;
  const int h = static_cast<int>(idx % H);
  const long long bs = idx / H;
  const int s = static_cast<int>(bs % S), b = static_cast<int>(bs / S);
  const size_t off = static_cast<size_t>(bs) * H * dh + static_cast<size_t>(h) * dh;
  const uint4* po = reinterpret_cast<const uint4*>(o + off);
  const uint4* pd = reinterpret_cast<const uint4*>(d_o + off);
  float acc = 0.f;
  for (int c = 0; c < dh / 8; ++c) {
    const uint4 a = po[c], g = pd[c];
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 x = __bfloat1622float2(a2[e]), y = __bfloat1622float2(g2[e]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  delta[(static_cast<size_t>(b) * H + h) * S + s] = acc;
}

// 3-D tensor maps over a [B, S, D] tensor: bf16 operand tiles (64 columns x
// 128 rows, 128-byte swizzle) and the fp32 dQ target (16 columns x 32 rows).
inline int make_tmap_bsd(CUtensorMap* map, const void* ptr, int B, int S, int D, bool fp32) {
  auto enc = tensor_map_encoder();
  if (enc == nullptr) return 1;
  const int eb = fp32 ? 4 : 2;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ((static_cast<size_t>(D) * eb) & 15) != 0)
    return 2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(D) * eb, static_cast<cuuint64_t>(S) * D * eb};
  cuuint32_t box[3] = {fp32 ? 16u : 64u, fp32 ? 32u : 128u, 1u};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16,
                   3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE,
                   fp32 ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3;
}

inline void drop_consts(float p_drop, uint32_t* thresh, float* scale) {
  if (p_drop <= 0.f) { *thresh = 0u; *scale = 1.f; return; }
  double t = static_cast<double>(p_drop) * 4294967296.0;
  if (t > 4294967295.0) t = 4294967295.0;
  if (t < 1.0) t = 1.0;
  *thresh = static_cast<uint32_t>(t);
  *scale = 1.f / (1.f - p_drop);
}

}  // namespace attn
}  // namespace dsb

extern "C" int dsb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse,
                                 int B, int H, int S, int dh, float p_drop,
                                 unsigned long long seed, int* status, cudaStream_t stream) {
  using namespace dsb::attn;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (dh < 16 || dh > 128 || (dh & 15)) return 700;
  FwdParams p;
  const int D = H * dh;
  if (make_tmap_bsd(&p.q, q, B, S, D, false) || make_tmap_bsd(&p.k, k, B, S, D, false) ||
      make_tmap_bsd(&p.v, v, B, S, D, false))
    return 701;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.lse = lse;
  p.B = B; p.H = H; p.S = S; p.dh = dh;
  p.scale = 1.f / sqrtf(static_cast<float>(dh));
  drop_consts(p_drop, &p.drop_thresh, &p.drop_scale);
  p.seed = seed;
  p.status = status;
  const dim3 grid((S + kTile - 1) / kTile, H, B);
  cudaError_t e;
  if (dh <= 64) {
    e = cudaFuncSetAttribute(attn_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FwdSmem<1>::kTotal);
    if (e != cudaSuccess) return 702;
    attn_fwd_kernel<1><<<grid, 160, FwdSmem<1>::kTotal, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(attn_fwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             FwdSmem<2>::kTotal);
    if (e != cudaSuccess) return 702;
    attn_fwd_kernel<2><<<grid, 160, FwdSmem<2>::kTotal, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 703;
}

extern "C" int dsb_attention_bwd(const void* q, const void* k, const void* v, const void* out,
                                 const void* d_out, const float* lse, float* delta, float* dq,
                                 void* dk, void* dv, int B, int H, int S, int dh, float p_drop,
                                 unsigned long long seed, int* status, cudaStream_t stream) {
  using namespace dsb::attn;
  if (B <= 0 || H <= 0 || S <= 0) return 0;
  if (dh < 16 || dh > 128 || (dh & 15)) return 700;
  BwdParams p;
  const int D = H * dh;
  if (make_tmap_bsd(&p.q, q, B, S, D, false) || make_tmap_bsd(&p.k, k, B, S, D, false) ||
      make_tmap_bsd(&p.v, v, B, S, D, false) || make_tmap_bsd(&p.d_o, d_out, B, S, D, false) ||
      make_tmap_bsd(&p.dq, dq, B, S, D, true))
    return 701;
  const long long n = static_cast<long long>(B) * S * H;
  attn_delta_kernel<<<static_cast<unsigned>((n + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(out), reinterpret_cast<const __nv_bfloat16*>(d_out),
      delta, B, H, S, dh);
  p.dk = reinterpret_cast<__nv_bfloat16*>(dk);
  p.dv = reinterpret_cast<__nv_bfloat16*>(dv);
  p.lse = lse;
  p.delta = delta;
  p.B = B; p.H = H; p.S = S; p.dh = dh;
  p.scale = 1.f / sqrtf(static_cast<float>(dh));
  drop_consts(p_drop, &p.drop_thresh, &p.drop_scale);
  p.seed = seed;
  p.status = status;
  const dim3 grid((S + kTile - 1) / kTile, H, B);
  cudaError_t e;
  if (dh <= 64) {
    e = cudaFuncSetAttribute(attn_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             BwdSmem<1>::kTotal);
    if (e != cudaSuccess) return 702;
    attn_bwd_kernel<1><<<grid, 160, BwdSmem<1>::kTotal, stream>>>(p);
  } else {
    e = cudaFuncSetAttribute(attn_bwd_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             BwdSmem<2>::kTotal);
    if (e != cudaSuccess) return 702;
    attn_bwd_kernel<2><<<grid, 160, BwdSmem<2>::kTotal, stream>>>(p);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : 703;
}
