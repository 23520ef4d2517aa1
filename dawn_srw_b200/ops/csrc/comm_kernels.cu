// Cross-GPU synchronisation over symmetric memory (NVLink peer stores/loads).
//
// dsb_peer_barrier: every rank writes `epoch` into slot [my_rank] of every
// peer's signal pad (st.release.sys) and then waits until all slots of its own
// pad have reached `epoch`.  The wait is bounded: after kPeerWaitCycles it
// gives up, writes kStatusPeerTimeout to the status word and returns, so a
// missing peer turns into a host-visible error instead of a hung GPU.
// The reference needs no such primitive (XLA inserts its collectives).
#include <cstdint>

#include "common/ptx.cuh"
#include "dsb_api.h"

namespace dsb {

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

constexpr long long kPeerWaitCycles = 4000000000LL;  // ~2 s

__global__ void peer_barrier_kernel(unsigned int* const* pads, int rank, int world,
                                    unsigned int epoch, int slot_base, int* status,
                                    long long wait_cycles) {
  const int t = threadIdx.x;
  __threadfence_system();   // everything this GPU wrote before the barrier is visible first
  if (t < world) {
    unsigned int* dst = pads[t] + slot_base + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
  }
  if (t < world) {
    const unsigned int* src = pads[rank] + slot_base + t;
    const long long t0 = clock64();
    unsigned int v = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if (clock64() - t0 > wait_cycles) {
        atomicExch(status, kStatusPeerTimeout);
        break;
      }
      __nanosleep(200);
    }
  }
  __syncthreads();
  __threadfence_system();
}


// ---------------------------------------------------------------------------
// One-shot all-reduce (sum) of a small fp32 vector over symmetric memory.
// CTA c owns elements [c * kArChunk, (c+1) * kArChunk): it copies them into
// this rank's staging buffer (two halves used in turn, selected by the epoch's
// parity), exchanges epoch flags with the same CTA of every peer (bounded wait;
// slots slot_base + c * world + rank) and then sums the peers' staging buffers
// in rank order, so all ranks get bit-identical results.  A rank cannot run
// more than one call ahead of a peer (it needs that peer's flag of the current
// call), hence two halves are enough.  CTAs never wait on one another.  Meant
// for per-token statistics, denominators and loss scalars.
constexpr int kArChunk = 4096;

__global__ void small_allreduce_kernel(float* const* stage, unsigned int* const* pads, int rank,
                                       int world, unsigned int epoch, int slot_base,
                                       const float* in, float* out /* may alias in */,
                                       int n, int cap, int* status, long long wait_cycles) {
  const int t = threadIdx.x;
  const int lo = blockIdx.x * kArChunk;
  const int hi = min(n, lo + kArChunk);
  const size_t half = static_cast<size_t>(epoch & 1u) * cap;
  float* mine = stage[rank] + half;
  for (int i = lo + t; i < hi; i += blockDim.x) mine[i] = in[i];
  __threadfence_system();
  __syncthreads();
  if (t < world) {
    const int slot = slot_base + blockIdx.x * world;
    unsigned int* dst = pads[t] + slot + rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
    const unsigned int* src = pads[rank] + slot + t;
    const long long t0 = clock64();
    unsigned int v = 0;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      if (static_cast<int>(v - epoch) >= 0) break;
      if (clock64() - t0 > wait_cycles) {
        atomicExch(status, kStatusPeerTimeout);
        break;
      }
      __nanosleep(100);
    }
  }
  __syncthreads();
  for (int i = lo + t; i < hi; i += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < world; ++r)
      acc += __ldcv(stage[r] + half + i);   // peer memory: never served from a stale L1 line
    out[i] = acc;
  }
}

// ---------------------------------------------------------------------------
// Partitioned optimizer step over peer memory (reduce-scatter + AdamW +
// all-gather without a library collective).  All ranks of a replica group keep
// the parameters and their gradients in symmetric fp32 buffers of identical
// layout; rank k owns elements [lo, lo + n) of them.
//
// zero_reduce_kernel: g_own[i] = scale * sum_r grads[r][lo + i] (rank order),
// and sq[0] += sum g_own^2.  Reads the peers' gradients with plain loads over
// NVLink; float4 when everything is 16-byte aligned.
__global__ void zero_reduce_kernel(const float* const* grads, int world, long long lo, long long n,
                                   float scale, float* __restrict__ g_own,
                                   float* __restrict__ sq) {
  float s = 0.f;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = n >> 2;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < world; ++r) {
      const float4 v = __ldcv(reinterpret_cast<const float4*>(grads[r] + lo) + i);
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(g_own)[i] = acc;
    s += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  s = warp_sum_f(s);
  __shared__ float sh[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) sh[warp] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
    for (int k = 0; k < (blockDim.x >> 5); ++k) tot += sh[k];
    atomicAdd(sq, tot);
  }
}

// zero_adam_scatter_kernel: AdamW on the owned slice (moments are local and
// slice-sized), the new parameters are stored to every rank's buffer.
__global__ void zero_adam_scatter_kernel(float* const* params, int world, int rank, long long lo,
                                         long long n, const float* __restrict__ g,
                                         float* __restrict__ m, float* __restrict__ v,
                                         const float* __restrict__ clip_scale, float lr, float b1,
                                         float b2, float eps, float wd, float bc1, float bc2) {
  const float cs = *clip_scale;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const long long n4 = n >> 2;
  const float4* p_own = reinterpret_cast<const float4*>(params[rank] + lo);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4;
       i += stride) {
    const float4 g4 = reinterpret_cast<const float4*>(g)[i];
    float4 m4 = reinterpret_cast<float4*>(m)[i], v4 = reinterpret_cast<float4*>(v)[i];
    float4 p4 = p_own[i];
    const float gg[4] = {g4.x * cs, g4.y * cs, g4.z * cs, g4.w * cs};
    float mm[4] = {m4.x, m4.y, m4.z, m4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
    float pp[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mm[k] = b1 * mm[k] + (1.f - b1) * gg[k];
      vv[k] = b2 * vv[k] + (1.f - b2) * gg[k] * gg[k];
      const float upd = (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps) + wd * pp[k];
      pp[k] -= lr * upd;
    }
    reinterpret_cast<float4*>(m)[i] = make_float4(mm[0], mm[1], mm[2], mm[3]);
    reinterpret_cast<float4*>(v)[i] = make_float4(vv[0], vv[1], vv[2], vv[3]);
    const float4 out = make_float4(pp[0], pp[1], pp[2], pp[3]);
    for (int r = 0; r < world; ++r) reinterpret_cast<float4*>(params[r] + lo)[i] = out;
  }
}

// out[i] = sum over slabs of in[w * n + i]: the local half of the fused
// reduce-scatter (the slabs were stored by the ranks' GEMM epilogues).
template <bool kInBf16, bool kOutBf16>
__global__ void sum_slabs_kernel(const void* __restrict__ in, int n_slabs, long long n,
                                 void* __restrict__ out) {
  const long long n8 = n >> 3;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < n_slabs; ++w) {
      if (kInBf16) {
        const uint4 v = reinterpret_cast<const uint4*>(
            static_cast<const __nv_bfloat16*>(in) + static_cast<size_t>(w) * n)[i];
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 f = __bfloat1622float2(h[k]);
          acc[2 * k] += f.x;
          acc[2 * k + 1] += f.y;
        }
      } else {
        const float4* src = reinterpret_cast<const float4*>(
            static_cast<const float*>(in) + static_cast<size_t>(w) * n) + 2 * i;
        const float4 a = src[0], b = src[1];
        acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w;
        acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
      }
    }
    if (kOutBf16) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      reinterpret_cast<uint4*>(out)[i] = o;
    } else {
      float4* dst = reinterpret_cast<float4*>(out) + 2 * i;
      dst[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
      dst[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}

// Owner side of the fused reduce-scatter of a route's output: sums the W partial
// slabs (bf16) and the W partial denominators of its tokens and divides after the
// reduction (the reference normalises before its all-reduce of bf16 outputs,
// models/dawn_spatial_v41_exp.py:579-586; a per-row factor commutes with the sum).
__global__ void sum_slabs_div_kernel(const __nv_bfloat16* __restrict__ in, int n_slabs, int rows,
                                     int cols, const float* __restrict__ den_in,
                                     const float* __restrict__ scale, float* __restrict__ out,
                                     float* __restrict__ den_out) {
  const int c8 = cols >> 3;
  const long long n8 = static_cast<long long>(rows) * c8;
  const long long slab = static_cast<long long>(rows) * cols;
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  const float sc = *scale;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8;
       i += stride) {
    const int row = static_cast<int>(i / c8);
    const int cc = static_cast<int>(i - static_cast<long long>(row) * c8);
    float den = 0.f;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int w = 0; w < n_slabs; ++w) {
      den += den_in[static_cast<size_t>(w) * rows + row];
      const uint4 v = reinterpret_cast<const uint4*>(in + w * slab)[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    const float f = sc / fmaxf(den, 1.f);
    float4* dst = reinterpret_cast<float4*>(out) + 2 * i;
    dst[0] = make_float4(acc[0] * f, acc[1] * f, acc[2] * f, acc[3] * f);
    dst[1] = make_float4(acc[4] * f, acc[5] * f, acc[6] * f, acc[7] * f);
    if (cc == 0) den_out[row] = den;
  }
}

}  // namespace dsb

extern "C" int dsb_peer_barrier(unsigned int* const* pads_dev, int rank, int world,
                                unsigned int epoch, int slot_base, int* status,
                                long long wait_cycles, cudaStream_t stream) {
  if (world < 1 || world > 32) return 600;
  if (wait_cycles <= 0) wait_cycles = dsb::kPeerWaitCycles;
  dsb::peer_barrier_kernel<<<1, 32, 0, stream>>>(pads_dev, rank, world, epoch, slot_base, status,
                                                 wait_cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}

extern "C" int dsb_small_allreduce(float* const* stage_dev, unsigned int* const* pads_dev, int rank,
                                   int world, unsigned int epoch, int slot_base, const float* in,
                                   float* out, int n, int cap, int* status, long long wait_cycles,
                                   cudaStream_t stream) {
  if (world < 1 || world > 32) return 600;
  if (n < 0 || n > cap) return 602;
  if (n == 0) return 0;
  if (wait_cycles <= 0) wait_cycles = dsb::kPeerWaitCycles;
  const int ctas = (n + dsb::kArChunk - 1) / dsb::kArChunk;
  if (ctas * world > 512) return 602;   // flag slots reserved for this primitive
  const int threads = n >= 512 ? 512 : (n <= 32 ? 32 : ((n + 31) / 32) * 32);
  dsb::small_allreduce_kernel<<<ctas, threads, 0, stream>>>(stage_dev, pads_dev, rank, world, epoch,
                                                         slot_base, in, out, n, cap, status,
                                                         wait_cycles);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}

static int zero_grid(long long n4) {
  long long g = (n4 + 255) / 256;
  if (g < 1) g = 1;
  return static_cast<int>(g < 148 * 8 ? g : 148 * 8);
}

extern "C" int dsb_zero_reduce(const float* const* grads_dev, int world, long long lo, long long n,
                               float scale, float* g_own, float* sq, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 3) || (lo & 3) || (reinterpret_cast<uintptr_t>(g_own) & 15)) return 603;
  dsb::zero_reduce_kernel<<<zero_grid(n >> 2), 256, 0, stream>>>(grads_dev, world, lo, n, scale,
                                                                 g_own, sq);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}

extern "C" int dsb_zero_adam_scatter(float* const* params_dev, int world, int rank, long long lo,
                                     long long n, const float* g, float* m, float* v,
                                     const float* clip_scale, float lr, float b1, float b2,
                                     float eps, float wd, float bc1, float bc2,
                                     cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((n & 3) || (lo & 3)) return 603;
  dsb::zero_adam_scatter_kernel<<<zero_grid(n >> 2), 256, 0, stream>>>(
      params_dev, world, rank, lo, n, g, m, v, clip_scale, lr, b1, b2, eps, wd, bc1, bc2);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}

extern "C" int dsb_sum_slabs(const void* in, int in_is_bf16, int n_slabs, long long n, void* out,
                             int out_is_bf16, cudaStream_t stream) {
  if (n <= 0 || n_slabs <= 0) return 0;
  if ((n & 7) || (reinterpret_cast<uintptr_t>(in) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return 603;
  const int grid = zero_grid(n >> 3);
  if (in_is_bf16 && out_is_bf16) dsb::sum_slabs_kernel<true, true><<<grid, 256, 0, stream>>>(in, n_slabs, n, out);
  else if (in_is_bf16) dsb::sum_slabs_kernel<true, false><<<grid, 256, 0, stream>>>(in, n_slabs, n, out);
  else if (out_is_bf16) dsb::sum_slabs_kernel<false, true><<<grid, 256, 0, stream>>>(in, n_slabs, n, out);
  else dsb::sum_slabs_kernel<false, false><<<grid, 256, 0, stream>>>(in, n_slabs, n, out);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}

extern "C" int dsb_sum_slabs_div(const void* in_bf16, int n_slabs, int rows, int cols,
                                 const float* den_in, const float* scale, float* out,
                                 float* den_out, cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || n_slabs <= 0) return 0;
  if ((cols & 7) || (reinterpret_cast<uintptr_t>(in_bf16) & 15) ||
      (reinterpret_cast<uintptr_t>(out) & 15))
    return 603;
  const long long n8 = static_cast<long long>(rows) * (cols >> 3);
  dsb::sum_slabs_div_kernel<<<zero_grid(n8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(in_bf16), n_slabs, rows, cols, den_in, scale, out, den_out);
  return cudaGetLastError() == cudaSuccess ? 0 : 601;
}
