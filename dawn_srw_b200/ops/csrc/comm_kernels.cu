// Cross-GPU synchronisation over symmetric memory (NVLink peer stores/loads).
//
// dsb_peer_barrier: every rank writes `epoch` into slot [my_rank] of every
// peer's signal pad (st.release.sys) and then waits until all slots of its own
// pad have reached `epoch`.  The wait is bounded: after kPeerWaitCycles it
// gives up, writes kStatusPeerTimeout to the status word and returns, so a
// missing peer turns into a host-visible error instead of a hung GPU.
// The reference needs no such primitive (XLA inserts its collectives).
#include "common/ptx.cuh"
#include "dsb_api.h"

namespace dsb {

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
