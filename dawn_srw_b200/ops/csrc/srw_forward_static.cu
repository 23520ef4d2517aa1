// Allocation-free variant of dsb_srw_forward: the p[T, U] scratch lives in a
// file-scope device array.  See srw_forward_static.h for the contract.
#include <stdio.h>

#include "srw_forward_static.h"

namespace {

// Part of the library image; resident on every device that loads it.
static __device__ __align__(256) unsigned char g_srw_scratch[DSB_SRW_STATIC_SCRATCH_BYTES];

thread_local char g_last_error[256] = "";

// Device address of g_srw_scratch on the current device.  In host code the
// name g_srw_scratch is only a handle for the runtime, never a pointer a kernel
// may use.  The address is asked for on every call (a cheap table look-up in
// the runtime) instead of being cached per ordinal: a cached pointer would
// outlive a context that was torn down and re-created on the same ordinal.
// Concurrent calls from several host threads are fine: nothing is shared here.
int scratch_for_current_device(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
    snprintf(g_last_error, sizeof(g_last_error), "no usable current CUDA device (ordinal %d)", dev);
    return DSB_STATIC_ERR_SYMBOL;
  }
  void* ptr = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&ptr, g_srw_scratch);  // `dev` is current
  if (e != cudaSuccess || ptr == nullptr) {
    snprintf(g_last_error, sizeof(g_last_error),
             "cudaGetSymbolAddress for the static SRW scratch failed on device %d: %s", dev,
             cudaGetErrorString(e));
    return DSB_STATIC_ERR_SYMBOL;
  }
  *out = ptr;
  return 0;
}

inline long long padded_units(int U) { return (static_cast<long long>(U) + 7) / 8 * 8; }

}  // namespace

extern "C" unsigned long long dsb_srw_forward_static_bytes_needed(int T, int U) {
  if (T <= 0 || U <= 0) return 0;
  return static_cast<unsigned long long>(T) * static_cast<unsigned long long>(padded_units(U)) * 2ull;
}

extern "C" unsigned long long dsb_srw_forward_static_capacity(void) {
  return DSB_SRW_STATIC_SCRATCH_BYTES;
}

extern "C" const char* dsb_srw_forward_static_last_error(void) { return g_last_error; }

extern "C" int dsb_srw_forward_static(const void* h, long long ldh, const void* emb,
                                      long long lde, const void* x, long long ldx,
                                      const void* read, long long ldr, const void* write,
                                      long long ldw, int T, int U, int r, int D, const float* tau,
                                      const float* inv_sigma, float* raw_out, long long ldo,
                                      float* den_sum, unsigned char* alive,
                                      const float* unit_mask, const DsbGate* gate, int* status,
                                      cudaStream_t stream) {
  g_last_error[0] = '\0';
  if (T <= 0 || U <= 0) return 0;
  const unsigned long long need = dsb_srw_forward_static_bytes_needed(T, U);
  if (need > DSB_SRW_STATIC_SCRATCH_BYTES) {
    snprintf(g_last_error, sizeof(g_last_error),
             "SRW forward with T=%d tokens and U=%d units needs %llu bytes of scratch; the static "
             "buffer holds %llu.  Split the tokens or use dsb_srw_forward with your own scratch.",
             T, U, need, static_cast<unsigned long long>(DSB_SRW_STATIC_SCRATCH_BYTES));
    return DSB_STATIC_ERR_TOO_LARGE;
  }
  void* scratch = nullptr;
  const int rc = scratch_for_current_device(&scratch);
  if (rc != 0) return rc;
  const int lrc = dsb_srw_forward(h, ldh, emb, lde, x, ldx, read, ldr, write, ldw, T, U, r, D, tau,
                                  inv_sigma, scratch, padded_units(U), raw_out, ldo, den_sum, alive,
                                  unit_mask, gate, status, stream);
  if (lrc != 0)
    snprintf(g_last_error, sizeof(g_last_error), "dsb_srw_forward returned %d", lrc);
  return lrc;
}
