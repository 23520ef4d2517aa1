// SRW forward for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference (which is a JAX program
// and never manages device memory itself).  It exists for hosts that embed the
// kernels where allocation is off the table: a serving loop that has handed the
// whole device to a memory pool it does not control, a latency-critical thread
// in which a cudaMalloc (a device-wide synchronising call) would stall other
// streams, or a plugin sandbox that forbids the allocator outright.
//
// dsb_srw_forward_static does the same work as dsb_srw_forward (one route of
// the SRW forward op: gate kernel, then the write GEMM) but keeps the gated
// operand tile p[T, U] in a buffer that is part of the library image instead of
// taking scratch from the caller.  It calls no cudaMalloc / cudaFree and no
// allocating library routine.
//
//   * Capacity: DSB_SRW_STATIC_SCRATCH_BYTES (64 MiB).  A call needs
//     T * round_up(U, 8) * 2 bytes; larger problems are refused with
//     DSB_STATIC_ERR_TOO_LARGE and nothing is launched.  Every GPU whose
//     context loads this library keeps those 64 MiB until the process exits.
//   * Every call looks up the buffer's device address (cudaGetSymbolAddress,
//     with the caller's device current); the first such look-up on a device
//     initialises the library image there, so make the first call on each
//     device outside any stream capture.
//   * The buffer is part of libdsb_kernels.so only (the C library); the Python
//     extension module does not carry a second copy.
//   * All calls on a device share the one buffer and it keeps whatever the last
//     call left there.  The kernels rewrite every element they later read, and
//     den_sum (an output) is cleared by the call itself, so nothing needs
//     pre-zeroing -- but two calls whose kernels overlap on the GPU (different
//     streams, or different host threads) race on the buffer.  Serialise them.
//   * Inputs and outputs are still the caller's: same shapes, strides and
//     alignment rules as dsb_srw_forward.
#pragma once
#include "dsb_api.h"

#ifdef __cplusplus
extern "C" {
#endif

#define DSB_SRW_STATIC_SCRATCH_BYTES (64ull << 20)
#define DSB_STATIC_ERR_TOO_LARGE 501   /* T * round_up(U,8) * 2 exceeds the static buffer */
#define DSB_STATIC_ERR_SYMBOL 502      /* the device address of the buffer could not be obtained */

int dsb_srw_forward_static(const void* h, long long ldh, const void* emb, long long lde,
                           const void* x, long long ldx, const void* read, long long ldr,
                           const void* write, long long ldw, int T, int U, int r, int D,
                           const float* tau, const float* inv_sigma, float* raw_out,
                           long long ldo, float* den_sum, unsigned char* alive,
                           const float* unit_mask, const DsbGate* gate /*host*/, int* status,
                           cudaStream_t stream);

// Bytes of static scratch a (T, U) problem needs, and the capacity.
unsigned long long dsb_srw_forward_static_bytes_needed(int T, int U);
unsigned long long dsb_srw_forward_static_capacity(void);
// Human-readable description of the last non-zero return of
// dsb_srw_forward_static on the calling thread ("" if none).
const char* dsb_srw_forward_static_last_error(void);

#ifdef __cplusplus
}
#endif
