// C ABI of the dawn_srw_b200 CUDA library.  All pointers are device pointers
// unless noted; every launcher is asynchronous on `stream` and returns 0 on a
// successful launch (non-zero: host-side argument / launch error).  Kernels
// report device-side failures (bounded waits that ran out) through the int
// `status` word the caller passes (0 = ok).
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct DsbGate {
  int kind;  // 0: clip(relu(s-tau),0,clip_max)  1: z*Phi(z), z=(s-tau)/sigma  2: two-stage
  float sharpness, act_threshold, act_cutoff, epsilon, max_intensity, clip_max, dead_threshold;
} DsbGate;

// Fused all-gather of the token operands of a gate kernel over `n_ranks` GPUs.
// Tensor t (0: x, 1: h, 2: dy) lives on every rank in a "full" bf16 buffer
// [n_ranks * rows_per_rank, cols[t]] (ld[t] elements between rows) of which
// the rank has filled only its own row block (the tensors are generic: any bf16
// operand of the kernel, or of the GEMMs that follow it); bufs[t] is a HOST array with the
// n_ranks device pointers of those buffers (peer pointers for other ranks).
// The kernel pulls the missing row blocks into bufs[t][my_rank] while it
// computes.  `ready` is local device memory with one uint32 per 128 rows and
// `epoch` must be larger than any value used before on that array.
typedef struct DsbGather {
  int n_ranks, my_rank, rows_per_rank, n_tensors;
  const void* const* bufs[3];
  long long ld[3];
  int cols[3];
  unsigned int* ready;
  unsigned int epoch;
  // optional: n_stats arrays of per-token float4 [n_ranks * rows_per_rank] that are gathered
  // along with the rows; stats[s] is a HOST array with the n_ranks device pointers
  int n_stats;
  const void* const* stats[3];
} DsbGather;

// C[M,N] (=|+=) alpha * row_scale[m] * (A . B^T)[m,n] + bias[n]
//   A: a_mn == 0 -> stored [M][K] (lda >= K);  a_mn == 1 -> stored [K][M] (lda >= M)
//   B: b_mn == 0 -> stored [N][K];             b_mn == 1 -> stored [K][N]
//   bf16 operands, fp32 accumulation; C is bf16 (c_is_bf16) or fp32.
//   Leading dimensions must be multiples of 8 elements, bases 16-byte aligned.
int dsb_gemm_bf16(const void* A, int a_mn, long long lda, const void* B, int b_mn, long long ldb,
                  int M, int N, int K, void* C, long long ldc, int c_is_bf16, int accumulate,
                  float alpha, const float* row_scale, const float* bias, int block_n,
                  int* status, cudaStream_t stream);

// SRW forward gate kernel: p[T,U] = gate(h.emb^T; tau, 1/sigma) * (x.read^T),
// den_sum[T] += sum_U den_term.  gate_sum / alive / unit_mask may be null.
int dsb_srw_fwd_gate(const void* h, long long ldh, const void* emb, long long lde, const void* x,
                     long long ldx, const void* read, long long ldr, int T, int U, int r, int D,
                     void* p_out, long long ldp, const float* tau, const float* inv_sigma,
                     float* den_sum, float* gate_sum, unsigned char* alive,
                     const float* unit_mask, const DsbGate* gate /*host*/, int* status,
                     cudaStream_t stream);

// SRW backward gate kernel: recomputes S and XR, adds DP = dy.write^T, writes
// p, dxr = DP*g and ds (all bf16 [T, ld_out]) and accumulates dtau_sum[T] -= sum_U ds.
// dsz_sum is accepted for ABI stability and left untouched: the caller derives
// sum_U ds*z from ds.emb and dtau (see ops/cuda_backend.py).
int dsb_srw_bwd_gate(const void* h, long long ldh, const void* emb, long long lde, const void* x,
                     long long ldx, const void* read, long long ldr, const void* dy,
                     long long lddy, const void* write, long long ldw, int T, int U, int r, int D,
                     void* p_out, void* dxr_out, void* ds_out, long long ld_out, const float* tau,
                     const float* inv_sigma, const float* dden, float* dtau_sum, float* dsz_sum,
                     const DsbGate* gate /*host*/, int* status, cudaStream_t stream);

// Gate kernels with the all-gather fused in (gather may be null: plain kernel).
// h / x (/ dy) must then be this rank's full buffers.
int dsb_srw_fwd_gate_gather(const void* h, long long ldh, const void* emb, long long lde,
                            const void* x, long long ldx, const void* read, long long ldr, int T,
                            int U, int r, int D, void* p_out, long long ldp, const float* tau,
                            const float* inv_sigma, float* den_sum, float* gate_sum,
                            unsigned char* alive, const float* unit_mask, const DsbGate* gate,
                            const DsbGather* gather /*host*/, int* status, cudaStream_t stream);
int dsb_srw_bwd_gate_gather(const void* h, long long ldh, const void* emb, long long lde,
                            const void* x, long long ldx, const void* read, long long ldr,
                            const void* dy, long long lddy, const void* write, long long ldw,
                            int T, int U, int r, int D, void* p_out, void* dxr_out, void* ds_out,
                            long long ld_out, const float* tau, const float* inv_sigma,
                            const float* dden, float* dtau_sum, float* dsz_sum,
                            const DsbGate* gate, const DsbGather* gather /*host*/, int* status,
                            cudaStream_t stream);

// 1 when a pool of U units runs on the 256-column gate kernels (CTA pairs, U >= 512);
// only those can keep / consume the read scalars below.
int dsb_srw_wide_tiles(int U);

// Forward gate kernel that can also keep the read scalars: xr_out (nullable)
// receives bf16 xr = x.read^T [T, ldxr] next to p.  Needs dsb_srw_wide_tiles(U).
// gather may be null.  `stats` (nullable; wide kernels only) replaces tau / inv_sigma by
// one float4 per token (tau, 1/sigma, -, -): the form in which a fused gather brings the
// per-token constants in together with the rows (DsbGather.stats).
// `diag` (nullable; wide kernels only): zeroed fp32 [T * 12 + 2]; receives the routing
// diagnostics as per-token sums over the units, 12 columns per token (gate sum, active,
// strong, band, z / intensity sum, two narrower bands, sum g log g, sum s^3, sum s^4, gate
// max, one spare), followed by two scalars (max intensity, count of capped intensities).
int dsb_srw_fwd_gate_xr(const void* h, long long ldh, const void* emb, long long lde,
                        const void* x, long long ldx, const void* read, long long ldr, int T,
                        int U, int r, int D, void* p_out, long long ldp, void* xr_out,
                        long long ldxr, const float* tau, const float* inv_sigma,
                        const void* stats, float* den_sum, float* gate_sum, float* diag,
                        unsigned char* alive, const float* unit_mask, const DsbGate* gate,
                        const DsbGather* gather /*host*/, int* status, cudaStream_t stream);

// Backward gate step from the read scalars the forward pass kept: one launch
// computing S = h.emb^T and DP = dy.write^T, writing p = g*xr, dxr = DP*g and ds
// (bf16 [T, ld_out]) and accumulating dtau_sum[T] -= sum_U ds.  No x / read
// operands: xr is read back instead of recomputed.  With a gather, every tensor
// it lists is pulled under its one epoch.  `stats` (nullable): float4 (tau, 1/sigma, dden, -)
// per token instead of the three arrays.
int dsb_srw_bwd_gate_xr(const void* h, long long ldh, const void* emb, long long lde,
                        const void* dy, long long lddy, const void* write, long long ldw,
                        const void* xr, long long ldxr, int T, int U, int r, int D, void* p_out,
                        void* dxr_out, void* ds_out, long long ld_out, const float* tau,
                        const float* inv_sigma, const float* dden, const void* stats,
                        float* dtau_sum, const DsbGate* gate, const DsbGather* gather /*host*/,
                        int* status, cudaStream_t stream);

// One route of the SRW forward op (gate kernel + write GEMM).  `p_scratch` is
// caller-provided scratch: bf16 [T, ldp] with ldp >= U and ldp % 8 == 0; its
// contents on return are unspecified.  den_sum[T] is cleared and filled here;
// raw_out is fp32 [T, ldo].  alive / unit_mask may be null.
int dsb_srw_forward(const void* h, long long ldh, const void* emb, long long lde, const void* x,
                    long long ldx, const void* read, long long ldr, const void* write,
                    long long ldw, int T, int U, int r, int D, const float* tau,
                    const float* inv_sigma, void* p_scratch, long long ldp, float* raw_out,
                    long long ldo, float* den_sum, unsigned char* alive, const float* unit_mask,
                    const DsbGate* gate /*host*/, int* status, cudaStream_t stream);

// GEMM whose output row blocks are stored to their owner ranks (first half of
// a fused reduce-scatter, see gemm_kernels.cu).  `outs` is a HOST array of
// n_ranks device pointers to the ranks' receive buffers [n_ranks *
// rows_per_rank, ldc] (bf16 or fp32; peer pointers included); this rank fills
// slot `my_rank` of each.  After a barrier the owner sums its slots:
int dsb_gemm_bf16_scatter(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                          long long ldb, int M, int N, int K, void* const* outs, int n_ranks,
                          int my_rank, int rows_per_rank, long long ldc, int out_is_bf16,
                          float alpha, const float* row_scale, int* status, cudaStream_t stream);
// Scatter GEMM that also sends one fp32 value per result row to the row's owner:
// aux_dsts[j][my_rank * rows_per_rank + local row] = aux_src[row] (aux_dsts: HOST array of
// n_ranks device pointers to fp32 [n_ranks * rows_per_rank] receive buffers).  Used for the
// partial per-token denominators / threshold cotangents, which are then summed like the slabs.
int dsb_gemm_bf16_scatter_aux(const void* A, int a_mn, long long lda, const void* B, int b_mn,
                              long long ldb, int M, int N, int K, void* const* outs, int n_ranks,
                              int my_rank, int rows_per_rank, long long ldc, int out_is_bf16,
                              float alpha, const float* row_scale, const float* aux_src,
                              float* const* aux_dsts, int* status, cudaStream_t stream);
// Second half of the fused reduce-scatter of a route's output with the sum-normalisation
// after the reduction: den[t] = sum_w den_in[w * rows + t];
// out[t, :] = scale[0] * sum_w in[w][t, :] / max(den[t], 1)   (in bf16 [n_slabs * rows, cols],
// cols a multiple of 8; out fp32 [rows, cols]; den_out fp32 [rows]; scale: device scalar).
int dsb_sum_slabs_div(const void* in_bf16, int n_slabs, int rows, int cols, const float* den_in,
                      const float* scale, float* out, float* den_out, cudaStream_t stream);
// out[i] = sum_w in[w * n + i], w < n_slabs; in bf16 or fp32, out bf16 or fp32
// (accumulated in fp32); n a multiple of 8, pointers 16-byte aligned.
int dsb_sum_slabs(const void* in, int in_is_bf16, int n_slabs, long long n, void* out,
                  int out_is_bf16, cudaStream_t stream);

// Tied LM head with the softmax statistics taken in the GEMM epilogue (no fp32 logits):
// logits_bf16 [M, ldl] = x[M, K] . emb[V, K]^T, lse / label_logit fp32 [M], argmax int64 [M];
// `partial`: scratch of M * ceil(V / 256) * 16 bytes.  labels < 0: no label (label_logit 0).
int dsb_lm_head_ce_fwd(const void* x, long long ldx, const void* emb, long long lde, int M, int V,
                       int K, const long long* labels, void* logits_bf16, long long ldl,
                       void* partial, float* lse, float* label_logit, long long* argmax,
                       int* status, cudaStream_t stream);
// In place: logits -> scale[row] * (softmax - onehot(label)) as bf16 (columns >= V zeroed).
int dsb_lm_head_ce_bwd_inplace(void* logits_bf16, long long ldl, int M, int V,
                               const long long* labels, const float* lse, const float* scale,
                               cudaStream_t stream);

// Bounded cross-GPU barrier over symmetric signal pads.  `pads_dev` is a DEVICE
// array of `world` pointers to the ranks' pads (uint32); slots
// [slot_base, slot_base + world) of every pad belong to this barrier stream.
// `epoch` must increase by one per call.  wait_cycles <= 0 selects the default.
int dsb_peer_barrier(unsigned int* const* pads_dev, int rank, int world, unsigned int epoch,
                     int slot_base, int* status, long long wait_cycles, cudaStream_t stream);

// One-shot sum all-reduce of n <= cap fp32 values over symmetric memory.
// `stage_dev`: DEVICE array of `world` pointers to the ranks' staging buffers
// (2 * cap floats each); pads / epoch / slot_base as for dsb_peer_barrier (use
// a slot range of its own: ceil(n / 4096) * world slots, at most 512).  All
// ranks get bit-identical sums.
int dsb_small_allreduce(float* const* stage_dev, unsigned int* const* pads_dev, int rank, int world,
                        unsigned int epoch, int slot_base, const float* in, float* out, int n,
                        int cap, int* status, long long wait_cycles, cudaStream_t stream);

// Partitioned optimizer step over peer memory.  `grads_dev` / `params_dev` are
// DEVICE arrays of `world` pointers to flat fp32 buffers of identical layout;
// this rank owns elements [lo, lo + n) (both multiples of 4).
//   dsb_zero_reduce:       g_own[i] = scale * sum_r grads[r][lo+i];  sq[0] += |g_own|^2
//   dsb_zero_adam_scatter: AdamW on the owned slice (m, v are slice-sized and
//                          local), new parameters stored to every rank.
// The caller orders them against the peers with dsb_peer_barrier.
int dsb_zero_reduce(const float* const* grads_dev, int world, long long lo, long long n, float scale,
                    float* g_own, float* sq, cudaStream_t stream);
int dsb_zero_adam_scatter(float* const* params_dev, int world, int rank, long long lo, long long n,
                          const float* g, float* m, float* v, const float* clip_scale, float lr,
                          float b1, float b2, float eps, float wd, float bc1, float bc2,
                          cudaStream_t stream);

#ifdef __cplusplus
}
#endif
