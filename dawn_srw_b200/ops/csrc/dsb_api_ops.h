// C ABI of the memory-bound kernels (see elementwise_kernels.cu).  Device
// pointers; asynchronous on `stream`; return 0 on a successful launch.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// y = (x - mean) * rstd * w + b, eps inside the sqrt; x fp32 [T,D], y bf16 [T,D].
int dsb_layernorm_fwd(const float* x, const float* w, const float* b, void* y_bf16, float* mean,
                      float* rstd, int T, int D, float eps, cudaStream_t stream);
// dx fp32 [T,D]; dw, db fp32 [D] are accumulated into (zero them first).
int dsb_layernorm_bwd(const void* dy_bf16, const float* x, const float* w, const float* mean,
                      const float* rstd, float* dx, float* dw, float* db, int T, int D,
                      cudaStream_t stream);
// Row statistics of fp32 logits [R, ld] with V valid columns: logsumexp, the
// label's logit (labels < 0 read column 0) and the arg-max.
int dsb_ce_fwd(const float* logits, long long ld, const long long* labels, int R, int V, float* lse,
               float* label_logit, long long* argmax, cudaStream_t stream);
// dl = scale[row] * (softmax - onehot) as bf16 [R, ldo] (columns V..ldo zeroed).
int dsb_ce_bwd(const float* logits, long long ld, const long long* labels, const float* lse,
               const float* scale, int R, int V, void* dl_bf16, long long ldo, cudaStream_t stream);
// AdamW step on one tensor; the global-norm clip factor is read from device memory.
int dsb_adamw(float* p, const float* g, float* m, float* v, long long n, const float* clip_scale,
              float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
              cudaStream_t stream);
// out[0] += sum(g^2)
int dsb_sqnorm_accumulate(const float* g, long long n, float* out, cudaStream_t stream);
// The same two operations over lists of tensors (host arrays of device pointers and element
// counts) in one launch per 160 tensors: a block takes a 64 K-element chunk of one tensor.
int dsb_adamw_multi(float* const* p, const float* const* g, float* const* m, float* const* v,
                    const long long* n, int count, const float* clip_scale, float lr, float b1,
                    float b2, float eps, float wd, float bc1, float bc2, cudaStream_t stream);
int dsb_sqnorm_multi(const float* const* g, const long long* n, int count, float* out,
                     cudaStream_t stream);

// out[t, :] = tok[ids[t], :] + pos[t % S, :]  (fp32, D % 4 == 0; ids clamped to [0, V)).
int dsb_embed_fwd(const long long* ids, const float* tok, const float* pos, float* out, int T, int S,
                  int D, int V, cudaStream_t stream);
// dtok[ids[t], :] += dy[t, :] (dtok zeroed by the caller); dpos[s, :] = sum_b dy[b*S+s, :].
int dsb_embed_bwd(const long long* ids, const float* dy, float* dtok, float* dpos, int B, int S,
                  int D, int V, cudaStream_t stream);
// total[0] += sum_{i != j} |sim_ij|; sgn (bf16 [m, ld_s]) = sign(sim) off the diagonal, 0 on it.
int dsb_offdiag_abs(const float* sim, long long ld, int m, void* sgn_bf16, long long ld_s,
                    float* total, cudaStream_t stream);
// dy_bf = bf16(dy * row_scale[t]); rowdot[t] = <dy[t], y[t]>   (dy, y fp32 [T, D], D % 4 == 0)
int dsb_route_bwd_prologue(const float* dy, const float* y, const float* row_scale,
                           void* dy_bf16, float* rowdot, int T, int D, cudaStream_t stream);

// y = res + dropout(x) (res may be null: y = dropout(x)); fp32, n % 4 == 0.  An element is kept
// (and scaled by 1 / (1 - p)) iff a hash of (seed, its index) is >= p * 2^32, so the gradient
// of x is the same call with res = null on the incoming gradient.
int dsb_dropout(const float* res, const float* x, float* y, long long n, unsigned long long seed,
                float p, cudaStream_t stream);

// Per-token score statistics from hg = h . (E^T E) (fp32 [N, r]) and bf16 h [N, ldh]:
//   mu = <h, esum> * inv_u,  var = <hg, h> * inv_u - mu^2,  sd = sqrt(max(var, 1e-12)) + 1e-8,
//   tau = mu + off * sd,  isd = 1 / sd;  hsum[r] += column sums of h (hsum may be null).
int dsb_score_stats_fwd(const float* hg, const void* h_bf16, long long ldh, const float* esum,
                        const float* off, float inv_u, int N, int r, float* tau, float* isd,
                        float* mu, float* sd, float* hsum, cudaStream_t stream);
// The same statistics for a handful of rows in one launch (generation), from fp32 h [T, R, r]
// (strides h_st, h_sr in elements, unit inner stride), off [T, R] (strides o_st, o_sr) and the
// fp32 Gram matrix.  Output rows are route-major: row ri * T + t; hb is bf16(h) [R * T, r].
int dsb_score_stats_rows(const float* h, long long h_st, long long h_sr, const float* off,
                         long long o_st, long long o_sr, const float* gram, const float* esum,
                         float inv_u, int T, int R, int r, float* tau, float* isd, void* hb_bf16,
                         cudaStream_t stream);
// Backward of the above.  d_tau, d_isd [N], d_hsum [r], d_hb (bf16 [N, r] cotangent of the
// bf16 copy of h) may be null.  Writes dh fp32 [N, r] (all terms summed), w = bf16(d_var * h)
// [N, ldw] (operand of dG = w^T h * inv_u), d_off [N]; accumulates d_esum [r] (zero it first).
int dsb_score_stats_bwd(const float* d_tau, const float* d_isd, const float* d_hsum,
                        const void* d_hb_bf16, const float* off, const float* mu, const float* sd,
                        const float* hg, const void* h_bf16, long long ldh, const float* esum,
                        float inv_u, int N, int r, float* dh, void* w_bf16, long long ldw,
                        float* d_off, float* d_esum, cudaStream_t stream);

// SRW pool op for a handful of token rows (decoding): one streaming pass over the pool.
// h [N, r], x [N, D] bf16 contiguous (row n of x belongs to row n of h), tau / isd [N];
// emb / read / write bf16 with row strides in elements (multiples of 8); unit_mask [U] or null.
// out[n, :] = (sum_u bf16(g * <x_n, r_u>) w_u) * scale / max(sum_u den_term, 1), fp32 [N, D];
// scale_ptr (device scalar) overrides scale when not null; den_out [N] may be null.
// part / den_part: scratch of dsb_srw_rows_blocks(N, D) * NR * D and * NR floats, NR = N rounded
// up to 1, 2 or 4.  N <= dsb_srw_rows_max(D) (4 up to d_model 1280, 2 up to 2048, else 0).
int dsb_srw_rows_max(int D);
int dsb_srw_rows_blocks(int N, int D);
struct DsbGate;
int dsb_srw_rows(const void* h, const void* x, const float* tau, const float* isd, const void* emb,
                 long long lde, const void* read, long long ldr, const void* write, long long ldw,
                 const float* unit_mask, int N, int U, int r, int D, const struct DsbGate* gate,
                 float scale, const float* scale_ptr, float* part, float* den_part, float* out,
                 float* den_out, cudaStream_t stream);

// One decoded token: k, v [B, H*dh] are appended to the fp32 caches [B, H, s_max, dh] at
// position pos[0] (device scalar), out [B, H*dh] = softmax(q K^T / sqrt(dh)) V over 0..pos.
int dsb_kv_decode_attention(const float* q, const float* k, const float* v, float* cache_k,
                            float* cache_v, const long long* pos, int B, int H, int dh, int s_max,
                            float* out, cudaStream_t stream);

// y[t, n] = <x_t, W_n> + bias[n] for N <= 4 rows (decoding): x bf16 [N, K] contiguous, W bf16
// [n_out, ldw], bias fp32 [n_out] or null, y fp32 [N, ldy]; K % 8 == 0, K <= 8192.
int dsb_gemv_rows(const void* x, const void* w, long long ldw, const float* bias, float* y,
                  long long ldy, int N, int n_out, int K, cudaStream_t stream);

// Causal self-attention (tcgen05 kernels).  q, k, v, out, d_out: bf16 [B, S, H*dh]
// (head h in columns [h*dh, (h+1)*dh)); dh a multiple of 16, at most 128.
// lse, delta: fp32 [B, H, S] (delta is scratch filled by the backward call).
// Dropout on the attention weights is a hash of (seed, batch*head, query, key):
// pass the forward call's p_drop and seed to the backward call.
int dsb_attention_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B,
                      int H, int S, int dh, float p_drop, unsigned long long seed, int* status,
                      cudaStream_t stream);
// dq: fp32 [B, S, H*dh], ZEROED by the caller (query tiles are reduce-added into
// it); dk, dv: bf16 [B, S, H*dh].
int dsb_attention_bwd(const void* q, const void* k, const void* v, const void* out,
                      const void* d_out, const float* lse, float* delta, float* dq, void* dk,
                      void* dv, int B, int H, int S, int dh, float p_drop,
                      unsigned long long seed, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
