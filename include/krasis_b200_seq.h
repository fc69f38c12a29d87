/*
 * krasis_b200 — C ABI of the ragged-batch sequence operators (libkrasis_b200_seq.so).
 *
 * One step of a serving engine carries portions of several prompts next to single decoded tokens.  These entry points take
 * that step as a flat token axis [T] plus small int32 tables on the device:
 *   tokens[T], positions[T] (position of each token in its own sequence), seq_of[T] (index of its sequence in the step),
 *   cu[S + 1] (first row of each sequence's portion), slots[S] (recurrent-state slot of each sequence),
 *   pages[S][max_pages] (page list of each sequence in a paged cache with `page_size` tokens per page).
 * Conventions follow krasis_b200.h: device pointers owned by the caller, stream-ordered on `stream` (a cudaStream_t), no hidden
 * synchronisation, 0 = ok, text of the last error via kb2_seq_last_error().  `dt` arguments: 0 = float32, 1 = bfloat16.
 * There is no CPU fallback.
 */
#ifndef KRASIS_B200_SEQ_H
#define KRASIS_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define KB2SEQ_API __attribute__((visibility("default")))
#else
#define KB2SEQ_API
#endif

#define KB2SEQ_OK 0
#define KB2SEQ_ERR_VALUE 2
#define KB2SEQ_ERR_CUDA 3

KB2SEQ_API const char* kb2_seq_last_error(void);
KB2SEQ_API long long kb2_seq_total_launches(void);

/* x[t, :] = table[tokens[t], :] * scale, fp32 out */
KB2SEQ_API int kb2_seq_embed(const void* table, int dt, const int* tokens, float* x, int T, int W, float scale, void* stream);

/* C[b] = A[b] (M x K, row stride lda) * B[b]^T (N x K, row stride ldb), fp32 accumulation; b < batch with element strides sA, sB, sC */
KB2SEQ_API int kb2_seq_gemm(const void* A, int dtA, long long lda, const void* B, int dtB, long long ldb, void* C, int dtC,
                            long long ldc, int M, int N, int K, int batch, long long sA, long long sB, long long sC, void* stream);

/* x += norm(y) [+ x0]; h = layer_norm(x; wb, bb).  y_mode 1: layer norm (wa, ba), 2: RMS norm (wa).  y, x0 and h may be null. */
KB2SEQ_API int kb2_seq_residual_norm(float* x, const float* y, int y_mode, const float* wa, const float* ba, const float* x0,
                                     const float* wb, const float* bb, void* h, int dt_h, int T, int W, float eps, void* stream);

/* out[t, f] = gelu_tanh(in[t, f]) * in[t, F + f] */
KB2SEQ_API int kb2_seq_act_mul(const void* in, int dt_in, void* out, int dt_out, int T, int F, void* stream);

/* out[t, d] = gelu_tanh(g[t, d]) * table[tokens[t], col0 + d] */
KB2SEQ_API int kb2_seq_side_gate(const float* g, const void* table, int dt_table, long long table_ld, const int* tokens, int col0,
                                 int dim, int T, void* out, int dt_out, void* stream);

/* proj [T, ldp] = [q: H x (dn + dr) | latent: r | shared rotated key: dr].  Writes the RMS-normed latent and the rotated key to the
 * cache rows of the tokens' positions and rotates the queries' rotated parts in place.  freq[rot_dims / 2], amplitude amp. */
KB2SEQ_API int kb2_seq_latent_prep(float* proj, long long ldp, int T, int H, int dn, int dr, int r, const float* cw, float eps,
                                   const double* freq, int rot_dims, float amp, const int* positions, const int* seq_of,
                                   const int* pages, int max_pages, int page_size, void* ckv, void* kr, int dt_cache, void* stream);

/* out[t, h, :r] = sum_j softmax_j(...) latent_j over the keys with 0 <= pos - j < window; the denominator also holds exp(sinks[h]).
 * With cu != NULL the tokens of sequences whose portion has skip_from tokens or more are left out (another kernel serves them).
 * nsplit > 1 cuts every token's key range into nsplit pieces that run as separate blocks (steps of few tokens: decoding) and are merged
 * by a second kernel; part_acc [T][nsplit][H][r] and part_ml [T][nsplit][H][2] (fp32) hold the pieces. */
KB2SEQ_API int kb2_seq_latent_window_attn(const float* q_abs, const float* proj, long long ldp, int T, int H, int dn, int dr, int r,
                                          const void* ckv, const void* kr, int dt_cache, const int* positions, const int* seq_of,
                                          const int* pages, int max_pages, int page_size, const float* sinks, float scale, int window,
                                          float* out, const int* cu, int skip_from, int nsplit, float* part_acc, float* part_ml,
                                          void* stream);

/* out[t, c] = silu(causal conv over time of proj[:, c], K taps) for c < C; tail [slots][C][K - 1] is read, then advanced */
KB2SEQ_API int kb2_seq_conv_silu(const float* proj, long long ldp, int T, int S, int C, int K, const float* taps, float* tail,
                                 const int* seq_of, const int* cu, const int* slots, float* out, void* stream);

/* gated delta rule over each sequence's portion; state [slots][H][dk][dv] fp32 is read and written back.
 * scratch (fp32, 2 T Hk dk + 2 T H + T H dv + 4 elements, 16-byte aligned) selects the register-state kernels when dk is 32, 64 or
 * 128 and dv a multiple of 32; with scratch == NULL, or other sizes, one block per (sequence, head) keeps the state in shared memory. */
KB2SEQ_API int kb2_seq_delta_rule(const float* conv, int C, const float* proj, long long ldp, int g_off, int a_off, int b_off, int T,
                                  int S, int H, int Hk, int dk, int dv, const float* A_log, const float* dt_bias, const float* norm_w,
                                  float eps, float* state, const int* cu, const int* slots, float* scratch, void* out, int dt_out,
                                  void* stream);

#ifdef __cplusplus
}
#endif
#endif
