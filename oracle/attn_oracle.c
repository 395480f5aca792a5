/*
 * CPU oracle for the attention forward/backward path of sergeytimoshin/autoresearch.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of the
 * reference's GPU kernels (kernels/ops.mojo) so that the CUDA library can be
 * checked against it.  It is never linked into, imported by, or called from the
 * shipped library; only the test-suite, the smoke check and the CPU-baseline leg
 * of the benchmark may use it.
 *
 * PARITY UNPINNED: the reference has no CPU implementation of this path, needs a
 * Mojo toolchain that is not available, and its own tests hold no known-answer
 * vectors for attention or RoPE (test_kernels.mojo:280-285 covers other kernels).
 * The restatement is therefore cross-checked against an independent fp64 dense
 * softmax and against autograd instead of against reference outputs.
 *
 * Every function exists in a "literal" form (one loop iteration per reference GPU
 * thread, identical operation order) and, for the redundant backward kernels, a
 * "row" form that computes each score once and then performs the same additions
 * in the same order.  With -ffp-contract=off both forms give bit-identical
 * results.  All arithmetic is IEEE fp32, as in the reference.
 *
 * Layout (ops.mojo:270-275, 295, 309): tensors are [B, T, H, D] contiguous,
 * element ((b*T + t)*H + h)*D + d;  LSE and D are [B, T, H].
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

ORACLE_API int oracle_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* Launchers such as torchrun export OMP_NUM_THREADS=1; the CPU-baseline legs call this to use
 * all host cores again.  n <= 0 leaves the setting alone. */
ORACLE_API void oracle_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

/* model.mojo:57-81 — angle = t / base^(2d/D) in fp64, cos/sin rounded to fp32.
 * Table shape [rows, D/2]. */
ORACLE_API void oracle_rope_table(float* cos_out, float* sin_out, int64_t rows,
                                  int64_t head_dim, double base) {
  int64_t half = head_dim / 2;
  for (int64_t t = 0; t < rows; ++t) {
    for (int64_t d = 0; d < half; ++d) {
      double freq = (double)t / pow(base, (double)(2 * d) / (double)head_dim);
      cos_out[t * half + d] = (float)cos(freq);
      sin_out[t * half + d] = (float)sin(freq);
    }
  }
}

/* ops.mojo:209-238.  The reference indexes the table with token_idx = b*T + t
 * (ops.mojo:227,233); seq_len > 0 selects pos = token_idx % seq_len, seq_len <= 0
 * reproduces the reference index literally.  In-place (out == in) is allowed. */
ORACLE_API void oracle_rope_fwd(float* out, const float* in, const float* cos_buf,
                                const float* sin_buf, int64_t num_tokens,
                                int64_t num_heads, int64_t head_dim, int64_t seq_len) {
  int64_t half = head_dim / 2;
  int64_t total = num_tokens * num_heads * half;
#pragma omp parallel for schedule(static)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t token_head = tid / half;
    int64_t d = tid % half;
    int64_t token = token_head / num_heads;
    int64_t pos = seq_len > 0 ? token % seq_len : token;
    int64_t base = token_head * head_dim;
    float x1 = in[base + d];
    float x2 = in[base + half + d];
    float c = cos_buf[pos * half + d];
    float s = sin_buf[pos * half + d];
    out[base + d] = x1 * c + x2 * s;
    out[base + half + d] = x1 * (-s) + x2 * c;
  }
}

/* ops.mojo:1091-1120 — transpose of the forward rotation. */
ORACLE_API void oracle_rope_bwd(float* grad_in, const float* grad_out, const float* cos_buf,
                                const float* sin_buf, int64_t num_tokens,
                                int64_t num_heads, int64_t head_dim, int64_t seq_len) {
  int64_t half = head_dim / 2;
  int64_t total = num_tokens * num_heads * half;
#pragma omp parallel for schedule(static)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t token_head = tid / half;
    int64_t d = tid % half;
    int64_t token = token_head / num_heads;
    int64_t pos = seq_len > 0 ? token % seq_len : token;
    int64_t base = token_head * head_dim;
    float dy1 = grad_out[base + d];
    float dy2 = grad_out[base + half + d];
    float c = cos_buf[pos * half + d];
    float s = sin_buf[pos * half + d];
    grad_in[base + d] = dy1 * c - dy2 * s;
    grad_in[base + half + d] = dy1 * s + dy2 * c;
  }
}

/* ops.mojo:244-323.  One iteration per (b, qp, h) reference thread; keys ascending;
 * causal break (:290), window skip (:292, admits keys qp-W..qp), scale 1/sqrt(D)
 * (:276), per-key online softmax with a normalised accumulator (:302-314),
 * LSE = m + log(l) (:320-323).  head_dim > 128 is a silent no-op (:267). */
ORACLE_API void oracle_flash_attn_fwd(float* output, float* lse_out, const float* q,
                                      const float* k, const float* v, int64_t B, int64_t T,
                                      int64_t num_heads, int64_t head_dim,
                                      int64_t window_size) {
  if (head_dim > 128) return;
  int64_t total = B * T * num_heads;
  float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t bt = tid / num_heads;
    int64_t h = tid % num_heads;
    int64_t b = bt / T;
    int64_t qp = bt % T;
    int64_t q_base = tid * head_dim;
    float m = -FLT_MAX; /* Float32.MIN: the lowest finite float */
    float l = 0.0f;
    float o_acc[128];
    for (int64_t d = 0; d < head_dim; ++d) o_acc[d] = 0.0f;
    for (int64_t kp = 0; kp < T; ++kp) {
      if (kp > qp) break;
      if (window_size > 0 && kp < qp - window_size) continue;
      int64_t k_base = (b * T * num_heads + kp * num_heads + h) * head_dim;
      float score = 0.0f;
      for (int64_t d = 0; d < head_dim; ++d) score += q[q_base + d] * k[k_base + d];
      score *= scale;
      float m_new = score > m ? score : m;
      float exp_old = expf(m - m_new);
      float exp_new = expf(score - m_new);
      float l_new = l * exp_old + exp_new;
      float alpha = (l * exp_old) / l_new;
      float beta = exp_new / l_new;
      for (int64_t d = 0; d < head_dim; ++d)
        o_acc[d] = alpha * o_acc[d] + beta * v[k_base + d];
      m = m_new;
      l = l_new;
    }
    for (int64_t d = 0; d < head_dim; ++d) output[q_base + d] = o_acc[d];
    lse_out[tid] = l > 0.0f ? m + logf(l) : -FLT_MAX;
  }
}

/* ops.mojo:329-346 — D[bth] = sum_d O*dO, d ascending. */
ORACLE_API void oracle_flash_attn_bwd_precompute_d(float* d_out, const float* output,
                                                   const float* grad_output, int64_t B,
                                                   int64_t T, int64_t num_heads,
                                                   int64_t head_dim) {
  int64_t total = B * T * num_heads;
#pragma omp parallel for schedule(static)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t base = tid * head_dim;
    float acc = 0.0f;
    for (int64_t d = 0; d < head_dim; ++d) acc += output[base + d] * grad_output[base + d];
    d_out[tid] = acc;
  }
}

/* ops.mojo:349-411, literal: one iteration per OUTPUT ELEMENT (b, qp, h, d); the
 * score and dA dot products are recomputed by each of the head_dim elements of a
 * row, exactly as the reference does. */
ORACLE_API void oracle_flash_attn_bwd_dq_literal(float* grad_q, const float* q, const float* k,
                                                 const float* v, const float* grad_output,
                                                 const float* lse, const float* d_buf,
                                                 int64_t B, int64_t T, int64_t num_heads,
                                                 int64_t head_dim, int64_t window_size) {
  int64_t total = B * T * num_heads * head_dim;
  float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 512)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t bth = tid / head_dim;
    int64_t d = tid % head_dim;
    int64_t bt = bth / num_heads;
    int64_t h = bth % num_heads;
    int64_t b = bt / T;
    int64_t qp = bt % T;
    int64_t q_base = bth * head_dim;
    float lse_val = lse[bth];
    float d_val = d_buf[bth];
    float acc = 0.0f;
    for (int64_t kp = 0; kp < T; ++kp) {
      if (kp > qp) break;
      if (window_size > 0 && kp < qp - window_size) continue;
      int64_t k_base = (b * T * num_heads + kp * num_heads + h) * head_dim;
      float score = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) score += q[q_base + dd] * k[k_base + dd];
      score *= scale;
      float a_val = expf(score - lse_val);
      float da = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) da += grad_output[q_base + dd] * v[k_base + dd];
      float ds = a_val * (da - d_val);
      acc += ds * k[k_base + d];
    }
    grad_q[tid] = acc * scale;
  }
}

/* Same sums in the same order as the literal form, with the per-(q,k) scalars
 * computed once per row instead of once per output element. */
ORACLE_API void oracle_flash_attn_bwd_dq(float* grad_q, const float* q, const float* k,
                                         const float* v, const float* grad_output,
                                         const float* lse, const float* d_buf, int64_t B,
                                         int64_t T, int64_t num_heads, int64_t head_dim,
                                         int64_t window_size) {
  if (head_dim > 128) return;
  int64_t total = B * T * num_heads;
  float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t bth = 0; bth < total; ++bth) {
    int64_t bt = bth / num_heads;
    int64_t h = bth % num_heads;
    int64_t b = bt / T;
    int64_t qp = bt % T;
    int64_t q_base = bth * head_dim;
    float lse_val = lse[bth];
    float d_val = d_buf[bth];
    float acc[128];
    for (int64_t d = 0; d < head_dim; ++d) acc[d] = 0.0f;
    for (int64_t kp = 0; kp < T; ++kp) {
      if (kp > qp) break;
      if (window_size > 0 && kp < qp - window_size) continue;
      int64_t k_base = (b * T * num_heads + kp * num_heads + h) * head_dim;
      float score = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) score += q[q_base + dd] * k[k_base + dd];
      score *= scale;
      float a_val = expf(score - lse_val);
      float da = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) da += grad_output[q_base + dd] * v[k_base + dd];
      float ds = a_val * (da - d_val);
      for (int64_t d = 0; d < head_dim; ++d) acc[d] += ds * k[k_base + d];
    }
    for (int64_t d = 0; d < head_dim; ++d) grad_q[q_base + d] = acc[d] * scale;
  }
}

/* ops.mojo:414-480, literal: one iteration per output element (b, kp, h, d);
 * queries qp in [kp, min(T, kp+W+1)) ascending (:450-455). */
ORACLE_API void oracle_flash_attn_bwd_dkv_literal(float* grad_k, float* grad_v, const float* q,
                                                  const float* k, const float* v,
                                                  const float* grad_output, const float* lse,
                                                  const float* d_buf, int64_t B, int64_t T,
                                                  int64_t num_heads, int64_t head_dim,
                                                  int64_t window_size) {
  int64_t total = B * T * num_heads * head_dim;
  float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 512)
  for (int64_t tid = 0; tid < total; ++tid) {
    int64_t bth = tid / head_dim;
    int64_t d = tid % head_dim;
    int64_t bt = bth / num_heads;
    int64_t h = bth % num_heads;
    int64_t b = bt / T;
    int64_t kp = bt % T;
    int64_t k_base = bth * head_dim;
    float dk_acc = 0.0f, dv_acc = 0.0f;
    int64_t qp_end = T;
    if (window_size > 0 && kp + window_size < T) qp_end = kp + window_size + 1;
    for (int64_t qp = kp; qp < qp_end; ++qp) {
      int64_t row = b * T * num_heads + qp * num_heads + h;
      int64_t q_base = row * head_dim;
      float lse_val = lse[row];
      float d_val = d_buf[row];
      float score = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) score += q[q_base + dd] * k[k_base + dd];
      score *= scale;
      float a_val = expf(score - lse_val);
      dv_acc += a_val * grad_output[q_base + d];
      float da = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) da += grad_output[q_base + dd] * v[k_base + dd];
      float ds = a_val * (da - d_val);
      dk_acc += ds * q[q_base + d];
    }
    grad_k[tid] = dk_acc * scale;
    grad_v[tid] = dv_acc;
  }
}

/* Row form of the above: same additions, same order, scalars computed once. */
ORACLE_API void oracle_flash_attn_bwd_dkv(float* grad_k, float* grad_v, const float* q,
                                          const float* k, const float* v,
                                          const float* grad_output, const float* lse,
                                          const float* d_buf, int64_t B, int64_t T,
                                          int64_t num_heads, int64_t head_dim,
                                          int64_t window_size) {
  if (head_dim > 128) return;
  int64_t total = B * T * num_heads;
  float scale = 1.0f / sqrtf((float)head_dim);
#pragma omp parallel for schedule(dynamic, 16)
  for (int64_t bth = 0; bth < total; ++bth) {
    int64_t bt = bth / num_heads;
    int64_t h = bth % num_heads;
    int64_t b = bt / T;
    int64_t kp = bt % T;
    int64_t k_base = bth * head_dim;
    float dk_acc[128], dv_acc[128];
    for (int64_t d = 0; d < head_dim; ++d) dk_acc[d] = dv_acc[d] = 0.0f;
    int64_t qp_end = T;
    if (window_size > 0 && kp + window_size < T) qp_end = kp + window_size + 1;
    for (int64_t qp = kp; qp < qp_end; ++qp) {
      int64_t row = b * T * num_heads + qp * num_heads + h;
      int64_t q_base = row * head_dim;
      float lse_val = lse[row];
      float d_val = d_buf[row];
      float score = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) score += q[q_base + dd] * k[k_base + dd];
      score *= scale;
      float a_val = expf(score - lse_val);
      for (int64_t d = 0; d < head_dim; ++d) dv_acc[d] += a_val * grad_output[q_base + d];
      float da = 0.0f;
      for (int64_t dd = 0; dd < head_dim; ++dd) da += grad_output[q_base + dd] * v[k_base + dd];
      float ds = a_val * (da - d_val);
      for (int64_t d = 0; d < head_dim; ++d) dk_acc[d] += ds * q[q_base + d];
    }
    for (int64_t d = 0; d < head_dim; ++d) {
      grad_k[k_base + d] = dk_acc[d] * scale;
      grad_v[k_base + d] = dv_acc[d];
    }
  }
}

/* Whole-path composition in the order model.mojo launches it:
 * forward  (model.mojo:668-677, 694-699): rope_fwd(q), rope_fwd(k) in place, flash_attn_fwd;
 * backward (model.mojo:915-935, 955-964): precompute_d, bwd_dq, bwd_dkv, then
 * rope_bwd in place on grad_q and grad_k.
 * q_rot/k_rot receive the rotated Q/K (what the reference saves for backward).
 * The gradients returned are with respect to the PRE-rotation q and k.  Row forms
 * are used for the backward.  rope position = t (token % T). */
ORACLE_API void oracle_attention_path(float* o, float* lse, float* d_buf, float* dq, float* dk,
                                      float* dv, float* q_rot, float* k_rot, const float* q,
                                      const float* k, const float* v, const float* d_o,
                                      const float* cos_buf, const float* sin_buf, int64_t B,
                                      int64_t T, int64_t H, int64_t D, int64_t window_size,
                                      int32_t apply_rope, int32_t do_backward) {
  int64_t n = B * T * H * D;
  if (apply_rope) {
    oracle_rope_fwd(q_rot, q, cos_buf, sin_buf, B * T, H, D, T);
    oracle_rope_fwd(k_rot, k, cos_buf, sin_buf, B * T, H, D, T);
  } else {
    memcpy(q_rot, q, (size_t)n * sizeof(float));
    memcpy(k_rot, k, (size_t)n * sizeof(float));
  }
  oracle_flash_attn_fwd(o, lse, q_rot, k_rot, v, B, T, H, D, window_size);
  if (!do_backward) return;
  oracle_flash_attn_bwd_precompute_d(d_buf, o, d_o, B, T, H, D);
  oracle_flash_attn_bwd_dq(dq, q_rot, k_rot, v, d_o, lse, d_buf, B, T, H, D, window_size);
  oracle_flash_attn_bwd_dkv(dk, dv, q_rot, k_rot, v, d_o, lse, d_buf, B, T, H, D, window_size);
  if (apply_rope) {
    oracle_rope_bwd(dq, dq, cos_buf, sin_buf, B * T, H, D, T);
    oracle_rope_bwd(dk, dk, cos_buf, sin_buf, B * T, H, D, T);
  }
}

/* ops.mojo:61-104 (rmsnorm_fwd) - y = x / sqrt(mean(x^2) + 1e-5), one block of 256 threads per row.
 * The sum of squares is formed exactly as the kernel forms it: thread t adds the elements t,
 * t + 256, ... in order (ops.mojo:77-80); the 256 partial sums are folded in shared memory,
 * upper half onto lower half, down to 32 (ops.mojo:84-89); the last 32 meet in warp.sum, taken
 * here as the usual butterfly (offsets 16, 8, 4, 2, 1).  PINNED by the reference's own known-answer
 * test for this kernel (test_kernels.mojo:140-181: rms = [2.7386, 2.5], out[0,0] = 0.3651,
 * out[1,3] = 2.0, each within 0.01), checked in tests/test_oracle.py.  In place (out == in) allowed. */
ORACLE_API void oracle_rmsnorm_fwd(float* out, float* rms_out, const float* in, int64_t num_rows,
                                   int64_t dim) {
#pragma omp parallel for schedule(static)
  for (int64_t row = 0; row < num_rows; ++row) {
    const float* x = in + row * dim;
    float part[256];
    for (int t = 0; t < 256; ++t) {
      float ss = 0.0f;
      for (int64_t i = t; i < dim; i += 256) ss += x[i] * x[i];
      part[t] = ss;
    }
    for (int active = 128; active >= 32; active >>= 1)
      for (int t = 0; t < active; ++t) part[t] += part[t + active];
    for (int off = 16; off >= 1; off >>= 1)
      for (int t = 0; t < off; ++t) part[t] += part[t + off];
    float mean_sq = part[0] / (float)dim;
    float rms = sqrtf(mean_sq + 1e-5f);
    if (rms_out) rms_out[row] = rms;
    for (int64_t i = 0; i < dim; ++i) out[row * dim + i] = x[i] / rms;
  }
}

/* The step before attention, in model.mojo's launch order (model.mojo:668-687): rope_fwd in place on
 * q and k (position = token % seq_len), then rmsnorm_fwd per (token, head) row of head_dim. */
ORACLE_API void oracle_qk_rope_norm(float* q_out, float* k_out, float* rms_q, float* rms_k, const float* q,
                                    const float* k, const float* cos_buf, const float* sin_buf,
                                    int64_t num_tokens, int64_t num_heads, int64_t head_dim, int64_t seq_len) {
  oracle_rope_fwd(q_out, q, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len);
  oracle_rope_fwd(k_out, k, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len);
  oracle_rmsnorm_fwd(q_out, rms_q, q_out, num_tokens * num_heads, head_dim);
  oracle_rmsnorm_fwd(k_out, rms_k, k_out, num_tokens * num_heads, head_dim);
}

/* ops.mojo:110-117 (linear_fwd): Y[m, n] = sum_k X[m, k] * W[n, k], k ascending, fp32.  This restates
 * what the kernel's docstring and its accumulation loop state (ops.mojo:118, 170-186); the kernel's
 * thread-to-output mapping covers only rows / columns 0..3 of every 8 (ops.mojo:134-143, 188-203),
 * which is not a convention a replacement could follow. */
ORACLE_API void oracle_linear_fwd(float* y, const float* x, const float* w, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m)
    for (int64_t n = 0; n < N; ++n) {
      float acc = 0.0f;
      for (int64_t k = 0; k < K; ++k) acc += x[m * K + k] * w[n * K + k];
      y[m * N + n] = acc;
    }
}

/* ops.mojo:870-878 (linear_bwd_dx): dX[m, k] = sum_n dY[m, n] * W[n, k], n ascending for every
 * element (the loops are ordered for locality; each element's own sum order is unchanged). */
ORACLE_API void oracle_linear_bwd_dx(float* dx, const float* dy, const float* w, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel for schedule(static)
  for (int64_t m = 0; m < M; ++m) {
    float* acc = dx + m * K;
    for (int64_t k = 0; k < K; ++k) acc[k] = 0.0f;
    for (int64_t n = 0; n < N; ++n) {
      const float g = dy[m * N + n];
      for (int64_t k = 0; k < K; ++k) acc[k] += g * w[n * K + k];
    }
  }
}

/* ops.mojo:953-961 (linear_bwd_dw): dW[n, k] += sum_m dY[m, n] * X[m, k], m ascending for every
 * element, the finished sum added into dW once (ops.mojo:1018-1033). */
ORACLE_API void oracle_linear_bwd_dw(float* dw, const float* dy, const float* x, int64_t M, int64_t N, int64_t K) {
#pragma omp parallel
  {
    float* acc = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
    for (int64_t n = 0; n < N; ++n) {
      for (int64_t k = 0; k < K; ++k) acc[k] = 0.0f;
      for (int64_t m = 0; m < M; ++m) {
        const float g = dy[m * N + n];
        for (int64_t k = 0; k < K; ++k) acc[k] += g * x[m * K + k];
      }
      for (int64_t k = 0; k < K; ++k) dw[n * K + k] += acc[k];
    }
    free(acc);
  }
}
