/*
 * arattn.h — C ABI of libarattn.so: flash-attention forward/backward for NVIDIA B200
 * (sm_100a), a drop-in for the attention entry points of sergeytimoshin/autoresearch
 * (kernels/ops.mojo), meant to be bound from Mojo with external_call / DLHandle.
 *
 * Conventions shared by every entry point
 *   - all tensor pointers are DEVICE pointers owned by the caller; nothing is
 *     retained after the call returns;
 *   - tensors are [B, T, H, D] contiguous, element ((b*T + t)*H + h)*D + d
 *     (ops.mojo:270-275, 295, 309); LSE and D are [B, T, H] fp32 (ops.mojo:321, 457);
 *   - head_dim must be 128 and the number of K/V heads must equal the number of Q
 *     heads (ops.mojo:295, 309 index K/V with num_heads);
 *   - window_size W: W <= 0 or W >= T means full causal (k <= q); otherwise query q
 *     sees keys q-W .. q, i.e. W+1 keys (ops.mojo:290-293, 450-453);
 *   - scores are scaled by 1/sqrt(D) before the softmax (ops.mojo:276); LSE is the
 *     natural-log sum-exp of the SCALED scores (ops.mojo:320-321);
 *   - outputs are overwritten, never accumulated into (ops.mojo:318, 411, 479-480);
 *   - `stream` is a cudaStream_t passed as void*; NULL is the legacy default stream.
 *     Calls only enqueue work unless AR_FLAG_SYNC is given (fused family) — the
 *     mirrors behave like the reference's enqueue_function: asynchronous;
 *   - every function returns an ar_status; on error ar_last_error() holds a message
 *     for the calling thread.  The library never aborts, traps or falls back to a
 *     CPU path: if no sm_100 device/driver is present the call fails with AR_ERR_CUDA.
 *
 * Arithmetic: Q, K, V, dO (and P, dS) enter the tensor cores as bf16; all
 * accumulation, softmax statistics, LSE, D and the gradient outputs are fp32.
 */
#ifndef ARATTN_H_
#define ARATTN_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AR_API __attribute__((visibility("default")))

typedef int32_t ar_status;
enum {
  AR_OK = 0,
  AR_ERR_BAD_ARG = -1,     /* null pointer, non-positive size, misaligned pointer */
  AR_ERR_UNSUPPORTED = -2, /* head_dim != 128, rope table too short, unknown dtype */
  AR_ERR_CUDA = -3,        /* a CUDA runtime/driver call failed (message has the detail) */
  AR_ERR_WORKSPACE = -4,   /* caller workspace too small / size beyond a fixed maximum */
  AR_ERR_TIMEOUT = -5      /* a bounded device-side wait gave up (reported by ar_device_status) */
};

enum { AR_F32 = 0, AR_BF16 = 1 };

enum {
  AR_FLAG_SYNC = 1u << 0,        /* synchronise the stream and check the device status word */
  AR_FLAG_ROPE_PREPASS = 1u << 1, /* rope_mode 1 only: rotate Q/K in a separate pre-pass kernel
                                    into the workspace instead of inside the attention kernels */
  /* ar_attn_bwd only: leave out one of its three stages.  The reference launches them as
   * separate kernels (model.mojo:915-935); a caller that needs only some of the gradients, or
   * that already holds D in d_buf, can skip the rest.  Skipped outputs are not written and
   * their pointers may be NULL (d_o/o are still needed unless D is skipped and unused). */
  AR_FLAG_BWD_SKIP_D = 1u << 2,   /* d_buf already holds D = rowsum(O * dO) */
  AR_FLAG_BWD_SKIP_DQ = 1u << 3,  /* do not compute dq */
  AR_FLAG_BWD_SKIP_DKV = 1u << 4  /* do not compute dk, dv */
};

AR_API int32_t ar_version(void);
AR_API const char* ar_last_error(void);

/* Reads and clears the device-side status word of the current device.  Returns
 * AR_ERR_TIMEOUT if any kernel since the last call abandoned a bounded wait.
 * Synchronises the device. */
AR_API ar_status ar_device_status(void);

/* No counterpart in the reference: lets an integrator exercise the handling of AR_ERR_TIMEOUT
 * without a misbehaving GPU.  Enqueues a one-warp kernel whose bounded wait (on a barrier that
 * nothing arrives at) is cut to about a millisecond; it runs out, sets the status word the way an
 * abandoned wait inside an attention kernel does, and the kernel returns normally - nothing
 * faults, traps or hangs.  which = 0 sets the word ar_device_status() reads, which = 1 the word
 * ar_noalloc_status() reads.  Until that word is read (and thereby cleared) every attention
 * kernel launched on the device returns at once without touching its outputs. */
AR_API ar_status ar_selftest_wait_timeout(int32_t which, void* stream);

/* ------------------------------------------------------------------------------------
 * (i) Exact mirrors of kernels/ops.mojo: fp32 tensors, same argument order, `Int`
 *     dims as int64_t, plus a trailing stream.  The attention mirrors stage their
 *     fp32 operands as bf16 in a library-managed device workspace (grown on demand
 *     with cudaMalloc, cached per device) and run the tensor-core kernels.
 * ------------------------------------------------------------------------------------ */

/* replaces rope_fwd (ops.mojo:209-217; launched at model.mojo:668-677).
 * out may alias in.  cos/sin: [rows, head_dim/2] fp32 (model.mojo:57-81).
 * The reference indexes the table with token = b*T + t (ops.mojo:227, 233), which
 * leaves the table for B*T > rows; seq_len > 0 uses pos = token % seq_len instead
 * (identical wherever the reference is in bounds for B == 1); seq_len <= 0 keeps
 * the literal index and requires the table to have num_tokens rows. */
AR_API ar_status ar_rope_fwd(float* out, const float* in, const float* cos_buf,
                             const float* sin_buf, int64_t num_tokens, int64_t num_heads,
                             int64_t head_dim, int64_t seq_len, void* stream);

/* replaces rope_bwd (ops.mojo:1091-1099; launched at model.mojo:955-964). */
AR_API ar_status ar_rope_bwd(float* grad_in, const float* grad_out, const float* cos_buf,
                             const float* sin_buf, int64_t num_tokens, int64_t num_heads,
                             int64_t head_dim, int64_t seq_len, void* stream);

/* The step before attention in one launch: replaces the two rope_fwd launches and the two per-head
 * rmsnorm_fwd launches on q and k (model.mojo:668-687; ops.mojo:209-217, 61-67) and writes the
 * bf16 operands the fused family reads, so that the trainer's fp32 q, k, v (outputs of its QKV
 * projections, model.mojo:643-645; in_dtype AR_F32, or AR_BF16 for a caller whose projections
 * already produce bf16) reach the tensor-core kernels with one pass over memory:
 *     q_rot = bf16( rope(q) / sqrt(mean(rope(q)^2) + eps) )   per (token, head) row, same for k
 *     v_bf16 = bf16(v)                                       (v, v_bf16 may both be NULL)
 * q_rot, k_rot, v_bf16: bf16 [num_tokens, num_heads, 128].  rms_q, rms_k (optional, fp32
 * [num_tokens, num_heads]) receive the row's sqrt(mean + eps), rmsnorm_fwd's rms_out.  eps is the
 * reference's 1e-5 (ops.mojo:97).  Position index as in ar_rope_fwd (seq_len).  Afterwards call
 * ar_attn_fwd with rope_mode 0 on (q_rot, k_rot, v_bf16); for the backward pass hand the same
 * q_rot, k_rot to ar_attn_bwd with rope_mode 1, which then returns dq, dk with rope_bwd applied -
 * what the reference computes, whose backward passes gradients straight through this
 * normalisation (model.mojo:937). */
AR_API ar_status ar_qk_norm_rope_cast(void* q_rot, void* k_rot, void* v_bf16, float* rms_q,
                                      float* rms_k, const void* q, const void* k, const void* v,
                                      int32_t in_dtype, const float* cos_buf, const float* sin_buf,
                                      int64_t num_tokens, int64_t num_heads, int64_t head_dim,
                                      int64_t seq_len, float eps, void* stream);

/* replaces flash_attn_fwd (ops.mojo:244-255; launched at model.mojo:694-699).
 * q, k are the already-rotated tensors. */
AR_API ar_status ar_flash_attn_fwd(float* output, float* lse_out, const float* q,
                                   const float* k, const float* v, int64_t B, int64_t T,
                                   int64_t num_heads, int64_t head_dim, int64_t window_size,
                                   void* stream);

/* No counterpart in the reference: ar_flash_attn_fwd for callers that must not allocate.
 * Some hosts of this library cannot call cudaMalloc when attention runs: code inside a region
 * where device allocation is forbidden or would synchronise the device (a latency-critical
 * serving loop, a section holding an allocator lock, a process whose memory budget is fixed
 * up front).  This entry point computes exactly what ar_flash_attn_fwd computes, but the bf16
 * staging copies of q, k, v live in a fixed array inside the library image instead of the
 * grown-on-demand workspace, and its device status word is a library symbol too, so the call
 * performs no cudaMalloc, no cudaFree and no other allocating call.
 *   - Limit: B * T * num_heads <= AR_NOALLOC_MAX_ROWS (16384 rows of 128, i.e. 4 MiB per staged
 *     tensor, 12 MiB in total, resident on every GPU that loads the library until exit).
 *     Larger problems are refused with AR_ERR_WORKSPACE and a message naming the limit.
 *   - The first call on a device looks the array's device address up (one-time set-up, with
 *     that device current); make that first call before any stream capture begins.
 *   - Every call on a device shares the one array, which keeps the previous call's contents
 *     (each call overwrites what it reads, nothing needs clearing).  Calls that overlap on
 *     the GPU (different streams, or threads) race on it: keep them ordered on one stream.
 *   - Its kernels record an abandoned device-side wait in the library's own status symbol,
 *     which ar_device_status() (an allocating call on first use) does not read: read it with
 *     ar_noalloc_status().  While that word is set, later allocation-free calls on the device do
 *     no work (their kernels return at once), so check it wherever the results matter. */
#define AR_NOALLOC_MAX_ROWS 16384
AR_API ar_status ar_flash_attn_fwd_noalloc(float* output, float* lse_out, const float* q,
                                           const float* k, const float* v, int64_t B, int64_t T,
                                           int64_t num_heads, int64_t head_dim,
                                           int64_t window_size, void* stream);

/* No counterpart in the reference: the ar_device_status() of the allocation-free entry point.
 * Waits for the current device, reads the status word that ar_flash_attn_fwd_noalloc's kernels
 * write and clears it when set; returns AR_ERR_TIMEOUT if a bounded device-side wait was abandoned
 * since the last call, AR_OK otherwise.  Like the entry point it serves it allocates nothing (the
 * word is a symbol of the library image; the copies go through cudaMemcpy). */
AR_API ar_status ar_noalloc_status(void);

/* replaces flash_attn_bwd_precompute_d (ops.mojo:329-337; model.mojo:915-919). */
AR_API ar_status ar_flash_attn_bwd_precompute_d(float* d_out, const float* output,
                                                const float* grad_output, int64_t B, int64_t T,
                                                int64_t num_heads, int64_t head_dim,
                                                void* stream);

/* replaces flash_attn_bwd_dq (ops.mojo:349-362; model.mojo:921-927). */
AR_API ar_status ar_flash_attn_bwd_dq(float* grad_q, const float* q, const float* k,
                                      const float* v, const float* grad_output,
                                      const float* lse, const float* d_buf, int64_t B,
                                      int64_t T, int64_t num_heads, int64_t head_dim,
                                      int64_t window_size, void* stream);

/* replaces flash_attn_bwd_dkv (ops.mojo:414-428; model.mojo:929-935). */
AR_API ar_status ar_flash_attn_bwd_dkv(float* grad_k, float* grad_v, const float* q,
                                       const float* k, const float* v,
                                       const float* grad_output, const float* lse,
                                       const float* d_buf, int64_t B, int64_t T,
                                       int64_t num_heads, int64_t head_dim,
                                       int64_t window_size, void* stream);

/* ------------------------------------------------------------------------------------
 * The projections either side of attention (QKV before it, c_proj after it, and any other linear
 * layer of the model) on the tensor cores: bf16 operands, fp32 accumulation.  Same argument order
 * as the reference's matmuls, plus element types: in_dtype (AR_BF16, or AR_F32 = staged as bf16 in
 * the library's scratch) for both inputs, out_dtype for the result.  All matrices row-major and
 * contiguous; N and K multiples of 8, the result's row length a multiple of 32; M arbitrary.
 * What the reference's docstrings state is computed (its kernels write only a quarter of each
 * output tile, ops.mojo:134-143).  With AR_F32 operands the output may be one of the inputs
 * (they are staged first: the in-place call at model.mojo:906 works as written); with AR_BF16
 * operands an aliased output is refused.  The scratch of the AR_F32 form is the same
 * per-device block the mirrors under (i) use: one thread and one stream per device at a time.
 * ------------------------------------------------------------------------------------ */

/* replaces linear_fwd (ops.mojo:110-117; launch_linear, model.mojo:162-174):
 * output[M,N] = input[M,K] weight[N,K]^T. */
AR_API ar_status ar_linear_fwd(void* output, const void* input, const void* weight, int64_t M,
                               int64_t N, int64_t K, int32_t in_dtype, int32_t out_dtype,
                               void* stream);

/* replaces linear_bwd_dx (ops.mojo:870-878; launch_linear_bwd_dx, model.mojo:177-189):
 * grad_input[M,K] = grad_output[M,N] weight[N,K]. */
AR_API ar_status ar_linear_bwd_dx(void* grad_input, const void* grad_output, const void* weight,
                                  int64_t M, int64_t N, int64_t K, int32_t in_dtype,
                                  int32_t out_dtype, void* stream);

/* replaces linear_bwd_dw (ops.mojo:953-961; launch_linear_bwd_dw, model.mojo:192-204):
 * grad_weight[N,K] += grad_output[M,N]^T input[M,K]; fp32, ACCUMULATED into grad_weight like the
 * reference's (zero it first for a plain product).  The sum over M is split over the SMs and
 * added with fp32 reductions, so its rounding can differ from run to run in the last bits. */
AR_API ar_status ar_linear_bwd_dw(float* grad_weight, const void* grad_output, const void* input,
                                  int64_t M, int64_t N, int64_t K, int32_t in_dtype, void* stream);

/* ------------------------------------------------------------------------------------
 * (ii) Fused family: one call for the forward launches of model.mojo:668-677 + 694-699
 *      and one for the backward launches of model.mojo:915-935 + 955-964.
 * ------------------------------------------------------------------------------------ */
typedef struct ar_attn_params {
  uint32_t struct_size; /* sizeof(ar_attn_params), checked */
  uint32_t flags;       /* AR_FLAG_* */
  int32_t io_dtype;     /* AR_BF16 or AR_F32: element type of q, k, v, o, d_o */
  int32_t grad_dtype;   /* AR_F32 or AR_BF16: element type of dq, dk, dv */
  int64_t B, T, H, D;   /* D must be 128 */
  int64_t window;       /* window_size as above (config.mojo:49-55 gives the per-layer value) */
  int32_t rope_mode;    /* 0: q, k already rotated (what ops.mojo's attention kernels get);
                           1: q, k are un-rotated; rotate with position t on the way in and
                              return dq, dk with respect to the un-rotated tensors, i.e.
                              rope_bwd already applied (model.mojo:955-964) */
  int32_t reserved;
  const float* cos_buf; /* [rope_rows, D/2] fp32, needed when rope_mode == 1 */
  const float* sin_buf;
  int64_t rope_rows;    /* must be >= T */
  void* workspace;      /* optional caller scratch; NULL = library-managed */
  uint64_t workspace_bytes;
  void* stream;
  /* Optional, rope_mode == 1 only: bf16 [B,T,H,D] buffers for the ROTATED q and k, the
   * counterpart of the reference's saved_q / saved_k (model.mojo:689-690).  ar_attn_fwd rotates
   * q, k into them in a pre-pass and runs attention on them; ar_attn_bwd given the same buffers
   * reads them instead of rotating q, k again (q, k themselves are then not read).  Either both
   * or neither; NULL keeps the self-contained behaviour. */
  void* q_rot;
  void* k_rot;
  /* Optional strides, in ELEMENTS, of q, k, v, o, d_o, dq, dk, dv, q_rot and k_rot (all the same);
   * all three zero means contiguous [B,T,H,D].  They let a caller hand over a head range cut out
   * of a wider [B,T,H_all,D] tensor - e.g. one rank's share when (batch, head) units are split
   * inside a batch - without copying it: stride_h must be D (the heads of a token adjacent),
   * stride_t = H_all * D, stride_b = T * stride_t (or more; both multiples of D).  lse and d_buf
   * are then the matching cut of [B,T,H_all]: element strides stride_b / D, stride_t / D, 1. */
  int64_t stride_b, stride_t, stride_h;
} ar_attn_params;

/* Bytes of scratch the given call needs (pass 0 = forward, 1 = backward). */
AR_API uint64_t ar_attn_workspace_bytes(const ar_attn_params* p, int32_t pass);

/* o: [B,T,H,D] io_dtype; lse: [B,T,H] fp32. */
AR_API ar_status ar_attn_fwd(const ar_attn_params* p, const void* q, const void* k,
                             const void* v, void* o, float* lse);

/* d_buf: [B,T,H] fp32 scratch owned by the caller (model.mojo:447, 511), overwritten
 * with D = rowsum(O * dO).  dq, dk, dv: [B,T,H,D] grad_dtype. */
AR_API ar_status ar_attn_bwd(const ar_attn_params* p, const void* q, const void* k,
                             const void* v, const void* o, const void* d_o, const float* lse,
                             float* d_buf, void* dq, void* dk, void* dv);

#ifdef __cplusplus
}
#endif
#endif /* ARATTN_H_ */
