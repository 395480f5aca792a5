/*
 * A C caller of libarattn.so that does exactly what the reference trainer does around attention,
 * kernel by kernel and argument by argument (model.mojo:668-699 forward, model.mojo:915-964
 * backward), with each Mojo kernel launch replaced by the C entry point of the same name.  It is
 * what the Mojo binding in mojo/attn_ffi.mojo does, written in a language that can be compiled
 * here.  tests/test_c_abi_call.py builds it against include/arattn.h, runs it on seeded inputs and
 * compares what it writes with the CPU oracle.
 *
 *   c_abi_call <in.bin> <out.bin> B T H W
 *   in.bin : fp32 q, k, v, dO [B,T,H,128] each, then cos, sin [T,64]
 *   out.bin: fp32 o [B,T,H,128], lse [B,T,H], d [B,T,H], dq, dk, dv [B,T,H,128]
 */
#include <cuda_runtime_api.h>
#include <stdio.h>
#include <stdlib.h>

#include "arattn.h"

#define CHECK_CUDA(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
  fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); return 2; } } while (0)
#define CHECK_AR(x) do { ar_status s_ = (x); if (s_ != AR_OK) { \
  fprintf(stderr, "%s: status %d: %s\n", #x, (int)s_, ar_last_error()); return 3; } } while (0)

static float* dev_from(const float* host, size_t n) {
  float* p = NULL;
  if (cudaMalloc((void**)&p, n * sizeof(float)) != cudaSuccess) return NULL;
  if (host && cudaMemcpy(p, host, n * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
  return p;
}

int main(int argc, char** argv) {
  if (argc != 7) { fprintf(stderr, "usage: %s in.bin out.bin B T H W\n", argv[0]); return 1; }
  const int64_t B = atoll(argv[3]), T = atoll(argv[4]), H = atoll(argv[5]), W = atoll(argv[6]), D = 128;
  const size_t n = (size_t)(B * T * H * D), rows = (size_t)(B * T * H), tab = (size_t)(T * D / 2);
  const size_t n_in = 4 * n + 2 * tab;
  float* host = (float*)malloc(n_in * sizeof(float));
  FILE* f = fopen(argv[1], "rb");
  if (!host || !f || fread(host, sizeof(float), n_in, f) != n_in) { fprintf(stderr, "cannot read %s\n", argv[1]); return 1; }
  fclose(f);

  /* the trainer's buffers (ForwardBuffers, model.mojo:443-481), all fp32, caller-owned */
  float *q = dev_from(host, n), *k = dev_from(host + n, n), *v = dev_from(host + 2 * n, n);
  float *grad_attn_out = dev_from(host + 3 * n, n);
  float *rope_cos = dev_from(host + 4 * n, tab), *rope_sin = dev_from(host + 4 * n + tab, tab);
  float *attn_out = dev_from(NULL, n), *lse = dev_from(NULL, rows), *d_buf = dev_from(NULL, rows);
  float *grad_q = dev_from(NULL, n), *grad_k = dev_from(NULL, n), *grad_v = dev_from(NULL, n);
  if (!q || !k || !v || !grad_attn_out || !rope_cos || !rope_sin || !attn_out || !lse || !d_buf || !grad_q ||
      !grad_k || !grad_v) { fprintf(stderr, "device allocation failed\n"); return 2; }
  const int64_t BT = B * T;
  void* stream = NULL;   /* the legacy default stream, as a Mojo caller without a stream handle uses */

  /* forward: model.mojo:668-677 then 694-699 (q, k rotated in place; position = token % T) */
  CHECK_AR(ar_rope_fwd(q, q, rope_cos, rope_sin, BT, H, D, T, stream));
  CHECK_AR(ar_rope_fwd(k, k, rope_cos, rope_sin, BT, H, D, T, stream));
  CHECK_AR(ar_flash_attn_fwd(attn_out, lse, q, k, v, B, T, H, D, W, stream));
  /* backward: model.mojo:915-935 then 955-964 (q, k are the saved rotated tensors) */
  CHECK_AR(ar_flash_attn_bwd_precompute_d(d_buf, attn_out, grad_attn_out, B, T, H, D, stream));
  CHECK_AR(ar_flash_attn_bwd_dq(grad_q, q, k, v, grad_attn_out, lse, d_buf, B, T, H, D, W, stream));
  CHECK_AR(ar_flash_attn_bwd_dkv(grad_k, grad_v, q, k, v, grad_attn_out, lse, d_buf, B, T, H, D, W, stream));
  CHECK_AR(ar_rope_bwd(grad_q, grad_q, rope_cos, rope_sin, BT, H, D, T, stream));
  CHECK_AR(ar_rope_bwd(grad_k, grad_k, rope_cos, rope_sin, BT, H, D, T, stream));
  CHECK_AR(ar_device_status());   /* waits for the device; AR_ERR_TIMEOUT if a kernel gave up a wait */

  f = fopen(argv[2], "wb");
  if (!f) { fprintf(stderr, "cannot write %s\n", argv[2]); return 1; }
  const float* outs[6] = {attn_out, lse, d_buf, grad_q, grad_k, grad_v};
  const size_t sizes[6] = {n, rows, rows, n, n, n};
  float* back = (float*)malloc(n * sizeof(float));
  for (int i = 0; i < 6; ++i) {
    CHECK_CUDA(cudaMemcpy(back, outs[i], sizes[i] * sizeof(float), cudaMemcpyDeviceToHost));
    if (fwrite(back, sizeof(float), sizes[i], f) != sizes[i]) return 1;
  }
  fclose(f);
  printf("c_abi_call ok (version %d)\n", (int)ar_version());
  return 0;
}
