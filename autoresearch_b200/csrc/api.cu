// C ABI of libarattn.so (declared in include/arattn.h): argument validation, per-device
// state (status word, scratch workspace), operand staging and kernel launches.
// There is no CPU path: every entry point either launches the sm_100a kernels or fails.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "../../include/arattn.h"
#include "attn_common.cuh"
#include "tmap.h"

namespace ar {

// ---- error reporting -------------------------------------------------------------------
static thread_local char g_err[512] = "";

static ar_status fail(ar_status code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
static ar_status cuda_fail(cudaError_t e, const char* what) {
  return fail(AR_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}
#define AR_CUDA(call, what)                          \
  do {                                               \
    cudaError_t e__ = (call);                        \
    if (e__ != cudaSuccess) return cuda_fail(e__, what); \
  } while (0)

// ---- per-device state --------------------------------------------------------------------
constexpr int kMaxDevices = 64;
struct DeviceState {
  uint32_t* status = nullptr;  // device status word
  void* ws = nullptr;          // library-managed scratch
  size_t ws_bytes = 0;
  bool arch_checked = false;
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_mu;

static ar_status device_state(DeviceState** out) {
  int dev = -1;
  AR_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(AR_ERR_CUDA, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  DeviceState& st = g_dev[dev];
  if (!st.arch_checked) {
    int major = 0;
    AR_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev),
            "cudaDeviceGetAttribute");
    if (major != 10)
      return fail(AR_ERR_CUDA, "device %d has compute capability %d.x; sm_100 is required", dev,
                  major);
    st.arch_checked = true;
  }
  if (!st.status) {
    AR_CUDA(cudaMalloc(&st.status, sizeof(uint32_t)), "cudaMalloc(status)");
    AR_CUDA(cudaMemset(st.status, 0, sizeof(uint32_t)), "cudaMemset(status)");
  }
  *out = &st;
  return AR_OK;
}

// Library-managed scratch: grown on demand, kept until process exit.  Growing frees the
// old block (cudaFree synchronises the device first, so earlier launches are finished).
static ar_status library_workspace(DeviceState* st, size_t bytes, void** out) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (st->ws_bytes < bytes) {
    if (st->ws) {
      AR_CUDA(cudaFree(st->ws), "cudaFree(workspace)");
      st->ws = nullptr;
      st->ws_bytes = 0;
    }
    const size_t rounded = (bytes + (size_t(1) << 20) - 1) & ~((size_t(1) << 20) - 1);
    AR_CUDA(cudaMalloc(&st->ws, rounded), "cudaMalloc(workspace)");
    st->ws_bytes = rounded;
  }
  *out = st->ws;
  return AR_OK;
}

static inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }
// Backward scratch always starts with the key-stationary copies of LSE*log2e and D:
// two [B, H, Tp] fp32 arrays, Tp = T rounded up to 64, each 1024-byte aligned.
static inline int64_t pad64(int64_t T) { return (T + 63) / 64 * 64; }
static inline size_t stats_each(int64_t B, int64_t T, int64_t H) {
  return align_up((size_t)B * H * pad64(T) * sizeof(float), 1024);
}
static inline size_t stats_bytes(int64_t B, int64_t T, int64_t H) { return 2 * stats_each(B, T, H); }

// ---- validation helpers ------------------------------------------------------------------
static ar_status check_dims(int64_t B, int64_t T, int64_t H, int64_t D) {
  if (B <= 0 || T <= 0 || H <= 0 || D <= 0)
    return fail(AR_ERR_BAD_ARG, "B, T, num_heads, head_dim must be positive (got %lld %lld %lld %lld)",
                (long long)B, (long long)T, (long long)H, (long long)D);
  if (D != kHeadDim)
    return fail(AR_ERR_UNSUPPORTED, "head_dim %lld is not supported (only 128)", (long long)D);
  if (T > (int64_t(1) << 24) || H > 65535 || B > 65535 || B * T * H > (int64_t(1) << 40))
    return fail(AR_ERR_UNSUPPORTED, "shape out of range (T <= 2^24, H, B <= 65535)");
  return AR_OK;
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static int norm_window(int64_t window, int64_t T) {
  return (window <= 0 || window >= T) ? 0 : static_cast<int>(window);
}

struct Maps {
  CUtensorMap q, k, v, d_o;
};
// Layout of the caller's tensors in rows of head_dim elements (see AttnDims); {0, 0} = contiguous.
struct Layout {
  int64_t pitch_t = 0, pitch_b = 0;
};
static ar_status make_map(CUtensorMap* m, const void* base, int64_t B, int64_t T, int64_t H, int box_rows,
                          const Layout& lay) {
  if (!make_tmap_bthd(m, base, B, T, H, kHeadDim, box_rows, lay.pitch_t, lay.pitch_b))
    return fail(AR_ERR_CUDA, "cuTensorMapEncodeTiled failed (driver entry point missing or bad tensor)");
  return AR_OK;
}
#define AR_TRY(expr)                  \
  do {                                \
    ar_status s__ = (expr);           \
    if (s__ != AR_OK) return s__;     \
  } while (0)

static ar_status finish(DeviceState* st, uint32_t flags, cudaStream_t stream) {
  if (!(flags & AR_FLAG_SYNC)) return AR_OK;
  AR_CUDA(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
  uint32_t word = 0;
  AR_CUDA(cudaMemcpy(&word, st->status, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  if (word != 0) {
    AR_CUDA(cudaMemset(st->status, 0, sizeof(uint32_t)), "cudaMemset(status)");
    return fail(AR_ERR_TIMEOUT, "a device-side bounded wait gave up (status word 0x%x)", word);
  }
  return AR_OK;
}

// ---- core drivers on bf16 operands ---------------------------------------------------------
static AttnDims make_dims(int64_t B, int64_t T, int64_t H, int window, const Layout& lay) {
  const int64_t pt = lay.pitch_t ? lay.pitch_t : H;
  return AttnDims{(int)B, (int)T, (int)H, window, (int)pt, (long long)(lay.pitch_b ? lay.pitch_b : T * pt)};
}

// `lay` is the layout of o and lse and of those of q, k, v whose flag in `caller` (bit 0: q, 1: k,
// 2: v) is set; the others are contiguous scratch.
static ar_status run_fwd(DeviceState* st, const __nv_bfloat16* q, const __nv_bfloat16* k,
                         const __nv_bfloat16* v, void* o, int o_f32, float* lse, int64_t B, int64_t T,
                         int64_t H, int window, const float* cos_buf, const float* sin_buf,
                         cudaStream_t stream, const Layout& lay = Layout(), unsigned caller = 0) {
  Maps m;
  const Layout contig;
  AR_TRY(make_map(&m.q, q, B, T, H, kTile, (caller & 1u) ? lay : contig));
  AR_TRY(make_map(&m.k, k, B, T, H, kTile, (caller & 2u) ? lay : contig));
  AR_TRY(make_map(&m.v, v, B, T, H, kTile, (caller & 4u) ? lay : contig));
  FwdParams p;
  p.dims = make_dims(B, T, H, window, lay);
  p.scale = 1.0f / sqrtf((float)kHeadDim);
  p.scale_log2e = p.scale * kLog2e;
  p.o = o;
  p.o_f32 = o_f32;
  p.lse = lse;
  p.cos_buf = cos_buf;
  p.sin_buf = sin_buf;
  p.status = st->status;
  AR_CUDA(launch_attn_fwd(m.q, m.k, m.v, p, cos_buf != nullptr, stream), "attn_fwd launch");
  return AR_OK;
}

static ar_status run_bwd(DeviceState* st, bool want_dq, bool want_dkv, const __nv_bfloat16* q,
                         const __nv_bfloat16* k, const __nv_bfloat16* v, const __nv_bfloat16* d_o,
                         const float* lse, const float* d_buf, const __nv_bfloat16* o_for_d, float* d_out, void* stats_ws,
                         void* dq, void* dk, void* dv, int grad_f32, int64_t B, int64_t T, int64_t H, int window,
                         const float* cos_buf, const float* sin_buf, cudaStream_t stream,
                         const Layout& lay = Layout(), unsigned caller = 0) {
  // `lay`: layout of lse, d_buf, o_for_d, the gradients, and of those of q, k, v, d_o whose flag in
  // `caller` (bit 0: q, 1: k, 2: v, 3: d_o) is set; the others are contiguous scratch.
  Maps m;   // the backward kernels move every operand in 64-row boxes
  const Layout contig;
  AR_TRY(make_map(&m.q, q, B, T, H, 64, (caller & 1u) ? lay : contig));
  AR_TRY(make_map(&m.k, k, B, T, H, 64, (caller & 2u) ? lay : contig));
  AR_TRY(make_map(&m.v, v, B, T, H, 64, (caller & 4u) ? lay : contig));
  AR_TRY(make_map(&m.d_o, d_o, B, T, H, 64, (caller & 8u) ? lay : contig));
  BwdParams p;
  p.dims = make_dims(B, T, H, window, lay);
  p.scale = 1.0f / sqrtf((float)kHeadDim);
  p.scale_log2e = p.scale * kLog2e;
  p.lse = lse;
  p.dvec = d_buf;
  float* lse2_t = static_cast<float*>(stats_ws);
  float* dvec_t = reinterpret_cast<float*>(static_cast<char*>(stats_ws) + stats_each(B, T, H));
  p.lse2_t = lse2_t;
  p.dvec_t = dvec_t;
  p.t_pad = (int)pad64(T);
  // With o_for_d the dQ kernel produces D and both key-stationary arrays on its way.
  if (!want_dq) o_for_d = nullptr;
  p.o_for_d = o_for_d;
  p.do_for_d = d_o;
  p.d_out = d_out;
  p.lse2_t_out = lse2_t;
  p.dvec_t_out = dvec_t;
  if (want_dkv && !o_for_d)
    AR_CUDA(launch_stats_transpose(lse2_t, dvec_t, lse, d_buf, (int)B, (int)T, (int)H, p.t_pad, stream,
                                   RowMap{(int)T, (int)H, p.dims.pitch_t, p.dims.pitch_b}),
            "stats transpose launch");
  p.dq = dq;
  p.dk = dk;
  p.dv = dv;
  p.grad_f32 = grad_f32;
  p.cos_buf = cos_buf;
  p.sin_buf = sin_buf;
  p.status = st->status;
  if (want_dq) AR_CUDA(launch_attn_bwd_dq(m.q, m.k, m.v, m.d_o, p, stream), "attn_bwd_dq launch");
  if (want_dkv) AR_CUDA(launch_attn_bwd_dkv(m.q, m.k, m.v, m.d_o, p, stream), "attn_bwd_dkv launch");
  return AR_OK;
}

static ar_status rope_mirror(float* out, const float* in, const float* cos_buf, const float* sin_buf,
                             int64_t num_tokens, int64_t num_heads, int64_t head_dim,
                             int64_t seq_len, int mode, void* stream) {
  if (!out || !in || !cos_buf || !sin_buf) return fail(AR_ERR_BAD_ARG, "null pointer");
  if (num_tokens <= 0 || num_heads <= 0 || head_dim <= 0 || (head_dim & 1))
    return fail(AR_ERR_BAD_ARG, "num_tokens, num_heads must be positive and head_dim positive and even");
  DeviceState* st;
  AR_TRY(device_state(&st));
  const long long rows = num_tokens * num_heads;
  const bool vec = (head_dim % 8 == 0) && aligned16(out) && aligned16(in) && aligned16(cos_buf) &&
                   aligned16(sin_buf);
  if (vec)
    AR_CUDA((launch_rope_cast<float, float>(out, in, cos_buf, sin_buf, rows, (int)num_heads,
                                            (int)head_dim, seq_len, mode, (cudaStream_t)stream)),
            "rope launch");
  else
    AR_CUDA(launch_rope_scalar(out, in, cos_buf, sin_buf, rows, (int)num_heads, (int)head_dim,
                               seq_len, mode, (cudaStream_t)stream),
            "rope launch");
  return AR_OK;
}

}  // namespace ar

using namespace ar;

extern "C" {

AR_API int32_t ar_version(void) { return 100; }
AR_API const char* ar_last_error(void) { return g_err; }

AR_API ar_status ar_device_status(void) {
  DeviceState* st;
  AR_TRY(device_state(&st));
  AR_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  uint32_t word = 0;
  AR_CUDA(cudaMemcpy(&word, st->status, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy(status)");
  if (word != 0) {
    AR_CUDA(cudaMemset(st->status, 0, sizeof(uint32_t)), "cudaMemset(status)");
    return fail(AR_ERR_TIMEOUT, "a device-side bounded wait gave up (status word 0x%x)", word);
  }
  return AR_OK;
}

AR_API ar_status ar_rope_fwd(float* out, const float* in, const float* cos_buf, const float* sin_buf,
                             int64_t num_tokens, int64_t num_heads, int64_t head_dim,
                             int64_t seq_len, void* stream) {
  return rope_mirror(out, in, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len, kRopeFwd,
                     stream);
}

AR_API ar_status ar_rope_bwd(float* grad_in, const float* grad_out, const float* cos_buf,
                             const float* sin_buf, int64_t num_tokens, int64_t num_heads,
                             int64_t head_dim, int64_t seq_len, void* stream) {
  return rope_mirror(grad_in, grad_out, cos_buf, sin_buf, num_tokens, num_heads, head_dim, seq_len,
                     kRopeBwd, stream);
}

AR_API ar_status ar_qk_norm_rope_cast(void* q_rot, void* k_rot, void* v_bf16, float* rms_q, float* rms_k,
                                      const void* q, const void* k, const void* v, int32_t in_dtype,
                                      const float* cos_buf, const float* sin_buf, int64_t num_tokens,
                                      int64_t num_heads, int64_t head_dim, int64_t seq_len, float eps,
                                      void* stream) {
  if (in_dtype != AR_F32 && in_dtype != AR_BF16) return fail(AR_ERR_UNSUPPORTED, "in_dtype %d unknown", in_dtype);
  if (!q_rot || !k_rot || !q || !k || !cos_buf || !sin_buf) return fail(AR_ERR_BAD_ARG, "null pointer");
  if ((v == nullptr) != (v_bf16 == nullptr)) return fail(AR_ERR_BAD_ARG, "v and v_bf16 must be given together");
  if (num_tokens <= 0 || num_heads <= 0) return fail(AR_ERR_BAD_ARG, "num_tokens, num_heads must be positive");
  if (head_dim != kHeadDim) return fail(AR_ERR_UNSUPPORTED, "head_dim %lld is not supported (only 128)", (long long)head_dim);
  if (!(eps >= 0.f)) return fail(AR_ERR_BAD_ARG, "eps must be non-negative");
  if (!aligned16(q_rot) || !aligned16(k_rot) || !aligned16(v_bf16) || !aligned16(q) || !aligned16(k) || !aligned16(v) ||
      !aligned16(cos_buf) || !aligned16(sin_buf))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  auto* qo = static_cast<__nv_bfloat16*>(q_rot);
  auto* ko = static_cast<__nv_bfloat16*>(k_rot);
  auto* vo = static_cast<__nv_bfloat16*>(v_bf16);
  const long long rows = num_tokens * num_heads;
  if (in_dtype == AR_F32)
    AR_CUDA(launch_qk_norm_rope_cast_128<float>(qo, ko, vo, rms_q, rms_k, (const float*)q, (const float*)k, (const float*)v,
                                                cos_buf, sin_buf, rows, (int)num_heads, seq_len, eps, (cudaStream_t)stream),
            "qk_norm_rope_cast launch");
  else
    AR_CUDA(launch_qk_norm_rope_cast_128<__nv_bfloat16>(qo, ko, vo, rms_q, rms_k, (const __nv_bfloat16*)q,
                                                        (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, cos_buf, sin_buf,
                                                        rows, (int)num_heads, seq_len, eps, (cudaStream_t)stream),
            "qk_norm_rope_cast launch");
  return AR_OK;
}

AR_API ar_status ar_flash_attn_fwd(float* output, float* lse_out, const float* q, const float* k,
                                   const float* v, int64_t B, int64_t T, int64_t num_heads,
                                   int64_t head_dim, int64_t window_size, void* stream) {
  if (!output || !lse_out || !q || !k || !v) return fail(AR_ERR_BAD_ARG, "null pointer");
  AR_TRY(check_dims(B, T, num_heads, head_dim));
  if (!aligned16(output) || !aligned16(q) || !aligned16(k) || !aligned16(v))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  const size_t n = (size_t)B * T * num_heads * head_dim;
  const size_t each = align_up(n * sizeof(__nv_bfloat16), 1024);
  void* ws;
  AR_TRY(library_workspace(st, 3 * each, &ws));
  auto* qb = reinterpret_cast<__nv_bfloat16*>(ws);
  auto* kb = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + each);
  auto* vb = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + 2 * each);
  cudaStream_t s = (cudaStream_t)stream;
  const long long rows = B * T * num_heads;
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(qb, q, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast q");
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(kb, k, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast k");
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(vb, v, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast v");
  return run_fwd(st, qb, kb, vb, output, 1, lse_out, B, T, num_heads, norm_window(window_size, T),
                 nullptr, nullptr, s);
}

// ---- allocation-free forward ----------------------------------------------------------------
// Scratch and status word are file-scope device symbols.  In host code their names are only
// host-side stand-ins, not device addresses: the address is looked up once per device with
// cudaGetSymbolAddress (that device current) and passed to the kernels like any pointer.
constexpr size_t kNoAllocTensorBytes = (size_t)AR_NOALLOC_MAX_ROWS * kHeadDim * sizeof(__nv_bfloat16);
static __device__ __align__(256) unsigned char g_noalloc_scratch[3 * kNoAllocTensorBytes];
static __device__ uint32_t g_noalloc_status;   // zero-initialised with the image

struct NoAllocState {
  void* scratch = nullptr;
  uint32_t* status = nullptr;
};
static NoAllocState g_noalloc[kMaxDevices];

static ar_status noalloc_state(NoAllocState** out) {
  int dev = -1;
  AR_CUDA(cudaGetDevice(&dev), "cudaGetDevice");
  if (dev < 0 || dev >= kMaxDevices) return fail(AR_ERR_CUDA, "device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_mu);
  NoAllocState& st = g_noalloc[dev];
  if (!st.scratch) {
    int major = 0;
    AR_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev), "cudaDeviceGetAttribute");
    if (major != 10)
      return fail(AR_ERR_CUDA, "device %d has compute capability %d.x; sm_100 is required", dev, major);
    void* scratch = nullptr;
    void* status = nullptr;
    AR_CUDA(cudaGetSymbolAddress(&scratch, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)");
    AR_CUDA(cudaGetSymbolAddress(&status, g_noalloc_status), "cudaGetSymbolAddress(status)");
    st.status = static_cast<uint32_t*>(status);
    st.scratch = scratch;
  }
  *out = &st;
  return AR_OK;
}

AR_API ar_status ar_flash_attn_fwd_noalloc(float* output, float* lse_out, const float* q, const float* k,
                                           const float* v, int64_t B, int64_t T, int64_t num_heads,
                                           int64_t head_dim, int64_t window_size, void* stream) {
  if (!output || !lse_out || !q || !k || !v) return fail(AR_ERR_BAD_ARG, "null pointer");
  AR_TRY(check_dims(B, T, num_heads, head_dim));
  if (!aligned16(output) || !aligned16(q) || !aligned16(k) || !aligned16(v))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  const int64_t rows = B * T * num_heads;
  if (rows > AR_NOALLOC_MAX_ROWS)
    return fail(AR_ERR_WORKSPACE,
                "B*T*num_heads = %lld exceeds the fixed scratch of the allocation-free entry point "
                "(AR_NOALLOC_MAX_ROWS = %d); use ar_flash_attn_fwd",
                (long long)rows, AR_NOALLOC_MAX_ROWS);
  NoAllocState* na;
  AR_TRY(noalloc_state(&na));
  char* base = static_cast<char*>(na->scratch);
  auto* qb = reinterpret_cast<__nv_bfloat16*>(base);
  auto* kb = reinterpret_cast<__nv_bfloat16*>(base + kNoAllocTensorBytes);
  auto* vb = reinterpret_cast<__nv_bfloat16*>(base + 2 * kNoAllocTensorBytes);
  cudaStream_t s = (cudaStream_t)stream;
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(qb, q, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast q");
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(kb, k, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast k");
  AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(vb, v, nullptr, nullptr, rows, (int)num_heads, 128, 0, kCastOnly, s)), "cast v");
  DeviceState view;            // only the status pointer is read by run_fwd
  view.status = na->status;
  return run_fwd(&view, qb, kb, vb, output, 1, lse_out, B, T, num_heads, norm_window(window_size, T),
                 nullptr, nullptr, s);
}

AR_API ar_status ar_noalloc_status(void) {
  NoAllocState* na;
  AR_TRY(noalloc_state(&na));
  AR_CUDA(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  uint32_t word = 0;
  AR_CUDA(cudaMemcpy(&word, na->status, sizeof(word), cudaMemcpyDeviceToHost), "cudaMemcpy(noalloc status)");
  if (word != 0) {
    const uint32_t zero = 0;
    AR_CUDA(cudaMemcpy(na->status, &zero, sizeof(zero), cudaMemcpyHostToDevice), "cudaMemcpy(clear noalloc status)");
    return fail(AR_ERR_TIMEOUT, "a device-side bounded wait gave up in an allocation-free call (status word 0x%x)", word);
  }
  return AR_OK;
}

// ---- self-test of the time-out path ------------------------------------------------------------
// One warp waits on an mbarrier that nothing ever arrives at, with a limit of about a millisecond
// instead of the kernels' 0.2 s.  The wait runs out, flags the status word exactly as an abandoned
// wait inside an attention kernel would, and the kernel returns normally.
constexpr long long kSelfTestLimitCycles = 2000000ll;
__global__ void __launch_bounds__(32, 1) selftest_wait_kernel(uint32_t* status) {
  __shared__ alignas(8) uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncwarp();
  WaitCtx w{status, smem_u32(&abort_flag)};
  (void)mbar_wait<0, kSelfTestLimitCycles>(w, smem_u32(&bar), 0);
}

AR_API ar_status ar_selftest_wait_timeout(int32_t which, void* stream) {
  uint32_t* word = nullptr;
  if (which == 0) {
    DeviceState* st;
    AR_TRY(device_state(&st));
    word = st->status;
  } else if (which == 1) {
    NoAllocState* na;
    AR_TRY(noalloc_state(&na));
    word = na->status;
  } else {
    return fail(AR_ERR_BAD_ARG, "which must be 0 (ar_device_status word) or 1 (ar_noalloc_status word)");
  }
  selftest_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(word);
  AR_CUDA(cudaGetLastError(), "selftest launch");
  return AR_OK;
}

AR_API ar_status ar_flash_attn_bwd_precompute_d(float* d_out, const float* output,
                                                const float* grad_output, int64_t B, int64_t T,
                                                int64_t num_heads, int64_t head_dim, void* stream) {
  if (!d_out || !output || !grad_output) return fail(AR_ERR_BAD_ARG, "null pointer");
  if (B <= 0 || T <= 0 || num_heads <= 0 || head_dim <= 0)
    return fail(AR_ERR_BAD_ARG, "B, T, num_heads, head_dim must be positive");
  if (head_dim % 4 != 0 || !aligned16(output) || !aligned16(grad_output))
    return fail(AR_ERR_UNSUPPORTED, "head_dim must be a multiple of 4 and tensors 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  AR_CUDA(launch_precompute_d<float>(d_out, output, grad_output, B * T * num_heads, (int)head_dim,
                                     (cudaStream_t)stream),
          "precompute_d launch");
  return AR_OK;
}

static ar_status bwd_mirror(bool want_dq, float* g0, float* g1, float* g2, const float* q,
                            const float* k, const float* v, const float* grad_output,
                            const float* lse, const float* d_buf, int64_t B, int64_t T, int64_t H,
                            int64_t D, int64_t window_size, void* stream) {
  if (!q || !k || !v || !grad_output || !lse || !d_buf) return fail(AR_ERR_BAD_ARG, "null pointer");
  AR_TRY(check_dims(B, T, H, D));
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(grad_output))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  const size_t n = (size_t)B * T * H * D;
  const size_t each = align_up(n * sizeof(__nv_bfloat16), 1024);
  void* ws;
  const size_t sb = stats_bytes(B, T, H);
  AR_TRY(library_workspace(st, sb + 4 * each, &ws));
  __nv_bfloat16* buf[4];
  for (int i = 0; i < 4; ++i)
    buf[i] = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + sb + i * each);
  const float* src[4] = {q, k, v, grad_output};
  cudaStream_t s = (cudaStream_t)stream;
  for (int i = 0; i < 4; ++i)
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(buf[i], src[i], nullptr, nullptr, B * T * H, (int)H, 128, 0, kCastOnly, s)), "cast");
  return run_bwd(st, want_dq, !want_dq, buf[0], buf[1], buf[2], buf[3], lse, d_buf, nullptr, nullptr, ws, g0, g1, g2, 1, B,
                 T, H, norm_window(window_size, T), nullptr, nullptr, s);
}

AR_API ar_status ar_flash_attn_bwd_dq(float* grad_q, const float* q, const float* k, const float* v,
                                      const float* grad_output, const float* lse, const float* d_buf,
                                      int64_t B, int64_t T, int64_t num_heads, int64_t head_dim,
                                      int64_t window_size, void* stream) {
  if (!grad_q || !aligned16(grad_q)) return fail(AR_ERR_BAD_ARG, "grad_q null or misaligned");
  return bwd_mirror(true, grad_q, nullptr, nullptr, q, k, v, grad_output, lse, d_buf, B, T, num_heads,
                    head_dim, window_size, stream);
}

AR_API ar_status ar_flash_attn_bwd_dkv(float* grad_k, float* grad_v, const float* q, const float* k,
                                       const float* v, const float* grad_output, const float* lse,
                                       const float* d_buf, int64_t B, int64_t T, int64_t num_heads,
                                       int64_t head_dim, int64_t window_size, void* stream) {
  if (!grad_k || !grad_v || !aligned16(grad_k) || !aligned16(grad_v))
    return fail(AR_ERR_BAD_ARG, "grad_k / grad_v null or misaligned");
  return bwd_mirror(false, nullptr, grad_k, grad_v, q, k, v, grad_output, lse, d_buf, B, T, num_heads,
                    head_dim, window_size, stream);
}

// ---- projections ---------------------------------------------------------------------------------
// mode 0: y[M,N] = x[M,K] w[N,K]^T   mode 1: dx[M,K] = dy[M,N] w[N,K]   mode 2: dw[N,K] += dy[M,N]^T x[M,K]
static ar_status linear_call(int mode, void* out, const void* a_in, const void* b_in, int64_t M, int64_t N, int64_t K,
                             int32_t in_dtype, int32_t out_dtype, void* stream) {
  if (!out || !a_in || !b_in) return fail(AR_ERR_BAD_ARG, "null pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(AR_ERR_BAD_ARG, "M, N, K must be positive");
  if (M > (int64_t(1) << 30) || N > (int64_t(1) << 24) || K > (int64_t(1) << 24))
    return fail(AR_ERR_UNSUPPORTED, "shape out of range");
  if (N % 8 != 0 || K % 8 != 0) return fail(AR_ERR_UNSUPPORTED, "N and K must be multiples of 8 (16-byte rows)");
  const int64_t out_cols = mode == 0 ? N : K;
  if (out_cols % 32 != 0) return fail(AR_ERR_UNSUPPORTED, "the output's row length (%lld) must be a multiple of 32", (long long)out_cols);
  if (in_dtype != AR_F32 && in_dtype != AR_BF16) return fail(AR_ERR_UNSUPPORTED, "in_dtype %d unknown", in_dtype);
  if (out_dtype != AR_F32 && out_dtype != AR_BF16) return fail(AR_ERR_UNSUPPORTED, "out_dtype %d unknown", out_dtype);
  if (mode == 2 && out_dtype != AR_F32) return fail(AR_ERR_UNSUPPORTED, "dw is accumulated in fp32");
  if (!aligned16(out) || !aligned16(a_in) || !aligned16(b_in)) return fail(AR_ERR_BAD_ARG, "pointers must be 16-byte aligned");
  // fp32 operands are staged as bf16 copies before the product starts, so the output may be one of
  // them (the reference's in-place c_proj backward, model.mojo:906); bf16 operands are read in place
  if (in_dtype == AR_BF16 && (out == a_in || out == b_in))
    return fail(AR_ERR_BAD_ARG, "the output aliases a bf16 operand");
  DeviceState* st;
  AR_TRY(device_state(&st));
  cudaStream_t s = (cudaStream_t)stream;
  // operand shapes (rows x inner): mode 0: a = x [M,K], b = w [N,K]; 1: a = dy [M,N], b = w [N,K]; 2: a = dy [M,N], b = x [M,K]
  const int64_t a_rows = M, a_inner = mode == 0 ? K : N;
  const int64_t b_rows = mode == 2 ? M : N, b_inner = K;
  const __nv_bfloat16 *ab = (const __nv_bfloat16*)a_in, *bb = (const __nv_bfloat16*)b_in;
  if (in_dtype == AR_F32) {   // stage both operands as bf16
    const size_t na = align_up((size_t)a_rows * a_inner * 2, 1024), nb = align_up((size_t)b_rows * b_inner * 2, 1024);
    void* ws;
    AR_TRY(library_workspace(st, na + nb, &ws));
    auto* sa = reinterpret_cast<__nv_bfloat16*>(ws);
    auto* sb = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + na);
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(sa, (const float*)a_in, nullptr, nullptr, a_rows, 1, (int)a_inner, 0, kCastOnly, s)), "stage a");
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(sb, (const float*)b_in, nullptr, nullptr, b_rows, 1, (int)b_inner, 0, kCastOnly, s)), "stage b");
    ab = sa; bb = sb;
  }
  // K-major operands move in boxes of (tile rows) x 64 inner elements, MN-major ones in 64 depth rows x 64
  CUtensorMap ma, mb;
  const int a_box = mode == 2 ? 64 : 128, b_box = mode == 0 ? 256 : 64;
  if (!make_tmap_bthd(&ma, ab, 1, a_rows, 1, a_inner, a_box) || !make_tmap_bthd(&mb, bb, 1, b_rows, 1, b_inner, b_box))
    return fail(AR_ERR_CUDA, "cuTensorMapEncodeTiled failed (driver entry point missing or bad tensor)");
  LinParams p;
  p.mode = mode;
  p.rows_a = (int)(mode == 2 ? N : M);
  p.cols_b = (int)out_cols;
  p.depth = (int)(mode == 0 ? K : (mode == 1 ? N : M));
  p.depth_chunk = (p.depth + 63) / 64 * 64;
  if (mode == 2) {   // split the long depth so that every SM has work; each chunk adds its partial tile
    const int tiles = ((p.rows_a + 127) / 128) * ((p.cols_b + 255) / 256);
    int chunks = (2 * 148 + tiles - 1) / tiles;
    const int max_chunks = (p.depth + 511) / 512;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks < 1) chunks = 1;
    p.depth_chunk = ((p.depth + chunks - 1) / chunks + 63) / 64 * 64;
  }
  p.c = out;
  p.c_f32 = out_dtype == AR_F32;
  p.ldc = (int)out_cols;
  p.accumulate = mode == 2;
  p.status = st->status;
  AR_CUDA(launch_linear(ma, mb, p, s), "linear launch");
  return AR_OK;
}

AR_API ar_status ar_linear_fwd(void* output, const void* input, const void* weight, int64_t M, int64_t N, int64_t K,
                               int32_t in_dtype, int32_t out_dtype, void* stream) {
  return linear_call(0, output, input, weight, M, N, K, in_dtype, out_dtype, stream);
}
AR_API ar_status ar_linear_bwd_dx(void* grad_input, const void* grad_output, const void* weight, int64_t M, int64_t N,
                                  int64_t K, int32_t in_dtype, int32_t out_dtype, void* stream) {
  return linear_call(1, grad_input, grad_output, weight, M, N, K, in_dtype, out_dtype, stream);
}
AR_API ar_status ar_linear_bwd_dw(float* grad_weight, const void* grad_output, const void* input, int64_t M, int64_t N,
                                  int64_t K, int32_t in_dtype, void* stream) {
  return linear_call(2, grad_weight, grad_output, input, M, N, K, in_dtype, AR_F32, stream);
}

// ---- fused family ------------------------------------------------------------------------------
static ar_status check_params(const ar_attn_params* p) {
  if (!p) return fail(AR_ERR_BAD_ARG, "params is null");
  if (p->struct_size != sizeof(ar_attn_params))
    return fail(AR_ERR_BAD_ARG, "struct_size %u does not match this library (%zu)", p->struct_size,
                sizeof(ar_attn_params));
  AR_TRY(check_dims(p->B, p->T, p->H, p->D));
  if (p->io_dtype != AR_F32 && p->io_dtype != AR_BF16)
    return fail(AR_ERR_UNSUPPORTED, "io_dtype %d unknown", p->io_dtype);
  if (p->grad_dtype != AR_F32 && p->grad_dtype != AR_BF16)
    return fail(AR_ERR_UNSUPPORTED, "grad_dtype %d unknown", p->grad_dtype);
  if (p->rope_mode != 0 && p->rope_mode != 1)
    return fail(AR_ERR_BAD_ARG, "rope_mode must be 0 or 1");
  if (p->rope_mode == 1) {
    if (!p->cos_buf || !p->sin_buf) return fail(AR_ERR_BAD_ARG, "rope_mode 1 needs cos_buf and sin_buf");
    if (p->rope_rows < p->T)
      return fail(AR_ERR_UNSUPPORTED, "rope table has %lld rows, T is %lld", (long long)p->rope_rows,
                  (long long)p->T);
    if (!aligned16(p->cos_buf) || !aligned16(p->sin_buf))
      return fail(AR_ERR_BAD_ARG, "rope tables must be 16-byte aligned");
  }
  if (p->stride_b != 0 || p->stride_t != 0 || p->stride_h != 0) {
    if (p->stride_h != p->D)
      return fail(AR_ERR_UNSUPPORTED, "stride_h must equal head_dim (the heads of one token adjacent)");
    if (p->stride_t % p->D != 0 || p->stride_t < p->H * p->D)
      return fail(AR_ERR_BAD_ARG, "stride_t must be a multiple of head_dim and at least H * head_dim");
    if (p->stride_b % p->D != 0 || p->stride_b < p->T * p->stride_t)
      return fail(AR_ERR_BAD_ARG, "stride_b must be a multiple of head_dim and at least T * stride_t");
  }
  if ((p->q_rot == nullptr) != (p->k_rot == nullptr))
    return fail(AR_ERR_BAD_ARG, "q_rot and k_rot must be given together");
  if (p->q_rot && p->rope_mode != 1) return fail(AR_ERR_BAD_ARG, "q_rot / k_rot need rope_mode 1");
  if (p->q_rot && (!aligned16(p->q_rot) || !aligned16(p->k_rot)))
    return fail(AR_ERR_BAD_ARG, "q_rot / k_rot must be 16-byte aligned");
  return AR_OK;
}

// The caller's layout from the stride fields (all zero: contiguous), and the row map of a helper
// kernel's tensor in that layout.
static Layout layout_of(const ar_attn_params* p) {
  Layout lay;
  if (p->stride_t != 0) {
    lay.pitch_t = p->stride_t / p->D;
    lay.pitch_b = p->stride_b / p->D;
  }
  return lay;
}
static RowMap row_map(const ar_attn_params* p, const Layout& lay) {
  if (lay.pitch_t == 0) return RowMap();
  return RowMap{(int)p->T, (int)p->H, (int)lay.pitch_t, (long long)lay.pitch_b};
}

// Scratch layout: `count` bf16 tensors of n elements, each 1024-byte aligned.
static uint64_t ws_need(const ar_attn_params* p, int32_t pass) {
  const size_t n = (size_t)p->B * p->T * p->H * p->D;
  const size_t each = align_up(n * sizeof(__nv_bfloat16), 1024);
  int count = 0;
  if (pass == 0) {
    if (p->io_dtype == AR_F32) count = 3;                                      // q, k, v staged
    else if (p->rope_mode == 1 && (p->flags & AR_FLAG_ROPE_PREPASS) && !p->q_rot) count = 2;  // rotated q, k
  } else {
    if (p->io_dtype == AR_F32) count = 4;   // q, k, v, dO staged
    else if (p->rope_mode == 1 && !p->q_rot) count = 2;  // rotated q, k
    return (uint64_t)stats_bytes(p->B, p->T, p->H) + (uint64_t)count * each;
  }
  return (uint64_t)count * each;
}

AR_API uint64_t ar_attn_workspace_bytes(const ar_attn_params* p, int32_t pass) {
  if (!p || p->B <= 0 || p->T <= 0 || p->H <= 0 || p->D <= 0) return 0;
  return ws_need(p, pass);
}

static ar_status get_ws(DeviceState* st, const ar_attn_params* p, int32_t pass, void** ws) {
  const uint64_t need = ws_need(p, pass);
  *ws = nullptr;
  if (need == 0) return AR_OK;
  if (p->workspace) {
    if (p->workspace_bytes < need)
      return fail(AR_ERR_WORKSPACE, "workspace has %llu bytes, %llu needed",
                  (unsigned long long)p->workspace_bytes, (unsigned long long)need);
    if ((reinterpret_cast<uintptr_t>(p->workspace) & 1023u) != 0)
      return fail(AR_ERR_BAD_ARG, "workspace must be 1024-byte aligned");
    *ws = p->workspace;
    return AR_OK;
  }
  return library_workspace(st, need, ws);
}

AR_API ar_status ar_attn_fwd(const ar_attn_params* p, const void* q, const void* k, const void* v,
                             void* o, float* lse) {
  AR_TRY(check_params(p));
  if (!q || !k || !v || !o || !lse) return fail(AR_ERR_BAD_ARG, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  void* ws;
  AR_TRY(get_ws(st, p, 0, &ws));
  cudaStream_t s = (cudaStream_t)p->stream;
  const size_t n = (size_t)p->B * p->T * p->H * p->D;
  const size_t each = align_up(n * sizeof(__nv_bfloat16), 1024);
  const long long rows = p->B * p->T * p->H;
  const int H = (int)p->H;
  const bool rope = p->rope_mode == 1;
  const Layout lay = layout_of(p);
  const RowMap cm = row_map(p, lay), none;   // caller's tensors / contiguous scratch
  const RowMap rot_map = p->q_rot ? cm : none;   // q_rot, k_rot share the caller's layout
  unsigned caller = 0;                       // which of q, k, v the attention kernel reads in the caller's layout
  const __nv_bfloat16 *qb, *kb, *vb;
  const float *fc = nullptr, *fs = nullptr;  // tables handed to the attention kernel (fused rope)
  if (p->io_dtype == AR_F32) {
    auto* b0 = p->q_rot ? static_cast<__nv_bfloat16*>(p->q_rot) : reinterpret_cast<__nv_bfloat16*>(ws);
    auto* b1 = p->k_rot ? static_cast<__nv_bfloat16*>(p->k_rot)
                        : reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + each);
    auto* b2 = reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + 2 * each);
    const int mode = rope ? kRopeFwd : kCastOnly;  // staging pass rotates while it casts
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b0, (const float*)q, p->cos_buf, p->sin_buf, rows, H, 128, p->T, mode, s, cm, rot_map)), "stage q");
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b1, (const float*)k, p->cos_buf, p->sin_buf, rows, H, 128, p->T, mode, s, cm, rot_map)), "stage k");
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b2, (const float*)v, nullptr, nullptr, rows, H, 128, 0, kCastOnly, s, cm, none)), "stage v");
    qb = b0; kb = b1; vb = b2;
    if (p->q_rot) caller |= 3u;
  } else {
    qb = (const __nv_bfloat16*)q; kb = (const __nv_bfloat16*)k; vb = (const __nv_bfloat16*)v;
    caller = 7u;
    if (rope && ((p->flags & AR_FLAG_ROPE_PREPASS) || p->q_rot)) {
      auto* b0 = p->q_rot ? static_cast<__nv_bfloat16*>(p->q_rot) : reinterpret_cast<__nv_bfloat16*>(ws);
      auto* b1 = p->k_rot ? static_cast<__nv_bfloat16*>(p->k_rot)
                          : reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(ws) + each);
      AR_CUDA(launch_rope_pair_bf16_128(b0, qb, b1, kb, p->cos_buf, p->sin_buf, rows / H, H, p->T, s, cm, rot_map), "rope q, k");
      qb = b0; kb = b1;
      if (!p->q_rot) caller = 4u;
    } else if (rope) {
      fc = p->cos_buf; fs = p->sin_buf;
    }
  }
  AR_TRY(run_fwd(st, qb, kb, vb, o, p->io_dtype == AR_F32, lse, p->B, p->T, p->H,
                 norm_window(p->window, p->T), fc, fs, s, lay, caller));
  return finish(st, p->flags, s);
}

AR_API ar_status ar_attn_bwd(const ar_attn_params* p, const void* q, const void* k, const void* v,
                             const void* o, const void* d_o, const float* lse, float* d_buf, void* dq,
                             void* dk, void* dv) {
  AR_TRY(check_params(p));
  const bool do_d = !(p->flags & AR_FLAG_BWD_SKIP_D);
  const bool do_dq = !(p->flags & AR_FLAG_BWD_SKIP_DQ);
  const bool do_dkv = !(p->flags & AR_FLAG_BWD_SKIP_DKV);
  if (!q || !k || !v || !d_o || !lse || !d_buf || (do_d && !o) || (do_dq && !dq) ||
      (do_dkv && (!dk || !dv)))
    return fail(AR_ERR_BAD_ARG, "null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o) || !aligned16(d_o) ||
      !aligned16(dq) || !aligned16(dk) || !aligned16(dv))
    return fail(AR_ERR_BAD_ARG, "tensor pointers must be 16-byte aligned");
  DeviceState* st;
  AR_TRY(device_state(&st));
  void* ws;
  AR_TRY(get_ws(st, p, 1, &ws));
  cudaStream_t s = (cudaStream_t)p->stream;
  const size_t n = (size_t)p->B * p->T * p->H * p->D;
  const size_t each = align_up(n * sizeof(__nv_bfloat16), 1024);
  char* tens = static_cast<char*>(ws) + stats_bytes(p->B, p->T, p->H);   // staged tensors follow the statistics
  const long long rows = p->B * p->T * p->H;
  const int H = (int)p->H;
  const bool rope = p->rope_mode == 1;
  const int rmode = rope ? kRopeFwd : kCastOnly;
  const Layout lay = layout_of(p);
  const RowMap cm = row_map(p, lay), none;   // caller's tensors / contiguous scratch
  unsigned caller = 0;                       // which of q, k, v, dO the kernels read in the caller's layout
  const __nv_bfloat16 *qb, *kb, *vb, *dob;
  const __nv_bfloat16* o_for_d = nullptr;
  if (p->io_dtype == AR_F32) {
    if (do_d) AR_CUDA(launch_precompute_d<float>(d_buf, (const float*)o, (const float*)d_o, rows, 128, s, cm), "precompute_d");
    __nv_bfloat16* b[4];
    for (int i = 0; i < 4; ++i) b[i] = reinterpret_cast<__nv_bfloat16*>(tens + i * each);
    if (p->q_rot) {   // rotated and staged by the forward pass
      b[0] = static_cast<__nv_bfloat16*>(p->q_rot);
      b[1] = static_cast<__nv_bfloat16*>(p->k_rot);
      caller |= 3u;
    } else {
      AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b[0], (const float*)q, p->cos_buf, p->sin_buf, rows, H, 128, p->T, rmode, s, cm, none)), "stage q");
      AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b[1], (const float*)k, p->cos_buf, p->sin_buf, rows, H, 128, p->T, rmode, s, cm, none)), "stage k");
    }
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b[2], (const float*)v, nullptr, nullptr, rows, H, 128, 0, kCastOnly, s, cm, none)), "stage v");
    AR_CUDA((launch_rope_cast<float, __nv_bfloat16>(b[3], (const float*)d_o, nullptr, nullptr, rows, H, 128, 0, kCastOnly, s, cm, none)), "stage dO");
    qb = b[0]; kb = b[1]; vb = b[2]; dob = b[3];
  } else {
    // D rides along in the dQ kernel when both are wanted (it holds the dO tile anyway)
    if (do_d && do_dq) o_for_d = (const __nv_bfloat16*)o;
    else if (do_d) AR_CUDA(launch_precompute_d<__nv_bfloat16>(d_buf, (const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, rows, 128, s, cm), "precompute_d");
    qb = (const __nv_bfloat16*)q; kb = (const __nv_bfloat16*)k;
    vb = (const __nv_bfloat16*)v; dob = (const __nv_bfloat16*)d_o;
    caller = 15u;
    if (rope && p->q_rot) {
      qb = static_cast<const __nv_bfloat16*>(p->q_rot);   // rotated in the forward pass
      kb = static_cast<const __nv_bfloat16*>(p->k_rot);
    } else if (rope) {
      auto* b0 = reinterpret_cast<__nv_bfloat16*>(tens);
      auto* b1 = reinterpret_cast<__nv_bfloat16*>(tens + each);
      AR_CUDA(launch_rope_pair_bf16_128(b0, qb, b1, kb, p->cos_buf, p->sin_buf, rows / H, H, p->T, s, cm, none), "rope q, k");
      qb = b0; kb = b1;
      caller = 12u;
    }
  }
  AR_TRY(run_bwd(st, do_dq, do_dkv, qb, kb, vb, dob, lse, d_buf, o_for_d, d_buf, ws, dq, dk, dv, p->grad_dtype == AR_F32,
                 p->B, p->T, p->H, norm_window(p->window, p->T), rope ? p->cos_buf : nullptr,
                 rope ? p->sin_buf : nullptr, s, lay, caller));
  return finish(st, p->flags, s);
}

}  // extern "C"
