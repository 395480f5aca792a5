// HBM-bound helper kernels around the tensor-core attention kernels:
//   rope_cast_kernel   : RoPE forward / inverse rotation and/or dtype cast (fp32 <-> bf16);
//                        mirrors rope_fwd / rope_bwd (ops.mojo:209-238, 1091-1120) and stages
//                        fp32 operands as bf16.
//   precompute_d_kernel: D[b,t,h] = sum_d O * dO (ops.mojo:329-346), one warp per row.
#include "attn_common.cuh"

namespace ar {

template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) {
    return *reinterpret_cast<const float4*>(p);
  }
  static __device__ __forceinline__ void store(float* p, float4 v) {
    *reinterpret_cast<float4*>(p) = v;
  }
};
template <>
struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    return make_float4(bf16_lo_to_f32(u.x), bf16_hi_to_f32(u.x), bf16_lo_to_f32(u.y),
                       bf16_hi_to_f32(u.y));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16x2(v.x, v.y), pack_bf16x2(v.z, v.w));
  }
};

// One thread handles 4 consecutive d of the first half and the matching 4 of the second
// half of one (token, head) row.  rows = num_tokens * num_heads, half = head_dim / 2
// (a multiple of 4).  pos = token % seq_len when seq_len > 0, else token.
template <typename InT, typename OutT>
__global__ void __launch_bounds__(256)
rope_cast_kernel(OutT* out, const InT* in, const float* __restrict__ cos_buf,
                 const float* __restrict__ sin_buf, long long rows, int num_heads, int half,
                 long long seq_len, int mode, const RowMap in_map, const RowMap out_map) {
  const int groups = half >> 2;
  const long long total = rows * groups;
  for (long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x; tid < total;
       tid += (long long)gridDim.x * blockDim.x) {
    const long long row = tid / groups;
    const int g = static_cast<int>(tid - row * groups);
    const long long base = map_row(in_map, row) * 2 * half + g * 4;
    const long long obase = map_row(out_map, row) * 2 * half + g * 4;
    float4 x1 = Vec4<InT>::load(in + base);
    float4 x2 = Vec4<InT>::load(in + base + half);
    if (mode != kCastOnly) {
      const long long token = row / num_heads;
      const long long pos = seq_len > 0 ? token % seq_len : token;
      const float4 c = __ldg(reinterpret_cast<const float4*>(cos_buf + pos * half + g * 4));
      float4 s = __ldg(reinterpret_cast<const float4*>(sin_buf + pos * half + g * 4));
      if (mode == kRopeBwd) s = make_float4(-s.x, -s.y, -s.z, -s.w);
      // forward: y1 = x1*c + x2*s ; y2 = -x1*s + x2*c.  backward is the same with -s.
      const float4 y1 = make_float4(x1.x * c.x + x2.x * s.x, x1.y * c.y + x2.y * s.y,
                                    x1.z * c.z + x2.z * s.z, x1.w * c.w + x2.w * s.w);
      const float4 y2 = make_float4(x2.x * c.x - x1.x * s.x, x2.y * c.y - x1.y * s.y,
                                    x2.z * c.z - x1.z * s.z, x2.w * c.w - x1.w * s.w);
      x1 = y1;
      x2 = y2;
    }
    Vec4<OutT>::store(out + obase, x1);
    Vec4<OutT>::store(out + obase + half, x2);
  }
}

// Forward rotation of two bf16 [tokens, H, 128] tensors (Q and K) in one launch.  One thread owns
// 8 consecutive d of the first half and the matching 8 of the second half of one token; it reads
// its 8 cos / 8 sin once and applies them to every head of both tensors with 16-byte accesses, so
// the table traffic is 1/(2H) of the data traffic instead of equal to it.  blockIdx.y picks Q or K.
__global__ void __launch_bounds__(256)
rope_pair_bf16_128_kernel(__nv_bfloat16* out0, const __nv_bfloat16* in0, __nv_bfloat16* out1,
                          const __nv_bfloat16* in1, const float* __restrict__ cos_buf,
                          const float* __restrict__ sin_buf, long long tokens, int num_heads, long long seq_len,
                          const RowMap in_map, const RowMap out_map) {
  const __nv_bfloat16* in = blockIdx.y == 0 ? in0 : in1;
  __nv_bfloat16* out = blockIdx.y == 0 ? out0 : out1;
  const long long total = tokens * 8;
  for (long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x; tid < total;
       tid += (long long)gridDim.x * blockDim.x) {
    const long long token = tid >> 3;
    const int g = static_cast<int>(tid & 7);
    const long long pos = seq_len > 0 ? token % seq_len : token;
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_buf + pos * 64 + g * 8));
    const float4 c1 = __ldg(reinterpret_cast<const float4*>(cos_buf + pos * 64 + g * 8 + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_buf + pos * 64 + g * 8));
    const float4 s1 = __ldg(reinterpret_cast<const float4*>(sin_buf + pos * 64 + g * 8 + 4));
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    const long long irow0 = map_row(in_map, token * num_heads), orow0 = map_row(out_map, token * num_heads);
    for (int h = 0; h < num_heads; ++h) {
      const long long base = (irow0 + h) * 128 + g * 8, obase = (orow0 + h) * 128 + g * 8;
      const uint4 a = *reinterpret_cast<const uint4*>(in + base);
      const uint4 b = *reinterpret_cast<const uint4*>(in + base + 64);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
      uint32_t ya[4], yb[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float x1l = bf16_lo_to_f32(aw[i]), x1h = bf16_hi_to_f32(aw[i]);
        const float x2l = bf16_lo_to_f32(bw[i]), x2h = bf16_hi_to_f32(bw[i]);
        // y1 = x1*c + x2*s ; y2 = x2*c - x1*s   (ops.mojo:237-238)
        ya[i] = pack_bf16x2(x1l * cs[2 * i] + x2l * sn[2 * i], x1h * cs[2 * i + 1] + x2h * sn[2 * i + 1]);
        yb[i] = pack_bf16x2(x2l * cs[2 * i] - x1l * sn[2 * i], x2h * cs[2 * i + 1] - x1h * sn[2 * i + 1]);
      }
      *reinterpret_cast<uint4*>(out + obase) = make_uint4(ya[0], ya[1], ya[2], ya[3]);
      *reinterpret_cast<uint4*>(out + obase + 64) = make_uint4(yb[0], yb[1], yb[2], yb[3]);
    }
  }
}

// Prologue of the attention path in one launch: the reference's rope_fwd on q and k followed by its
// per-head rmsnorm_fwd on q and k (model.mojo:668-687; ops.mojo:209-238, 61-104), with the result
// cast to the bf16 operands the tensor-core kernels read, and v cast alongside (blockIdx.y picks
// q, k or v).  One thread owns 8 consecutive d of the first half of a (token, head) row and the
// matching 8 of the second half - the two halves a rotation pairs - so the rotation is local to
// the thread; the sum of squares of a row meets across its 8 threads by shuffles.  As in the
// reference the row is rotated first and normalised by sqrt(mean(y^2) + eps) of the ROTATED row
// (a rotation keeps the sum of squares, so this differs from normalising first only by rounding).
// rms_q / rms_k (optional) receive that square root per row, as rmsnorm_fwd's rms_out does.
template <typename InT>
__global__ void __launch_bounds__(256)
qk_norm_rope_cast_128_kernel(__nv_bfloat16* q_out, __nv_bfloat16* k_out, __nv_bfloat16* v_out, float* rms_q,
                             float* rms_k, const InT* __restrict__ q, const InT* __restrict__ k,
                             const InT* __restrict__ v, const float* __restrict__ cos_buf,
                             const float* __restrict__ sin_buf, long long rows, int num_heads, long long seq_len,
                             float eps) {
  const int which = blockIdx.y;   // 0: q, 1: k, 2: v
  const InT* in = which == 0 ? q : (which == 1 ? k : v);
  __nv_bfloat16* out = which == 0 ? q_out : (which == 1 ? k_out : v_out);
  float* rms_out = which == 0 ? rms_q : (which == 1 ? rms_k : nullptr);
  const long long total = rows * 8;   // a multiple of 8: the 8 threads of a row always run together
  for (long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x; tid < total;
       tid += (long long)gridDim.x * blockDim.x) {
    const long long row = tid >> 3;
    const int g = static_cast<int>(tid & 7);
    const long long base = row * 128 + g * 8;
    const float4 a0 = Vec4<InT>::load(in + base), a1 = Vec4<InT>::load(in + base + 4);
    const float4 b0 = Vec4<InT>::load(in + base + 64), b1 = Vec4<InT>::load(in + base + 68);
    float x1[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
    float x2[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
    if (which < 2) {
      const long long token = row / num_heads;
      const long long pos = seq_len > 0 ? token % seq_len : token;
      const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_buf + pos * 64 + g * 8));
      const float4 c1 = __ldg(reinterpret_cast<const float4*>(cos_buf + pos * 64 + g * 8 + 4));
      const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_buf + pos * 64 + g * 8));
      const float4 s1 = __ldg(reinterpret_cast<const float4*>(sin_buf + pos * 64 + g * 8 + 4));
      const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
      const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float y1 = x1[i] * cs[i] + x2[i] * sn[i];    // ops.mojo:237-238
        const float y2 = x2[i] * cs[i] - x1[i] * sn[i];
        x1[i] = y1;
        x2[i] = y2;
        ss += y1 * y1 + y2 * y2;
      }
      // the 8 threads of a row are 8 consecutive lanes of one warp
      ss += __shfl_xor_sync(0xffffffffu, ss, 1);
      ss += __shfl_xor_sync(0xffffffffu, ss, 2);
      ss += __shfl_xor_sync(0xffffffffu, ss, 4);
      const float rms = sqrtf(ss * (1.0f / 128.0f) + eps);  // ops.mojo:96-97
      if (rms_out != nullptr && g == 0) rms_out[row] = rms;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        x1[i] = x1[i] / rms;                                 // ops.mojo:101-102 divides
        x2[i] = x2[i] / rms;
      }
    }
    *reinterpret_cast<uint4*>(out + base) = make_uint4(pack_bf16x2(x1[0], x1[1]), pack_bf16x2(x1[2], x1[3]),
                                                       pack_bf16x2(x1[4], x1[5]), pack_bf16x2(x1[6], x1[7]));
    *reinterpret_cast<uint4*>(out + base + 64) = make_uint4(pack_bf16x2(x2[0], x2[1]), pack_bf16x2(x2[2], x2[3]),
                                                            pack_bf16x2(x2[4], x2[5]), pack_bf16x2(x2[6], x2[7]));
  }
}

template <typename InT>
cudaError_t launch_qk_norm_rope_cast_128(__nv_bfloat16* q_out, __nv_bfloat16* k_out, __nv_bfloat16* v_out, float* rms_q,
                                         float* rms_k, const InT* q, const InT* k, const InT* v,
                                         const float* cos_buf, const float* sin_buf, long long rows, int num_heads,
                                         long long seq_len, float eps, cudaStream_t stream) {
  long long blocks = (rows * 8 + 255) / 256;
  const long long cap = 148LL * 16;   // grid-stride beyond 16 blocks (of 256 threads) per SM
  dim3 grid(static_cast<unsigned>(blocks < 1 ? 1 : (blocks > cap ? cap : blocks)), v != nullptr ? 3 : 2);
  qk_norm_rope_cast_128_kernel<InT><<<grid, 256, 0, stream>>>(q_out, k_out, v_out, rms_q, rms_k, q, k, v, cos_buf, sin_buf,
                                                              rows, num_heads, seq_len, eps);
  return cudaGetLastError();
}
template cudaError_t launch_qk_norm_rope_cast_128<float>(__nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, float*, float*,
                                                         const float*, const float*, const float*, const float*,
                                                         const float*, long long, int, long long, float, cudaStream_t);
template cudaError_t launch_qk_norm_rope_cast_128<__nv_bfloat16>(__nv_bfloat16*, __nv_bfloat16*, __nv_bfloat16*, float*, float*,
                                                                 const __nv_bfloat16*, const __nv_bfloat16*,
                                                                 const __nv_bfloat16*, const float*, const float*,
                                                                 long long, int, long long, float, cudaStream_t);

// Scalar form for head dims whose half is not a multiple of 4 (fp32 only; the rope mirrors).
__global__ void __launch_bounds__(256)
rope_scalar_kernel(float* out, const float* in,
                   const float* __restrict__ cos_buf, const float* __restrict__ sin_buf,
                   long long rows, int num_heads, int half, long long seq_len, int mode) {
  const long long total = rows * half;
  for (long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x; tid < total;
       tid += (long long)gridDim.x * blockDim.x) {
    const long long row = tid / half;
    const int d = static_cast<int>(tid - row * half);
    const long long token = row / num_heads;
    const long long pos = seq_len > 0 ? token % seq_len : token;
    const float x1 = in[row * 2 * half + d], x2 = in[row * 2 * half + half + d];
    const float c = cos_buf[pos * half + d];
    const float s = mode == kRopeBwd ? -sin_buf[pos * half + d] : sin_buf[pos * half + d];
    out[row * 2 * half + d] = x1 * c + x2 * s;
    out[row * 2 * half + half + d] = x2 * c - x1 * s;
  }
}

static int grid_for(long long total, int block) {
  long long g = (total + block - 1) / block;
  const long long cap = 148LL * 32;  // grid-stride beyond 32 blocks per SM
  return static_cast<int>(g < 1 ? 1 : (g > cap ? cap : g));
}

template <typename InT, typename OutT>
cudaError_t launch_rope_cast(OutT* out, const InT* in, const float* cos_buf, const float* sin_buf,
                             long long rows, int num_heads, int head_dim, long long seq_len,
                             int mode, cudaStream_t stream, RowMap in_map, RowMap out_map) {
  const int half = head_dim / 2;
  const long long total = rows * (half >> 2);
  rope_cast_kernel<InT, OutT><<<grid_for(total, 256), 256, 0, stream>>>(
      out, in, cos_buf, sin_buf, rows, num_heads, half, seq_len, mode, in_map, out_map);
  return cudaGetLastError();
}
cudaError_t launch_rope_pair_bf16_128(__nv_bfloat16* out0, const __nv_bfloat16* in0, __nv_bfloat16* out1,
                                      const __nv_bfloat16* in1, const float* cos_buf, const float* sin_buf,
                                      long long tokens, int num_heads, long long seq_len, cudaStream_t stream,
                                      RowMap in_map, RowMap out_map) {
  dim3 grid(grid_for(tokens * 8, 256), 2);
  rope_pair_bf16_128_kernel<<<grid, 256, 0, stream>>>(out0, in0, out1, in1, cos_buf, sin_buf, tokens, num_heads,
                                                      seq_len, in_map, out_map);
  return cudaGetLastError();
}
template cudaError_t launch_rope_cast<float, float>(float*, const float*, const float*, const float*,
                                                    long long, int, int, long long, int, cudaStream_t, RowMap, RowMap);
template cudaError_t launch_rope_cast<float, __nv_bfloat16>(__nv_bfloat16*, const float*, const float*,
                                                            const float*, long long, int, int,
                                                            long long, int, cudaStream_t, RowMap, RowMap);
template cudaError_t launch_rope_cast<__nv_bfloat16, __nv_bfloat16>(__nv_bfloat16*, const __nv_bfloat16*,
                                                                    const float*, const float*,
                                                                    long long, int, int, long long,
                                                                    int, cudaStream_t, RowMap, RowMap);

cudaError_t launch_rope_scalar(float* out, const float* in, const float* cos_buf,
                               const float* sin_buf, long long rows, int num_heads, int head_dim,
                               long long seq_len, int mode, cudaStream_t stream) {
  const int half = head_dim / 2;
  rope_scalar_kernel<<<grid_for(rows * half, 256), 256, 0, stream>>>(out, in, cos_buf, sin_buf, rows,
                                                                     num_heads, half, seq_len, mode);
  return cudaGetLastError();
}

// D[row] = sum_d O[row,d] * dO[row,d] (ops.mojo:343-346), fp32 accumulation.  Each thread takes 16
// bytes of O and of dO per step; a row of 128 elements is covered by 16 (bf16) or 32 (fp32)
// adjacent lanes, which then combine their partial sums with shuffles.  head_dim = 128 path.
template <typename T>
__global__ void __launch_bounds__(256)
precompute_d128_kernel(float* __restrict__ d_out, const T* __restrict__ o, const T* __restrict__ d_o,
                       long long rows, const RowMap map) {
  constexpr int kPer = 16 / sizeof(T);       // elements per thread: 8 bf16 or 4 fp32
  constexpr int kLanes = 128 / kPer;         // threads per row: 16 or 32
  const long long tid0 = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const int seg = static_cast<int>(tid0 % kLanes);
  const long long rows_per_sweep = nthreads / kLanes;
  const long long n_iter = (rows + rows_per_sweep - 1) / rows_per_sweep;
  // every thread runs the same number of iterations (the shuffles need the full warp)
  for (long long i = 0; i < n_iter; ++i) {
    const long long row = tid0 / kLanes + i * rows_per_sweep;
    float acc = 0.f;
    const long long mrow = row < rows ? map_row(map, row) : 0;
    if (row < rows) {
      const uint4 a = *reinterpret_cast<const uint4*>(o + mrow * 128 + seg * kPer);
      const uint4 g = *reinterpret_cast<const uint4*>(d_o + mrow * 128 + seg * kPer);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (sizeof(T) == 2)
          acc += bf16_lo_to_f32(aw[i]) * bf16_lo_to_f32(gw[i]) + bf16_hi_to_f32(aw[i]) * bf16_hi_to_f32(gw[i]);
        else
          acc += __uint_as_float(aw[i]) * __uint_as_float(gw[i]);
      }
    }
#pragma unroll
    for (int off = kLanes / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (seg == 0 && row < rows) d_out[mrow] = acc;
  }
}

// Generic head_dim (a multiple of 4): one warp per row.
template <typename T>
__global__ void __launch_bounds__(256)
precompute_d_kernel(float* __restrict__ d_out, const T* __restrict__ o, const T* __restrict__ d_o,
                    long long rows, int head_dim, const RowMap map) {
  const int lane = threadIdx.x & 31;
  const long long warp0 = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = warp0; row < rows; row += nwarps) {
    const long long mrow = map_row(map, row);
    float acc = 0.f;
    for (int d = lane * 4; d < head_dim; d += 128) {
      const float4 a = Vec4<T>::load(o + mrow * head_dim + d);
      const float4 g = Vec4<T>::load(d_o + mrow * head_dim + d);
      acc += a.x * g.x + a.y * g.y + a.z * g.z + a.w * g.w;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    if (lane == 0) d_out[mrow] = acc;
  }
}

template <typename T>
cudaError_t launch_precompute_d(float* d_out, const T* o, const T* d_o, long long rows, int head_dim,
                                cudaStream_t stream, RowMap map) {
  if (head_dim == 128) {
    constexpr int kLanes = 128 / (16 / (int)sizeof(T));
    const long long threads = rows * kLanes;
    long long blocks = (threads + 255) / 256;
    const long long cap = 148LL * 16;
    if (blocks > cap) blocks = cap;
    precompute_d128_kernel<T><<<(int)(blocks < 1 ? 1 : blocks), 256, 0, stream>>>(d_out, o, d_o, rows, map);
  } else {
    precompute_d_kernel<T><<<grid_for(rows * 32, 256), 256, 0, stream>>>(d_out, o, d_o, rows, head_dim, map);
  }
  return cudaGetLastError();
}
template cudaError_t launch_precompute_d<float>(float*, const float*, const float*, long long, int,
                                                cudaStream_t, RowMap);
template cudaError_t launch_precompute_d<__nv_bfloat16>(float*, const __nv_bfloat16*,
                                                        const __nv_bfloat16*, long long, int,
                                                        cudaStream_t, RowMap);


// One thread per (b, h, tp): gathers LSE and D from [B,T,H] into [B,H,Tp] (coalesced writes).  The LSE
// is stored as the addend of the dK/dV kernel's exponent: kTruncGainLog2 - LSE * log2(e).
__global__ void __launch_bounds__(256)
stats_transpose_kernel(float* __restrict__ lse2_t, float* __restrict__ dvec_t, const float* __restrict__ lse,
                       const float* __restrict__ dvec, int B, int T, int H, int t_pad, const RowMap map) {
  const long long total = (long long)B * H * t_pad;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int tp = static_cast<int>(i % t_pad);
    const long long bh = i / t_pad;
    const int hh = static_cast<int>(bh % H);
    const long long bb = bh / H;
    float l = -INFINITY, d = 0.f;   // padding rows: exponent -inf, P = 0
    if (tp < T) {
      const long long src = map_row(map, (bb * T + tp) * H + hh);
      l = kTruncGainLog2 - lse[src] * kLog2e;
      d = dvec[src];
    }
    lse2_t[i] = l;
    dvec_t[i] = d;
  }
}

cudaError_t launch_stats_transpose(float* lse2_t, float* dvec_t, const float* lse, const float* dvec,
                                   int B, int T, int H, int t_pad, cudaStream_t stream, RowMap map) {
  stats_transpose_kernel<<<grid_for((long long)B * H * t_pad, 256), 256, 0, stream>>>(lse2_t, dvec_t, lse,
                                                                                      dvec, B, T, H, t_pad, map);
  return cudaGetLastError();
}

}  // namespace ar
