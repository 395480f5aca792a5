// Shared constants, parameter blocks and smem helpers of the attention kernels.
#pragma once
#include "ptx.cuh"

namespace ar {

constexpr int kTile = 128;          // rows per MMA tile (queries or keys)
constexpr int kHeadDim = 128;       // the only supported head_dim (ops.mojo:267, 285)
constexpr int kHalfBytes = 16384;   // 128 rows x 64 bf16: one TMA box
constexpr int kTileBytes = 32768;   // 128 rows x 128 bf16: two boxes (d 0..63, d 64..127)
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnDims {
  int B, T, H;
  int window;  // normalised: 0 = full causal, else 1 <= window <= T-1 (keys q-window .. q)
  // Layout of the caller's tensors in rows of head_dim elements: row (b, t, h) is row
  // b * pitch_b + t * pitch_t + h of q, k, v, o, dO and the gradients, and element
  // b * pitch_b + t * pitch_t + h of LSE and D.  Contiguous [B,T,H,D]: pitch_t = H, pitch_b = T * H;
  // a head range cut out of a wider tensor keeps the wider tensor's pitches.
  int pitch_t;
  long long pitch_b;
};
__host__ __device__ __forceinline__ size_t row_of(const AttnDims& d, int b, int t, int h) {
  return (size_t)b * (size_t)d.pitch_b + (size_t)t * (size_t)d.pitch_t + (size_t)h;
}

// How a helper kernel finds row r = (b * T + t) * H + h of one of its tensors: T == 0 means the
// tensor is contiguous (row r is row r), otherwise the pitches above apply.
struct RowMap {
  int T = 0, H = 0, pitch_t = 0;
  long long pitch_b = 0;
};
__host__ __device__ __forceinline__ long long map_row(const RowMap& m, long long r) {
  if (m.T == 0) return r;
  const long long token = r / m.H, h = r - token * m.H;
  const long long b = token / m.T, t = token - b * m.T;
  return b * m.pitch_b + t * m.pitch_t + h;
}


// ---- kernel parameter blocks and launchers (definitions in attn_fwd.cu / attn_bwd.cu /
// ---- elementwise.cu) -----------------------------------------------------------------
struct FwdParams {
  AttnDims dims;
  float scale;        // 1/sqrt(D)
  float scale_log2e;  // scale * log2(e)
  void* o;            // [B,T,H,D] bf16 or fp32
  int o_f32;
  float* lse;         // [B,T,H]
  const float* cos_buf;  // [rows >= T, 64]; non-null selects rotate-on-load
  const float* sin_buf;
  uint32_t* status;
};

struct BwdParams {
  AttnDims dims;
  float scale;
  float scale_log2e;
  const float* lse;    // [B,T,H] natural log of the scaled scores
  const float* dvec;   // [B,T,H] D = rowsum(O * dO)
  const float* lse2_t; // [B,H,Tp] kTruncGainLog2 - LSE * log2(e), Tp = T rounded up to 64, padded with -inf
  const float* dvec_t; // [B,H,Tp] D, padded with 0      (both only read by the dK/dV kernel)
  // Non-null: the dQ kernel computes D = rowsum(O * dO) itself from this bf16 O (and its resident dO
  // tile), writes it to d_out and writes both key-stationary arrays for the dK/dV kernel that follows.
  const __nv_bfloat16* o_for_d;
  const __nv_bfloat16* do_for_d;   // dO in global memory (the tensor behind the dO map)
  float* d_out;        // [B,T,H]
  float* lse2_t_out;   // [B,H,Tp]
  float* dvec_t_out;   // [B,H,Tp]
  int t_pad;           // Tp
  void* dq;            // [B,T,H,D]
  void* dk;
  void* dv;
  int grad_f32;        // element type of dq/dk/dv
  const float* cos_buf;  // non-null: apply rope_bwd to dq / dk with position t
  const float* sin_buf;
  uint32_t* status;
};

enum RopeMode { kCastOnly = 0, kRopeFwd = 1, kRopeBwd = 2 };

cudaError_t launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                            const FwdParams& p, bool rope, cudaStream_t stream);
cudaError_t launch_attn_bwd_dq(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                               const CUtensorMap& mdo, const BwdParams& p, cudaStream_t stream);
cudaError_t launch_attn_bwd_dkv(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                                const CUtensorMap& mdo, const BwdParams& p, cudaStream_t stream);
template <typename InT, typename OutT>
cudaError_t launch_rope_cast(OutT* out, const InT* in, const float* cos_buf, const float* sin_buf,
                             long long rows, int num_heads, int head_dim, long long seq_len,
                             int mode, cudaStream_t stream, RowMap in_map = RowMap(), RowMap out_map = RowMap());
// Forward rotation of bf16 Q and K ([tokens, H, 128] each) in one launch.
cudaError_t launch_rope_pair_bf16_128(__nv_bfloat16* out0, const __nv_bfloat16* in0, __nv_bfloat16* out1,
                                      const __nv_bfloat16* in1, const float* cos_buf, const float* sin_buf,
                                      long long tokens, int num_heads, long long seq_len, cudaStream_t stream,
                                      RowMap in_map = RowMap(), RowMap out_map = RowMap());
// rope_fwd + per-head rmsnorm_fwd on q, k and the bf16 cast of q, k, v in one launch (head_dim 128);
// v / v_out may be null (q and k only); rms_q / rms_k may be null.
template <typename InT>
cudaError_t launch_qk_norm_rope_cast_128(__nv_bfloat16* q_out, __nv_bfloat16* k_out, __nv_bfloat16* v_out, float* rms_q,
                                         float* rms_k, const InT* q, const InT* k, const InT* v,
                                         const float* cos_buf, const float* sin_buf, long long rows, int num_heads,
                                         long long seq_len, float eps, cudaStream_t stream);
cudaError_t launch_rope_scalar(float* out, const float* in, const float* cos_buf,
                               const float* sin_buf, long long rows, int num_heads, int head_dim,
                               long long seq_len, int mode, cudaStream_t stream);
template <typename T>
cudaError_t launch_precompute_d(float* d_out, const T* o, const T* d_o, long long rows, int head_dim,
                                cudaStream_t stream, RowMap map = RowMap());
// [B,T,H] LSE and D -> key-stationary layout [B,H,Tp]: LSE * log2(e) (pad +inf) and D (pad 0).
cudaError_t launch_stats_transpose(float* lse2_t, float* dvec_t, const float* lse, const float* dvec,
                                   int B, int T, int H, int t_pad, cudaStream_t stream, RowMap map = RowMap());

// The projection GEMMs (linear.cu): C[rows_a, cols_b] (+)= A B over `depth`, in one of three operand
// arrangements (mode 0: Y = X W^T, 1: dX = dY W, 2: dW += dY^T X).
struct LinParams {
  int mode;
  int rows_a, cols_b, depth;
  int depth_chunk;   // depth handled by one work item (a multiple of 64; < depth only for mode 2)
  void* c;           // output, row-major, leading dimension ldc elements
  int c_f32;         // element type of c (mode 2: always fp32)
  int ldc;
  int accumulate;    // add into c with fp32 reductions instead of storing (mode 2)
  uint32_t* status;
};
cudaError_t launch_linear(const CUtensorMap& map_a, const CUtensorMap& map_b, const LinParams& p, cudaStream_t stream);

// Launches a persistent kernel with programmatic stream serialization allowed (see ptx.cuh).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = AR_PDL;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) &
                                    ~static_cast<uintptr_t>(1023));
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared::cta.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared::cta.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// Rotate row `row` of a 128x128 bf16 tile in shared memory (two swizzled 64-column
// halves at tile_addr and tile_addr + kHalfBytes) by the RoPE angle of position `pos`:
//   forward (ops.mojo:237-238):  y1 = x1*c + x2*s ; y2 = -x1*s + x2*c
// with x1 = columns [0,64), x2 = columns [64,128) and c, s = cos/sin[pos, 0..63].
// A column pair (d, d+64) sits at the same swizzled offset of the two halves.
__device__ __forceinline__ void rope_rotate_row_smem(uint32_t tile_addr, uint32_t row,
                                                     const float* __restrict__ cos_row,
                                                     const float* __restrict__ sin_row) {
#pragma unroll 2
  for (uint32_t c = 0; c < 8; ++c) {
    const uint32_t off = row * 128u + ((c ^ (row & 7u)) << 4);
    uint4 a = lds128(tile_addr + off);
    uint4 b = lds128(tile_addr + kHalfBytes + off);
    const float4 c0 = __ldg(reinterpret_cast<const float4*>(cos_row + c * 8));
    const float4 c1 = __ldg(reinterpret_cast<const float4*>(cos_row + c * 8 + 4));
    const float4 s0 = __ldg(reinterpret_cast<const float4*>(sin_row + c * 8));
    const float4 s1 = __ldg(reinterpret_cast<const float4*>(sin_row + c * 8 + 4));
    const float cs[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    uint32_t aw[4] = {a.x, a.y, a.z, a.w};
    uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float x1l = bf16_lo_to_f32(aw[i]), x1h = bf16_hi_to_f32(aw[i]);
      const float x2l = bf16_lo_to_f32(bw[i]), x2h = bf16_hi_to_f32(bw[i]);
      const float y1l = x1l * cs[2 * i] + x2l * sn[2 * i];
      const float y1h = x1h * cs[2 * i + 1] + x2h * sn[2 * i + 1];
      const float y2l = x2l * cs[2 * i] - x1l * sn[2 * i];
      const float y2h = x2h * cs[2 * i + 1] - x1h * sn[2 * i + 1];
      aw[i] = pack_bf16x2(y1l, y1h);
      bw[i] = pack_bf16x2(y2l, y2h);
    }
    sts128(tile_addr + off, make_uint4(aw[0], aw[1], aw[2], aw[3]));
    sts128(tile_addr + kHalfBytes + off, make_uint4(bw[0], bw[1], bw[2], bw[3]));
  }
}

// Copies rows [r0, r0 + 32) of one staged 128-byte column block (row r at r * 128 bytes, its 16-byte
// chunk j at position j ^ (r & 7)) to global
// memory with plain vector stores, NJ 16-byte chunks per row starting at chunk j0: each instruction
// writes 32 / NJ complete row segments.  Called by the warp that staged these rows (after a
// __syncwarp), so no CTA-wide barrier is needed, and nothing has to be waited for afterwards: the
// data is in registers when the stores issue, unlike a bulk store, whose read of shared memory the
// CTA would have to outwait before it may exit.
template <int NJ>
__device__ __forceinline__ void store_staged_rows(uint32_t block_addr, int r0, int lane, int j0, uint8_t* gblock,
                                                  size_t row_stride_bytes, int rows_valid) {
  constexpr int kRowsPerInstr = 32 / NJ;
  uint4 v[NJ];
#pragma unroll
  for (int k = 0; k < NJ; ++k) {
    const uint32_t row = r0 + kRowsPerInstr * k + lane / NJ;
    const uint32_t j = j0 + lane % NJ;
    v[k] = lds128(block_addr + row * 128u + ((j ^ (row & 7u)) << 4));
  }
#pragma unroll
  for (int k = 0; k < NJ; ++k) {
    const int row = r0 + kRowsPerInstr * k + lane / NJ;
    const int j = j0 + lane % NJ;
    if (row < rows_valid) *reinterpret_cast<uint4*>(gblock + (size_t)row * row_stride_bytes + j * 16) = v[k];
  }
}

// Writes 32 consecutive values per lane (lane = row of this warp's 32-row block; first output
// column at byte offset 0 of `grow0`) as fp32 or bf16 through the warp's 2 KB transposition buffer.
// An SM retires only about 32 bytes of global stores per clock, and half that when a store
// instruction is made of 64-byte pieces, so fp32 rows go out as full 128-byte lines: the two
// half-warps stage their 16 rows in turn (16-byte chunks XOR-swizzled by the row), and each store
// instruction writes four complete rows.  bf16 rows (64 bytes) go out in one pass of eight rows per
// instruction.
__device__ __forceinline__ void warp_store_32cols(uint32_t epi, int lane, const float (&v)[32], uint8_t* grow0,
                                                  size_t row_stride_bytes, int rows_valid, int out_f32) {
  if (out_f32) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if ((lane >> 4) == half) {
        const uint32_t rl = lane & 15;
#pragma unroll
        for (uint32_t j = 0; j < 8; ++j)
          sts128(epi + rl * 128u + ((j ^ (rl & 7u)) << 4),
                 make_uint4(__float_as_uint(v[4 * j]), __float_as_uint(v[4 * j + 1]), __float_as_uint(v[4 * j + 2]),
                            __float_as_uint(v[4 * j + 3])));
      }
      __syncwarp();
      uint4 t[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t rl = 4 * k + (lane >> 3), j = lane & 7;
        t[k] = lds128(epi + rl * 128u + ((j ^ (rl & 7u)) << 4));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int row = 16 * half + 4 * k + (lane >> 3), j = lane & 7;
        if (row < rows_valid) *reinterpret_cast<uint4*>(grow0 + (size_t)row * row_stride_bytes + j * 16) = t[k];
      }
      __syncwarp();
    }
  } else {
    const uint32_t wsw = (lane >> 1) & 3u;
#pragma unroll
    for (uint32_t j = 0; j < 4; ++j)
      sts128(epi + lane * 64u + ((j ^ wsw) << 4),
             make_uint4(pack_bf16x2(v[8 * j], v[8 * j + 1]), pack_bf16x2(v[8 * j + 2], v[8 * j + 3]),
                        pack_bf16x2(v[8 * j + 4], v[8 * j + 5]), pack_bf16x2(v[8 * j + 6], v[8 * j + 7])));
    __syncwarp();
    uint4 t[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t row = 8 * k + (lane >> 2), j = lane & 3;
      t[k] = lds128(epi + row * 64u + ((j ^ ((row >> 1) & 3u)) << 4));
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int row = 8 * k + (lane >> 2), j = lane & 3;
      if (row < rows_valid) *reinterpret_cast<uint4*>(grow0 + (size_t)row * row_stride_bytes + j * 16) = t[k];
    }
    __syncwarp();
  }
}

// In-register inverse rotation of a full fp32 row (rope_bwd, ops.mojo:1119-1120):
//   dx1 = dy1*c - dy2*s ; dx2 = dy1*s + dy2*c
__device__ __forceinline__ void rope_bwd_pair(float& g1, float& g2, float c, float s) {
  const float a = g1 * c - g2 * s;
  const float b = g1 * s + g2 * c;
  g1 = a;
  g2 = b;
}

// Write-out of the column pairs (d, d + 64), d in [col0, col0 + 16), of a warp's 32 rows (lane = row)
// with the inverse rotation of rope_bwd (ops.mojo:1119-1120) applied AFTER the transposition, where a
// lane holds four consecutive columns of one row: the cos / sin values it needs are then 16 bytes that
// eight rows' worth of lanes fetch as whole 64-byte segments (`cs`, `sn`: fetched by the caller with
// rot_table_fetch, early, so that their latency is hidden), instead of every lane gathering its own
// row of the table (32 lines per instruction, several thousand cycles per item).  The rows leave 16
// at a time through 2 KB of the warp's buffer (1 KB per half of the pair); fp32 rows as 64-byte
// segments, bf16 rows as 32-byte segments.
struct RotTable {
  float4 c[2][2], s[2][2];   // [16-row half][8-row group]
};
__device__ __forceinline__ void rot_table_fetch(RotTable& t, const float* cos_buf, const float* sin_buf, int row0_warp,
                                                int lane, int col0, int T) {
#pragma unroll
  for (int h = 0; h < 2; ++h)
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int pos = min(row0_warp + 16 * h + 8 * k + (lane >> 2), T - 1);
      const size_t off = (size_t)pos * 64 + col0 + 4 * (lane & 3);
      t.c[h][k] = __ldg(reinterpret_cast<const float4*>(cos_buf + off));
      t.s[h][k] = __ldg(reinterpret_cast<const float4*>(sin_buf + off));
    }
}
template <bool kRot>
__device__ __forceinline__ void warp_store_pair16(uint32_t epi, int lane, const float (&lo)[16], const float (&hi)[16],
                                                  const RotTable& rot, uint8_t* grow0, size_t row_stride_bytes,
                                                  int col0, int rows_valid, int out_f32) {
  const int esize = out_f32 ? 4 : 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if ((lane >> 4) == h) {
      const uint32_t rl = lane & 15, wsw = (rl >> 1) & 3u;
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        sts128(epi + rl * 64u + ((j ^ wsw) << 4),
               make_uint4(__float_as_uint(lo[4 * j]), __float_as_uint(lo[4 * j + 1]), __float_as_uint(lo[4 * j + 2]),
                          __float_as_uint(lo[4 * j + 3])));
        sts128(epi + 1024u + rl * 64u + ((j ^ wsw) << 4),
               make_uint4(__float_as_uint(hi[4 * j]), __float_as_uint(hi[4 * j + 1]), __float_as_uint(hi[4 * j + 2]),
                          __float_as_uint(hi[4 * j + 3])));
      }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint32_t rl = 8 * k + (lane >> 2), j = lane & 3;
      const uint32_t off = rl * 64u + ((j ^ ((rl >> 1) & 3u)) << 4);
      const uint4 a = lds128(epi + off), b = lds128(epi + 1024u + off);
      float x[4] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w)};
      float y[4] = {__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w)};
      if (kRot) {
        const float4 c = rot.c[h][k], s = rot.s[h][k];
        rope_bwd_pair(x[0], y[0], c.x, s.x);
        rope_bwd_pair(x[1], y[1], c.y, s.y);
        rope_bwd_pair(x[2], y[2], c.z, s.z);
        rope_bwd_pair(x[3], y[3], c.w, s.w);
      }
      const int row = 16 * h + (int)rl;
      if (row < rows_valid) {
        uint8_t* g = grow0 + (size_t)row * row_stride_bytes + (size_t)(col0 + 4 * j) * esize;
        if (out_f32) {
          *reinterpret_cast<float4*>(g) = make_float4(x[0], x[1], x[2], x[3]);
          *reinterpret_cast<float4*>(g + 64 * 4) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
          *reinterpret_cast<uint2*>(g) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
          *reinterpret_cast<uint2*>(g + 64 * 2) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
        }
      }
    }
    __syncwarp();
  }
}
// The same with the rotation decided at run time (one copy of the code for rotated and plain rows).
__device__ __forceinline__ void warp_store_pair16_rt(bool rot_on, uint32_t epi, int lane, const float (&lo)[16],
                                                     const float (&hi)[16], const RotTable& rot, uint8_t* grow0,
                                                     size_t row_stride_bytes, int col0, int rows_valid, int out_f32) {
  const int esize = out_f32 ? 4 : 2;
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    if ((lane >> 4) == h) {
      const uint32_t rl = lane & 15, wsw = (rl >> 1) & 3u;
#pragma unroll
      for (uint32_t j = 0; j < 4; ++j) {
        sts128(epi + rl * 64u + ((j ^ wsw) << 4),
               make_uint4(__float_as_uint(lo[4 * j]), __float_as_uint(lo[4 * j + 1]), __float_as_uint(lo[4 * j + 2]),
                          __float_as_uint(lo[4 * j + 3])));
        sts128(epi + 1024u + rl * 64u + ((j ^ wsw) << 4),
               make_uint4(__float_as_uint(hi[4 * j]), __float_as_uint(hi[4 * j + 1]), __float_as_uint(hi[4 * j + 2]),
                          __float_as_uint(hi[4 * j + 3])));
      }
    }
    __syncwarp();
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const uint32_t rl = 8 * k + (lane >> 2), j = lane & 3;
      const uint32_t off = rl * 64u + ((j ^ ((rl >> 1) & 3u)) << 4);
      const uint4 a = lds128(epi + off), b = lds128(epi + 1024u + off);
      float x[4] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w)};
      float y[4] = {__uint_as_float(b.x), __uint_as_float(b.y), __uint_as_float(b.z), __uint_as_float(b.w)};
      if (rot_on) {
        const float4 c = rot.c[h][k], s = rot.s[h][k];
        rope_bwd_pair(x[0], y[0], c.x, s.x);
        rope_bwd_pair(x[1], y[1], c.y, s.y);
        rope_bwd_pair(x[2], y[2], c.z, s.z);
        rope_bwd_pair(x[3], y[3], c.w, s.w);
      }
      const int row = 16 * h + (int)rl;
      if (row < rows_valid) {
        uint8_t* g = grow0 + (size_t)row * row_stride_bytes + (size_t)(col0 + 4 * j) * esize;
        if (out_f32) {
          *reinterpret_cast<float4*>(g) = make_float4(x[0], x[1], x[2], x[3]);
          *reinterpret_cast<float4*>(g + 64 * 4) = make_float4(y[0], y[1], y[2], y[3]);
        } else {
          *reinterpret_cast<uint2*>(g) = make_uint2(pack_bf16x2(x[0], x[1]), pack_bf16x2(x[2], x[3]));
          *reinterpret_cast<uint2*>(g + 64 * 2) = make_uint2(pack_bf16x2(y[0], y[1]), pack_bf16x2(y[2], y[3]));
        }
      }
    }
    __syncwarp();
  }
}


// Static schedule of a persistent kernel: round k hands the items [k*G, (k+1)*G) to the G CTAs, in
// CTA order in even rounds and in reverse order in odd rounds, so that with items sorted by
// decreasing work every CTA alternates between the heavy and the light end of a round.  Returns the
// item of this CTA in round k, -2 if the round has none for it, -1 when all rounds are done.
__device__ __forceinline__ int sched_item(int k, int n_items) {
  const int G = gridDim.x, base = k * G;
  if (base >= n_items) return -1;
  const int idx = (k & 1) ? base + (G - 1 - (int)blockIdx.x) : base + (int)blockIdx.x;
  return idx < n_items ? idx : -2;
}

// Teardown shared by the tensor-core kernels: if any wait was abandoned, give copies
// and MMAs still in flight time to land before shared/tensor memory is released.
__device__ __forceinline__ void drain_if_aborted(uint32_t abort_smem) {
  if (ld_shared_u32(abort_smem) != 0u) {
    for (int i = 0; i < 64; ++i) __nanosleep(10000);
  }
}

}  // namespace ar
