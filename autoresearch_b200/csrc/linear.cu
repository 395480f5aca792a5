// The projections either side of attention as tcgen05 GEMMs for sm_100a, replacing the
// reference's tiled matmuls linear_fwd, linear_bwd_dx and linear_bwd_dw (ops.mojo:110-203,
// 870-950, 953-1033; launched at model.mojo:643-645, 704 and 906-907, 967-990):
//   forward   Y[M,N]  = X[M,K] W[N,K]^T      A = X  (K-major),  B = W  (K-major),  depth K
//   dX        dX[M,K] = dY[M,N] W[N,K]       A = dY (K-major),  B = W  (MN-major), depth N
//   dW        dW[N,K] += dY[M,N]^T X[M,K]    A = dY (MN-major), B = X  (MN-major), depth M
// bf16 operands, fp32 accumulation in tensor memory.  What the reference documents is computed
// (its kernels leave three quarters of every output tile unwritten, ops.mojo:134-143, 188-203).
//
// One persistent kernel for the three: a CTA per SM walks output tiles of 128 x 256 (one
// tcgen05.mma shape, M=128 N=256 K=16), depth in stages of 64 through a 4-stage TMA ring
// (48 KB per stage: 16 KB of A, 32 KB of B, 128-byte swizzle).  Warp 0 issues the TMA loads, warp 1
// the MMAs (8 KB A + ... per instruction from shared memory: tensor-bound at N=256), warps 2-5 write
// finished tiles out.  The accumulator is double-buffered in tensor memory (2 x 256 columns), so the
// write-out of one tile overlaps the products of the next.
// A K-major operand tile is rows x 64 depth elements (one TMA box); an MN-major operand tile is
// 64 depth rows x 64-element column blocks (one box per block, LBO = one block), as TMA writes them.
// dW adds into its output (the reference accumulates gradients: model.mojo:826-827): its depth M
// is split into chunks over the CTAs and every chunk adds its partial tile with vector fp32
// reductions (red.global.add.v4.f32), so the sum over chunks is not in a fixed order.
#include "attn_common.cuh"

namespace ar {

constexpr int kLinStages = 4;
constexpr int kLinBM = 128, kLinBN = 256, kLinBK = 64;
constexpr int kLinThreads = 192;   // warp 0 TMA, warp 1 MMA issuer, warps 2-5 write-out
constexpr int kLinABytes = kLinBM * kLinBK * 2;   // 16 KB
constexpr int kLinBBytes = kLinBN * kLinBK * 2;   // 32 KB

struct LinSmem {
  alignas(1024) uint8_t a[kLinStages][kLinABytes];
  alignas(1024) uint8_t b[kLinStages][kLinBBytes];
  alignas(1024) uint8_t epi[4][2048];   // write-out transposition buffers, one per write-out warp
  alignas(8) uint64_t full[kLinStages], empty[kLinStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// One work item: output tile (ta, tb) and depth chunk ch.
struct LinItem {
  int row0, col0, d0, d1;
};
__device__ __forceinline__ LinItem lin_item(int item, const LinParams& p) {
  LinItem it;
  const int tiles_b = (p.cols_b + kLinBN - 1) / kLinBN;
  const int tiles = ((p.rows_a + kLinBM - 1) / kLinBM) * tiles_b;
  const int ch = item / tiles, t = item - ch * tiles;   // chunk-major: the tiles of one chunk run together
  it.row0 = (t / tiles_b) * kLinBM;
  it.col0 = (t % tiles_b) * kLinBN;
  it.d0 = ch * p.depth_chunk;
  it.d1 = min(p.depth, it.d0 + p.depth_chunk);
  return it;
}

// Adds 32 consecutive fp32 values per lane (lane = row of this warp's 32-row block) into global
// memory, full 128-byte lines per instruction, through the warp's 2 KB transposition buffer.
__device__ __forceinline__ void warp_red_32cols(uint32_t epi, int lane, const float (&v)[32], float* grow0,
                                                size_t row_stride_elems, int rows_valid) {
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
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t rl = 4 * k + (lane >> 3), j = lane & 7;
      const uint4 t = lds128(epi + rl * 128u + ((j ^ (rl & 7u)) << 4));
      const int row = 16 * half + (int)rl;
      if (row < rows_valid) {
        float* dst = grow0 + (size_t)row * row_stride_elems + j * 4;
        asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(__uint_as_float(t.x)),
                     "f"(__uint_as_float(t.y)), "f"(__uint_as_float(t.z)), "f"(__uint_as_float(t.w))
                     : "memory");
      }
    }
    __syncwarp();
  }
}

__global__ void __launch_bounds__(kLinThreads, 1)
linear_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const LinParams p,
              const int n_items) {
  extern __shared__ uint8_t smem_raw[];
  LinSmem& sm = *reinterpret_cast<LinSmem*>(align1024(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  WaitCtx w{p.status, smem_u32(&sm.abort_flag)};

  if (threadIdx.x == 0) {
    for (int s = 0; s < kLinStages; ++s) {
      mbar_init(smem_u32(&sm.full[s]), 1);
      mbar_init(smem_u32(&sm.empty[s]), 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.acc_full[i]), 1);
      mbar_init(smem_u32(&sm.acc_empty[i]), 4);   // the four write-out warps have read the accumulator
    }
    sm.abort_flag = 0u;
    fence_mbar_init();
    prefetch_tmap(&map_a);
    prefetch_tmap(&map_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&sm.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // an earlier abandoned wait (status word still set): the producer stays idle and everyone gives up
  if (threadIdx.x == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) sm.abort_flag = 1u;
  __syncthreads();
  const bool live = ld_shared_u32(smem_u32(&sm.abort_flag)) == 0u;
  const uint32_t tmem = sm.tmem_base;
  const bool a_mn = p.mode == 2, b_mn = p.mode != 0;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    int g = 0;
    bool ok = live;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x) {
      const LinItem it = lin_item(item, p);
      for (int d = it.d0; d < it.d1; d += kLinBK, ++g) {
        const int s = g % kLinStages;
        if (!mbar_wait(w, smem_u32(&sm.empty[s]), ((g / kLinStages) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t bar = smem_u32(&sm.full[s]);
          mbar_arrive_expect_tx(bar, kLinABytes + kLinBBytes);
          const uint32_t a = smem_u32(sm.a[s]), b = smem_u32(sm.b[s]);
          if (!a_mn) {
            tma_load_4d(a, &map_a, bar, d, 0, it.row0, 0);                    // 128 rows x 64 depth
          } else {
#pragma unroll
            for (int c = 0; c < 2; ++c) tma_load_4d(a + c * 8192, &map_a, bar, it.row0 + 64 * c, 0, d, 0);   // 64 depth rows x 64
          }
          if (!b_mn) {
            tma_load_4d(b, &map_b, bar, d, 0, it.col0, 0);                    // 256 rows x 64 depth
          } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) tma_load_4d(b + c * 8192, &map_b, bar, it.col0 + 64 * c, 0, d, 0);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    const uint32_t idesc = make_idesc_bf16(kLinBM, kLinBN, a_mn ? 1u : 0u, b_mn ? 1u : 0u);
    int g = 0, n = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++n) {
      const LinItem it = lin_item(item, p);
      const int buf = n & 1;
      // the write-out of the tile before the previous one has left this accumulator
      if (n >= 2 && !mbar_wait(w, smem_u32(&sm.acc_empty[buf]), ((n >> 1) - 1) & 1)) break;
      tc_fence_after();
      const uint32_t acc = tmem + buf * kLinBN;
      bool first = true;
      for (int d = it.d0; d < it.d1; d += kLinBK, ++g) {
        const int s = g % kLinStages;
        if (!mbar_wait(w, smem_u32(&sm.full[s]), (g / kLinStages) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t a = smem_u32(sm.a[s]), b = smem_u32(sm.b[s]);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t ad = a_mn ? make_sdesc_sw128(a + ks * 2048, 8192, 1024) : make_sdesc_sw128(a + ks * 32, 0, 1024);
          const uint64_t bd = b_mn ? make_sdesc_sw128(b + ks * 2048, 8192, 1024) : make_sdesc_sw128(b + ks * 32, 0, 1024);
          umma_ss_elect(acc, ad, bd, idesc, (first && ks == 0) ? 0u : 1u);
        }
        first = false;
        umma_commit_elect(smem_u32(&sm.empty[s]));
      }
      if (!ok) break;
      umma_commit_elect(smem_u32(&sm.acc_full[buf]));
    }
  } else {
    // ------------------------------------------------------------------ write-out warps
    const int q = warp & 3;   // TMEM lane quadrant of this warp: warps 2, 3, 4, 5 -> 2, 3, 0, 1
    const uint32_t lane_off = static_cast<uint32_t>(q * 32) << 16;
    const uint32_t epi = smem_u32(sm.epi[q]);
    const int esize = p.c_f32 ? 4 : 2;
    int n = 0;
    bool ok = true;
    for (int item = blockIdx.x; ok && item < n_items; item += gridDim.x, ++n) {
      const LinItem it = lin_item(item, p);
      const int buf = n & 1;
      if (!mbar_wait(w, smem_u32(&sm.acc_full[buf]), (n >> 1) & 1)) break;
      tc_fence_after();
      const uint32_t acc = tmem + buf * kLinBN + lane_off;
      const int wrow0 = it.row0 + 32 * q;
      const int rows_valid = p.rows_a - wrow0;
#pragma unroll 1
      for (int c = 0; c < kLinBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32_wait(acc + 32 * c, r);
        if (c == kLinBN / 32 - 1) {   // the accumulator may be overwritten
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm.acc_empty[buf]));
        }
        const int col = it.col0 + 32 * c;
        if (col >= p.cols_b) continue;   // whole 32-column chunks only: cols_b is a multiple of 32
        float v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
        if (p.accumulate) {
          warp_red_32cols(epi, lane, v, static_cast<float*>(p.c) + (size_t)wrow0 * p.ldc + col, (size_t)p.ldc, rows_valid);
        } else {
          warp_store_32cols(epi, lane, v, static_cast<uint8_t*>(p.c) + ((size_t)wrow0 * p.ldc + col) * esize,
                            (size_t)p.ldc * esize, rows_valid, p.c_f32);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  drain_if_aborted(w.abort_smem);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

cudaError_t launch_linear(const CUtensorMap& ma, const CUtensorMap& mb, const LinParams& p, cudaStream_t stream) {
  const size_t smem = sizeof(LinSmem) + 1024;
  static int sm_count_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int& sm_count = sm_count_dev[dev & 63];
  if (sm_count == 0) {
    cudaError_t e = cudaFuncSetAttribute(linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int tiles = ((p.rows_a + kLinBM - 1) / kLinBM) * ((p.cols_b + kLinBN - 1) / kLinBN);
  const int chunks = (p.depth + p.depth_chunk - 1) / p.depth_chunk;
  const int n_items = tiles * chunks;
  const int grid = n_items < sm_count ? n_items : sm_count;
  linear_kernel<<<grid, kLinThreads, smem, stream>>>(ma, mb, p, n_items);
  return cudaGetLastError();
}

}  // namespace ar
