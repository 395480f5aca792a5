// Known-answer kernel for the tcgen05 building blocks the attention kernels rely on.
// One CTA multiplies two 128x128 bf16 matrices held in global memory and writes the
// 128x128 fp32 product, exercising one operand-placement variant per launch:
//   a_mode 0: A from shared memory, K-major   (A_mem[m][k], k contiguous)
//   a_mode 1: A from shared memory, MN-major  (A_mem[k][m], m contiguous)
//   a_mode 2: A from tensor memory            (A_mem[m][k]; packed bf16x2 written with tcgen05.st)
//   b_mode 0: B K-major                       (B_mem[n][k], k contiguous)
//   b_mode 1: B MN-major                      (B_mem[k][n], n contiguous)
// In every case D[m][n] = sum_k A(m,k) * B(k,n).  Built into its own shared object
// that only the test-suite loads.
#include "ptx.cuh"

namespace ar {

constexpr int kKatThreads = 128;

struct KatSmem {
  alignas(1024) uint8_t a[2][16384];
  alignas(1024) uint8_t b[2][16384];
  alignas(8) uint64_t bar_load;
  alignas(8) uint64_t bar_mma;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

__global__ void __launch_bounds__(kKatThreads, 1)
kat_umma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                const __nv_bfloat16* a_gmem, float* out, int a_mode, int b_mode,
                uint32_t* status) {

  extern __shared__ uint8_t smem_raw[];
  KatSmem& sm = *reinterpret_cast<KatSmem*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const uint32_t warp = threadIdx.x >> 5;
  const uint32_t bar_load = smem_u32(&sm.bar_load);
  const uint32_t bar_mma = smem_u32(&sm.bar_mma);
  WaitCtx wctx{status, smem_u32(&sm.abort_flag)};

  if (threadIdx.x == 0) {
    mbar_init(bar_load, 1);
    mbar_init(bar_mma, 1);
    sm.abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&sm.tmem_base), 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sm.tmem_base;
  const uint32_t tmem_d = tmem;        // columns [0,128): fp32 accumulator
  const uint32_t tmem_a = tmem + 128;  // columns [128,192): A as packed bf16 (a_mode 2)

  if (threadIdx.x == 0) {
    uint32_t bytes = (a_mode == 2) ? 32768u : 65536u;
    mbar_arrive_expect_tx(bar_load, bytes);
    if (a_mode != 2) {
      tma_load_4d(smem_u32(sm.a[0]), &map_a, bar_load, 0, 0, 0, 0);
      tma_load_4d(smem_u32(sm.a[1]), &map_a, bar_load, 64, 0, 0, 0);
    }
    tma_load_4d(smem_u32(sm.b[0]), &map_b, bar_load, 0, 0, 0, 0);
    tma_load_4d(smem_u32(sm.b[1]), &map_b, bar_load, 64, 0, 0, 0);
  }
  if (a_mode == 2) {
    // Thread r owns row r of A: lane r of TMEM, column c holds elements (2c, 2c+1).
    const uint32_t row = threadIdx.x;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(a_gmem + row * 128);
    const uint32_t lane_addr = tmem_a + ((warp * 32u) << 16);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t regs[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) regs[i] = src[c * 16 + i];
      tmem_st16(lane_addr + c * 16, regs);
    }
    tmem_wait_st();
    tc_fence_before();
  }
  __syncthreads();

  bool ok = true;
  if (warp == 0) {
    ok = mbar_wait(wctx, bar_load, 0);
    tc_fence_after();
    if (ok && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(128, 128, a_mode == 1 ? 1u : 0u, b_mode == 1 ? 1u : 0u);
      const uint32_t a_base = smem_u32(sm.a[0]);
      const uint32_t b_base = smem_u32(sm.b[0]);
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        uint64_t bdesc = (b_mode == 0)
                             ? make_sdesc_sw128(b_base + (ks >> 2) * 16384 + (ks & 3) * 32, 0, 1024)
                             : make_sdesc_sw128(b_base + ks * 2048, 16384, 1024);
        if (a_mode == 2) {
          umma_ts(tmem_d, tmem_a + ks * 8, bdesc, idesc, ks > 0);
        } else {
          uint64_t adesc = (a_mode == 0)
                               ? make_sdesc_sw128(a_base + (ks >> 2) * 16384 + (ks & 3) * 32, 0, 1024)
                               : make_sdesc_sw128(a_base + ks * 2048, 16384, 1024);
          umma_ss(tmem_d, adesc, bdesc, idesc, ks > 0);
        }
      }
      umma_commit(bar_mma);
    }
    __syncwarp();
  }
  ok = mbar_wait(wctx, bar_mma, 0);
  tc_fence_after();
  if (ok) {
    const uint32_t row = threadIdx.x;
    const uint32_t lane_addr = tmem_d + ((warp * 32u) << 16);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      uint32_t regs[32];
      tmem_ld32_wait(lane_addr + c * 32, regs);
#pragma unroll
      for (int i = 0; i < 32; ++i) out[row * 128 + c * 32 + i] = __uint_as_float(regs[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

}  // namespace ar

#include "tmap.h"

// Test-only entry point.  a, b: device [128,128] bf16 row-major; out: device [128,128] fp32.
// status: device u32, zeroed by the caller.
extern "C" __attribute__((visibility("default"))) int32_t ar_kat_umma(const void* a, const void* b,
                                                                      float* out, int32_t a_mode,
                                                                      int32_t b_mode,
                                                                      uint32_t* status,
                                                                      void* stream) {
  CUtensorMap ma, mb;
  // Treat each matrix as a [B=1, T=128, H=1, D=128] tensor: box = 64 columns x 128 rows.
  if (!ar::make_tmap_bthd(&ma, a, 1, 128, 1, 128, 128)) return -3;
  if (!ar::make_tmap_bthd(&mb, b, 1, 128, 1, 128, 128)) return -3;
  size_t smem = sizeof(ar::KatSmem) + 1024;
  cudaError_t e = cudaFuncSetAttribute(ar::kat_umma_kernel,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return -3;
  ar::kat_umma_kernel<<<1, ar::kKatThreads, smem, (cudaStream_t)stream>>>(
      ma, mb, (const __nv_bfloat16*)a, out, a_mode, b_mode, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
