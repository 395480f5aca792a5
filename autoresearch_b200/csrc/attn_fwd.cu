// Forward attention for sm_100a: O = softmax(mask(Q K^T / sqrt(D))) V and the natural-log
// LSE of the scaled scores, replacing rope_fwd + flash_attn_fwd (ops.mojo:209-238, 244-323).
//
// Persistent kernel: one CTA per SM walks a static list of work items - 256 consecutive queries
// of one (batch, head): two 128-row tiles A and B - heaviest first.  The TMA warp and the MMA
// issuers run ahead into the next item while the softmax warps still write out the previous one.
// Warp roles:
//   warps 0-3   softmax of tile A (thread r = query row r: no shuffles needed for row
//               statistics because tcgen05.ld 32x32b hands each thread a whole row)
//   warps 4-7   softmax of tile B
//   warps 8-11  kRope: rotate each K tile in shared memory after it lands;
//               otherwise: write-out of both tiles (O / l, LSE), so that the softmax warps go
//               straight on to the next item
//   warp  12    TMA producer: Q per item, K/V tiles through a 2-stage ring that runs on across items
//   warps 13,14 tcgen05.mma issuers, one per Q tile (warp 13 owns the TMEM allocation)
// Registers are moved from the data-movement warpgroups to the softmax warpgroups
// (setmaxnreg), which hold a whole 128-column score row per thread.
// Tensor memory (512 columns): S_A [0,128) S_B [128,256) O_A [256,384) O_B [384,512);
// P (bf16) overwrites the first 64 columns of its S.
// Per KV tile j and Q tile X:  S_X = Q_X K_j^T (SS MMA)  ->  softmax warps read S_X, write
// P_X, rescale O_X  ->  O_X += P_X V_j (A operand from TMEM, V as MN-major B operand).
// KV tiles outside the causal / sliding-window band of a Q tile are never visited; only
// tiles crossed by a mask edge pay for element masking.
// At the end of an item the O rows are divided by the row sum and written out with plain coalesced
// stores through a per-warp transposition buffer.  Without rotate-on-load the otherwise idle
// warpgroup 8-11 does that: the softmax threads leave their row statistics in shared memory and
// start the next item at once, so the two tiles keep taking turns across item boundaries instead of
// one tile running alone (at the latency of its S -> P -> PV chain) while the other writes out.
// With rotate-on-load that warpgroup is busy and each softmax thread writes its own row out.
#include "attn_common.cuh"

namespace ar {

constexpr int kFwdStages = 2;
constexpr int kFwdThreads = 512;  // four warpgroups (see the role list above)
constexpr int kWarpRot0 = 8;      // warps 8-11: K rotation (idle without rotate-on-load)
constexpr int kWarpTma = 12;
constexpr int kWarpMma = 13;      // warps 13, 14: MMA issuers of tile A, tile B; warp 15 idle
// Largest growth of a row maximum (in log2 units of the scaled scores) that is absorbed
// without rescaling O: P is then computed against the stale maximum and stays <= 2^8.
constexpr float kLazyRescaleLog2 = 8.0f;

struct FwdSmem {
  alignas(1024) uint8_t q[2][kTileBytes];
  alignas(1024) uint8_t k[kFwdStages][kTileBytes];
  alignas(1024) uint8_t v[kFwdStages][kTileBytes];
  alignas(1024) uint8_t epi[8][4096];   // write-out transposition buffers, one per softmax warp
  alignas(8) uint64_t q_full, q_free;
  uint64_t q_ready[2];
  uint64_t k_full[kFwdStages], k_rot[kFwdStages], k_empty[kFwdStages];
  uint64_t v_full[kFwdStages], v_empty[kFwdStages];
  uint64_t s_full[2], p_ready[2][2], o_final[2], o_free[2];   // p_ready: one per 64-key half of P
  uint64_t stat_ready[2];   // the tile's row statistics of this item are in shared memory (write-out warps)
  uint32_t exp_cnt[2];   // per tile: exponential phases finished so far x 4 warps (monotonic)
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// One work item: 256 queries starting at q0 of head h of batch b; per Q tile X its KV tile range.
struct FwdItem {
  int q0, h, b;
  int jlo_t[2], jhi_t[2];   // jhi_t < jlo_t: tile inactive (past the end of the sequence)
  bool act[2];
  int jlo, jhi;             // union of the two ranges: the KV tiles the item streams
};
__device__ __forceinline__ FwdItem fwd_item(int item, const AttnDims& d, int n_qb) {
  FwdItem it;
  const int bh = d.B * d.H;
  const int qi = item / bh, r = item - qi * bh;   // items are ordered by query block, late (long) blocks first
  it.b = r / d.H;
  it.h = r - it.b * d.H;
  it.q0 = (n_qb - 1 - qi) * 256;
#pragma unroll
  for (int X = 0; X < 2; ++X) {
    const int qlo = it.q0 + kTile * X;
    it.act[X] = qlo < d.T;
    const int klo = d.window > 0 ? max(0, qlo - d.window) : 0;
    const int khi = min(qlo + kTile - 1, d.T - 1);
    it.jlo_t[X] = klo >> 7;
    it.jhi_t[X] = it.act[X] ? (khi >> 7) : (klo >> 7) - 1;
  }
  it.jlo = it.jlo_t[0];
  it.jhi = it.act[1] ? it.jhi_t[1] : it.jhi_t[0];
  return it;
}

template <bool kRope>
__global__ void __launch_bounds__(kFwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const FwdParams p, const int n_items, const int n_qb) {
  extern __shared__ uint8_t smem_raw[];
  FwdSmem& sm = *reinterpret_cast<FwdSmem*>(align1024(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int T = p.dims.T, window = p.dims.window;

  grid_dep_launch_dependents();   // all CTAs of this grid are resident: the next kernel may be scheduled
  WaitCtx w{p.status, smem_u32(&sm.abort_flag)};

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.q_full), 1);
    mbar_init(smem_u32(&sm.q_free), 2);          // each issuer has issued the item's last S product
    for (int X = 0; X < 2; ++X) {
      mbar_init(smem_u32(&sm.q_ready[X]), 128);
      mbar_init(smem_u32(&sm.s_full[X]), 1);
      // every softmax thread arrives (measured 8 % faster for the whole kernel than one elected
      // lane per warp behind a __syncwarp)
      mbar_init(smem_u32(&sm.p_ready[X][0]), 128);
      mbar_init(smem_u32(&sm.p_ready[X][1]), 128);
      mbar_init(smem_u32(&sm.o_final[X]), 1);
      mbar_init(smem_u32(&sm.o_free[X]), 4);       // the tile's O rows have left tensor memory
      mbar_init(smem_u32(&sm.stat_ready[X]), 4);
    }
    for (int s = 0; s < kFwdStages; ++s) {
      mbar_init(smem_u32(&sm.k_full[s]), 1);
      mbar_init(smem_u32(&sm.k_rot[s]), 128);
      mbar_init(smem_u32(&sm.k_empty[s]), 2);  // one release per Q tile
      mbar_init(smem_u32(&sm.v_full[s]), 1);
      mbar_init(smem_u32(&sm.v_empty[s]), 2);
    }
    sm.exp_cnt[0] = 0;
    sm.exp_cnt[1] = 0;
    sm.abort_flag = 0u;
    fence_mbar_init();
    prefetch_tmap(&map_q);
    prefetch_tmap(&map_k);
    prefetch_tmap(&map_v);
  }
  if (warp == kWarpMma) {
    tmem_alloc(smem_u32(&sm.tmem_base), 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dep_wait();   // everything above overlapped the previous kernel's tail; its results are visible from here
  // An earlier abandoned wait (this or a previous kernel's, status word still set): do no work.  The
  // word is read only now, when the previous kernel's writes are visible.  Without data from the TMA
  // warp no hand-shake of this CTA can complete, so it is enough that the producers stay idle: every
  // other role gives up at its first wait.
  if (threadIdx.x == 0 && *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) sm.abort_flag = 1u;
  __syncthreads();
  const bool live = ld_shared_u32(smem_u32(&sm.abort_flag)) == 0u;
  const uint32_t tmem = sm.tmem_base;

  if (warp < 8) {
    // ------------------------------------------------------------------ softmax warps
    if (kRope) setmaxnreg_inc<200>(); else setmaxnreg_inc<192>();   // without rotate-on-load the write-out warps take the difference
    const int X = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t tS = tmem + X * 128 + lane_off;
    const uint32_t tO = tmem + 256 + X * 128 + lane_off;
    const uint32_t s_full = smem_u32(&sm.s_full[X]);
    const uint32_t p_ready = smem_u32(&sm.p_ready[X][0]);
    const uint32_t epi = smem_u32(sm.epi[warp]);
    const f32x2 sc2 = f2_pack(p.scale_log2e, p.scale_log2e);
    // iterations done so far by this tile and by the other one, items in which this tile was
    // active, items: barrier phases follow these counts
    int g_own = 0, g_oth = 0, nx = 0, n = 0;
    bool ok = true;
    for (int kk = 0; ok; ++kk) {
      const int item = sched_item(kk, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const FwdItem wi = fwd_item(item, p.dims, n_qb);
      // constant indices only, so that the item stays in registers
      const bool act_x = X == 0 ? wi.act[0] : wi.act[1];
      const int jlo_x = X == 0 ? wi.jlo_t[0] : wi.jlo_t[1], jhi_x = X == 0 ? wi.jhi_t[0] : wi.jhi_t[1];
      const int n_it = act_x ? jhi_x - jlo_x + 1 : 0;
      const int n_other = X == 0 ? (wi.act[1] ? wi.jhi_t[1] - wi.jlo_t[1] + 1 : 0) : (wi.act[0] ? wi.jhi_t[0] - wi.jlo_t[0] + 1 : 0);
      if (!act_x) {
        // Ragged end of the sequence: this tile has no rows.  A parity wait is only valid for a
        // waiter that has seen the previous phase complete, so the idle tile still follows every
        // phase the other roles complete in this item.
        if (kRope && !mbar_wait(w, smem_u32(&sm.q_full), n & 1)) { ok = false; break; }
        g_oth += n_other;
        ++n;
        continue;
      }
      const int qlo = wi.q0 + kTile * X;
      const int qrow = qlo + r;
      if (kRope) {
        if (!mbar_wait(w, smem_u32(&sm.q_full), n & 1)) { ok = false; break; }
        if (qrow < T)
          rope_rotate_row_smem(smem_u32(sm.q[X]), r, p.cos_buf + (size_t)qrow * 64, p.sin_buf + (size_t)qrow * 64);
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&sm.q_ready[X]));
      }

      // m_ref: the reference maximum P is computed against (raw score units).  It trails the
      // true running maximum by at most kLazyRescaleLog2 (in log2 units after scaling).
      float m_ref = -INFINITY, l_run = 0.f;
      for (int it = 0; it < n_it; ++it) {
        const int kbase = (jlo_x + it) * kTile;
        // s_full's commit covers every MMA issued before it, so O_X += P V of the previous
        // step is complete as well once this wait returns.
        if (!mbar_wait(w, s_full, (g_own + it) & 1)) { ok = false; break; }
        tc_fence_after();
        uint32_t sr[128];
        tmem_ld128_wait(tS, sr);
        const bool edge_hi = kbase + kTile - 1 > qlo;
        const bool edge_lo = window > 0 && kbase < qlo + kTile - 1 - window;
        if (edge_hi || edge_lo) {
          const int hi = qrow - kbase;                                     // visible: col <= hi
          const int lo = window > 0 ? qrow - window - kbase : -(1 << 30);  // visible: col >= lo
          // The rows of a warp are consecutive, so a 32-column chunk that lane 0 sees up to its
          // last column (lane 31 from its first) is visible to the whole warp and is skipped; the
          // causal and the window edge are tested separately, one compare per element.
          const int hi0 = hi - lane, lo31 = lo - lane + 31;                // warp-uniform bounds
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int cb = 32 * c;
            if (edge_hi && cb + 31 > hi0) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cb + i > hi) sr[cb + i] = 0xff800000u;   // -inf
            }
            if (edge_lo && cb < lo31) {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (cb + i < lo) sr[cb + i] = 0xff800000u;
            }
          }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 128; i += 8) {
          mx0 = fmax3(mx0, __uint_as_float(sr[i]), __uint_as_float(sr[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(sr[i + 2]), __uint_as_float(sr[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(sr[i + 4]), __uint_as_float(sr[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(sr[i + 6]), __uint_as_float(sr[i + 7]));
        }
        const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
        // rescale only when the maximum grew by more than the lazy threshold
        float alpha = 1.f;
        if (mx > m_ref && (mx - m_ref) * p.scale_log2e > kLazyRescaleLog2) {
          alpha = ex2_approx((m_ref - mx) * p.scale_log2e);   // m_ref = -inf gives 0
          m_ref = mx;
        }
        // Rare: the running maximum outgrew the lazy threshold, rescale O before any P V of this
        // step is issued (the P V of the previous step is complete: s_full's commit covered it).
        if (it > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
          // 16 columns at a time: the score row already holds 128 registers
#pragma unroll 1
          for (int c = 0; c < 8; ++c) {
            uint32_t a[16];
            tmem_ld16_wait(tO + c * 16, a);
#pragma unroll
            for (int i = 0; i < 16; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * alpha);
            tmem_st16(tO + c * 16, a);
          }
        }
        // The exponential phases of the two tiles take turns (A0 B0 A1 B1 ...): left alone they
        // fall into step, both tiles competing for the special-function unit and then both
        // queueing their MMAs, so that neither unit ever overlaps the other.  Tile A opens an
        // item only after tile B has finished the previous one, which also keeps every waiter
        // within one phase of its barrier.
        // (monotonic counters, four increments per phase, rather than parity barriers: the idle
        // tile of a ragged item does not follow the other's phases, and a parity wait is only
        // valid for a waiter that has seen the previous phase complete)
        if (X == 0) {
          if (it == 0 || it - 1 < n_other) {
            if (!counter_wait(w, smem_u32(&sm.exp_cnt[1]), 4u * (uint32_t)(g_oth + it))) { ok = false; break; }
          }
        } else {
          if (it < n_other && !counter_wait(w, smem_u32(&sm.exp_cnt[0]), 4u * (uint32_t)(g_oth + it + 1))) { ok = false; break; }
        }
        // P = 2^(s*scale*log2e - m*scale*log2e) * kTruncGain, truncated to bf16 (see ptx.cuh).  Every
        // exponential is an ex2.approx: the special-function unit sustains about 31 per clock per SM
        // (rate probe), which is not what bounds this loop, and moving a share of them to a cubic on
        // the FMA pipe (tried at 1/8, 2/8, 3/8) only adds instructions.  Each 64-key half is handed to
        // the issuer as soon as it is written.
        const float neg_ms = ((m_ref == -INFINITY) ? 0.f : -m_ref * p.scale_log2e) + kTruncGainLog2;
        const f32x2 nm2 = f2_pack(neg_ms, neg_ms);
        f32x2 sum_a = 0ull, sum_b = 0ull;   // two lanes of +0.0f each
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t pk[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const f32x2 x = f2_fma(f2_pack_u(sr[c * 64 + 2 * i], sr[c * 64 + 2 * i + 1]), sc2, nm2);
            float x0, x1;
            f2_unpack(x, x0, x1);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            if (i & 1) sum_b = f2_add(sum_b, f2_pack(p0, p1));
            else sum_a = f2_add(sum_a, f2_pack(p0, p1));
            pk[i] = pack_bf16x2_trunc(p0, p1);
          }
          tmem_st32(tS + c * 32, pk);
          if (c == 1) {
            __syncwarp();
            if (lane == 0) atomicAdd(&sm.exp_cnt[X], 1u);
          }
          tmem_wait_st();
          tc_fence_before();
          mbar_arrive(p_ready + 8 * c);
        }
        float sum0, sum1;
        f2_unpack(f2_add(sum_a, sum_b), sum0, sum1);
        l_run = l_run * alpha + (sum0 + sum1);
      }
      if (!ok) break;

      if (!kRope) {
        // Hand the row statistics to the write-out warps.  They live in the transposition buffers
        // of softmax warps 4-7, unused in this mode: [tile][l | m][row].  The previous item's
        // statistics have been read once o_free has completed its phase (long ago: the first P V of
        // this item waited for the same phase).
        if (nx > 0 && !mbar_wait(w, smem_u32(&sm.o_free[X]), (nx - 1) & 1)) { ok = false; break; }
        float* stat = reinterpret_cast<float*>(sm.epi[4]) + X * 256;
        stat[r] = l_run;
        stat[128 + r] = m_ref;
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.stat_ready[X]));
        g_own += n_it;
        g_oth += n_other;
        ++nx;
        ++n;
        continue;
      }
      // epilogue: O / l and LSE = m * scale + ln(l)   (ops.mojo:316-321)
      if (!mbar_wait(w, smem_u32(&sm.o_final[X]), nx & 1)) { ok = false; break; }
      tc_fence_after();
      uint32_t og[128];
      tmem_ld128_wait(tO, og);
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.o_free[X]));   // the next item may overwrite O_X
      l_run *= kTruncGainInv;   // the row sum was accumulated from the inflated P
      const float inv_l = 1.f / l_run;
      {
        const int esize = p.o_f32 ? 4 : 2;
        const size_t row_stride = (size_t)p.dims.pitch_t * 128 * esize;
        const int wrow0 = qlo + 32 * (warp & 3);   // first row of this warp's 32-row block
        uint8_t* gout = static_cast<uint8_t*>(p.o) + row_of(p.dims, wi.b, wrow0, wi.h) * 128 * esize;
        const uint32_t wbase = epi + lane * 128u;
        const uint32_t sw = lane & 7u;
        if (p.o_f32) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j)
              sts128(wbase + ((j ^ sw) << 4),
                     make_uint4(__float_as_uint(__uint_as_float(og[c * 32 + 4 * j]) * inv_l),
                                __float_as_uint(__uint_as_float(og[c * 32 + 4 * j + 1]) * inv_l),
                                __float_as_uint(__uint_as_float(og[c * 32 + 4 * j + 2]) * inv_l),
                                __float_as_uint(__uint_as_float(og[c * 32 + 4 * j + 3]) * inv_l)));
            __syncwarp();
            store_staged_rows<8>(epi, 0, lane, 0, gout + c * 128, row_stride, T - wrow0);
            __syncwarp();
          }
        } else {
#pragma unroll
          for (int c = 0; c < 2; ++c) {
#pragma unroll
            for (uint32_t j = 0; j < 8; ++j) {
              const int o = c * 64 + 8 * j;
              sts128(wbase + ((j ^ sw) << 4),
                     make_uint4(pack_bf16x2(__uint_as_float(og[o]) * inv_l, __uint_as_float(og[o + 1]) * inv_l),
                                pack_bf16x2(__uint_as_float(og[o + 2]) * inv_l, __uint_as_float(og[o + 3]) * inv_l),
                                pack_bf16x2(__uint_as_float(og[o + 4]) * inv_l, __uint_as_float(og[o + 5]) * inv_l),
                                pack_bf16x2(__uint_as_float(og[o + 6]) * inv_l, __uint_as_float(og[o + 7]) * inv_l)));
            }
            __syncwarp();
            store_staged_rows<8>(epi, 0, lane, 0, gout + c * 128, row_stride, T - wrow0);
            __syncwarp();
          }
        }
      }
      if (qrow < T) p.lse[row_of(p.dims, wi.b, qrow, wi.h)] = m_ref * p.scale + logf(l_run);
      g_own += n_it;
      g_oth += n_other;
      ++nx;
      ++n;
    }
  }
  else if (warp >= 12) {
    setmaxnreg_dec<56>();
    if (warp == kWarpTma) {
      // ------------------------------------------------------------------ TMA producer
      int g = 0, n = 0;   // KV tiles and items issued so far
      bool ok = live;
      for (int kk = 0; ok; ++kk) {
        const int item = sched_item(kk, n_items);
        if (item == -1) break;
        if (item == -2) continue;
        const FwdItem wi = fwd_item(item, p.dims, n_qb);
        // Q may be replaced once the previous item's last S products have completed
        if (n > 0 && !mbar_wait(w, smem_u32(&sm.q_free), (n - 1) & 1)) break;
        if (lane == 0) {
          mbar_arrive_expect_tx(smem_u32(&sm.q_full), 2 * kTileBytes);
#pragma unroll
          for (int X = 0; X < 2; ++X) {
            tma_load_4d(smem_u32(sm.q[X]), &map_q, smem_u32(&sm.q_full), 0, wi.h, wi.q0 + kTile * X, wi.b);
            tma_load_4d(smem_u32(sm.q[X]) + kHalfBytes, &map_q, smem_u32(&sm.q_full), 64, wi.h, wi.q0 + kTile * X, wi.b);
          }
        }
        for (int j = wi.jlo; j <= wi.jhi; ++j, ++g) {
          const int s = g % kFwdStages;
          const uint32_t par = ((g / kFwdStages) & 1) ^ 1;
          if (!mbar_wait(w, smem_u32(&sm.k_empty[s]), par)) { ok = false; break; }
          if (lane == 0) {
            mbar_arrive_expect_tx(smem_u32(&sm.k_full[s]), kTileBytes);
            tma_load_4d(smem_u32(sm.k[s]), &map_k, smem_u32(&sm.k_full[s]), 0, wi.h, j * kTile, wi.b);
            tma_load_4d(smem_u32(sm.k[s]) + kHalfBytes, &map_k, smem_u32(&sm.k_full[s]), 64, wi.h, j * kTile, wi.b);
          }
          if (!mbar_wait(w, smem_u32(&sm.v_empty[s]), par)) { ok = false; break; }
          if (lane == 0) {
            mbar_arrive_expect_tx(smem_u32(&sm.v_full[s]), kTileBytes);
            tma_load_4d(smem_u32(sm.v[s]), &map_v, smem_u32(&sm.v_full[s]), 0, wi.h, j * kTile, wi.b);
            tma_load_4d(smem_u32(sm.v[s]) + kHalfBytes, &map_v, smem_u32(&sm.v_full[s]), 64, wi.h, j * kTile, wi.b);
          }
        }
        ++n;
      }
    } else if (warp == kWarpMma || warp == kWarpMma + 1) {
      // -------------------------------------------------------------- MMA issuers
      // One issuing warp per Q tile: a single thread sustains only about one tcgen05.mma
      // per 90-115 cycles, two issuers keep the tensor pipe fed.  All 32 lanes run the
      // loop; elect.sync inside each asm statement predicates the instruction onto one
      // lane, so the descriptors stay warp-uniform.
      const int X = warp - kWarpMma;
      constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, 128, 0, 1);
      const uint32_t tS = tmem + X * 128, tO = tmem + 256 + X * 128;
      const uint32_t qa = smem_u32(sm.q[X]);
      int g0 = 0, gx = 0, nx = 0, n = 0;   // KV tiles before this item; iterations / active items of tile X; items
      bool ok = true;
      for (int kk = 0; ok; ++kk) {
        const int item = sched_item(kk, n_items);
        if (item == -1) break;
        if (item == -2) continue;
        const FwdItem wi = fwd_item(item, p.dims, n_qb);
        const int n_kv = wi.jhi - wi.jlo + 1;
        const bool act_x = X == 0 ? wi.act[0] : wi.act[1];
        const int jlo_x = X == 0 ? wi.jlo_t[0] : wi.jlo_t[1], jhi_x = X == 0 ? wi.jhi_t[0] : wi.jhi_t[1];
        if (!act_x) {
          // Ragged end of the sequence: this tile has no rows in the item.  Its issuer still takes
          // part in every hand-shake of the item - it waits for Q and for each KV tile and makes this
          // tile's share of the releases - so that no barrier completes a phase this warp has not
          // seen (a parity wait is only valid for a waiter that saw the previous phase complete).
          if (!mbar_wait(w, smem_u32(&sm.q_full), n & 1)) { ok = false; break; }
          if (lane == 0) mbar_arrive(smem_u32(&sm.q_free));
          for (int t = 0; ok && t < n_kv; ++t) {
            const int s = (g0 + t) % kFwdStages;
            const uint32_t par = static_cast<uint32_t>(((g0 + t) / kFwdStages) & 1);
            if (!mbar_wait(w, kRope ? smem_u32(&sm.k_rot[s]) : smem_u32(&sm.k_full[s]), par) ||
                !mbar_wait(w, smem_u32(&sm.v_full[s]), par)) { ok = false; break; }
            if (lane == 0) {
              mbar_arrive(smem_u32(&sm.k_empty[s]));
              mbar_arrive(smem_u32(&sm.v_empty[s]));
            }
          }
          if (!ok) break;
          g0 += n_kv;
          ++n;
          continue;
        }
        if (kRope) {
          if (!mbar_wait(w, smem_u32(&sm.q_ready[X]), nx & 1)) { ok = false; break; }
        } else {
          if (!mbar_wait(w, smem_u32(&sm.q_full), n & 1)) { ok = false; break; }
        }
        auto stage_of = [&](int j) { return (g0 + j - wi.jlo) % kFwdStages; };
        auto parity_of = [&](int j) { return static_cast<uint32_t>(((g0 + j - wi.jlo) / kFwdStages) & 1); };
        auto active = [&](int j) { return j >= jlo_x && j <= jhi_x; };

        // S_X = Q_X K_j^T : 8 MMAs of K=16 over head_dim
        auto issue_qk = [&](int j) -> bool {
          const int s = stage_of(j);
          const uint32_t kbar = kRope ? smem_u32(&sm.k_rot[s]) : smem_u32(&sm.k_full[s]);
          if (!mbar_wait(w, kbar, parity_of(j))) return false;
          tc_fence_after();
          const uint32_t ka = smem_u32(sm.k[s]);
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
            umma_ss_elect(tS, make_sdesc_sw128(qa + off, 0, 1024), make_sdesc_sw128(ka + off, 0, 1024),
                          idesc_qk, ks > 0);
          }
          umma_commit_elect(smem_u32(&sm.s_full[X]));
          umma_commit_elect(smem_u32(&sm.k_empty[s]));
          if (j == jhi_x) {   // last read of Q_X in this item
            umma_commit_elect(smem_u32(&sm.q_free));
          }
          return true;
        };

        for (int j = wi.jlo; j <= wi.jhi; ++j) {
          const int s = stage_of(j);
          if (!active(j)) {
            // this tile does not use KV tile j: follow its phases (see above), then release its
            // share of the stage
            if (!mbar_wait(w, kRope ? smem_u32(&sm.k_rot[s]) : smem_u32(&sm.k_full[s]), parity_of(j)) ||
                !mbar_wait(w, smem_u32(&sm.v_full[s]), parity_of(j))) { ok = false; break; }
            if (lane == 0) {
              mbar_arrive(smem_u32(&sm.k_empty[s]));
              mbar_arrive(smem_u32(&sm.v_empty[s]));
            }
            continue;
          }
          const int itx = j - jlo_x;
          if (itx == 0 && !issue_qk(j)) { ok = false; break; }
          if (!mbar_wait(w, smem_u32(&sm.p_ready[X][0]), (gx + itx) & 1)) { ok = false; break; }
          if (!mbar_wait(w, smem_u32(&sm.v_full[s]), parity_of(j))) { ok = false; break; }
          // the item's first P V overwrites O_X: the previous item's rows must have left
          if (itx == 0 && nx > 0 && !mbar_wait(w, smem_u32(&sm.o_free[X]), (nx - 1) & 1)) { ok = false; break; }
          tc_fence_after();
          // O_X (+)= P_X V_j : P from TMEM (8 columns = 16 keys per MMA), V MN-major; the second
          // 64 keys follow when the softmax warps have written them
          const uint32_t va = smem_u32(sm.v[s]);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_ts_elect(tO, tS + ks * 8, make_sdesc_sw128(va + ks * 2048, kHalfBytes, 1024), idesc_pv,
                          (itx > 0 || ks > 0) ? 1u : 0u);
          if (!mbar_wait(w, smem_u32(&sm.p_ready[X][1]), (gx + itx) & 1)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int ks = 4; ks < 8; ++ks)
            umma_ts_elect(tO, tS + ks * 8, make_sdesc_sw128(va + ks * 2048, kHalfBytes, 1024), idesc_pv, 1u);
          if (j == jhi_x) umma_commit_elect(smem_u32(&sm.o_final[X]));
          umma_commit_elect(smem_u32(&sm.v_empty[s]));
          // S_X of the next KV tile overwrites the columns P_X occupies: it is issued by the
          // same thread after the P V MMAs, and MMAs of one thread complete in issue order.
          if (active(j + 1) && j + 1 <= wi.jhi && !issue_qk(j + 1)) { ok = false; break; }
        }
        if (!ok) break;
        g0 += n_kv;
        gx += jhi_x - jlo_x + 1;
        ++nx;
        ++n;
      }
    }
  } else {
    // ------------------------------------------------------------------ K rotation / write-out warps
    if (kRope) setmaxnreg_dec<56>(); else setmaxnreg_dec<72>();
    const int r = threadIdx.x - kWarpRot0 * 32;
    if (!kRope) {
      // ------------------------------------------------------------------ write-out warps
      // Thread r takes row r of tile A, then of tile B: O / l as bf16 or fp32 and
      // LSE = m * scale + ln(l) (ops.mojo:316-321).  O is read 32 columns at a time and leaves
      // through this warp's transposition buffer; the accumulator is released to the next item as
      // soon as its last columns are in registers.
      const int wq = warp - kWarpRot0;
      const uint32_t lane_off = static_cast<uint32_t>(wq * 32) << 16;
      const uint32_t epi = smem_u32(sm.epi[wq]);
      const uint32_t wbase = epi + lane * 128u, sw = lane & 7u;
      int nxe0 = 0, nxe1 = 0;
      bool ok = true;
      for (int kk = 0; ok; ++kk) {
        const int item = sched_item(kk, n_items);
        if (item == -1) break;
        if (item == -2) continue;
        const FwdItem wi = fwd_item(item, p.dims, n_qb);
        // Neither loop is unrolled: this code runs once per tile and item, and code that is not
        // resident costs about 100 cycles per 128 bytes of it to fetch, so one small body run
        // eight times is cheaper than eight copies run once.
#pragma unroll 1
        for (int X = 0; X < 2; ++X) {
          if (!(X == 0 ? wi.act[0] : wi.act[1])) continue;
          const int ph = (X == 0 ? nxe0 : nxe1) & 1;
          if (!mbar_wait(w, smem_u32(&sm.stat_ready[X]), ph)) { ok = false; break; }
          const float* stat = reinterpret_cast<const float*>(sm.epi[4]) + X * 256;
          const float l_row = stat[r] * kTruncGainInv;   // the row sum was accumulated from the inflated P
          const float m_row = stat[128 + r];
          if (!mbar_wait(w, smem_u32(&sm.o_final[X]), ph)) { ok = false; break; }
          tc_fence_after();
          const float inv_l = 1.f / l_row;
          const uint32_t tO = tmem + 256 + X * 128 + lane_off;
          const int qlo = wi.q0 + kTile * X, qrow = qlo + r;
          const int esize = p.o_f32 ? 4 : 2;
          const size_t row_stride = (size_t)p.dims.pitch_t * 128 * esize;
          const int wrow0 = qlo + 32 * wq;   // first row of this warp's 32-row block
          uint8_t* gout = static_cast<uint8_t*>(p.o) + row_of(p.dims, wi.b, wrow0, wi.h) * 128 * esize;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t og[32];
            tmem_ld32_wait(tO + c * 32, og);
            if (c == 3) {   // the next item may overwrite O_X
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(smem_u32(&sm.o_free[X]));
            }
            if (p.o_f32) {
#pragma unroll
              for (uint32_t j = 0; j < 8; ++j)
                sts128(wbase + ((j ^ sw) << 4),
                       make_uint4(__float_as_uint(__uint_as_float(og[4 * j]) * inv_l),
                                  __float_as_uint(__uint_as_float(og[4 * j + 1]) * inv_l),
                                  __float_as_uint(__uint_as_float(og[4 * j + 2]) * inv_l),
                                  __float_as_uint(__uint_as_float(og[4 * j + 3]) * inv_l)));
              __syncwarp();
              store_staged_rows<8>(epi, 0, lane, 0, gout + c * 128, row_stride, T - wrow0);
              __syncwarp();
            } else {
              // two 32-column chunks make one 128-byte block of bf16
#pragma unroll
              for (uint32_t j = 0; j < 4; ++j) {
                const int o = 8 * j;
                sts128(wbase + (((j + 4 * (c & 1)) ^ sw) << 4),
                       make_uint4(pack_bf16x2(__uint_as_float(og[o]) * inv_l, __uint_as_float(og[o + 1]) * inv_l),
                                  pack_bf16x2(__uint_as_float(og[o + 2]) * inv_l, __uint_as_float(og[o + 3]) * inv_l),
                                  pack_bf16x2(__uint_as_float(og[o + 4]) * inv_l, __uint_as_float(og[o + 5]) * inv_l),
                                  pack_bf16x2(__uint_as_float(og[o + 6]) * inv_l, __uint_as_float(og[o + 7]) * inv_l)));
              }
              if (c & 1) {
                __syncwarp();
                store_staged_rows<8>(epi, 0, lane, 0, gout + (c >> 1) * 128, row_stride, T - wrow0);
                __syncwarp();
              }
            }
          }
          if (qrow < T) p.lse[row_of(p.dims, wi.b, qrow, wi.h)] = m_row * p.scale + logf(l_row);
          if (X == 0) ++nxe0; else ++nxe1;
        }
      }
    } else {
      int g = 0;
      bool ok = true;
      for (int kk = 0; ok; ++kk) {
        const int item = sched_item(kk, n_items);
        if (item == -1) break;
        if (item == -2) continue;
        const FwdItem wi = fwd_item(item, p.dims, n_qb);
        for (int j = wi.jlo; j <= wi.jhi; ++j, ++g) {
          const int s = g % kFwdStages;
          if (!mbar_wait(w, smem_u32(&sm.k_full[s]), (g / kFwdStages) & 1)) { ok = false; break; }
          const int t = j * kTile + r;
          if (t < T)
            rope_rotate_row_smem(smem_u32(sm.k[s]), r, p.cos_buf + (size_t)t * 64, p.sin_buf + (size_t)t * 64);
          fence_proxy_async_smem();
          mbar_arrive(smem_u32(&sm.k_rot[s]));
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  drain_if_aborted(w.abort_smem);
  if (warp == kWarpMma) tmem_dealloc(tmem, 512);
}


size_t attn_fwd_smem_bytes() { return sizeof(FwdSmem) + 1024; }

cudaError_t launch_attn_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                            const FwdParams& p, bool rope, cudaStream_t stream) {
  const size_t smem = attn_fwd_smem_bytes();
  static int sm_count_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int& sm_count = sm_count_dev[dev & 63];
  if (sm_count == 0) {
    cudaError_t e = cudaFuncSetAttribute(attn_fwd_kernel<false>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(attn_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int n_qb = (p.dims.T + 255) / 256;
  const int n_items = n_qb * p.dims.H * p.dims.B;
  const int grid = n_items < sm_count ? n_items : sm_count;
  return rope ? launch_pdl(attn_fwd_kernel<true>, grid, kFwdThreads, smem, stream, mq, mk, mv, p, n_items, n_qb)
              : launch_pdl(attn_fwd_kernel<false>, grid, kFwdThreads, smem, stream, mq, mk, mv, p, n_items, n_qb);
}

}  // namespace ar
