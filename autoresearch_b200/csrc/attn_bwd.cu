// dK, dV for sm_100a, replacing flash_attn_bwd_dkv and the rope_bwd on grad_k that follows it
// (ops.mojo:414-480, 1091-1120).  Deterministic, no atomics.
//
// Persistent kernel: one CTA per SM walks a static list of work items (key tile, head, batch),
// heaviest first, so that the fixed cost of an item - the first loads' latency at its start, the
// last products and the write-out of 128 KB of gradients at its end - overlaps the neighbouring
// items instead of leaving the tensor pipe idle: the TMA warp and the two MMA issuers run ahead
// into the next item while the compute warpgroups still drain the previous one.
//
// Per item the CTA keeps 128 keys (K, V tiles) and streams Q, dO in sub-tiles of 64 queries through
// a 4-stage TMA ring that runs on across items; the per-query kTruncGainLog2 - LSE*log2e and D ride
// along as two 256-byte bulk copies on the same mbarrier.  Products are formed transposed so that
// P^T / dS^T land with lanes = keys:
//   G1 = S^T  = K Q^T    SS MMA, 128 x 64, issuer 0
//   G2 = dP^T = V dO^T   SS MMA, 128 x 64, issuer 1
//   compute warps:  P^T = exp2(G1 * scale*log2e - LSE*log2e),  dS^T = P^T * (G2 - D)  -> bf16 in TMEM
//   dV += P^T dO (issuer 0),  dK += dS^T Q (issuer 1)      TS MMA, A from TMEM, B MN-major
// G1/G2 are double-buffered in tensor memory (even / odd sub-tiles), so the MMAs of sub-tile
// h+1 run while sub-tile h is being exponentiated; the two compute warpgroups split every
// sub-tile by columns (32 each) to keep the G -> exp -> accumulate chain of a buffer short.
// Tensor memory: dV [0,128) dK [128,256) | buffer b at 256+128b: G1 64 cols, G2 64 cols;
// P^T (bf16) overwrites G1 in place (columns [0,16) and [32,48): each warpgroup packs its own 32
// columns into its first 16), dS^T likewise in G2.  Issuer 0 only ever touches G1/P/dV and
// issuer 1 only G2/dS/dK, and MMAs of one thread complete in issue order, so overwriting a
// buffer two sub-tiles later needs no extra wait.
// Where a key can be seen by fewer than 16 queries in all (the last keys of a sequence; every key
// under a window below 15) dS^T is carried as two bf16 terms - the rounded value and its rounding
// residual, the latter in the 16 columns of G2 each warpgroup has left over - and P^T is rounded
// instead of truncated: such a key has nothing to average a bf16 rounding over, and with |dK| near
// 10 one rounding of dS (2^-9 relative) would be the whole error budget.
// Thread r of a compute warpgroup owns TMEM lane r (one key).  At the end of an item the compute
// threads pull their accumulator rows into registers (which frees tensor memory for the next
// item's accumulation), multiply dK by 1/sqrt(D) (ops.mojo:479), apply the inverse rotation of
// rope_bwd when asked, and write the rows out through a small per-warp transposition buffer with
// plain coalesced stores - nothing the CTA has to wait for, unlike a bulk store.
#include <type_traits>

#include "attn_common.cuh"

namespace ar {

constexpr int kSub = 64;                      // rows of a streamed sub-tile
constexpr int kSubBytes = kSub * 128 * 2;     // 16 KB: two 8 KB boxes (d 0..63, d 64..127)
constexpr int kSubHalf = kSub * 64 * 2;       // 8 KB
constexpr int kBwdStages = 4;
constexpr int kBwdThreads = 384;  // warps 0-3, 4-7 compute; 8 TMA; 9, 10 MMA issuers; 11 idle
constexpr int kEpiBytes = 2048;   // per compute warp: 32 rows x 64 bytes

struct BwdSmem {
  alignas(1024) uint8_t x1[kTileBytes];             // K
  alignas(1024) uint8_t x2[kTileBytes];             // V
  alignas(1024) uint8_t y1[kBwdStages][kSubBytes];  // Q sub-tiles
  alignas(1024) uint8_t y2[kBwdStages][kSubBytes];  // dO sub-tiles
  alignas(1024) uint8_t epi[8][kEpiBytes];          // write-out transposition buffers
  alignas(128) float stats[kBwdStages][2][kSub];    // per stage: exponent addend and D of its 64 queries
  alignas(8) uint64_t x_full, x_free;
  uint64_t y_full[kBwdStages], y_empty[kBwdStages];
  uint64_t g_full[2], ready[2], acc_done, acc_free;
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// One work item: the key tile kt of head h of batch b, and the 64-query sub-tiles that see it.
struct DkvItem {
  int row0, h, b, hlo, n_sub;
};
__device__ __forceinline__ DkvItem dkv_item(int item, const AttnDims& d) {
  DkvItem it;
  const int bh = d.B * d.H;
  const int kt = item / bh, r = item - kt * bh;   // items are ordered by key tile: most queries first
  it.b = r / d.H;
  it.h = r - it.b * d.H;
  it.row0 = kt * kTile;
  const int hi_row = d.window > 0 ? min(d.T - 1, it.row0 + kTile - 1 + d.window) : d.T - 1;
  it.hlo = it.row0 / kSub;
  it.n_sub = hi_row / kSub - it.hlo + 1;
  return it;
}

__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                    const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                    const BwdParams p, const int n_items) {
  extern __shared__ uint8_t smem_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(align1024(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int T = p.dims.T, window = p.dims.window, H = p.dims.H;

  grid_dep_launch_dependents();   // all CTAs of this grid are resident: the next kernel may be scheduled
  WaitCtx w{p.status, smem_u32(&sm.abort_flag)};
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.x_full), 1);
    mbar_init(smem_u32(&sm.x_free), 2);        // both issuers have issued the item's last product
    for (int s = 0; s < kBwdStages; ++s) {
      mbar_init(smem_u32(&sm.y_full[s]), 1);
      mbar_init(smem_u32(&sm.y_empty[s]), 2);  // one release per issuing warp
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.g_full[i]), 2);   // G1 and G2 each commit once
      mbar_init(smem_u32(&sm.ready[i]), 256);
    }
    mbar_init(smem_u32(&sm.acc_done), 2);      // both accumulations of the item are complete
    mbar_init(smem_u32(&sm.acc_free), 256);    // every compute thread holds its accumulator row
    sm.abort_flag = 0u;
    fence_mbar_init();
    prefetch_tmap(&map_k);
    prefetch_tmap(&map_v);
    prefetch_tmap(&map_q);
    prefetch_tmap(&map_do);
  }
  if (warp == 9) {
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
  constexpr uint32_t kColAcc0 = 0, kColAcc1 = 128, kColBuf = 256;
  // Queries y0 .. y0+63 against the keys row0 .. row0+127: can the sub-tile hold the queries of a key
  // that fewer than 16 queries see in all?  Those are the last 15 keys of a sequence (in the last key
  // tile) and, under a window below 15, every key (its queries lie in the sub-tiles a mask edge crosses).
  auto two_term_item = [&](int row0) { return (window > 0 && window < 15) || row0 + kTile >= T; };
  auto edge_sub = [&](int y0, int row0) {
    if (window > 0 && window < 15) return y0 < row0 + kTile - 1 || y0 + kSub - 1 > row0 + window;
    return row0 + kTile >= T;
  };

  if (warp >= 8) {
  // One setmaxnreg instruction per warpgroup: the compute warpgroups take the registers the
  // data-movement warpgroup gives up.
  setmaxnreg_dec<88>();
  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    int g = 0, n = 0;   // sub-tiles and items issued so far: ring stage and barrier phases follow them
    bool ok = live;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DkvItem wi = dkv_item(item, p.dims);
      // K, V may be replaced once the previous item's last products have completed
      if (n > 0 && !mbar_wait(w, smem_u32(&sm.x_free), (n - 1) & 1)) break;
      if (lane == 0) {
        const uint32_t bar = smem_u32(&sm.x_full);
        mbar_arrive_expect_tx(bar, 2 * kTileBytes);
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int rb = 0; rb < 2; ++rb) {
            const uint32_t off = half * kHalfBytes + rb * kSubHalf;
            tma_load_4d(smem_u32(sm.x1) + off, &map_k, bar, half * 64, wi.h, wi.row0 + rb * kSub, wi.b);
            tma_load_4d(smem_u32(sm.x2) + off, &map_v, bar, half * 64, wi.h, wi.row0 + rb * kSub, wi.b);
          }
      }
      for (int it = 0; it < wi.n_sub; ++it, ++g) {
        const int s = g % kBwdStages;
        if (!mbar_wait(w, smem_u32(&sm.y_empty[s]), ((g / kBwdStages) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t bar = smem_u32(&sm.y_full[s]);
          const int r = (wi.hlo + it) * kSub;
          mbar_arrive_expect_tx(bar, 2 * kSubBytes + 2 * kSub * 4);
          // per-query exponent addend and D of this sub-tile ride along with the tiles
          const size_t off = ((size_t)wi.b * H + wi.h) * p.t_pad + r;
          bulk_load(smem_u32(sm.stats[s][0]), p.lse2_t + off, kSub * 4, bar);
          bulk_load(smem_u32(sm.stats[s][1]), p.dvec_t + off, kSub * 4, bar);
          tma_load_4d(smem_u32(sm.y1[s]), &map_q, bar, 0, wi.h, r, wi.b);
          tma_load_4d(smem_u32(sm.y1[s]) + kSubHalf, &map_q, bar, 64, wi.h, r, wi.b);
          tma_load_4d(smem_u32(sm.y2[s]), &map_do, bar, 0, wi.h, r, wi.b);
          tma_load_4d(smem_u32(sm.y2[s]) + kSubHalf, &map_do, bar, 64, wi.h, r, wi.b);
        }
      }
      ++n;
    }
  } else if (warp == 9 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    // All lanes run the loop; each MMA / commit is predicated onto one elected lane.
    const int I = warp - 9;
    constexpr uint32_t idesc_g = make_idesc_bf16(128, kSub, 0, 0);    // 128 x 64, K-major operands
    constexpr uint32_t idesc_acc = make_idesc_bf16(128, 128, 0, 1);   // 128 x 128, B MN-major
    const uint32_t xa = smem_u32(I == 0 ? sm.x1 : sm.x2);
    const uint32_t acc_col = I == 1 ? kColAcc1 : kColAcc0;   // issuer 0: dV += P dO; issuer 1: dK += dS Q
    int g0 = 0, n = 0;   // global index of the item's first sub-tile; items done
    bool ok = true;

    // accumulate sub-tile `it` of the current item (global index gg)
    auto accumulate = [&](int it, int gg, bool two_terms) -> bool {
      const int s = gg % kBwdStages, bf = gg & 1;
      if (!mbar_wait(w, smem_u32(&sm.ready[bf]), (gg >> 1) & 1)) return false;
      // the item's first accumulation overwrites dV / dK: the previous item's rows must have left
      if (it == 0 && n > 0 && !mbar_wait(w, smem_u32(&sm.acc_free), (n - 1) & 1)) return false;
      tc_fence_after();
      const uint32_t a_tmem = tmem + kColBuf + bf * 128 + I * 64;   // P in G1, dS in G2
      const uint32_t yb = smem_u32(I == 0 ? sm.y2[s] : sm.y1[s]);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)   // k-steps 0,1: columns [0,16); k-steps 2,3: columns [32,48)
        umma_ts_elect(tmem + acc_col, a_tmem + (ks >> 1) * 32 + (ks & 1) * 8,
                      make_sdesc_sw128(yb + ks * 2048, kSubHalf, 1024), idesc_acc, (it > 0 || ks > 0) ? 1u : 0u);
      if (I == 1 && two_terms) {   // residual term of dS^T: columns [16,32) and [48,64) of G2
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ts_elect(tmem + acc_col, a_tmem + (ks >> 1) * 32 + 16 + (ks & 1) * 8,
                        make_sdesc_sw128(yb + ks * 2048, kSubHalf, 1024), idesc_acc, 1u);
      }
      umma_commit_elect(smem_u32(&sm.y_empty[s]));
      return true;
    };

    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DkvItem wi = dkv_item(item, p.dims);
      if (!mbar_wait(w, smem_u32(&sm.x_full), n & 1)) { ok = false; break; }
      for (int it = 0; it < wi.n_sub; ++it) {
        const int gg = g0 + it, s = gg % kBwdStages, bf = gg & 1;
        if (!mbar_wait(w, smem_u32(&sm.y_full[s]), (gg / kBwdStages) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ya = smem_u32(I == 0 ? sm.y1[s] : sm.y2[s]);
        const uint32_t g_tmem = tmem + kColBuf + bf * 128 + I * 64;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ss_elect(g_tmem, make_sdesc_sw128(xa + (ks >> 2) * kHalfBytes + (ks & 3) * 32, 0, 1024),
                        make_sdesc_sw128(ya + (ks >> 2) * kSubHalf + (ks & 3) * 32, 0, 1024), idesc_g, ks > 0);
        umma_commit_elect(smem_u32(&sm.g_full[bf]));
        if (it == wi.n_sub - 1) umma_commit_elect(smem_u32(&sm.x_free));   // last read of K / V
        if (it > 0 && !accumulate(it - 1, gg - 1, edge_sub((wi.hlo + it - 1) * kSub, wi.row0))) { ok = false; break; }
      }
      if (!ok || !accumulate(wi.n_sub - 1, g0 + wi.n_sub - 1, edge_sub((wi.hlo + wi.n_sub - 1) * kSub, wi.row0))) { ok = false; break; }
      umma_commit_elect(smem_u32(&sm.acc_done));
      g0 += wi.n_sub;
      ++n;
    }
  }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    setmaxnreg_inc<208>();
    const int wg = warp >> 2;                 // handles columns [32 wg, 32 wg + 32) of every sub-tile
    const int r = threadIdx.x & 127;          // TMEM lane = key row of the tile
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t epi = smem_u32(sm.epi[warp]);
    const f32x2 sc2 = f2_pack(p.scale_log2e, p.scale_log2e);
    int g0 = 0, n = 0;
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DkvItem wi = dkv_item(item, p.dims);
      const int row0 = wi.row0, row = row0 + r;
      // The loop over the item's sub-tiles exists in two copies, chosen once per item: only the rare
      // items that can hold two-term sub-tiles (see the head of the file) pay for the second pass.
      auto sub_loop = [&](auto may_two) {
      constexpr bool kMayTwo = decltype(may_two)::value;
      for (int it = 0; it < wi.n_sub; ++it) {
        const int gg = g0 + it, bf = gg & 1, s = gg % kBwdStages;
        // The per-query statistics of this stage arrived with its tiles (same mbarrier), before the
        // products are complete: they are fetched into registers now, because a shared-memory load
        // issued while the tensor pipe streams its operands takes far longer than the arithmetic
        // that would wait for it.
        if (!mbar_wait(w, smem_u32(&sm.y_full[s]), (gg / kBwdStages) & 1)) { ok = false; break; }
        float4 st_l[8], st_d[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          st_l[i] = *reinterpret_cast<const float4*>(&sm.stats[s][0][wg * 32 + 4 * i]);
          st_d[i] = *reinterpret_cast<const float4*>(&sm.stats[s][1][wg * 32 + 4 * i]);
        }
        if (!mbar_wait(w, smem_u32(&sm.g_full[bf]), (gg >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const int ybase = (wi.hlo + it) * kSub + wg * 32;   // first query of this thread's 32 columns
        const uint32_t buf = tmem + lane_off + kColBuf + bf * 128 + wg * 32;
        // row = key, column = query: visible iff q >= key and (no window or q <= key + window)
        const bool need_mask = (ybase < row0 + kTile - 1) || (window > 0 && ybase + 31 > row0 + window);
        const int lo = row - ybase;
        const int hi = window > 0 ? row + window - ybase : (1 << 30);
        uint32_t sr[32], dr[32];
        tmem_ld32x2_wait(buf, sr, buf + 64, dr);
        // Masking is a separate, rarely taken pass so that the main loop stays branch-free.  The
        // rows of a warp are consecutive: when lane 31 sees the chunk from its first column (lane 0
        // up to its last) the whole warp does, and that edge needs no per-element test.
        if (need_mask) {
          const int lo31 = lo - lane + 31, hi0 = hi - lane;   // warp-uniform bounds
          if (lo31 > 0) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < lo) sr[i] = 0xff800000u;   // -inf: P = 0
          }
          if (hi0 < 31) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i > hi) sr[i] = 0xff800000u;
          }
        }
        // Two-lane fp32 arithmetic throughout; P' = kTruncGain * P is truncated to bf16 (the gain
        // makes the truncation unbiased, see ptx.cuh), dS' = P' * (dP - D) is rounded; every
        // exponential is an ex2.approx.
        uint32_t pp[16], pd[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const f32x2 nl[2] = {f2_pack(st_l[i].x, st_l[i].y), f2_pack(st_l[i].z, st_l[i].w)};
          const f32x2 dd[2] = {f2_pack(st_d[i].x, st_d[i].y), f2_pack(st_d[i].z, st_d[i].w)};
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int j = 4 * i + 2 * e;
            const f32x2 x = f2_fma(f2_pack_u(sr[j], sr[j + 1]), sc2, nl[e]);
            float x0, x1;
            f2_unpack(x, x0, x1);
            const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
            float s0, s1;
            f2_unpack(f2_mul(f2_pack(p0, p1), f2_sub(f2_pack_u(dr[j], dr[j + 1]), dd[e])), s0, s1);
            pp[2 * i + e] = pack_bf16x2_trunc(p0, p1);
            pd[2 * i + e] = pack_bf16x2(s0, s1);
            if (kMayTwo) {   // kept for the second pass of a two-term sub-tile
              sr[j] = __float_as_uint(p0);
              sr[j + 1] = __float_as_uint(p1);
              dr[j] = __float_as_uint(s0);
              dr[j + 1] = __float_as_uint(s1);
            }
          }
        }
        const bool two_terms = kMayTwo && edge_sub((wi.hlo + it) * kSub, row0);   // CTA-uniform
        uint32_t pl[16];
        if (two_terms) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            // P^T rounded (the gain that makes truncation unbiased taken out again) ...
            pp[i] = pack_bf16x2_alu(__uint_as_float(sr[2 * i]) * kTruncGainInv, __uint_as_float(sr[2 * i + 1]) * kTruncGainInv);
            // ... and the rounding residual of dS^T (exact in fp32)
            pl[i] = pack_bf16x2_alu(__uint_as_float(dr[2 * i]) - bf16_lo_to_f32(pd[i]),
                                    __uint_as_float(dr[2 * i + 1]) - bf16_hi_to_f32(pd[i]));
          }
        }
        tmem_st16(buf, pp);        // P^T feeds dV
        tmem_st16(buf + 64, pd);   // dS^T feeds dK
        if (two_terms) tmem_st16(buf + 64 + 16, pl);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sm.ready[bf]));
      }
      };
      if (two_term_item(row0)) sub_loop(std::true_type{});
      else sub_loop(std::false_type{});
      if (!ok) break;
      g0 += wi.n_sub;
      if (!mbar_wait(w, smem_u32(&sm.acc_done), n & 1)) { ok = false; break; }
      tc_fence_after();
      // Warpgroup 0 writes out dV, warpgroup 1 dK (scaled, rotated back), 16 + 16 columns (a block and
      // the block 64 columns on, which a rotation pairs) per pass of a loop that is NOT unrolled: code
      // that runs once per item is fetched from far away (about 100 cycles per 128 bytes of it), so
      // four passes through one small body cost less than one pass through a body four times the
      // size.  The accumulator is released after the last pass has it in registers; the next item's
      // first accumulation needs P^T / dS^T from these same warps and cannot start earlier anyway.
      const uint32_t acc = tmem + lane_off + (wg == 0 ? kColAcc0 : kColAcc1);
      const int esize = p.grad_f32 ? 4 : 2;
      const size_t row_stride = (size_t)p.dims.pitch_t * 128 * esize;
      const int wrow0 = row0 + 32 * (warp & 3);   // first row of this warp's 32-row block
      uint8_t* gout = static_cast<uint8_t*>(wg == 0 ? p.dv : p.dk) +
                      row_of(p.dims, wi.b, wrow0, wi.h) * 128 * esize;
      const int rows_valid = T - wrow0;
      const float mul = wg == 0 ? 1.f : p.scale * kTruncGainInv;   // dS carried the gain of P'
      const bool rot = wg == 1 && p.cos_buf != nullptr;
#pragma unroll 1
      for (int cg = 0; cg < 4; ++cg) {
        RotTable rt;
        if (rot) rot_table_fetch(rt, p.cos_buf, p.sin_buf, wrow0, lane, 16 * cg, T);
        uint32_t a[16], b[16];
        tmem_ld16x2_wait(acc + 16 * cg, a, acc + 64 + 16 * cg, b);
        if (cg == 3) {
          tc_fence_before();
          mbar_arrive(smem_u32(&sm.acc_free));
        }
        float lo_v[16], hi_v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          lo_v[i] = __uint_as_float(a[i]) * mul;
          hi_v[i] = __uint_as_float(b[i]) * mul;
        }
        warp_store_pair16_rt(rot, epi, lane, lo_v, hi_v, rt, gout, row_stride, 16 * cg, rows_valid, p.grad_f32);
      }
      ++n;
    }
  }
  tc_fence_before();
  __syncthreads();
  drain_if_aborted(w.abort_smem);
  if (warp == 9) tmem_dealloc(tmem, 512);
}

// The four operand maps are built with 64-row boxes (make_tmap_bthd(..., box_rows = 64)).
cudaError_t launch_attn_bwd_dkv(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                                const CUtensorMap& mdo, const BwdParams& p, cudaStream_t stream) {
  const size_t smem = sizeof(BwdSmem) + 1024;
  static int sm_count_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int& sm_count = sm_count_dev[dev & 63];
  if (sm_count == 0) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int n_items = ((p.dims.T + kTile - 1) / kTile) * p.dims.H * p.dims.B;
  const int grid = n_items < sm_count ? n_items : sm_count;
  return launch_pdl(attn_bwd_dkv_kernel, grid, kBwdThreads, smem, stream, mk, mv, mq, mdo, p, n_items);
}


}  // namespace ar
