// dQ for sm_100a, replacing flash_attn_bwd_dq and the rope_bwd that follows it
// (ops.mojo:349-411, 1091-1120).  Deterministic, no atomics.
//
// Persistent kernel: one CTA per SM walks a static list of work items (query tile, head, batch),
// heaviest first; the TMA warp and the MMA issuers run ahead into the next item while the compute
// warpgroups still write out the previous one, so that an item's fixed costs (first-load latency,
// last products, write-out of the gradient tile) overlap its neighbours.
//
// Per item the CTA keeps 128 queries (Q and dO tiles) and streams K, V tiles of 128 keys through
// TMA rings (3 K stages, 2 V stages) that run on across items.  Per KV tile:
//   S  = Q  K^T   (SS MMA 128x128x128, issuer warp 17)     -> TMEM S
//   dP = dO V^T   (SS MMA 128x128x128, issuer warp 18)     -> TMEM dP
//   compute warps (thread r = query row r; four warpgroups, warpgroup w takes key columns
//   [32w, 32w+32): the element-wise stage is latency-bound, more resident warps hide it):
//       pull their S / dP columns into registers and at once release the S/dP region, so the
//       products of the NEXT tile run while this tile is exponentiated;
//       dS = exp2(S*scale*log2e - LSE*log2e) * (dP - D)  -> bf16 into its own TMEM region
//   dQ += dS K    (TS MMA, A = dS from TMEM, K as MN-major B, issuer warp 19)
// Every product is a full N=128 instruction: on this part an MMA costs about 100 cycles of its
// issuing thread whatever N is, which is why the three MMA streams have three issuing warps.
// Tensor memory: dQ [0,128)  S [128,256)  dP [256,384)  dS (bf16) [384,448)  dS residual [448,512).
// Where a query can see fewer than 16 keys in all (the first queries of a sequence; every query
// under a window below 15) dS is carried as two bf16 terms, the rounded value and the rounding
// residual, each through its own dQ product: such a query has nothing to average the bf16 rounding
// of dS over, and with |dQ| near 10 a single rounding (2^-9 relative) would already be the whole
// error budget.  Everywhere else (at least 16 visible keys per row) one term is carried.
// When asked (bf16 tensors, D and dQ both wanted) four otherwise idle warps compute
// D = rowsum(O * dO) for the queries of the item after the one in flight, replacing
// flash_attn_bwd_precompute_d (ops.mojo:329-346) and the key-stationary re-layout the dK/dV
// kernel needs.
// At the end of an item the four warpgroups pull the dQ rows into registers, a quarter of the columns
// each (which frees the accumulator for the next item), multiply by 1/sqrt(D) (ops.mojo:411), apply
// the inverse rotation of rope_bwd when asked, and write the rows out with plain coalesced stores
// through per-warp transposition buffers.  Those live in the V-ring slot that held the item's last V tile: the next
// item needs that slot only for its second V tile, and the TMA warp holds that one load back until
// the write-out is done.
#include <type_traits>

#include "attn_common.cuh"

namespace ar {

constexpr int kDqWGs = 4;                      // compute warpgroups: each takes 32 key columns of a tile
constexpr int kDqCW = 4 * kDqWGs;              // first non-compute warp: TMA; then S, dP, dQ issuers; 4 idle
constexpr int kDqThreads = (kDqCW + 8) * 32;
constexpr int kDqCols = kTile / kDqWGs;        // columns per compute thread
constexpr int kDqKStages = 3;   // K stays until the dQ MMAs of its tile are done
constexpr int kDqVStages = 2;   // V is free as soon as dP of its tile is done

struct DqSmem {
  alignas(1024) uint8_t q[kTileBytes];
  alignas(1024) uint8_t d_o[kTileBytes];
  alignas(1024) uint8_t k[kDqKStages][kTileBytes];
  alignas(1024) uint8_t v[kDqVStages][kTileBytes];
  alignas(8) uint64_t x_full, x_free;
  uint64_t k_full[kDqKStages], k_empty[kDqKStages], v_full[kDqVStages], v_empty[kDqVStages];
  uint64_t g_full, g_free, ready[2], ds_free[2], acc_done, acc_free, epi_free, d_ready[2], d_taken[2];   // ready, ds_free: per dS buffer (even / odd tiles); d_*: per D buffer (even / odd items)
  alignas(16) float d_row[2][kTile];   // D of the item's 128 queries when this kernel computes it (even / odd items)
  uint32_t tmem_base;
  uint32_t abort_flag;
};

// One work item: the query tile qt of head h of batch b and the key tiles it sees.
struct DqItem {
  int row0, h, b, jlo, n_it;
};
__device__ __forceinline__ DqItem dq_item(int item, const AttnDims& d, int n_qt) {
  DqItem it;
  const int bh = d.B * d.H;
  const int qi = item / bh, r = item - qi * bh;   // items are ordered by query tile, late (long) tiles first
  it.b = r / d.H;
  it.h = r - it.b * d.H;
  it.row0 = (n_qt - 1 - qi) * kTile;
  const int klo = d.window > 0 ? max(0, it.row0 - d.window) : 0;
  const int khi = min(it.row0 + kTile - 1, d.T - 1);
  it.jlo = klo >> 7;
  it.n_it = (khi >> 7) - it.jlo + 1;
  return it;
}

__global__ void __launch_bounds__(kDqThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                   const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                   const BwdParams p, const int n_items, const int n_qt) {
  extern __shared__ uint8_t smem_raw[];
  DqSmem& sm = *reinterpret_cast<DqSmem*>(align1024(smem_raw));
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int T = p.dims.T, window = p.dims.window, H = p.dims.H;

  grid_dep_launch_dependents();   // all CTAs of this grid are resident: the next kernel may be scheduled
  WaitCtx w{p.status, smem_u32(&sm.abort_flag)};
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&sm.x_full), 1);
    mbar_init(smem_u32(&sm.x_free), 2);      // the S and the dP issuer have issued the item's last product
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.d_ready[i]), 4);     // the four D warps have written the item's D
      mbar_init(smem_u32(&sm.d_taken[i]), kDqCW); // every compute warp has read it
    }
    for (int s = 0; s < kDqKStages; ++s) {
      mbar_init(smem_u32(&sm.k_full[s]), 1);
      mbar_init(smem_u32(&sm.k_empty[s]), 2);   // released by the S issuer and the dQ issuer
    }
    for (int s = 0; s < kDqVStages; ++s) {
      mbar_init(smem_u32(&sm.v_full[s]), 1);
      mbar_init(smem_u32(&sm.v_empty[s]), 1);   // released by the dP issuer
    }
    mbar_init(smem_u32(&sm.g_full), 2);      // S and dP each commit once
    // per-tile barriers: every compute thread arrives (measured 2 % faster for the whole kernel
    // than one elected lane per warp behind a __syncwarp)
    mbar_init(smem_u32(&sm.g_free), kDqCW * 32);  // every compute thread has its columns in registers
    for (int i = 0; i < 2; ++i) {
      mbar_init(smem_u32(&sm.ready[i]), kDqCW * 32);   // dS of a tile written into buffer i
      mbar_init(smem_u32(&sm.ds_free[i]), 1);          // the dQ MMAs of that tile have consumed it
    }
    mbar_init(smem_u32(&sm.acc_done), 1);
    mbar_init(smem_u32(&sm.acc_free), kDqCW);    // every compute warp holds its share of the dQ rows
    mbar_init(smem_u32(&sm.epi_free), kDqCW);    // ... and has read its transposition buffer
    sm.abort_flag = 0u;
    fence_mbar_init();
    prefetch_tmap(&map_q);
    prefetch_tmap(&map_do);
    prefetch_tmap(&map_k);
    prefetch_tmap(&map_v);
  }
  if (warp == kDqCW + 1) {
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
  // dS of tile g goes to buffer g & 1 (64 columns each), so that the element-wise stage of a tile does
  // not wait for the dQ products of the tile before it; a two-term tile puts its residual into the
  // other buffer and so needs both.
  constexpr uint32_t kColDQ = 0, kColS = 128, kColDP = 256, kColDS = 384;
  // Tile kb .. kb+127 against the queries row0 .. row0+127: can it hold the keys of a query that sees
  // fewer than 16 keys in all?  Those are the first 15 queries of a sequence (their keys lie in the
  // first tile) and, under a window below 15, every query (its keys lie in the tiles a mask edge
  // crosses).
  auto two_term_tile = [&](int kb, int row0) {
    if (window > 0 && window < 15) return kb + kTile - 1 > row0 || kb < row0 + kTile - 1 - window;
    return row0 == 0 && kb == 0;
  };

  if (warp >= kDqCW) {
  // registers move from the data-movement / issuing warpgroups to the compute warpgroups
  setmaxnreg_dec<48>();
  if (warp == kDqCW) {
    // ------------------------------------------------------------------ TMA producer
    // 128-row tile at `rows` of one (b,h): four 64-row boxes (two d-halves x two row blocks)
    auto load_tile = [&](uint32_t dst, const CUtensorMap* map, uint32_t bar, int rows, int hh, int bb) {
#pragma unroll
      for (int half = 0; half < 2; ++half)
#pragma unroll
        for (int rb = 0; rb < 2; ++rb)
          tma_load_4d(dst + half * kHalfBytes + rb * 8192, map, bar, half * 64, hh, rows + rb * 64, bb);
    };
    int g = 0, n = 0;        // tiles and items issued so far: ring stages and barrier phases follow them
    int epi_item = -1, epi_slot = 0;   // write-out not yet waited for, and the V slot it stages in
    bool ok = live;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DqItem wi = dq_item(item, p.dims, n_qt);
      // Q, dO may be replaced once the previous item's last S / dP products have completed
      if (n > 0 && !mbar_wait(w, smem_u32(&sm.x_free), (n - 1) & 1)) break;
      if (lane == 0) {
        const uint32_t bar = smem_u32(&sm.x_full);
        mbar_arrive_expect_tx(bar, 2 * kTileBytes);
        load_tile(smem_u32(sm.q), &map_q, bar, wi.row0, wi.h, wi.b);
        load_tile(smem_u32(sm.d_o), &map_do, bar, wi.row0, wi.h, wi.b);
      }
      for (int it = 0; it < wi.n_it; ++it, ++g) {
        const int sk = g % kDqKStages, sv = g % kDqVStages;
        if (!mbar_wait(w, smem_u32(&sm.k_empty[sk]), ((g / kDqKStages) & 1) ^ 1)) { ok = false; break; }
        if (lane == 0) {
          const uint32_t bar = smem_u32(&sm.k_full[sk]);
          mbar_arrive_expect_tx(bar, kTileBytes);
          load_tile(smem_u32(sm.k[sk]), &map_k, bar, (wi.jlo + it) * kTile, wi.h, wi.b);
        }
        if (!mbar_wait(w, smem_u32(&sm.v_empty[sv]), ((g / kDqVStages) & 1) ^ 1)) { ok = false; break; }
        // This slot may still hold the transposition buffers of the previous item's write-out.  The
        // wait is also settled before the item's last tile is issued, whichever slot that takes:
        // once that tile is under way this item can complete and be written out in its turn, and a
        // parity wait must not fall a phase behind its barrier.
        if (epi_item >= 0 && (sv == epi_slot || it == wi.n_it - 1)) {
          if (!mbar_wait(w, smem_u32(&sm.epi_free), epi_item & 1)) { ok = false; break; }
          epi_item = -1;
        }
        if (lane == 0) {
          const uint32_t bar = smem_u32(&sm.v_full[sv]);
          mbar_arrive_expect_tx(bar, kTileBytes);
          load_tile(smem_u32(sm.v[sv]), &map_v, bar, (wi.jlo + it) * kTile, wi.h, wi.b);
        }
      }
      if (!ok) break;
      epi_item = n;
      epi_slot = (g - 1) % kDqVStages;   // slot of this item's last V tile
      ++n;
    }
  } else if (warp == kDqCW + 1 || warp == kDqCW + 2) {
    // ------------------------------------------------------------------ S / dP issuers
    const int I = warp - (kDqCW + 1);
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, 0, 0);
    const uint32_t xa = smem_u32(I == 0 ? sm.q : sm.d_o);
    const uint32_t g_tmem = tmem + (I == 0 ? kColS : kColDP);
    int g = 0, n = 0;
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DqItem wi = dq_item(item, p.dims, n_qt);
      if (!mbar_wait(w, smem_u32(&sm.x_full), n & 1)) break;
      for (int it = 0; it < wi.n_it; ++it, ++g) {
        const int s = I == 0 ? g % kDqKStages : g % kDqVStages;
        const uint32_t full = I == 0 ? smem_u32(&sm.k_full[s]) : smem_u32(&sm.v_full[s]);
        if (!mbar_wait(w, full, (g / (I == 0 ? kDqKStages : kDqVStages)) & 1)) { ok = false; break; }
        // S / dP of the previous tile (of this or the previous item) must be in the compute threads' registers
        if (g > 0 && !mbar_wait(w, smem_u32(&sm.g_free), (g - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ya = smem_u32(I == 0 ? sm.k[s] : sm.v[s]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kHalfBytes + (ks & 3) * 32;
          umma_ss_elect(g_tmem, make_sdesc_sw128(xa + off, 0, 1024), make_sdesc_sw128(ya + off, 0, 1024),
                        idesc, ks > 0);
        }
        umma_commit_elect(smem_u32(&sm.g_full));
        umma_commit_elect(I == 0 ? smem_u32(&sm.k_empty[s]) : smem_u32(&sm.v_empty[s]));
        if (it == wi.n_it - 1) umma_commit_elect(smem_u32(&sm.x_free));   // last read of Q / dO
      }
      ++n;
    }
  } else if (warp == kDqCW + 3) {
    // ------------------------------------------------------------------ dQ issuer
    constexpr uint32_t idesc = make_idesc_bf16(128, 128, 0, 1);   // B (K) MN-major
    int g = 0, n = 0;
    bool ok = true;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DqItem wi = dq_item(item, p.dims, n_qt);
      for (int it = 0; it < wi.n_it; ++it, ++g) {
        const int s = g % kDqKStages;
        const uint32_t bsel = g & 1;
        // ready follows g_full, which follows k_full: K of this stage is in place
        if (!mbar_wait(w, smem_u32(&sm.ready[bsel]), (g >> 1) & 1)) { ok = false; break; }
        // the item's first product overwrites dQ: the previous item's rows must have left
        if (it == 0 && n > 0 && !mbar_wait(w, smem_u32(&sm.acc_free), (n - 1) & 1)) { ok = false; break; }
        tc_fence_after();
        const uint32_t ka = smem_u32(sm.k[s]);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts_elect(tmem + kColDQ, tmem + kColDS + 64 * bsel + ks * 8, make_sdesc_sw128(ka + ks * 2048, kHalfBytes, 1024),
                        idesc, (it > 0 || ks > 0) ? 1u : 0u);
        if (two_term_tile((wi.jlo + it) * kTile, wi.row0)) {   // the residual term of dS
#pragma unroll
          for (int ks = 0; ks < 8; ++ks)
            umma_ts_elect(tmem + kColDQ, tmem + kColDS + 64 * (bsel ^ 1u) + ks * 8,
                          make_sdesc_sw128(ka + ks * 2048, kHalfBytes, 1024), idesc, 1u);
        }
        umma_commit_elect(smem_u32(&sm.ds_free[bsel]));
        umma_commit_elect(smem_u32(&sm.k_empty[s]));
      }
      if (!ok) break;
      umma_commit_elect(smem_u32(&sm.acc_done));
      ++n;
    }
  } else if (warp >= kDqCW + 4 && p.o_for_d != nullptr) {
    // ------------------------------------------------------------------ D warps
    // D[row] = sum_d O[row,d] * dO[row,d] (ops.mojo:329-346) for an item's 128 queries, one item
    // ahead of the compute warps and off their critical path.  Each instruction reads two complete
    // 256-byte rows (16 lanes x 16 bytes) from global memory (dO is in L2: the TMA warp streams the
    // same tile); the 16 partial sums of a row meet by shuffles.  D goes to shared memory for the
    // compute threads, to d_out, and with the exponent addend to the key-stationary arrays that
    // the dK/dV kernel streams.
    const int wq = warp - (kDqCW + 4);             // rows [32 wq, 32 wq + 32) of the tile
    const int half = lane >> 4, ch = lane & 15;
    int n = 0;
    bool ok = live;   // these warps read and write global memory without waiting for anyone
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DqItem di = dq_item(item, p.dims, n_qt);
      float mine = 0.f;   // D of row 32 wq + lane
#pragma unroll 1
      for (int bt = 0; bt < 4; ++bt) {
        uint4 ov[4], dv[4];
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          const int row_g = di.row0 + 32 * wq + 8 * bt + 2 * pp + half;
          if (row_g < T) {
            const size_t ri = row_of(p.dims, di.b, row_g, di.h);
            ov[pp] = __ldg(reinterpret_cast<const uint4*>(p.o_for_d + ri * 128) + ch);
            dv[pp] = __ldg(reinterpret_cast<const uint4*>(p.do_for_d + ri * 128) + ch);
          } else {
            ov[pp] = make_uint4(0, 0, 0, 0);
            dv[pp] = make_uint4(0, 0, 0, 0);
          }
        }
#pragma unroll
        for (int pp = 0; pp < 4; ++pp) {
          const uint32_t ow[4] = {ov[pp].x, ov[pp].y, ov[pp].z, ov[pp].w}, dw[4] = {dv[pp].x, dv[pp].y, dv[pp].z, dv[pp].w};
          float acc = 0.f;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            acc += bf16_lo_to_f32(ow[i]) * bf16_lo_to_f32(dw[i]) + bf16_hi_to_f32(ow[i]) * bf16_hi_to_f32(dw[i]);
#pragma unroll
          for (int off = 8; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
          // lanes 0..15 hold the sum of row 8 bt + 2 pp, lanes 16..31 that of the next row
          const float lo_row = __shfl_sync(0xffffffffu, acc, 0), hi_row = __shfl_sync(0xffffffffu, acc, 16);
          if (lane == 8 * bt + 2 * pp) mine = lo_row;
          if (lane == 8 * bt + 2 * pp + 1) mine = hi_row;
        }
      }
      const int row_l = 32 * wq + lane, row_g = di.row0 + row_l;
      const bool valid = row_g < T;
      // the compute warps must have taken the D of the item before the previous one (same buffer;
      // each buffer has its own barriers, so that a waiter is never two phases behind)
      if (n > 1 && !mbar_wait(w, smem_u32(&sm.d_taken[n & 1]), ((n >> 1) - 1) & 1)) break;
      sm.d_row[n & 1][row_l] = valid ? mine : 0.f;
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&sm.d_ready[n & 1]));
      if (row_g < p.t_pad) {
        const size_t ti = ((size_t)di.b * H + di.h) * p.t_pad + row_g;
        float addend = -INFINITY;
        if (valid) {
          const size_t ri = row_of(p.dims, di.b, row_g, di.h);
          p.d_out[ri] = mine;
          addend = kTruncGainLog2 - p.lse[ri] * kLog2e;
        }
        p.dvec_t_out[ti] = valid ? mine : 0.f;
        p.lse2_t_out[ti] = addend;
      }
      ++n;
    }
  }
  } else {
    // ------------------------------------------------------------------ compute warpgroups
    // setmaxnreg.inc blocks until the registers exist: the totals after re-allocation must not
    // exceed what the CTA was launched with (768 x 80 = 512 x 96 + 256 x 48), or the kernel deadlocks.
    setmaxnreg_inc<96>();
    const int wg = warp >> 2;
    const int r = threadIdx.x & 127;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const f32x2 sc2 = f2_pack(p.scale_log2e, p.scale_log2e);
    int g = 0, n = 0;
    bool ok = true;
    bool prev_two = false;   // the tile before this one (of this or the previous item) used both dS buffers
    const bool fuse_d = p.o_for_d != nullptr;
    for (int k = 0; ok; ++k) {
      const int item = sched_item(k, n_items);
      if (item == -1) break;
      if (item == -2) continue;
      const DqItem wi = dq_item(item, p.dims, n_qt);
      const int row0 = wi.row0, row = row0 + r;
      const bool valid = row < T;
      const size_t row_index = row_of(p.dims, wi.b, min(row, T - 1), wi.h);
      // exp(s*scale - lse) = exp2(s*scale*log2e - lse*log2e); rows past T get lse = +inf, i.e. P = 0
      const float lse2 = valid ? p.lse[row_index] * kLog2e : INFINITY;
      float d_row = (!fuse_d && valid) ? p.dvec[row_index] : 0.f;
      const f32x2 nl2 = f2_pack(kTruncGainLog2 - lse2, kTruncGainLog2 - lse2);
      f32x2 dd2 = f2_pack(d_row, d_row);
      // The loop over the item's key tiles exists in two copies, chosen once per item: items that can
      // hold two-term tiles (see the head of the file; they are rare) also form the rounding
      // residual of dS, which costs registers the common copy should not pay for.
      auto tile_loop = [&](auto may_two) {
      constexpr bool kMayTwo = decltype(may_two)::value;
      for (int it = 0; it < wi.n_it; ++it, ++g) {
        const int ybase = (wi.jlo + it) * kTile + wg * kDqCols;   // first key of this warpgroup's columns
        if (!mbar_wait(w, smem_u32(&sm.g_full), g & 1)) { ok = false; break; }
        tc_fence_after();
        const bool two_terms = kMayTwo && two_term_tile((wi.jlo + it) * kTile, row0);   // CTA-uniform
        uint32_t sr[kDqCols], dr[kDqCols];
        tmem_ld32x2_wait(tmem + lane_off + kColS + wg * 32, sr, tmem + lane_off + kColDP + wg * 32, dr);
        tc_fence_before();
        mbar_arrive(smem_u32(&sm.g_free));
        if (it == 0 && fuse_d) {   // D of this item, computed by the D warps of this CTA an item ahead
          if (!mbar_wait(w, smem_u32(&sm.d_ready[n & 1]), (n >> 1) & 1)) { ok = false; break; }
          d_row = sm.d_row[n & 1][r];
          dd2 = f2_pack(d_row, d_row);
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&sm.d_taken[n & 1]));
        }
        // visible keys of this query within the 32 columns: lo <= col <= hi
        const bool edge_hi = ybase + kDqCols - 1 > row0;
        const bool edge_lo = window > 0 && ybase < row0 + kTile - 1 - window;
        const int hi = row - ybase;
        const int lo = window > 0 ? row - window - ybase : -(1 << 30);
        // Masking is a separate, rarely taken pass over the registers so that the main loop stays
        // branch-free.  The rows of a warp are consecutive, so a chunk that lane 0 sees up to its
        // last column (lane 31 from its first) is visible to the whole warp and is skipped.
        if (edge_hi && 31 > hi - lane) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i > hi) sr[i] = 0xff800000u;   // -inf: P = 0
        }
        if (edge_lo && 0 < lo - lane + 31) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < lo) sr[i] = 0xff800000u;
        }
        // dS' = P' (dP - D) with P' = kTruncGain * 2^(s*scale*log2e - lse*log2e), rounded to bf16 (the
        // gain is divided out at the write-out); two-lane fp32 arithmetic, every exponential an
        // ex2.approx.
        uint32_t pd[kDqCols / 2], pl[kDqCols / 2];
#pragma unroll
        for (int i = 0; i < kDqCols / 2; ++i) {
          const f32x2 x = f2_fma(f2_pack_u(sr[2 * i], sr[2 * i + 1]), sc2, nl2);
          float x0, x1;
          f2_unpack(x, x0, x1);
          const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);
          float s0, s1;
          f2_unpack(f2_mul(f2_pack(p0, p1), f2_sub(f2_pack_u(dr[2 * i], dr[2 * i + 1]), dd2)), s0, s1);
          pd[i] = pack_bf16x2(s0, s1);
          if (kMayTwo)   // the rounding residual dS - bf16(dS), exact in fp32
            pl[i] = pack_bf16x2_alu(s0 - bf16_lo_to_f32(pd[i]), s1 - bf16_hi_to_f32(pd[i]));
        }
        // Buffer g & 1 was last read by the dQ MMAs of tile g - 2.  The other buffer belongs to tile
        // g - 1: its MMAs must be done as well if that tile also kept its residual in this buffer, or if
        // this tile is about to put its own residual there.  (One barrier per buffer: a waiter on a
        // single barrier would fall two phases behind, which a parity wait cannot express.)
        const uint32_t bsel = g & 1;
        if (g > 1 && !mbar_wait(w, smem_u32(&sm.ds_free[bsel]), ((g >> 1) - 1) & 1)) { ok = false; break; }
        if (g > 0 && (prev_two || two_terms) &&
            !mbar_wait(w, smem_u32(&sm.ds_free[bsel ^ 1u]), ((g - 1) >> 1) & 1)) { ok = false; break; }
        tmem_st16(tmem + lane_off + kColDS + 64 * bsel + wg * 16, pd);
        if (kMayTwo && two_terms) tmem_st16(tmem + lane_off + kColDS + 64 * (bsel ^ 1u) + wg * 16, pl);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&sm.ready[bsel]));
        prev_two = two_terms;
      }
      };
      if (row0 == 0 || (window > 0 && window < 15)) tile_loop(std::true_type{});
      else tile_loop(std::false_type{});
      if (!ok) break;
      {
        // Write-out by all four warpgroups: warpgroup c takes the column pairs (d, d + 64) with d in
        // [16c, 16c + 16) of its rows.  The table values of the inverse rotation are fetched (in the
        // layout the rows have after their transposition, see warp_store_pair16) before the wait for
        // the item's last products.
        const bool rot = p.cos_buf != nullptr;
        const int wrow0 = row0 + 32 * (warp & 3);
        RotTable rt;
        if (rot) rot_table_fetch(rt, p.cos_buf, p.sin_buf, wrow0, lane, wg * 16, T);
        if (!mbar_wait(w, smem_u32(&sm.acc_done), n & 1)) { ok = false; break; }
        tc_fence_after();
        uint32_t a[16], bq[16];
        tmem_ld16x2_wait(tmem + lane_off + kColDQ + wg * 16, a, tmem + lane_off + kColDQ + 64 + wg * 16, bq);
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.acc_free));
        float lo_v[16], hi_v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          lo_v[i] = __uint_as_float(a[i]) * (p.scale * kTruncGainInv);   // dS carried the gain of P'
          hi_v[i] = __uint_as_float(bq[i]) * (p.scale * kTruncGainInv);
        }
        // transposition buffer of this warp: 2 KB of the V slot that held the item's last V tile
        const uint32_t epi = smem_u32(sm.v[(g - 1) % kDqVStages]) + warp * 2048u;
        const int esize = p.grad_f32 ? 4 : 2;
        uint8_t* gout = static_cast<uint8_t*>(p.dq) + row_of(p.dims, wi.b, wrow0, wi.h) * 128 * esize;
        const size_t row_stride = (size_t)p.dims.pitch_t * 128 * esize;
        if (rot) warp_store_pair16<true>(epi, lane, lo_v, hi_v, rt, gout, row_stride, wg * 16, T - wrow0, p.grad_f32);
        else warp_store_pair16<false>(epi, lane, lo_v, hi_v, rt, gout, row_stride, wg * 16, T - wrow0, p.grad_f32);
        fence_proxy_async_smem();   // the slot is next written by a bulk tensor load
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&sm.epi_free));
      }
      ++n;
    }
  }
  tc_fence_before();
  __syncthreads();
  drain_if_aborted(w.abort_smem);
  if (warp == kDqCW + 1) tmem_dealloc(tmem, 512);
}


// The operand maps are built with 64-row boxes.
cudaError_t launch_attn_bwd_dq(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                               const CUtensorMap& mdo, const BwdParams& p, cudaStream_t stream) {
  const size_t smem = sizeof(DqSmem) + 1024;
  static int sm_count_dev[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int& sm_count = sm_count_dev[dev & 63];
  if (sm_count == 0) {
    cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
  }
  const int n_qt = (p.dims.T + kTile - 1) / kTile;
  const int n_items = n_qt * p.dims.H * p.dims.B;
  const int grid = n_items < sm_count ? n_items : sm_count;
  return launch_pdl(attn_bwd_dq_kernel, grid, kDqThreads, smem, stream, mq, mdo, mk, mv, p, n_items, n_qt);
}

}  // namespace ar
