// Tensor-core forward of the Mamba-3 SSD scan (sm_100a: tcgen05 MMA, TMEM accumulators, bulk copies).
//
// A CTA walks (batch, head) stripes in 128-row tiles (128 / R time steps, rows rho = (t, r)), with the
// fp32 state resident in TMEM as H^T [d_state x head_dim], so the forward pass moves no chunk-state
// traffic beyond the per-tile checkpoint the backward pass asks for.  Per tile:
//   copy    raw rows of B, C (and theta) land in staging buffers by bulk tensor copies of row maps (one box
//           per 64 elements of a row, 128-byte swizzle), requested a tile ahead by the copy warp
//   ahead   per-token scalars by the look-ahead warp a tile ahead; the (cos, sin) table of the wrapped
//           cumulative angle by the epilogue warps, while the previous tile's second group of products
//           runs                                                        (scan.rs:491-522, fused.rs:588-619)
//   stage   C^, B^ (rotated by -phi, ranks de-interleaved), X~, sigma_w X~ as bf16 operands
//   MMA     Yoff = C^ H^T-contraction,  G = C^ B^^T   (issuer warp)      (scan.rs:199, :256-261)
//   regs    M = G o band -> operand; Yoff *= exp(acum); H *= exp(cd)     (fused.rs:2044-2070)
//   MMA     Y += M X~ ;  H^T += B^^T (sigma_w X~)                        (scan.rs:202-216)
//   store   y = Y + D x staged in the row map's layout and sent off by bulk tensor stores; the bf16 copy
//           of H refreshed for the next tile
// bf16 operands, fp32 accumulation and state; shapes: head_dim 64, d_state 128, R in {1,2,4}.
// Warp roles, barriers and the distribution of stripes (or time segments of stripes) over CTAs:
// m3_tc_roles.cuh.  Rank 1 with real dynamics has a second form (m3_tc_fwd_direct.cu) whose rows need no
// conversion and land in operand layout by bulk TENSOR copies.
#include "m3_tc.h"
#include "m3_tc_roles.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_XW = 81920, OFF_H = 98304, OFF_TAB = 114688;
template <int R>
struct FwdSmem {
  static constexpr uint32_t kTab = (kRows / R) * kNH * 4;                  // (cos, sin) table of one tile
  static constexpr uint32_t kTheta = (kRows / R) * kNH * 2;                // raw theta rows, at the table's start
  static constexpr uint32_t kRaw = RawTile<R>::bytes(kN);                  // staged raw rows of B (and again of C)
  static constexpr uint32_t off_raw_b = OFF_TAB + kTab, off_raw_c = off_raw_b + kRaw, off_sc = off_raw_c + kRaw;
  // two sets of per-token scalars, the angle pass's exchange space ([4][64] sums, [64] running angle),
  // then mbarriers and the TMEM slot
  static constexpr uint32_t off_q = off_sc + 2 * kNumScal * kScal * 4;
  static constexpr uint32_t bytes = off_q + (4 * kNH + kNH) * 4 + 64;   // bars, TMEM slot, hand-over outcome
  static_assert(bytes <= 232448, "forward shared memory exceeds the 227 KB a CTA can have");
};
constexpr uint32_t TM_G = 0, TM_Y = 128, TM_H = 192, TM_COLS = 256;

template <int R, bool ROT, bool SPLIT>
__global__ void __launch_bounds__(kCtaThreads, 1) tc_fwd_kernel(const __grid_constant__ TcFwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  using SM = FwdSmem<R>;
  constexpr int LT = kRows / R;  // time steps per tile
  uint8_t *sC = smem + OFF_C, *sB = smem + OFF_B, *sX = smem + OFF_X, *sXw = smem + OFF_XW, *sH = smem + OFF_H;
  float* sTab = reinterpret_cast<float*>(smem + OFF_TAB);
  uint8_t *rawB = smem + SM::off_raw_b, *rawC = smem + SM::off_raw_c;
  float* sc = reinterpret_cast<float*>(smem + SM::off_sc);
  auto scal_set = [&](int i) {
    float* q = sc + i * kNumScal * kScal;
    return TileScalars{q, q + kScal, q + 2 * kScal, q + 3 * kScal, q + 4 * kScal, q + 5 * kScal, q + 6 * kScal,
                       q + 7 * kScal, q + 8 * kScal};
  };
  float* s_q = reinterpret_cast<float*>(smem + SM::off_q);
  float* s_carry = s_q + 4 * kNH;
  // [0], [1]: tensor-core phases; [2]: arrival of a tile's raw rows of B and C; [3]: of its theta rows
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_carry + kNH);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);
  int* s_ok = reinterpret_cast<int*>(tmem_slot + 1);  // outcome of a hand-over wait, for the epilogue warps

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.T, H = p.H;
  const int ntiles = (T + LT - 1) / LT;
  const uint32_t wait_limit = p.wait_limit;
  // Every role walks the same sequence of tiles: the tiles of this CTA's items, one item after the other,
  // as two nested loops, so that what belongs to the item (stripe, head, direction) is invariant where the
  // tiles are walked; g counts the tiles this CTA has gone through and picks barrier phases and scalar sets.
  // A head that walks right to left sees scan position s at time T-1-s: its rows are reached with a
  // negative token stride, everything else (tiles, scalars, checkpoints) is in scan order.
  // SPLIT: stripes cut in time, a grid of at most one CTA per SM that works through its items.  Otherwise
  // one CTA per stripe, whose single item is known without a decode and whose loops run once.
  const int nseg = SPLIT ? p.nseg : 1;
  const int BH = p.B * H, nitems = BH * nseg;
  auto item_of = [&](int item) {
    if (SPLIT) return decode_item(item, BH, H, ntiles, nseg, p.tps, 0);
    ItemInfo r;
    r.bh = item; r.b = item / H; r.h = item - r.b * H; r.seg = 0; r.k_lo = 0; r.k_hi = ntiles;
    return r;
  };

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_init(&bars[3], 1);
  }
  if (warp == 0) tmem_alloc(tmem_slot, TM_COLS);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  if (warp == kCopyWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Copy warp: the raw rows of a tile - the next item's first one included - are requested as soon as
    // the tile before it is staged (staging buffers and angle table spent), one request per lane; theta
    // rows land at the start of the table's buffer.
    // --------------------------------------------------------------------------------------------
    int g = 0, requested = 0;
    bool copies_ok = true;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo it = item_of(item);
      const int b = it.b, h = it.h;
      const bool rev = h >= H - p.rev;
      for (int k = it.k_lo; k < it.k_hi; ++k, ++g) {
        if (g > 0) {
          bar_sync(BAR_OPS, kEpiThreads + 64);  // the tile before this one is staged
          // its rows have landed unless the epilogue warps gave up on them: a barrier is armed again only
          // once its current phase is complete
          if (copies_ok) copies_ok = warp_all(mbar_wait(&bars[2], (g - 1) & 1) && (!ROT || mbar_wait(&bars[3], (g - 1) & 1)));
        }
        if (copies_ok) {
          if (lane == 0) {
            mbar_expect_tx(&bars[2], 2u * SM::kRaw);
            if (ROT) mbar_expect_tx(&bars[3], SM::kTheta);
          }
          __syncwarp();
          int l0 = request_raw_tile<R>(0, rawB, &p.tm_b, &bars[2], kN, b, h, T, k * LT, rev);
          l0 += request_raw_tile<R>(l0, rawC, &p.tm_c, &bars[2], kN, b, h, T, k * LT, rev);
          if (ROT && lane == l0) tma_load_rows(sTab, &p.tm_th, &bars[3], 0, h, rev ? T - k * LT - LT : k * LT, b);
          __syncwarp();
          ++requested;
        }
      }
    }
    if (g > 0) bar_sync(BAR_OPS, kEpiThreads + 64);  // the last tile
    // no copy of this CTA may be in flight when it lets go of its shared memory
    if (requested > 0) {
      mbar_wait(&bars[2], (requested - 1) & 1);
      if (ROT) mbar_wait(&bars[3], (requested - 1) & 1);
    }
  } else if (warp == kScalarWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Look-ahead warp: the scalars of the g-th tile go into set g & 1 as soon as the epilogue warps have
    // let go of it (BAR_FREE), and are announced on BAR_AHEAD; dt and lambda of the item's next tile are
    // requested right away and wait in registers.
    // --------------------------------------------------------------------------------------------
    ScalarLoads<R> ld;
    int g = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo it = item_of(item);
      const int b = it.b, h = it.h;
      const bool rev = h >= H - p.rev;
      const float A = -expf(p.a_log[h]);
      lookahead_load<R>(ld, p.dt, p.lam, p.disc, b, h, H, T, it.k_lo * LT, rev);
      for (int k = it.k_lo; k < it.k_hi; ++k, ++g) {
        if (g > 0) bar_sync(BAR_FREE, kPairCount);
        lookahead_scalars<R>(scal_set(g & 1), ld, A, T, k * LT);
        bar_arrive(bar_ahead(g), kPairCount);
        if (k + 1 < it.k_hi) lookahead_load<R>(ld, p.dt, p.lam, p.disc, b, h, H, T, (k + 1) * LT, rev);
      }
    }
  } else if (warp > kIssuerWarp) {
    regs_for_helpers();  // the idle warp of the helpers' group
  } else if (warp == kIssuerWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Issuer: both groups of products of every tile, and the state checkpoint.
    // --------------------------------------------------------------------------------------------
    int done = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo it = item_of(item);
      for (int k = it.k_lo; k < it.k_hi; ++k, ++done) {
      bar_sync(BAR_OPS, kEpiThreads + 64);  // operands of the tile staged
      if (lane == 0) {
        tc_fence_after();
        const Operand aC = k_major(smem_u32(sC), kN);
        gemm_issue(tm + TM_Y, aC, mn_major(smem_u32(sH), kP), make_idesc(64, 0, 1), kN, false);
        gemm_issue(tm + TM_G, aC, k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
        umma_commit(&bars[0]);
        if (p.ckpt_h) {
          // the bf16 state entering this tile, for the backward pass: one contiguous 16 KB bulk copy out of
          // the state's operand copy, which is next written after the second group of products
          bulk_store(p.ckpt_h + ((size_t)it.bh * ntiles + k) * kN * kP, sH, kN * kP * 2);
          bulk_commit();
        }
      }
      __syncwarp();
      bar_sync(BAR_MID, kPairCount);  // M = G o band staged; decays applied
      if (lane == 0) {
        if (p.ckpt_h) bulk_wait_read();  // the checkpoint has left the state's bf16 copy
        tc_fence_after();
        gemm_issue(tm + TM_Y, k_major(smem_u32(sC), kRows), mn_major(smem_u32(sX), kP), make_idesc(64, 0, 1), kRows, true);
        gemm_issue(tm + TM_H, mn_major(smem_u32(sB), kN), mn_major(smem_u32(sXw), kP), make_idesc(64, 1, 1), kRows, true);
        umma_commit(&bars[1]);
      }
      __syncwarp();
      }
    }
    // Nothing of this CTA may be in flight when it lets go of its shared memory and TMEM.
    if (done > 0) {
      mbar_wait(&bars[0], (done - 1) & 1);
      mbar_wait(&bars[1], (done - 1) & 1);
    }
    if (lane == 0) bulk_wait_all();
  } else {
    regs_for_epilogue();
    // --------------------------------------------------------------------------------------------
    // Epilogue warps.
    // --------------------------------------------------------------------------------------------
    const int quad = warp & 3, ch = warp >> 2;
    const int row = quad * 32 + lane;
    bool dead = false;  // a bounded wait of this warp gave up: it keeps the barriers going, nothing else
    // The angle table of tile kk of stripe sbh, the gg-th tile of this CTA, from its theta rows and its
    // scalars (which this call waits for).
    auto angle_table = [&](int gg, int sbh, int kk, bool srev) {
      bar_sync(bar_ahead(gg), kPairCount);  // scalars of the tile
      if (ROT) {
        if (!dead) dead = !warp_all(mbar_wait(&bars[3], gg & 1, wait_limit));
        if (!dead)
          epi_angle_table<R>(sTab, s_q, s_carry, s_carry, scal_set(gg & 1).dt, T, kk * LT, srev,
                             p.ckpt_angle ? p.ckpt_angle + ((size_t)sbh * ntiles + kk) * kNH : nullptr,
                             p.angle_out ? p.angle_out + (size_t)sbh * kNH : nullptr);
        else
          epi_sync();  // the pass's own barrier
      }
    };
    RawPX<R> raw_x;     // x of the next tile travels in registers
    int total = 0;      // tiles this CTA goes through in all
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo it = item_of(item);
      total += it.k_hi - it.k_lo;
    }
    int g = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo it = item_of(item);
      const int bh = it.bh, b = it.b, h = it.h, seg = it.seg, k_lo = it.k_lo, k_hi = it.k_hi;
      const bool rev = h >= H - p.rev;
      const int Hs = rev ? -H : H;
      // token-head index (row of a [B, T, H, ...] tensor) of scan position 0; position s is s * Hs rows further
      const size_t tok_base = ((size_t)b * T + (rev ? T - 1 : 0)) * H + h;
      auto tok_at = [&](int s) { return tok_base + (size_t)((ptrdiff_t)s * Hs); };
      const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
      const bool hand_over = seg + 1 < nseg;
      // ---- the item's first tile: the state and the running angle start from the caller's (first segment)
      //      or from what the previous segment handed over (bounded wait for its flag); the tile's angle
      //      table, which every later tile has ready from its predecessor's step 3 ----------------------------
      {
        issue_px<R>(raw_x, p.x, tok_at(k_lo * LT), Hs, T, k_lo * LT);
        if (seg > 0) {
          if (tid == 0) *s_ok = wait_flag(p.seg_flag + (size_t)bh * nseg + seg - 1, wait_limit << 4) ? 1 : 0;
          epi_sync();
          if (!*s_ok) dead = true;
        }
        if (ROT && tid < kNH)
          s_carry[tid] = seg > 0 ? __ldcg(p.seg_angle + ((size_t)bh * nseg + seg - 1) * kNH + tid)
                                 : (p.angle0 ? p.angle0[(size_t)bh * kNH + tid] : 0.0f);
        epi_sync();
        angle_table(g, bh, k_lo, rev);
        if (g == 0 && total > 1) epi_signal(BAR_FREE, kPairCount, dead);  // set 1 has never been used
        epi_sync();
        const float* src = seg > 0 ? p.seg_state + ((size_t)bh * nseg + seg - 1) * kP * kN
                                   : (p.h0 ? p.h0 + (size_t)bh * kP * kN : nullptr);
        float first = 0.0f;
        if (seg == 0 && p.h0) {
          const size_t i0 = tok_at(0);
          const float l0 = p.disc == 0 ? 1.0f : (p.disc == 1 ? 0.5f : bf(p.lam, i0));
          first = (1.0f - l0) * bf(p.dt, i0);
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int p0 = 32 * ch + 16 * cc;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            float s_ = 0.0f;
            if (src) {
              const size_t o = (size_t)(p0 + j) * kN + row;
              s_ = __ldcg(src + o);
              if (seg == 0) s_ += first * p.lu0[(size_t)bh * kP * kN + o];
            }
            v[j] = s_;
          }
          store_row16(sH, row, p0, kP, v);
          tmem_st16(tmem_addr(tm, quad * 32, TM_H + p0), v);
        }
        tmem_wait_st();
      }
      for (int k = k_lo; k < k_hi; ++k, ++g) {
      const int t0 = k * LT;
      const TileScalars ts = scal_set(g & 1);
      float *s_ac = ts.ac, *s_eac = ts.eac;
      const size_t tok0 = tok_at(t0);  // token-head index of l = 0 (stride Hs per step)
      // ---- 1. stage the operands ---------------------------------------------------------------
      if (!dead) dead = !warp_all(mbar_wait(&bars[2], g & 1, wait_limit));
      if (!dead) convert_bc<R, ROT>(rawB, rawC, sB, sC, sTab, rev);
      fence_async_smem();
      tc_fence_before();
      epi_signal(BAR_OPS, kEpiThreads + 64, dead);
      // X~ and sigma_w X~ are operands of the second group only: they are staged while the first group runs
      if (g > 0) {  // sigma_w X~ goes where the previous tile's y was staged: its stores must have read it
        if (warp == 0) bulk_wait_read();
        epi_sync();
      }
      if (!dead) commit_px<R>(raw_x, sX, sXw, ts.sw);
      if (!dead && k + 1 < k_hi) issue_px<R>(raw_x, p.x, tok0 + (size_t)LT * Hs, Hs, T, t0 + LT);
      // ---- 2. band, decays ---------------------------------------------------------------------
      // this row's scalars and the chunks' row factors need no product: they are taken before the wait
      const int l = row / R;
      const float acl = s_ac[l];
      const float eac = s_eac[l];
      const float ecd = __expf(fmaxf(s_ac[LT - 1], -60.0f));
      float rfs[4];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) rfs[cc] = row_factor(acl, s_ac[(64 * ch + 16 * cc) / R + 16 / R - 1]);
      if (!dead) dead = !warp_all(mbar_wait(&bars[0], g & 1, wait_limit));
      if (!dead) {
        tc_fence_after();
        const int lmax = (quad * 32 + 31) / R;  // last time step held by this warp
        float g[4][16], yv[2][16], hv[2][16];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int c0 = 64 * ch + 16 * cc;
          if (c0 / R <= lmax) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_G + c0), g[cc]);
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_Y + 32 * ch + 16 * cc), yv[cc]);
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_H + 32 * ch + 16 * cc), hv[cc]);
        }
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_fence(g[cc]);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) { tmem_ld_fence(yv[cc]); tmem_ld_fence(hv[cc]); }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int p0 = 32 * ch + 16 * cc;
#pragma unroll
          for (int j = 0; j < 16; j += 2) {  // packed fp32 pairs
            const float2 y2 = __fmul2_rn(make_float2(yv[cc][j], yv[cc][j + 1]), make_float2(eac, eac));
            const float2 h2 = __fmul2_rn(make_float2(hv[cc][j], hv[cc][j + 1]), make_float2(ecd, ecd));
            yv[cc][j] = y2.x; yv[cc][j + 1] = y2.y;
            hv[cc][j] = h2.x; hv[cc][j + 1] = h2.y;
          }
          tmem_st16(tmem_addr(tm, quad * 32, TM_Y + p0), yv[cc]);
          tmem_st16(tmem_addr(tm, quad * 32, TM_H + p0), hv[cc]);
        }
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int c0 = 64 * ch + 16 * cc;
          float m[16];
          if (c0 / R > lmax) {
#pragma unroll
            for (int j = 0; j < 16; ++j) m[j] = 0.0f;
          } else {
            ColScalars<R> cs;
            load_col_scalars<R>(cs, ts, c0);
            const int s0 = c0 / R;
            const float rf = rfs[cc];  // one exponential per chunk
            if (s0 + 16 / R - 1 < (quad * 32) / R) {
              // strictly below the diagonal for all 32 rows of this warp: the weight needs no selects and,
              // for one rank, is shared by every row up to the row factor
              const float2 rf2 = make_float2(rf, rf);  // two columns per instruction (packed fp32 pairs)
#pragma unroll
              for (int j = 0; j < 16; j += 2) {
                const int sa = j / R, sb = (j + 1) / R;
                const float2 wc = __fmul2_rn(make_float2(cs.w[sa], cs.w[sb]), make_float2(cs.cf[sa], cs.cf[sb]));
                const float2 m2 = __fmul2_rn(make_float2(g[cc][j], g[cc][j + 1]), __fmul2_rn(wc, rf2));
                m[j] = m2.x; m[j + 1] = m2.y;
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {  // branch-free: select between below / on / above the diagonal
                const int si = j / R, s = s0 + si;
                const float wgt = s < l ? cs.w[si] * (rf * cs.cf[si]) : (s == l ? cs.g[si] : 0.0f);
                m[j] = g[cc][j] * wgt;
              }
            }
          }
          float lo[8], hi[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = m[j]; hi[j] = m[8 + j]; }
          store_chunk(sC, tile_off(row, c0, kRows), lo);
          store_chunk(sC, tile_off(row, c0 + 8, kRows), hi);
        }
        tmem_wait_st();
      }
      fence_async_smem();
      tc_fence_before();
      epi_signal(BAR_MID, kPairCount, dead);
      // this tile's scalars are spent with the band: the look-ahead warp, whose code runs cold and slowly, may
      // overwrite their set with those of the tile after next from here on
      if (g + 2 < total) epi_signal(BAR_FREE, kPairCount, dead);
      // ---- 3. the next tile's angle table, while the second group of products runs (a tile that opens an
      //         item builds its own: its predecessor, which may be this very item, must have handed over) ---
      if (k + 1 < k_hi) angle_table(g + 1, bh, k + 1, rev);
      // ---- 4. outputs ----------------------------------------------------------------------------
      const bool hands = hand_over && k + 1 == k_hi;
      if (!dead) dead = !warp_all(mbar_wait(&bars[1], g & 1, wait_limit));
      if (!dead) {
        tc_fence_after();
        float yv[2][16], hv[2][16];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_Y + 32 * ch + 16 * cc), yv[cc]);
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_H + 32 * ch + 16 * cc), hv[cc]);
        }
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) { tmem_ld_fence(yv[cc]); tmem_ld_fence(hv[cc]); }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int p0 = 32 * ch + 16 * cc;
          float (&v)[16] = yv[cc];
          if (p.d_skip) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
              float xv[8];
              load_chunk(sX, tile_off(row, p0 + 8 * hh, kP), xv);
#pragma unroll
              for (int j = 0; j < 8; j += 2) {
                const float2 a2 = __ffma2_rn(make_float2(dsk, dsk), make_float2(xv[j], xv[j + 1]),
                                             make_float2(v[8 * hh + j], v[8 * hh + j + 1]));
                v[8 * hh + j] = a2.x; v[8 * hh + j + 1] = a2.y;
              }
            }
          }
          if constexpr (R != 2) stage_out16<R>(sXw, row, p0, v, rev);  // sigma_w X~ is spent: its buffer stages y
          // refresh the bf16 copy of the state: this thread's row n, 16 columns p at a time
          store_row16(sH, row, p0, kP, hv[cc]);
          if (k == ntiles - 1 && p.h_out) {
#pragma unroll
            for (int j = 0; j < 16; ++j) p.h_out[((size_t)bh * kP + p0 + j) * kN + row] = hv[cc][j];
          }
          if (hands) {  // the state leaving this segment, for whichever CTA runs the next one
            float* dst = p.seg_state + ((size_t)bh * nseg + seg) * kP * kN;
#pragma unroll
            for (int j = 0; j < 16; ++j) __stcg(dst + (size_t)(p0 + j) * kN + row, hv[cc][j]);
          }
        }
        if constexpr (R == 2) stage_out32<R>(sXw, row, 32 * ch, yv[0], yv[1], rev);  // rank 2: both halves at once
        if (k == ntiles - 1 && p.lu_out) {
          // last_u = sum_r x_{T-1}^(r) (x) B^_{T-1}^(r), from the staged operands (scan.rs:621-638)
          const int ll = T - 1 - t0;
          for (int e = tid; e < kP * kN; e += kEpiThreads) {
            const int pp = e / kN, nn = e % kN;
            float s_ = 0.0f;
#pragma unroll
            for (int rr = 0; rr < R; ++rr) {
              const float xv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(ll * R + rr, pp, kP)));
              const float bv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(ll * R + rr, nn, kN)));
              s_ += xv * bv;
            }
            p.lu_out[(size_t)bh * kP * kN + e] = s_;
          }
        }
      }
      if (hands) {
        if (ROT && tid < kNH) __stcg(p.seg_angle + ((size_t)bh * nseg + seg) * kNH + tid, s_carry[tid]);
        __threadfence();
      }
      fence_async_smem();  // the staged rows of y, for the stores that read them
      epi_sync();
      if (tile_leaves_by_map<R>(p.out_maps, rev, T, t0)) {
        if (warp == 0 && !dead) {
          store_out_tile<R>(0, sXw, &p.tm_y, kP, b, h, T, t0, rev);
          bulk_commit();
        }
      } else {
        if (!dead) copy_out_rows<R>(sXw, p.y, kP, tok0, Hs, T, t0, rev);
        epi_sync();
      }
      if (hands && tid == 0) raise_handover(p.seg_flag + (size_t)bh * nseg + seg);  // even if this CTA gave up: nobody waits in vain
      }
    }
    if (warp == 0) bulk_wait_all();  // the last tiles' stores
    if (dead && lane == 0 && p.err) raise_flag(p.err);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

template <int R>
cudaError_t launch_r(cudaStream_t st, const TcFwdParams& p, bool rot) {
  auto kern = p.nseg > 1 ? (rot ? tc_fwd_kernel<R, true, true> : tc_fwd_kernel<R, false, true>) : (rot ? tc_fwd_kernel<R, true, false> : tc_fwd_kernel<R, false, false>);
  constexpr uint32_t bytes = FwdSmem<R>::bytes;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return e;
  kern<<<p.grid, kCtaThreads, bytes, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

void tc_segment_plan(int BH, int tiles, bool allow_split, int* nseg, int* tps, int* grid, size_t* scratch_bytes) {
  static const int sms = [] {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) n = 148;
    return n;
  }();
  int want = 1;
  // Segments of one stripe run one after the other, so cutting adds no parallelism: it only evens out the
  // last round when there are more stripes than SMs.
  while (allow_split && BH > sms && (long long)BH * want < 6LL * sms && tiles / (want * 2) >= 4) want *= 2;
  const int per = (tiles + want - 1) / want;
  const int n = (tiles + per - 1) / per;
  *nseg = n;
  *tps = per;
  // whole stripes: one CTA each, handed out by the hardware; cut stripes: one CTA per SM at most, each
  // working through its items in order
  const long long items = (long long)BH * n;
  *grid = n == 1 ? BH : (int)(items < sms ? items : sms);
  if (scratch_bytes)
    *scratch_bytes = n > 1 ? (size_t)BH * n * ((size_t)kP * kN * 4 + kNH * 4 + 4) : 0;
}

cudaError_t tc_forward(cudaStream_t st, const TcFwdParams& p, bool rot) {
  if (p.use_tma && p.R == 1 && !rot) return tc_forward_direct(st, p);
  switch (p.R) {
    case 1: return launch_r<1>(st, p, rot);
    case 2: return launch_r<2>(st, p, rot);
    case 4: return launch_r<4>(st, p, rot);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace m3
