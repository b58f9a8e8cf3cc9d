// Tensor-core forward of the Mamba-3 SSD scan (sm_100a: tcgen05 MMA, TMEM accumulators).
//
// One CTA walks one (batch, head) stripe in 128-row tiles (128 / R time steps, rows
// rho = (t, r)), with the fp32 state resident in TMEM as H^T [d_state x head_dim], so the
// forward pass moves no chunk-state traffic beyond the per-tile checkpoint the backward
// pass asks for.  Per tile:
//   stage   C^, B^ (rotated by -phi, ranks de-interleaved), X~, sigma_w X~ as bf16 operands
//   MMA     Yoff = C^ H^T-contraction,  G = C^ B^^T                      (scan.rs:199, :256-261)
//   regs    M = G o band -> operand; Yoff *= exp(acum); H *= exp(cd)     (fused.rs:2044-2070)
//   MMA     Y += M X~ ;  H^T += B^^T (sigma_w X~)                        (scan.rs:202-216)
//   store   y = Y + D x ; refresh the bf16 copy of H for the next tile
// bf16 operands, fp32 accumulation and state; shapes: head_dim 64, d_state 128, R in {1,2,4}.
#include <cstdlib>

#include "m3_tc.h"
#include "m3_tc_stage.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_XW = 81920, OFF_H = 98304, OFF_PHI = 114688,
                   OFF_SC = 147456;
// scalar arrays: dt, lam, a, ac, g, w, sw, eac ; then carry[64], quarter sums[4][64]
constexpr uint32_t kSmemBytes = OFF_SC + (2 * kNumScal * kScal + 64 + 256) * 4 + 64;
constexpr uint32_t TM_G = 0, TM_Y = 128, TM_H = 192, TM_COLS = 256;
// The TMA-fed variant (rank 1, real dynamics): C^, B^ and X~ are the raw rows, landed in operand layout
// by bulk tensor copies, and exist twice so that the next tile arrives while this one computes; no
// angle buffer.
constexpr uint32_t TO_C0 = 0, TO_C1 = 65536, TO_X0 = 131072, TO_X1 = 147456,  // B^ follows its C^ at + 32768
                   TO_XW = 163840, TO_H = 180224, TO_SC = 196608;
constexpr uint32_t kSmemBytesTma = TO_SC + (2 * kNumScal * kScal + 64 + 256) * 4 + 64;
constexpr uint32_t kTileBytesTma = 2 * kRows * kN * 2 + kRows * kP * 2;  // C, B and x of one tile

#ifdef M3_TC_TIMING
__device__ long long g_tc_timing[16];
#define TICK(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) { long long c_ = clock64(); g_tc_timing[i] += c_ - tick_; tick_ = c_; } } while (0)
#define TOCK(i) do { if (blockIdx.x == 0 && threadIdx.x == 224) { long long c_ = clock64(); g_tc_timing[i] += c_ - tock_; tock_ = c_; } } while (0)
#else
#define TICK(i) do { } while (0)
#define TOCK(i) do { } while (0)
#endif

template <int R, bool ROT, bool TMA>
__global__ void __launch_bounds__(256, 1) tc_fwd_kernel(const __grid_constant__ TcFwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  static_assert(!TMA || (R == 1 && !ROT), "the TMA-fed variant serves rank 1 with real dynamics");
  constexpr int LT = kRows / R;  // time steps per tile
  uint8_t* sC = smem + (TMA ? TO_C0 : OFF_C);    // C^ operand, later M = G o band
  uint8_t* sB = smem + (TMA ? TO_C0 + 32768 : OFF_B);
  uint8_t* sX = smem + (TMA ? TO_X0 : OFF_X);
  uint8_t* sXw = smem + (TMA ? TO_XW : OFF_XW);
  uint8_t* sH = smem + (TMA ? TO_H : OFF_H);    // bf16 H [p][n]
  float* sPhi = reinterpret_cast<float*>(smem + OFF_PHI);  // not used by the TMA-fed variant
  float* sc = reinterpret_cast<float*>(smem + (TMA ? TO_SC : OFF_SC));
  // Two sets of per-token scalars: the next tile's are computed while this tile's products run.
  auto scal_set = [&](int i) {
    float* q = sc + i * kNumScal * kScal;
    return TileScalars{q, q + kScal, q + 2 * kScal, q + 3 * kScal, q + 4 * kScal, q + 5 * kScal, q + 6 * kScal,
                       q + 7 * kScal, q + 8 * kScal};
  };
  float* s_carry = sc + 2 * kNumScal * kScal;  // [64] running angle
  float* s_q = s_carry + 64;             // [4][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_q + 256);  // [0], [1]: tensor-core phases; [2], [3]: tile arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  // A head that walks right to left sees scan position s at time T-1-s: its rows are reached
  // with a negative token stride, everything else (tiles, scalars, checkpoints) is in scan order.
  const bool rev = h >= H - p.rev;
  const int Hs = rev ? -H : H;
  auto tok_at = [&](int s) { return ((size_t)b * T + (rev ? T - 1 - s : s)) * H + h; };
  const int ntiles = (T + LT - 1) / LT;
  const float A = -expf(p.a_log[h]);
  const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 32 + lane;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_init(&bars[3], 1);
  }
  if (warp == 0) tmem_alloc(tmem_slot, TM_COLS);
  if (ROT && tid < kNH) s_carry[tid] = p.angle0 ? p.angle0[(size_t)bh * kNH + tid] : 0.0f;
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  // ---- seed state: H^T[n][p] in TMEM and its bf16 copy [p][n] in shared memory
  {
    float first = 0.0f;
    if (p.h0) {
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
        float s = 0.0f;
        if (p.h0) {
          const size_t o = ((size_t)bh * kP + (p0 + j)) * kN + row;
          s = p.h0[o] + first * p.lu0[o];
        }
        v[j] = s;
        *reinterpret_cast<__nv_bfloat16*>(sH + tile_off(p0 + j, row, kN)) = __float2bfloat16_rn(s);
      }
      tmem_st16(tmem_addr(tm, quad * 32, TM_H + p0), v);
    }
    tmem_wait_st();
  }
  fence_async_smem();
  __syncthreads();  // the bf16 seed is read by the checkpoint's bulk copy and the first product

  if (p.stagger > 0) {  // spread the CTAs' memory phases: a fixed, bounded delay per CTA group
    const long long until = clock64() + (long long)(blockIdx.x & 3) * p.stagger;
    while (clock64() < until) {}
  }
  bool failed = false;
  float nx_dt, nx_lam;  // dt / lambda of the next tile, loaded one tile ahead
  load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, 0, rev);
  // Raw inputs of the NEXT tile travel in registers while the current tile computes.
  RawBC<R, ROT> raw_bc;
  RawPX<R> raw_x;
  RawTheta<R> raw_th;
  // TMA-fed variant: one thread asks for the three tiles of a time block; they land in operand layout.
  auto request_tile = [&](int kk) {
    uint64_t* bar = &bars[2 + (kk & 1)];
    uint8_t* base = smem + ((kk & 1) ? TO_C1 : TO_C0);
    const int tg = (b * T + kk * LT) / 8;  // token group of the tile's first row (T % 8 == 0)
    mbar_expect_tx(bar, kTileBytesTma);
    tma_load_tile(base, &p.tm_c, bar, h * (kN / 8), tg);
    tma_load_tile(base + 32768, &p.tm_b, bar, h * (kN / 8), tg);
    tma_load_tile(smem + ((kk & 1) ? TO_X1 : TO_X0), &p.tm_x, bar, h * (kP / 8), tg);
  };
  int requested = 0;  // tiles asked for so far (the same in every thread)
  if (TMA) {
    if (tid == 0) request_tile(0);
    requested = 1;
  } else {
    const size_t tok_first = tok_at(0);
    issue_bc<R, ROT>(raw_bc, p.b, p.c, tok_first, Hs, T, 0);
    issue_px<R>(raw_x, p.x, tok_first, Hs, T, 0);
    if (ROT) issue_theta<R>(raw_th, p.theta, tok_first, Hs, T, 0);
  }
  // Scalars and angles always run one tile ahead, inside the waits for the tensor core.
  auto prepare_scalars = [&](int k1) {
    tile_scalars<R>(scal_set(k1 & 1), nx_dt, nx_lam, A, T, k1 * LT);
    load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, (k1 + 1) * LT, rev);
  };
  auto prepare_angles = [&](int k1) {  // needs raw_th of tile k1 and the scalars of tile k1
    if (ROT) {
      commit_theta<R>(raw_th, sPhi);
      if (p.ckpt_angle && tid < kNH) p.ckpt_angle[((size_t)bh * ntiles + k1) * kNH + tid] = s_carry[tid];
      __syncthreads();
      const float ncarry = tile_angles_smem<R>(sPhi, s_q, s_carry, scal_set(k1 & 1).dt, T, k1 * LT,
                                               p.angle_out ? p.angle_out + (size_t)bh * kNH : nullptr);
      __syncthreads();
      if ((tid >> 6) == 3) s_carry[tid & 63] = ncarry;
    }
  };
  prepare_scalars(0);
  prepare_angles(0);
  __syncthreads();
#ifdef M3_TC_TIMING
  long long tick_ = clock64();
  long long tock_ = clock64();
#endif
  for (int k = 0; k < ntiles; ++k) {
    const int t0 = k * LT;
    const TileScalars ts = scal_set(k & 1);
    float *s_ac = ts.ac, *s_eac = ts.eac;
    TICK(0);
    const size_t tok0 = tok_at(t0);  // token-head index of l = 0 (stride Hs per step)
    if (TMA) {
      sC = smem + ((k & 1) ? TO_C1 : TO_C0);
      sB = sC + 32768;
      sX = smem + ((k & 1) ? TO_X1 : TO_X0);
      // the other set was last touched by tile k-1, whose products and reads are complete
      if (k + 1 < ntiles) {
        if (tid == 0) request_tile(k + 1);
        requested = k + 2;
      }
    }
    // ---- 1. the tile's raw inputs were put in flight one tile ago -----------------------------
    if (p.ckpt_h) {  // the bf16 state entering this tile, for the backward pass
      // one contiguous 16 KB bulk copy, in flight until the state's bf16 copy is refreshed in step 7
      if (tid == 0) {
        bulk_store(p.ckpt_h + ((size_t)bh * ntiles + k) * kN * kP, sH, kN * kP * 2);
        bulk_commit();
      }
    }
    TICK(1);
    TICK(2);
    TICK(3);
    // ---- 3. convert and store the operands -----------------------------------------------------
    if (TMA) {
      {
        const bool ok = mbar_wait(&bars[2 + (k & 1)], (k >> 1) & 1);
        if (__syncthreads_or(!ok)) { failed = true; break; }
      }
      const int nv = T - t0;  // rows of this tile that exist; the box ran on into the next sequence
      if (nv < kRows) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int q = tid; q < kRows * (kN / 8); q += 256) {
          const int r = q / (kN / 8), g8 = q % (kN / 8);
          if (r >= nv) {
            *reinterpret_cast<uint4*>(sC + tile_off(r, 8 * g8, kN)) = z;
            *reinterpret_cast<uint4*>(sB + tile_off(r, 8 * g8, kN)) = z;
            if (g8 < kP / 8) *reinterpret_cast<uint4*>(sX + tile_off(r, 8 * g8, kP)) = z;
          }
        }
        __syncthreads();
      }
    } else {
      commit_bc<R, ROT>(raw_bc, sB, sC, sPhi);
      commit_px<R>(raw_x, sX, sXw, ts.sw);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    TICK(4);
    // ---- 4. MMA phase 1: Yoff = C^ . H (over n), G = C^ B^^T -------------------------
    if (tid == 0) {
      tc_fence_after();
      const Operand aC = k_major(smem_u32(sC), kN);
      gemm_issue(tm + TM_Y, aC, k_major(smem_u32(sH), kN), make_idesc(64, 0, 0), kN, false);
      gemm_issue(tm + TM_G, aC, k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
      umma_commit(&bars[0]);
    }
    if (TMA) {
      // sigma_w X~, the scaled copy of x for the state update, is first needed by the second pair of
      // products: it is made while the first pair runs
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int q = tid + 256 * i;  // 16-byte chunk of the [128 x 64] tile: [r/8][c/8][r%8]
        const int r = (q >> 6) * 8 + (q & 7);
        float v[8];
        load_chunk(sX, (uint32_t)q * 16u, v);
        const float sw = ts.sw[r];
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] *= sw;
        store_chunk(sXw, (uint32_t)q * 16u, v);
      }
    }
    if (k + 1 < ntiles) {  // next tile's loads: in flight during both products and epilogues
      if (!TMA) {
        const size_t tok1 = tok0 + (size_t)LT * Hs;
        issue_bc<R, ROT>(raw_bc, p.b, p.c, tok1, Hs, T, t0 + LT);
        issue_px<R>(raw_x, p.x, tok1, Hs, T, t0 + LT);
        if (ROT) issue_theta<R>(raw_th, p.theta, tok1, Hs, T, t0 + LT);
      }
      prepare_scalars(k + 1);   // while G and Yoff are being computed
    }
    {
      const bool ok = mbar_wait(&bars[0], k & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    TICK(5);
    // ---- 5. band, decays, checkpoint ---------------------------------------------------
    {
      const int l = row / R;
      const float acl = s_ac[l];
      const int lmax = (quad * 32 + 31) / R;  // last time step held by this warp
      float g[4][16], yv[2][16], hv[2][16];
      TOCK(9);
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
      TOCK(10);
      const float eac = s_eac[l];
      const float ecd = __expf(fmaxf(s_ac[LT - 1], -60.0f));
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
      TOCK(11);
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
          const float rf = row_factor(acl, s_ac[s0 + 16 / R - 1]);  // one exponential per chunk
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
#ifdef ABL_NOSTORE
        if (lo[0] + hi[0] + lo[3] + hi[5] == 123.456f)
#endif
        {
        store_chunk(sC, tile_off(row, c0, kRows), lo);
        store_chunk(sC, tile_off(row, c0 + 8, kRows), hi);
        }
      }
      TOCK(12);
      tmem_wait_st();
      TOCK(13);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    TOCK(14);
    TICK(6);
    // ---- 6. MMA phase 2: Y += M X~ ; H^T += B^^T (sigma_w X~) ------------------------------
    if (tid == 0) {
      tc_fence_after();
      gemm_issue(tm + TM_Y, k_major(smem_u32(sC), kRows), mn_major(smem_u32(sX), kP), make_idesc(64, 0, 1), kRows, true);
      gemm_issue(tm + TM_H, mn_major(smem_u32(sB), kN), mn_major(smem_u32(sXw), kP), make_idesc(64, 1, 1), kRows, true);
      umma_commit(&bars[1]);
    }
    if (k + 1 < ntiles) prepare_angles(k + 1);  // while Y and the state update are being computed
    if (p.ckpt_h && tid == 0) bulk_wait_read();   // the checkpoint has left the state's bf16 copy
    {
      const bool ok = mbar_wait(&bars[1], k & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    TICK(7);
    // ---- 7. outputs -----------------------------------------------------------------------
    {
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
        stage_store16<kP>(sXw, row, p0, v);  // sigma_w X~ is spent: its buffer stages y
        // refresh the bf16 copy of the state (lane = n = row, columns = p)
#pragma unroll
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<__nv_bfloat16*>(sH + tile_off(p0 + j, row, kN)) = __float2bfloat16_rn(hv[cc][j]);
        if (k == ntiles - 1 && p.h_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) p.h_out[((size_t)bh * kP + p0 + j) * kN + row] = hv[cc][j];
        }
      }
      if (k == ntiles - 1 && p.lu_out) {
        // last_u = sum_r x_{T-1}^(r) (x) B^_{T-1}^(r), from the staged operands (scan.rs:621-638)
        const int ll = T - 1 - t0;
        for (int e = tid; e < kP * kN; e += 256) {
          const int pp = e / kN, n = e % kN;
          float s = 0.0f;
#pragma unroll
          for (int rr = 0; rr < R; ++rr) {
            const float xv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(ll * R + rr, pp, kP)));
            const float bv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(ll * R + rr, n, kN)));
            s += xv * bv;
          }
          p.lu_out[(size_t)bh * kP * kN + e] = s;
        }
      }
    }
    __syncthreads();
    copy_out<R, kP>(sXw, p.y, tok0, Hs, T, t0);
    fence_async_smem();  // this tile's writes to its operand set and to the state's bf16 copy, before bulk copies touch them
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    TICK(8);
  }
  if (failed && tid == 0 && p.err) atomicExch(p.err, 1);
  if (TMA && failed) {
    // A wait gave up: the bulk copies already requested still target this CTA's shared memory.
    // Give each of them one more bounded wait before the CTA lets go of it.
    for (int kk = requested > 2 ? requested - 2 : 0; kk < requested; ++kk) mbar_wait(&bars[2 + (kk & 1)], (kk >> 1) & 1);
  }
  if (tid == 0) bulk_wait_all();  // a checkpoint copy may still be reading this CTA's shared memory
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

template <int R>
cudaError_t launch_r(cudaStream_t st, const TcFwdParams& p, bool rot) {
  auto kern = rot ? tc_fwd_kernel<R, true, false> : tc_fwd_kernel<R, false, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytes, st>>>(p);
  return cudaGetLastError();
}

cudaError_t launch_tma(cudaStream_t st, const TcFwdParams& p) {
  auto kern = tc_fwd_kernel<1, false, true>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytesTma);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytesTma, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

#ifdef M3_TC_TIMING
extern "C" void m3_debug_timing(long long* out, int reset) {
  long long z[16] = {0};
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out, g_tc_timing, sizeof(z));
  if (reset) cudaMemcpyToSymbol(g_tc_timing, z, sizeof(z));
}
#endif

int tc_stagger_cycles(bool backward) {
  static const int env = [] {
    const char* v = getenv("M3_TC_STAGGER");
    return v ? atoi(v) : -1;
  }();
  if (env >= 0) return backward ? 2 * env : env;
  return backward ? 6000 : 3000;
}

bool tc_make_tile_map(CUtensorMap* map, const void* base, int B, int T, int H, int cols) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess) fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || T % 8 || cols % 8 || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
  const cuuint64_t dims[4] = {8, 8, (cuuint64_t)H * cols / 8, (cuuint64_t)B * T / 8};
  const cuuint64_t strides[3] = {(cuuint64_t)H * cols * 2, 16, (cuuint64_t)8 * H * cols * 2};
  const cuuint32_t box[4] = {8, 8, (cuuint32_t)cols / 8, 16};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t tc_forward(cudaStream_t st, const TcFwdParams& p, bool rot) {
  if (p.use_tma && p.R == 1 && !rot) return launch_tma(st, p);
  switch (p.R) {
    case 1: return launch_r<1>(st, p, rot);
    case 2: return launch_r<2>(st, p, rot);
    case 4: return launch_r<4>(st, p, rot);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace m3
