// Tensor-core backward of the Mamba-3 SSD scan (sm_100a: tcgen05 MMA, TMEM accumulators).
//
// The hand-written adjoint of the folded scan, one CTA per (batch, head) stripe walking its
// 128-row tiles in REVERSE with the gradient of the state, dH^T [d_state x head_dim] fp32,
// resident in TMEM.  The reference derives this pass from its tape (rules in
// src/autograd/ops.rs:204-264, :1066-1139, kernels src/tensor/ops/fused.rs:627-672,
// :2080-2138, :2513-2549); here it is two MMA phases per tile:
//   A:  G = C^ B^^T,  dM = dY~ X~^T,  T1 = dY~ H_k
//       regs: M = G o band, dG = dM o band, band adjoint sums, dC^ base = exp(acum) T1,
//             dS = dH (bf16 operand), d cd = exp(cd) <dH, H_k>, dH *= exp(cd)
//   B:  dX~ = M^T dY~ (+ sw . B^ dS^T),  dB^ = dG^T C^ + (sw X~) dS,  dC^ += dG B^,
//       dH^T += C^^T (exp(acum) dY~)
//       regs: un-rotate dB^, dC^ by +phi, collect d phi, reverse-scan it, per-token scalars.
#include "m3_tc.h"
#include "m3_tc_stage.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_DY = 81920, OFF_XW = 98304, OFF_DYE = 114688,
                   OFF_M = 131072, OFF_DG = 163840, OFF_HS = 196608, OFF_SC = 212992;
constexpr int kScalFloats = 2 * kNumScal * kScal + 256 * 4 + 512 + 256 + 132 + 132 + 16 + 64 + 64 + 256;
static_assert(OFF_SC + kScalFloats * 4 + 64 <= 232448, "backward shared memory exceeds the 227 KB a CTA can have");
constexpr uint32_t kSmemBytes = OFF_SC + kScalFloats * 4 + 64;
constexpr uint32_t TM_G = 0, TM_DM = 128, TM_T1 = 256, TM_DH = 384, TM_COLS = 512;
// phase B reuse: dB^ accumulates over G's columns, dX~ and U over dM's.
constexpr uint32_t TM_DB = 0, TM_DX = 128, TM_U = 192;


// Rank 1 with real dynamics: C^ and B^ are the raw rows, landed in operand layout by bulk tensor copies that
// are requested as soon as the previous tile has read its own, the checkpoint by a plain bulk copy; x and
// dy come through registers.
__global__ void __launch_bounds__(256, 1) tc_bwd_direct_kernel(const __grid_constant__ TcBwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int R = 1;  // rank 1 with real dynamics is the only shape this form serves
  constexpr int LT = kRows / R;
  uint8_t *sC = smem + OFF_C, *sB = smem + OFF_B, *sX = smem + OFF_X, *sXw = smem + OFF_XW, *sDY = smem + OFF_DY,
          *sDYe = smem + OFF_DYE, *sM = smem + OFF_M, *sDG = smem + OFF_DG, *sHS = smem + OFF_HS;
  float* sc = reinterpret_cast<float*>(smem + OFF_SC);
  // Two sets of per-token scalars: the next tile's are computed while this tile's phase-B products run.
  auto scal_set = [&](int i) {
    float* q = sc + i * kNumScal * kScal;
    return TileScalars{q, q + kScal, q + 2 * kScal, q + 3 * kScal, q + 4 * kScal, q + 5 * kScal, q + 6 * kScal,
                       q + 7 * kScal, q + 8 * kScal};
  };
  float* part_row = sc + 2 * kNumScal * kScal;   // [2][128]
  float* part_t1 = part_row + 256;    // [2][128]
  float* part_q = part_t1 + 256;      // [2][128]
  float* part_dg = part_q + 256;      // [2][128]
  float* part_col = part_dg + 256;    // [4][128]
  float* part_rot = part_col + 512;   // [2][128]
  float* s_dacum = part_rot + 256;    // [132]
  float* s_dast = s_dacum + 132;      // [132]
  float* s_red = s_dast + 132;        // [16]
  float* s_carry = s_red + 16;        // [64] angle entering the tile
  float* s_dcar = s_carry + 64;       // [64] sum of d phi over later tiles
  float* s_q = s_dcar + 64;           // [4][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_q + 256);  // [0], [1]: tensor-core phases; [2]: unused; [3]: checkpoint; [4]: C, B
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  // Right-to-left heads: scan position s is time T-1-s, reached with a negative token stride.
  const bool rev = h >= H - p.rev;
  const int Hs = rev ? -H : H;
  auto tok_at = [&](int s) { return ((size_t)b * T + (rev ? T - 1 - s : s)) * H + h; };
  const int ntiles = (T + LT - 1) / LT;
  const int Tp = ntiles * LT;
  const float A = -expf(p.a_log[h]);
  const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 32 + lane;
  const int rl = row / R;  // time step within the tile of this thread's row

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 1);
    mbar_init(&bars[3], 1);
    mbar_init(&bars[4], 1);
  }
  if (warp == 0) tmem_alloc(tmem_slot, TM_COLS);
  if (tid < kNH) s_dcar[tid] = 0.0f;
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  // dH^T <- gradient reaching the returned h (or zero)
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int p0 = 32 * ch + 16 * cc;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = p.dh ? p.dh[((size_t)bh * kP + p0 + j) * kN + row] : 0.0f;
    tmem_st16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
  }
  tmem_wait_st();

  bool failed = false;
  float nx_dt, nx_lam;  // dt / lambda of the next tile to process, loaded one tile ahead
  load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, (ntiles - 1) * LT, rev);
  // One thread asks for a tile's rows / its checkpoint.
  auto request_cb = [&](int kk) {
    const int tg = (b * T + kk * LT) / 8;  // token group of the tile's first row (T % 8 == 0)
    mbar_expect_tx(&bars[4], 2 * kRows * kN * 2);
    tma_load_tile(sC, &p.tm_c, &bars[4], h * (kN / 8), tg);
    tma_load_tile(sB, &p.tm_b, &bars[4], h * (kN / 8), tg);
  };
  auto request_ckpt = [&](int kk) {
    mbar_expect_tx(&bars[3], kN * kP * 2);
    bulk_load(sHS, p.ckpt_h + ((size_t)bh * ntiles + kk) * kN * kP, kN * kP * 2, &bars[3]);
  };
  auto prepare_scalars = [&](int kk, int slot) {  // tile kk's scalars, then the loads of the tile after it
    tile_scalars<R>(scal_set(slot), nx_dt, nx_lam, A, T, kk * LT);
    load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, (kk - 1) * LT, rev);
  };
  prepare_scalars(ntiles - 1, 0);
  int ckpt_requested = 0, cb_requested = 0;  // the same in every thread
  bool early_cb = false;
  if (tid == 0) {
    request_cb(ntiles - 1);
    request_ckpt(ntiles - 1);
  }
  ckpt_requested = cb_requested = 1;
  for (int k = ntiles - 1, it = 0; k >= 0; --k, ++it) {
    const int t0 = k * LT;
    const size_t tok0 = tok_at(t0);
    const bool last_tile = (k == ntiles - 1);
    const int l_end = T - 1 - t0;  // row of the final token when last_tile
    // ---- 1. every global load of the tile in flight, then scalars and angles ---------------------
    RawPX<R> raw_x, raw_dy;
    // x and dy come through registers even here: a bulk tensor copy moves these tiles in 16-byte
    // pieces, and the copy engine's piece rate, not memory, then sets when the tile can start.  The
    // rows were asked into L2 one tile ago, and the scaled copies are made from the same registers.
    issue_px<R>(raw_x, p.x, tok0, Hs, T, t0);
    issue_px<R>(raw_dy, p.dy, tok0, Hs, T, t0);
    const TileScalars ts = scal_set(it & 1);  // filled during the previous tile's phase-B wait (or the prologue)
    __syncthreads();
    // ---- 2-3. operands ------------------------------------------------------------------------------
    {
      const bool ok = mbar_wait(&bars[4], it & 1) && mbar_wait(&bars[3], it & 1);
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
        }
      }
    }
    commit_px<R>(raw_x, sX, sXw, ts.sw);      // with the scaled copies sigma_w X~ and exp(acum) dY~
    commit_px<R>(raw_dy, sDY, sDYe, ts.eac);
    if (k > 0) {  // the next tile's x (threads 0-127) and dy rows, one 128-byte line each, into L2
      const __nv_bfloat16* g = (tid < 128) ? p.x : p.dy;
      prefetch_l2(g + (tok0 - (size_t)LT * Hs + (size_t)(tid & 127) * Hs) * kP);
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- 4. MMA phase A ------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      gemm_issue(tm + TM_G, k_major(smem_u32(sC), kN), k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
      gemm_issue(tm + TM_DM, k_major(smem_u32(sDY), kP), k_major(smem_u32(sX), kP), make_idesc(128, 0, 0), kP, false);
      gemm_issue(tm + TM_T1, k_major(smem_u32(sDY), kP), k_major(smem_u32(sHS), kP), make_idesc(128, 0, 0), kP, false);
      umma_commit(&bars[0]);
    }
    // Without a rotation nothing reuses dG's buffer before the next band epilogue, so the 32 KB of dC
    // staged there by the previous tile leave now, while every warp would only wait for the products.
    if (it > 0 && p.dc) copy_out<R, kN>(sDG, p.dc, tok0 + (size_t)LT * Hs, Hs, T, t0 + LT);
    {
      const bool ok = mbar_wait(&bars[0], it & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    // ---- 5. epilogue A -------------------------------------------------------------------------
    const float acl = ts.ac[rl];
    const float cd = ts.ac[LT - 1];
    const float ecd = expc(cd);
    float dcd_part = 0.0f;
    {
      const int lmax = (quad * 32 + 31) / R;
      float rowE = 0.0f, dgp = 0.0f;
#pragma unroll 1
      for (int cb = 0; cb < 2; ++cb) {
        const int c0 = 64 * ch + 32 * cb;
        float dbd[32];
        if (c0 / R > lmax) {
          const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
          for (int q8 = 0; q8 < 4; ++q8) {
            store_chunk(sM, tile_off(row, c0 + 8 * q8, kRows), z);
            store_chunk(sDG, tile_off(row, c0 + 8 * q8, kRows), z);
          }
          part_col[quad * 128 + c0 + lane] = 0.0f;
          continue;
        }
        float gq[2][16], dmq[2][16];
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_G + c0 + 16 * hb), gq[hb]);
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DM + c0 + 16 * hb), dmq[hb]);
        }
        tmem_wait_ld();
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) { tmem_ld_fence(gq[hb]); tmem_ld_fence(dmq[hb]); }
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          const float (&g)[16] = gq[hb];
          const float (&dm)[16] = dmq[hb];
          float mv[16], dgv[16];
          ColScalars<R> cs;
          load_col_scalars<R>(cs, ts, c0 + 16 * hb);
          const int s0 = (c0 + 16 * hb) / R;
          const float rf = row_factor(acl, ts.ac[s0 + 16 / R - 1]);  // one exponential per chunk
          // A chunk whose last step precedes the first row of this warp lies strictly below the
          // diagonal for all 32 rows (the case of most chunks of the lower rows): no selects needed.
          if (s0 + 16 / R - 1 < (quad * 32) / R) {
            // two columns per instruction (packed fp32 pairs): the epilogues are bound by instruction issue
            const float2 rf2 = make_float2(rf, rf);
            float2 rowE2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const int sa = j / R, sb = (j + 1) / R;
              const float2 w2 = make_float2(cs.w[sa], cs.w[sb]);
              const float2 dec = __fmul2_rn(rf2, make_float2(cs.cf[sa], cs.cf[sb]));
              const float2 wgt = __fmul2_rn(w2, dec);
              const float2 g2 = make_float2(g[j], g[j + 1]), dm2 = make_float2(dm[j], dm[j + 1]);
              const float2 d2 = __fmul2_rn(dm2, __fmul2_rn(g2, dec));
              const float2 m2 = __fmul2_rn(g2, wgt), dg2 = __fmul2_rn(dm2, wgt);
              rowE2 = __ffma2_rn(d2, w2, rowE2);
              mv[j] = m2.x; mv[j + 1] = m2.y;
              dgv[j] = dg2.x; dgv[j + 1] = dg2.y;
              dbd[16 * hb + j] = d2.x; dbd[16 * hb + j + 1] = d2.y;
            }
            rowE += rowE2.x + rowE2.y;
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {  // branch-free selects: below / on / above the diagonal
              const int si = j / R, s = s0 + si;
              const bool below = s < rl, on = s == rl;
              const float dec = rf * cs.cf[si];
              const float wgt = below ? cs.w[si] * dec : (on ? cs.g[si] : 0.0f);
              const float gd = g[j] * dec;
              const float d_ = below ? dm[j] * gd : 0.0f;
              mv[j] = g[j] * wgt;
              dgv[j] = dm[j] * wgt;
              rowE += d_ * cs.w[si];
              dgp += on ? dm[j] * g[j] : 0.0f;
              dbd[16 * hb + j] = d_;
            }
          }
          float lo[8], hi[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = mv[j]; hi[j] = mv[8 + j]; }
          store_chunk(sM, tile_off(row, c0 + 16 * hb, kRows), lo);
          store_chunk(sM, tile_off(row, c0 + 16 * hb + 8, kRows), hi);
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = dgv[j]; hi[j] = dgv[8 + j]; }
          store_chunk(sDG, tile_off(row, c0 + 16 * hb, kRows), lo);
          store_chunk(sDG, tile_off(row, c0 + 16 * hb + 8, kRows), hi);
        }
        const float colsum = warp_column_sums(dbd);
        part_col[quad * 128 + c0 + lane] = colsum;
      }
      part_row[ch * 128 + row] = rowE;
      part_dg[ch * 128 + row] = dgp;
      // carry-out term: T1 = dY~ H_k ; d acum += exp(acum) <T1, C^> ; dC^ base = exp(acum) T1
      float t1[4][16], dhv[2][16];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_T1 + 64 * ch + 16 * cc), t1[cc]);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DH + 32 * ch + 16 * cc), dhv[cc]);
      tmem_wait_ld();
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) tmem_ld_fence(t1[cc]);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) tmem_ld_fence(dhv[cc]);
      const float eac = ts.eac[rl];
      const float2 eac2 = make_float2(eac, eac);
      float2 dot2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int n0 = 64 * ch + 16 * cc;
        float c1[8], c2[8];
        load_chunk(sC, tile_off(row, n0, kN), c1);
        load_chunk(sC, tile_off(row, n0 + 8, kN), c2);
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          dot2 = __ffma2_rn(make_float2(t1[cc][j], t1[cc][j + 1]), make_float2(c1[j], c1[j + 1]), dot2);
          dot2 = __ffma2_rn(make_float2(t1[cc][8 + j], t1[cc][9 + j]), make_float2(c2[j], c2[j + 1]), dot2);
        }
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float2 v = __fmul2_rn(make_float2(t1[cc][j], t1[cc][j + 1]), eac2);
          t1[cc][j] = v.x; t1[cc][j + 1] = v.y;
        }
        tmem_st16(tmem_addr(tm, quad * 32, TM_T1 + n0), t1[cc]);
      }
      part_t1[ch * 128 + row] = dot2.x + dot2.y;
      // state gradient: lanes are n, columns p; H_k and dS_k are kept [n][p]
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float hk[16];
        load_chunk(sHS, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&hk[0]));
        load_chunk(sHS, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&hk[8]));
#pragma unroll
        for (int j = 0; j < 16; ++j) dcd_part += dhv[cc][j] * hk[j];  // <dH, H_k>
        store_row16(sHS, row, p0, kP, dhv[cc]);                        // dS_k replaces H_k
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float2 v = __fmul2_rn(make_float2(dhv[cc][j], dhv[cc][j + 1]), make_float2(ecd, ecd));
          dhv[cc][j] = v.x; dhv[cc][j + 1] = v.y;
        }
        tmem_st16(tmem_addr(tm, quad * 32, TM_DH + p0), dhv[cc]);
      }
    }
    tmem_wait_st();
    const float dcd = ecd * inside(cd) * cta_sum(dcd_part, s_red);
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- 6. MMA phase B ------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      const uint32_t aM = smem_u32(sM), aDG = smem_u32(sDG), aC = smem_u32(sC), aB = smem_u32(sB), aHS = smem_u32(sHS);
      gemm_issue(tm + TM_DX, mn_major(aM, kRows), mn_major(smem_u32(sDY), kP), make_idesc(64, 1, 1), kRows, false);
      gemm_issue(tm + TM_U, k_major(aB, kN), mn_major(aHS, kP), make_idesc(64, 0, 1), kN, false);
      gemm_issue(tm + TM_DB, mn_major(aDG, kRows), mn_major(aC, kN), make_idesc(128, 1, 1), kRows, false);
      gemm_issue(tm + TM_DB, k_major(smem_u32(sXw), kP), k_major(aHS, kP), make_idesc(128, 0, 0), kP, true);
      gemm_issue(tm + TM_T1, k_major(aDG, kRows), mn_major(aB, kN), make_idesc(128, 0, 1), kRows, true);
      gemm_issue(tm + TM_DH, mn_major(aC, kN), mn_major(smem_u32(sDYe), kP), make_idesc(64, 1, 1), kRows, true);
      umma_commit(&bars[1]);
    }
    if (k > 0) prepare_scalars(k - 1, (it + 1) & 1);  // while the five products run
    {
      const bool ok = mbar_wait(&bars[1], it & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    if (k > 0) {
      // C^ and B^ of this tile have been read for the last time (only the gradient through last_u of the
      // final token looks at B^ again): their successors can start to arrive now.
      early_cb = !(last_tile && p.dlu);
      if (early_cb) {
        if (tid == 0) request_cb(k - 1);
        ++cb_requested;
      }
    }
    // ---- 7. epilogue B -------------------------------------------------------------------------
    const bool at_end = last_tile && rl == l_end;
    // Column blocks of this thread in a [128 x 128] gradient tile.
    auto gcol = [&](int q4) { return 64 * ch + 16 * q4; };
    float acc[2][16], u[2][16], gq[4][16];
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DX + 32 * ch + 16 * cc), acc[cc]);
      tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_U + 32 * ch + 16 * cc), u[cc]);
    }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DB + gcol(q4)), gq[q4]);
    tmem_wait_ld();
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) { tmem_ld_fence(acc[cc]); tmem_ld_fence(u[cc]); }
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) tmem_ld_fence(gq[q4]);
    float dD_part = 0.0f;
    {  // dx = M^T dY~ + sw (B^ dS^T) + D dy ; q = <U, x>
      const float sw = ts.sw[rl];
      const float2 sw2 = make_float2(sw, sw), dsk2 = make_float2(dsk, dsk);
      float2 qp2 = make_float2(0.0f, 0.0f), dD2 = make_float2(0.0f, 0.0f);
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float xv[16], dyv[16];
        load_chunk(sX, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&xv[0]));
        load_chunk(sX, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&xv[8]));
        load_chunk(sDY, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&dyv[0]));
        load_chunk(sDY, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&dyv[8]));
#pragma unroll
        for (int j = 0; j < 16; j += 2) {
          const float2 u2 = make_float2(u[cc][j], u[cc][j + 1]), x2 = make_float2(xv[j], xv[j + 1]);
          const float2 dy2 = make_float2(dyv[j], dyv[j + 1]);
          qp2 = __ffma2_rn(u2, x2, qp2);
          dD2 = __ffma2_rn(dy2, x2, dD2);
          const float2 a2 = __ffma2_rn(sw2, u2, __ffma2_rn(dsk2, dy2, make_float2(acc[cc][j], acc[cc][j + 1])));
          acc[cc][j] = a2.x; acc[cc][j + 1] = a2.y;
        }
        if (at_end && p.dlu) {  // gradient through last_u = sum_r x (x) B^ at the final token
#pragma unroll 1
          for (int j = 0; j < 16; ++j) {
            const float* gl = p.dlu + ((size_t)bh * kP + p0 + j) * kN;
            float s_ = 0.0f;
            for (int n = 0; n < kN; ++n)
              s_ += gl[n] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(row, n, kN)));
            float add[16];
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) add[jj] = (jj == j) ? s_ : 0.0f;
#pragma unroll
            for (int jj = 0; jj < 16; ++jj) acc[cc][jj] += add[jj];
          }
        }
        stage_store16<kP>(sHS, row, p0, acc[cc]);  // dS is spent: its buffer stages dx
      }
      part_q[ch * 128 + row] = qp2.x + qp2.y;
      dD_part = dD2.x + dD2.y;
    }
    {  // dB^ (TM_DB, operand sB, out db) then dC^ (TM_T1, operand sC, out dc)
      float gc[4][16];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_T1 + gcol(q4)), gc[q4]);  // in flight during dB^
      auto finish = [&](float (&g)[4][16], const uint8_t* sop, uint8_t* stg, bool is_b) {
        if (is_b && at_end && p.dlu) {  // d last_u reaches B^ of the final token: += dlu^T x
#pragma unroll 1
          for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll 1
            for (int j = 0; j < 16; ++j) {
              const int n = gcol(q4) + j;
              float s_ = 0.0f;
              for (int pp = 0; pp < kP; ++pp)
                s_ += p.dlu[((size_t)bh * kP + pp) * kN + n] *
                      __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(row, pp, kP)));
#pragma unroll
              for (int a4 = 0; a4 < 4; ++a4)
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) g[a4][jj] += (a4 == q4 && jj == j) ? s_ : 0.0f;
            }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) stage_store16<kN>(stg, row, gcol(q4), g[q4]);
      };
      finish(gq, sB, sXw, true);     // sigma_w X~ and exp(acum) dY~ are spent: 32 KB to stage dB
      tmem_wait_ld();
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) tmem_ld_fence(gc[q4]);
      finish(gc, sC, sDG, false);    // dG is spent: its buffer stages dC
      fence_async_smem();  // this tile's reads of its rows, before bulk copies replace them
      __syncthreads();
      if (k > 0) {  // the next tile's rows arrive during the copy-out and the per-token scalars
        if (tid == 0) {
          if (!early_cb) request_cb(k - 1);
        }
        if (!early_cb) ++cb_requested;
      }
      if (p.dx) copy_out<R, kP>(sHS, p.dx, tok0, Hs, T, t0);
      if (p.db) copy_out<R, kN>(sXw, p.db, tok0, Hs, T, t0);
      if (p.dc && k == 0) copy_out<R, kN>(sDG, p.dc, tok0, Hs, T, t0);
      fence_async_smem();  // dx was staged where the next checkpoint lands
      __syncthreads();
      if (k > 0) {
        if (tid == 0) request_ckpt(k - 1);
        ++ckpt_requested;
      }
    }
    const float dD_tile = cta_sum(dD_part, s_red);  // also orders part_* for what follows
    if (tid == 0) p.partD[(size_t)bh * ntiles + k] = dD_tile;
    // ---- 8. reverse cumulative sum of d phi over time -> d theta, and the dt term -----------------
    // ---- 9. per-token scalars of the tile ---------------------------------------------------------
    if (tid < LT) {
      const int l = tid;
      float rows = 0.0f, t1 = 0.0f, q = 0.0f, dgv = 0.0f, col = 0.0f;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int ro = l * R + r;
        rows += part_row[ro] + part_row[128 + ro];
        t1 += part_t1[ro] + part_t1[128 + ro];
        q += part_q[ro] + part_q[128 + ro];
        dgv += part_dg[ro] + part_dg[128 + ro];
        col += part_col[ro] + part_col[128 + ro] + part_col[256 + ro] + part_col[384 + ro];
      }
      const float ac = ts.ac[l], w = ts.w[l];
      const float raw = cd - ac;
      const float sg = expc(raw);
      const float dast = sg * w * q * inside(raw);
      const float dac = ts.eac[l] * inside(ac) * t1;
      s_dacum[l] = rows - w * col + dac - dast;
      s_dast[l] = dast;
      const size_t o = (size_t)bh * Tp + t0 + l;
      p.dw[o] = col + sg * q;
      p.dg[o] = dgv;
    }
    __syncthreads();
    if (warp == 0) {  // reverse inclusive scan of d acum (+ the chunk-decay terms on the last step)
      constexpr int EPL = LT / 32;
      float tail = 0.0f;
      for (int i = lane; i < LT; i += 32) tail += s_dast[i];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tail += __shfl_xor_sync(0xffffffffu, tail, o);
      tail += dcd;
      float loc[EPL];
      float run = 0.0f;
#pragma unroll
      for (int i = EPL - 1; i >= 0; --i) {
        const int l = lane * EPL + i;
        run += s_dacum[l] + (l == LT - 1 ? tail : 0.0f);
        loc[i] = run;
      }
      float tot = run;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_down_sync(0xffffffffu, tot, o);
        if (lane + o < 32) tot += n;
      }
      const float base = tot - run;
      float pa = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        const int l = lane * EPL + i;
        const float da = base + loc[i];
        p.da[(size_t)bh * Tp + t0 + l] = da;
        pa += da * ts.dt[l];
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) pa += __shfl_xor_sync(0xffffffffu, pa, o);
      if (lane == 0) p.partA[(size_t)bh * ntiles + k] = pa;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  // ---- gradient of the seed state -----------------------------------------------------------------
  if (!failed) {
    float first = 0.0f;
    if (p.h0) {
      const size_t i0 = tok_at(0);
      const float l0 = p.disc == 0 ? 1.0f : (p.disc == 1 ? 0.5f : bf(p.lam, i0));
      first = (1.0f - l0) * bf(p.dt, i0);
    }
    float ip = 0.0f;
#pragma unroll
    for (int cc = 0; cc < 2; ++cc) {
      const int p0 = 32 * ch + 16 * cc;
      float v[16];
      tmem_ld16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const size_t o = ((size_t)bh * kP + p0 + j) * kN + row;
        if (p.dh0) p.dh0[o] = v[j];
        if (p.dlu0) p.dlu0[o] = first * v[j];
        if (p.lu0) ip += v[j] * p.lu0[o];
      }
    }
    const float tot = cta_sum(ip, s_red);
    if (tid == 0) p.ip0[bh] = tot;
  }
  if (failed && tid == 0 && p.err) raise_flag(p.err);
  if (failed) {
    // A wait gave up: bulk copies already requested still target this CTA's shared memory.  Give the
    // latest request of each kind one more bounded wait before the CTA lets go of it.
    if (cb_requested > 0) mbar_wait(&bars[4], (cb_requested - 1) & 1);
    if (ckpt_requested > 0) mbar_wait(&bars[3], (ckpt_requested - 1) & 1);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

cudaError_t launch_tma(cudaStream_t st, const TcBwdParams& p) {
  auto kern = tc_bwd_direct_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytes, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_backward_direct(cudaStream_t st, const TcBwdParams& p) { return launch_tma(st, p); }

}  // namespace m3
