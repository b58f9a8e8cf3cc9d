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

constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_XW = 81920, OFF_DY = 98304, OFF_DYE = 114688,
                   OFF_M = 131072, OFF_DG = 163840, OFF_HS = 196608, OFF_SC = 212992;
constexpr int kScalFloats = 8 * kScal + 256 * 4 + 512 + 256 + 132 + 132 + 16 + 64 + 64 + 256;
constexpr uint32_t kSmemBytes = OFF_SC + kScalFloats * 4 + 64;
constexpr uint32_t TM_G = 0, TM_DM = 128, TM_T1 = 256, TM_DH = 384, TM_COLS = 512;
// phase B reuse: dB^ accumulates over G's columns, dX~ and U over dM's.
constexpr uint32_t TM_DB = 0, TM_DX = 128, TM_U = 192;

template <int R, bool ROT>
__global__ void __launch_bounds__(256, 1) tc_bwd_kernel(TcBwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int LT = kRows / R;
  uint8_t *sC = smem + OFF_C, *sB = smem + OFF_B, *sX = smem + OFF_X, *sXw = smem + OFF_XW, *sDY = smem + OFF_DY,
          *sDYe = smem + OFF_DYE, *sM = smem + OFF_M, *sDG = smem + OFF_DG, *sHS = smem + OFF_HS;
  float* sPhi = reinterpret_cast<float*>(smem + OFF_M);    // alive while staging and again after phase B
  float* sDphi = reinterpret_cast<float*>(smem + OFF_DG);  // alive after phase B
  float* sc = reinterpret_cast<float*>(smem + OFF_SC);
  TileScalars ts{sc, sc + kScal, sc + 2 * kScal, sc + 3 * kScal, sc + 4 * kScal, sc + 5 * kScal, sc + 6 * kScal,
                 sc + 7 * kScal};
  float* part_row = sc + 8 * kScal;   // [2][128]
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
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_q + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  const int ntiles = (T + LT - 1) / LT;
  const int Tp = ntiles * LT;
  const float A = -expf(p.a_log[h]);
  const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 32 + lane;
  const int rl = row / R, rr = row % R;  // time step within the tile and rank of this thread's row

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
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
  for (int k = ntiles - 1, it = 0; k >= 0; --k, ++it) {
    const int t0 = k * LT;
    const size_t tok0 = ((size_t)b * T + t0) * H + h;
    const bool last_tile = (k == ntiles - 1);
    const int l_end = T - 1 - t0;  // row of the final token when last_tile
    // ---- 1-3. scalars, angles, operands -----------------------------------------------------
    tile_scalars<R>(ts, p.dt, p.lam, p.disc, A, b, h, H, T, t0);
    if (ROT) {
      if (tid < kNH) s_carry[tid] = p.ckpt_angle[((size_t)bh * ntiles + k) * kNH + tid];
      __syncthreads();
      tile_angles<R>(sPhi, s_q, s_carry, ts.dt, p.theta, b, h, H, T, t0, nullptr);
    }
    __syncthreads();
    stage_bc<R, ROT>(sB, sC, p.b, p.c, sPhi, tok0, H, T, t0);
    stage_px<R>(sX, sXw, p.x, ts.sw, tok0, H, T, t0);
    stage_px<R>(sDY, sDYe, p.dy, ts.eac, tok0, H, T, t0);
    {  // H_k (state entering the tile) as a bf16 [p][n] operand
      const float* hk = p.ckpt_h + ((size_t)bh * ntiles + k) * kN * kP;
      for (int e = tid; e < kN * 8; e += 256) {
        const int n = e >> 3, p0 = (e & 7) * 8;
        const float4 a4 = *reinterpret_cast<const float4*>(hk + (size_t)n * kP + p0);
        const float4 b4 = *reinterpret_cast<const float4*>(hk + (size_t)n * kP + p0 + 4);
        const float v[8] = {a4.x, a4.y, a4.z, a4.w, b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<__nv_bfloat16*>(sHS + tile_off(p0 + j, n, kN)) = __float2bfloat16_rn(v[j]);
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- 4. MMA phase A ------------------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
      gemm_issue(tm + TM_G, k_major(smem_u32(sC), kN), k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
      gemm_issue(tm + TM_DM, k_major(smem_u32(sDY), kP), k_major(smem_u32(sX), kP), make_idesc(128, 0, 0), kP, false);
      gemm_issue(tm + TM_T1, k_major(smem_u32(sDY), kP), mn_major(smem_u32(sHS), kN), make_idesc(128, 0, 1), kP, false);
      umma_commit(&bars[0]);
    }
    {
      const bool ok = mbar_wait(&bars[0], it & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    // ---- 5. epilogue A -------------------------------------------------------------------------
    const float acl = ts.ac[rl];
    const float cd = ts.ac[LT - 1];
    const float ecd = expc(cd);
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
#pragma unroll
        for (int hb = 0; hb < 2; ++hb) {
          float g[16], dm[16], mv[16], dgv[16];
          tmem_ld16(tmem_addr(tm, quad * 32, TM_G + c0 + 16 * hb), g);
          tmem_ld16(tmem_addr(tm, quad * 32, TM_DM + c0 + 16 * hb), dm);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int s = (c0 + 16 * hb + j) / R;
            float m_ = 0.0f, dg_ = 0.0f, d_ = 0.0f;
            if (s < rl) {
              const float dec = expc(acl - ts.ac[s]);
              const float ws = ts.w[s];
              const float gd = g[j] * dec;
              m_ = gd * ws;
              dg_ = dm[j] * dec * ws;
              d_ = dm[j] * gd;
              rowE += d_ * ws;
            } else if (s == rl) {
              m_ = g[j] * ts.g[s];
              dg_ = dm[j] * ts.g[s];
              dgp += dm[j] * g[j];
            }
            mv[j] = m_; dgv[j] = dg_; dbd[16 * hb + j] = d_;
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
      const float eac = ts.eac[rl];
      float dot = 0.0f;
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        const int n0 = 64 * ch + 16 * cc;
        float v[16], c1[8], c2[8];
        tmem_ld16(tmem_addr(tm, quad * 32, TM_T1 + n0), v);
        load_chunk(sC, tile_off(row, n0, kN), c1);
        load_chunk(sC, tile_off(row, n0 + 8, kN), c2);
#pragma unroll
        for (int j = 0; j < 8; ++j) { dot += v[j] * c1[j] + v[8 + j] * c2[j]; }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= eac;
        tmem_st16(tmem_addr(tm, quad * 32, TM_T1 + n0), v);
      }
      part_t1[ch * 128 + row] = dot;
    }
    float dcd_part = 0.0f;
    {  // state gradient: lanes are n, columns p
      const float* hk = p.ckpt_h + (((size_t)bh * ntiles + k) * kN + row) * kP;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float v[16];
        tmem_ld16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float4 h4 = *reinterpret_cast<const float4*>(hk + p0 + 4 * j);
          dcd_part += v[4 * j] * h4.x + v[4 * j + 1] * h4.y + v[4 * j + 2] * h4.z + v[4 * j + 3] * h4.w;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<__nv_bfloat16*>(sHS + tile_off(p0 + j, row, kN)) = __float2bfloat16_rn(v[j]);  // dS_k
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= ecd;
        tmem_st16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
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
      gemm_issue(tm + TM_U, k_major(aB, kN), k_major(aHS, kN), make_idesc(64, 0, 0), kN, false);
      gemm_issue(tm + TM_DB, mn_major(aDG, kRows), mn_major(aC, kN), make_idesc(128, 1, 1), kRows, false);
      gemm_issue(tm + TM_DB, k_major(smem_u32(sXw), kP), mn_major(aHS, kN), make_idesc(128, 0, 1), kP, true);
      gemm_issue(tm + TM_T1, k_major(aDG, kRows), mn_major(aB, kN), make_idesc(128, 0, 1), kRows, true);
      gemm_issue(tm + TM_DH, mn_major(aC, kN), mn_major(smem_u32(sDYe), kP), make_idesc(64, 1, 1), kRows, true);
      umma_commit(&bars[1]);
    }
    {
      const bool ok = mbar_wait(&bars[1], it & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    // ---- 7. epilogue B -------------------------------------------------------------------------
    if (ROT) {  // the angles again (their buffer held M in between)
      tile_angles<R>(sPhi, s_q, s_carry, ts.dt, p.theta, b, h, H, T, t0, nullptr);
      __syncthreads();
    }
    const int t = t0 + rl;
    const bool live = t < T;
    const bool at_end = last_tile && rl == l_end;
    float dD_part = 0.0f;
    {  // dx = M^T dY~ + sw (B^ dS^T) + D dy ; q = <U, x>
      const float sw = ts.sw[rl];
      float qp = 0.0f;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float acc[16], u[16], xv[16], dyv[16];
        tmem_ld16(tmem_addr(tm, quad * 32, TM_DX + p0), acc);
        tmem_ld16(tmem_addr(tm, quad * 32, TM_U + p0), u);
        {
          float a8[8], b8[8];
          load_chunk(sX, tile_off(row, p0, kP), a8);
          load_chunk(sX, tile_off(row, p0 + 8, kP), b8);
#pragma unroll
          for (int j = 0; j < 8; ++j) { xv[j] = a8[j]; xv[8 + j] = b8[j]; }
          load_chunk(sDY, tile_off(row, p0, kP), a8);
          load_chunk(sDY, tile_off(row, p0 + 8, kP), b8);
#pragma unroll
          for (int j = 0; j < 8; ++j) { dyv[j] = a8[j]; dyv[8 + j] = b8[j]; }
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          qp += u[j] * xv[j];
          dD_part += dyv[j] * xv[j];
          acc[j] += sw * u[j] + dsk * dyv[j];
        }
        if (at_end && p.dlu) {  // gradient through last_u = sum_r x (x) B^ at the final token
          for (int j = 0; j < 16; ++j) {
            const float* gl = p.dlu + ((size_t)bh * kP + p0 + j) * kN;
            float s = 0.0f;
            for (int n = 0; n < kN; ++n)
              s += gl[n] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(row, n, kN)));
            acc[j] += s;
          }
        }
        if (live && p.dx) {
          __nv_bfloat16* dst = p.dx + (tok0 + (size_t)rl * H) * kP * R;
          if (R == 1) {
            uint4 q0, q1;
            q0.x = pack_bf16(acc[0], acc[1]); q0.y = pack_bf16(acc[2], acc[3]); q0.z = pack_bf16(acc[4], acc[5]); q0.w = pack_bf16(acc[6], acc[7]);
            q1.x = pack_bf16(acc[8], acc[9]); q1.y = pack_bf16(acc[10], acc[11]); q1.z = pack_bf16(acc[12], acc[13]); q1.w = pack_bf16(acc[14], acc[15]);
            reinterpret_cast<uint4*>(dst + p0)[0] = q0;
            reinterpret_cast<uint4*>(dst + p0)[1] = q1;
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(size_t)(p0 + j) * R + rr] = __float2bfloat16_rn(acc[j]);
          }
        }
      }
      part_q[ch * 128 + row] = qp;
    }
    {  // dB^ (TM_DB, operand sB, out db) and dC^ (TM_T1, operand sC, out dc)
      float dphi[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) dphi[j] = 0.0f;
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        const uint32_t tcol = which ? TM_T1 : TM_DB;
        const uint8_t* sop = which ? sC : sB;
        __nv_bfloat16* gout = which ? p.dc : p.db;
        __nv_bfloat16* dst = gout ? gout + (tok0 + (size_t)rl * H) * kN * R : nullptr;
        if (ROT) {
#pragma unroll
          for (int mc = 0; mc < 2; ++mc) {
            const int m0 = 32 * ch + 16 * mc;
            float g1[16], g2[16], o1[16], o2[16];
            tmem_ld16(tmem_addr(tm, quad * 32, tcol + m0), g1);
            tmem_ld16(tmem_addr(tm, quad * 32, tcol + kNH + m0), g2);
            {
              float a8[8], b8[8];
              load_chunk(sop, tile_off(row, m0, kN), a8);
              load_chunk(sop, tile_off(row, m0 + 8, kN), b8);
#pragma unroll
              for (int j = 0; j < 8; ++j) { o1[j] = a8[j]; o1[8 + j] = b8[j]; }
              load_chunk(sop, tile_off(row, kNH + m0, kN), a8);
              load_chunk(sop, tile_off(row, kNH + m0 + 8, kN), b8);
#pragma unroll
              for (int j = 0; j < 8; ++j) { o2[j] = a8[j]; o2[8 + j] = b8[j]; }
            }
            if (which == 0 && at_end && p.dlu) {
              for (int j = 0; j < 16; ++j) {
                float s1 = 0.0f, s2 = 0.0f;
                for (int pp = 0; pp < kP; ++pp) {
                  const float xv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(row, pp, kP)));
                  s1 += p.dlu[((size_t)bh * kP + pp) * kN + m0 + j] * xv;
                  s2 += p.dlu[((size_t)bh * kP + pp) * kN + kNH + m0 + j] * xv;
                }
                g1[j] += s1; g2[j] += s2;
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              dphi[16 * mc + j] += g1[j] * o2[j] - g2[j] * o1[j];
              float sn, cs;
              __sincosf(sPhi[rl * kNH + m0 + j], &sn, &cs);
              const float u1 = g1[j] * cs - g2[j] * sn, u2 = g1[j] * sn + g2[j] * cs;
              g1[j] = u1; g2[j] = u2;
            }
            if (live && dst) {
              if (R == 1) {
                uint4 q0, q1;
                q0.x = pack_bf16(g1[0], g1[1]); q0.y = pack_bf16(g1[2], g1[3]); q0.z = pack_bf16(g1[4], g1[5]); q0.w = pack_bf16(g1[6], g1[7]);
                q1.x = pack_bf16(g1[8], g1[9]); q1.y = pack_bf16(g1[10], g1[11]); q1.z = pack_bf16(g1[12], g1[13]); q1.w = pack_bf16(g1[14], g1[15]);
                reinterpret_cast<uint4*>(dst + m0)[0] = q0;
                reinterpret_cast<uint4*>(dst + m0)[1] = q1;
                q0.x = pack_bf16(g2[0], g2[1]); q0.y = pack_bf16(g2[2], g2[3]); q0.z = pack_bf16(g2[4], g2[5]); q0.w = pack_bf16(g2[6], g2[7]);
                q1.x = pack_bf16(g2[8], g2[9]); q1.y = pack_bf16(g2[10], g2[11]); q1.z = pack_bf16(g2[12], g2[13]); q1.w = pack_bf16(g2[14], g2[15]);
                reinterpret_cast<uint4*>(dst + kNH + m0)[0] = q0;
                reinterpret_cast<uint4*>(dst + kNH + m0)[1] = q1;
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  dst[(size_t)(m0 + j) * R + rr] = __float2bfloat16_rn(g1[j]);
                  dst[(size_t)(kNH + m0 + j) * R + rr] = __float2bfloat16_rn(g2[j]);
                }
              }
            }
          }
        } else {
#pragma unroll 1
          for (int cc = 0; cc < 4; ++cc) {
            const int n0 = 64 * ch + 16 * cc;
            float g1[16];
            tmem_ld16(tmem_addr(tm, quad * 32, tcol + n0), g1);
            if (which == 0 && at_end && p.dlu) {
              for (int j = 0; j < 16; ++j) {
                float s1 = 0.0f;
                for (int pp = 0; pp < kP; ++pp)
                  s1 += p.dlu[((size_t)bh * kP + pp) * kN + n0 + j] *
                        __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(row, pp, kP)));
                g1[j] += s1;
              }
            }
            if (live && dst) {
              if (R == 1) {
                uint4 q0, q1;
                q0.x = pack_bf16(g1[0], g1[1]); q0.y = pack_bf16(g1[2], g1[3]); q0.z = pack_bf16(g1[4], g1[5]); q0.w = pack_bf16(g1[6], g1[7]);
                q1.x = pack_bf16(g1[8], g1[9]); q1.y = pack_bf16(g1[10], g1[11]); q1.z = pack_bf16(g1[12], g1[13]); q1.w = pack_bf16(g1[14], g1[15]);
                reinterpret_cast<uint4*>(dst + n0)[0] = q0;
                reinterpret_cast<uint4*>(dst + n0)[1] = q1;
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) dst[(size_t)(n0 + j) * R + rr] = __float2bfloat16_rn(g1[j]);
              }
            }
          }
        }
      }
      if (ROT) {
        // d phi of a time step sums its R rows (adjacent lanes); it then overwrites dG's buffer,
        // which the phase-B products have finished reading.
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = dphi[j];
#pragma unroll
          for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          dphi[j] = v;
        }
        __syncthreads();  // every thread is done reading sB / sC / sM-as-phi? (phi stays; dG region is free)
        if (rr == 0) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float v = live ? dphi[j] : 0.0f;
            if (at_end && p.dangle) v += p.dangle[(size_t)bh * kNH + 32 * ch + j];
            sDphi[rl * kNH + 32 * ch + j] = v;
          }
        }
      }
    }
    const float dD_tile = cta_sum(dD_part, s_red);  // also orders part_* and sDphi for what follows
    if (tid == 0) p.partD[(size_t)bh * ntiles + k] = dD_tile;
    // ---- 8. reverse cumulative sum of d phi over time -> d theta, and the dt term -----------------
    if (ROT) {
      constexpr int LQ = LT / 4;
      const int q = tid >> 6, m = tid & 63;
      float run = 0.0f;
      for (int i = LQ - 1; i >= 0; --i) {
        const int l = q * LQ + i;
        run += sDphi[l * kNH + m];
        sDphi[l * kNH + m] = run;
      }
      s_q[q * 64 + m] = run;
      __syncthreads();
      float off = s_dcar[m];
      for (int qq = 3; qq > q; --qq) off += s_q[qq * 64 + m];
      for (int i = 0; i < LQ; ++i) {
        const int l = q * LQ + i, tt = t0 + l;
        const float ds = sDphi[l * kNH + m] + off;
        float prod = 0.0f;
        if (tt < T) {
          const size_t ti = (tok0 + (size_t)l * H) * kNH + m;
          if (p.dtheta) p.dtheta[ti] = __float2bfloat16_rn(ds * ts.dt[l]);
          prod = ds * bf(p.theta, ti);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) prod += __shfl_xor_sync(0xffffffffu, prod, o);
        if (lane == 0) part_rot[((tid >> 5) & 1) * 128 + l] = prod;
      }
      const float total = off + s_q[0 * 64 + m];  // for q == 0: carry + all four quarters
      __syncthreads();
      if (q == 0) {
        s_dcar[m] = total;
        if (k == 0 && p.dangle0) p.dangle0[(size_t)bh * kNH + m] = total;
      }
    }
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
      if (ROT) p.ddt_rot[o] = part_rot[l] + part_rot[128 + l];
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
      const size_t i0 = ((size_t)b * T) * H + h;
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
  if (failed && tid == 0 && p.err) atomicExch(p.err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

template <int R>
cudaError_t launch_r(cudaStream_t st, const TcBwdParams& p, bool rot) {
  auto kern = rot ? tc_bwd_kernel<R, true> : tc_bwd_kernel<R, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytes, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_backward(cudaStream_t st, const TcBwdParams& p, bool rot) {
  switch (p.R) {
    case 1: return launch_r<1>(st, p, rot);
    case 2: return launch_r<2>(st, p, rot);
    case 4: return launch_r<4>(st, p, rot);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace m3
