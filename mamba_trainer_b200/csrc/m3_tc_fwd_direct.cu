// Tensor-core forward of the Mamba-3 SSD scan, direct form: rank 1 with real dynamics
// (sm_100a: tcgen05 MMA, TMEM accumulators, bulk tensor copies).
//
// Without a rotation and with one rank, C^ = C, B^ = B and X~ = x: the rows need no conversion, only
// the operand layout, and a 4-D tiled tensor map lands a [128 tokens x cols] tile of a dense
// [B, T, H, cols] tensor in exactly that layout (tc_make_tile_map).  C, B and x exist twice in shared
// memory, so tile k+1 arrives while tile k computes; no thread touches the raw rows except for the
// scaled copy sigma_w x.  Needs every head left to right, T a multiple of 8 and 16-byte aligned
// tensors; everything else takes the role-split kernel of m3_tc_fwd.cu.  The arithmetic per tile is
// the same (scan.rs:192-268): Yoff = C H, G = C B^T, M = G o band, Y += M x, H^T += B^T (sigma_w x).
// 256 threads: warps 1-7 compute the next tile's scalars while thread 0 issues the products.
#include "m3_tc.h"
#include "m3_tc_stage.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr uint32_t TM_G = 0, TM_Y = 128, TM_H = 192, TM_COLS = 256;
constexpr uint32_t TO_C0 = 0, TO_C1 = 65536, TO_X0 = 131072, TO_X1 = 147456,  // B follows its C at + 32768
                   TO_XW = 163840, TO_H = 180224, TO_SC = 196608;
constexpr uint32_t kSmemBytesDirect = TO_SC + (2 * kNumScal * kScal) * 4 + 64;
constexpr uint32_t kTileBytesDirect = 2 * kRows * kN * 2 + kRows * kP * 2;  // C, B and x of one tile

__global__ void __launch_bounds__(256, 1) tc_fwd_direct_kernel(const __grid_constant__ TcFwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int R = 1, LT = kRows;
  uint8_t *sC, *sB, *sX;
  uint8_t* sXw = smem + TO_XW;
  uint8_t* sH = smem + TO_H;    // bf16 H [n][p]: a thread's 16 columns are two 16-byte pieces of its row
  float* sc = reinterpret_cast<float*>(smem + TO_SC);
  // Two sets of per-token scalars: the next tile's are computed while this tile's products run.
  auto scal_set = [&](int i) {
    float* q = sc + i * kNumScal * kScal;
    return TileScalars{q, q + kScal, q + 2 * kScal, q + 3 * kScal, q + 4 * kScal, q + 5 * kScal, q + 6 * kScal,
                       q + 7 * kScal, q + 8 * kScal};
  };
  uint64_t* bars = reinterpret_cast<uint64_t*>(sc + 2 * kNumScal * kScal);  // [0], [1]: tensor-core phases; [2], [3]: tile arrivals
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  auto tok_at = [&](int s) { return ((size_t)b * T + s) * H + h; };
  const int ntiles = (T + LT - 1) / LT;
  const float A = -expf(p.a_log[h]);
  const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 32 + lane;
  const uint32_t wait_limit = p.wait_limit;

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
      }
      store_row16(sH, row, p0, kP, v);
      tmem_st16(tmem_addr(tm, quad * 32, TM_H + p0), v);
    }
    tmem_wait_st();
  }
  fence_async_smem();
  __syncthreads();  // the bf16 seed is read by the checkpoint's bulk copy and the first product

  bool failed = false;
  int fail_bar = -1;      // the tensor-core barrier whose phase was in flight when a wait gave up
  uint32_t fail_parity = 0;
  float nx_dt, nx_lam;  // dt / lambda of the next tile, loaded one tile ahead
  load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, 0, false);
  // one thread asks for the three tiles of a time block; they land in operand layout
  auto request_tile = [&](int kk) {
    uint64_t* bar = &bars[2 + (kk & 1)];
    uint8_t* base = smem + ((kk & 1) ? TO_C1 : TO_C0);
    const int tg = (b * T + kk * LT) / 8;  // token group of the tile's first row (T % 8 == 0)
    mbar_expect_tx(bar, kTileBytesDirect);
    tma_load_tile(base, &p.tm_c, bar, h * (kN / 8), tg);
    tma_load_tile(base + 32768, &p.tm_b, bar, h * (kN / 8), tg);
    tma_load_tile(smem + ((kk & 1) ? TO_X1 : TO_X0), &p.tm_x, bar, h * (kP / 8), tg);
  };
  if (tid == 0) request_tile(0);
  int requested = 1;  // tiles asked for so far (the same in every thread)
  // Scalars always run one tile ahead, inside the waits for the tensor core.
  auto prepare_scalars = [&](int k1) {
    tile_scalars<R>(scal_set(k1 & 1), nx_dt, nx_lam, A, T, k1 * LT);
    load_dt_lam<R>(nx_dt, nx_lam, p.dt, p.lam, p.disc, b, h, H, T, (k1 + 1) * LT, false);
  };
  prepare_scalars(0);
  __syncthreads();
  for (int k = 0; k < ntiles; ++k) {
    const int t0 = k * LT;
    const TileScalars ts = scal_set(k & 1);
    float *s_ac = ts.ac, *s_eac = ts.eac;
    const size_t tok0 = tok_at(t0);
    sC = smem + ((k & 1) ? TO_C1 : TO_C0);
    sB = sC + 32768;
    sX = smem + ((k & 1) ? TO_X1 : TO_X0);
    // the other set was last touched by tile k-1, whose products and reads are complete
    if (k + 1 < ntiles) {
      if (tid == 0) request_tile(k + 1);
      requested = k + 2;
    }
    if (p.ckpt_h && tid == 0) {  // the bf16 state entering this tile, for the backward pass
      bulk_store(p.ckpt_h + ((size_t)bh * ntiles + k) * kN * kP, sH, kN * kP * 2);
      bulk_commit();
    }
    {
      const bool ok = mbar_wait(&bars[2 + (k & 1)], (k >> 1) & 1, wait_limit);
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
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- MMA phase 1: Yoff = C . H (over n), G = C B^T
    if (tid == 0) {
      tc_fence_after();
      const Operand aC = k_major(smem_u32(sC), kN);
      gemm_issue(tm + TM_Y, aC, mn_major(smem_u32(sH), kP), make_idesc(64, 0, 1), kN, false);
      gemm_issue(tm + TM_G, aC, k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
      umma_commit(&bars[0]);
    }
    // sigma_w x, the scaled copy of x for the state update, is first needed by the second pair of
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
    if (k + 1 < ntiles) prepare_scalars(k + 1);   // while G and Yoff are being computed
    {
      const bool ok = mbar_wait(&bars[0], k & 1, wait_limit);
      if (__syncthreads_or(!ok)) { failed = true; fail_bar = 0; fail_parity = k & 1; break; }
    }
    tc_fence_after();
    // ---- band, decays
    {
      const int l = row;
      const float acl = s_ac[l];
      const int lmax = quad * 32 + 31;  // last time step held by this warp
      float g[4][16], yv[2][16], hv[2][16];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int c0 = 64 * ch + 16 * cc;
        if (c0 <= lmax) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_G + c0), g[cc]);
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
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        const int c0 = 64 * ch + 16 * cc;
        float m[16];
        if (c0 > lmax) {
#pragma unroll
          for (int j = 0; j < 16; ++j) m[j] = 0.0f;
        } else {
          ColScalars<R> cs;
          load_col_scalars<R>(cs, ts, c0);
          const float rf = row_factor(acl, s_ac[c0 + 15]);  // one exponential per chunk
          if (c0 + 15 < quad * 32) {
            // strictly below the diagonal for all 32 rows of this warp: no selects, and the weight is
            // shared by every row up to the row factor
            const float2 rf2 = make_float2(rf, rf);
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const float2 wc = __fmul2_rn(make_float2(cs.w[j], cs.w[j + 1]), make_float2(cs.cf[j], cs.cf[j + 1]));
              const float2 m2 = __fmul2_rn(make_float2(g[cc][j], g[cc][j + 1]), __fmul2_rn(wc, rf2));
              m[j] = m2.x; m[j + 1] = m2.y;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {  // branch-free: select between below / on / above the diagonal
              const int s = c0 + j;
              const float wgt = s < l ? cs.w[j] * (rf * cs.cf[j]) : (s == l ? cs.g[j] : 0.0f);
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
    __syncthreads();
    // ---- MMA phase 2: Y += M x ; H^T += B^T (sigma_w x)
    if (tid == 0) {
      tc_fence_after();
      gemm_issue(tm + TM_Y, k_major(smem_u32(sC), kRows), mn_major(smem_u32(sX), kP), make_idesc(64, 0, 1), kRows, true);
      gemm_issue(tm + TM_H, mn_major(smem_u32(sB), kN), mn_major(smem_u32(sXw), kP), make_idesc(64, 1, 1), kRows, true);
      umma_commit(&bars[1]);
    }
    if (p.ckpt_h && tid == 0) bulk_wait_read();   // the checkpoint has left the state's bf16 copy
    {
      const bool ok = mbar_wait(&bars[1], k & 1, wait_limit);
      if (__syncthreads_or(!ok)) { failed = true; fail_bar = 1; fail_parity = k & 1; break; }
    }
    tc_fence_after();
    // ---- outputs
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
        stage_store16<kP>(sXw, row, p0, v);  // sigma_w x is spent: its buffer stages y
        store_row16(sH, row, p0, kP, hv[cc]);
        if (k == ntiles - 1 && p.h_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) p.h_out[((size_t)bh * kP + p0 + j) * kN + row] = hv[cc][j];
        }
      }
      if (k == ntiles - 1 && p.lu_out) {
        // last_u = x_{T-1} (x) B_{T-1}, from the staged operands (scan.rs:621-638)
        const int ll = T - 1 - t0;
        for (int e = tid; e < kP * kN; e += 256) {
          const int pp = e / kN, n = e % kN;
          const float xv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(ll, pp, kP)));
          const float bv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(ll, n, kN)));
          p.lu_out[(size_t)bh * kP * kN + e] = xv * bv;
        }
      }
    }
    __syncthreads();
    copy_out<R, kP>(sXw, p.y, tok0, H, T, t0);
    fence_async_smem();  // this tile's writes to its operand set and to the state's bf16 copy, before bulk copies touch them
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (failed && tid == 0 && p.err) raise_flag(p.err);
  if (failed) {
    // A wait gave up: products already issued still write this CTA's TMEM, and bulk copies already
    // requested still target its shared memory.  Give each of them one more wait, on the full limit,
    // before the CTA lets go of either.
    if (fail_bar >= 0) mbar_wait(&bars[fail_bar], fail_parity);
    for (int kk = requested > 2 ? requested - 2 : 0; kk < requested; ++kk) mbar_wait(&bars[2 + (kk & 1)], (kk >> 1) & 1);
  }
  if (tid == 0) bulk_wait_all();  // a checkpoint copy may still be reading this CTA's shared memory
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

}  // namespace

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

bool tc_make_row_map(CUtensorMap* map, const void* base, int B, int T, int H, int cols, int steps, bool swizzle) {
  typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeFn encode = [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess) fn = nullptr;
    return reinterpret_cast<EncodeFn>(fn);
  }();
  if (!encode || cols % 64 || steps < 1 || steps > 256 || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)H, (cuuint64_t)T, (cuuint64_t)B};
  const cuuint64_t strides[3] = {(cuuint64_t)cols * 2, (cuuint64_t)H * cols * 2, (cuuint64_t)T * H * cols * 2};
  const cuuint32_t box[4] = {64, 1, (cuuint32_t)steps, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                CU_TENSOR_MAP_L2_PROMOTION_NONE,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

cudaError_t tc_forward_direct(cudaStream_t st, const TcFwdParams& p) {
  auto kern = tc_fwd_direct_kernel;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytesDirect);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytesDirect, st>>>(p);
  return cudaGetLastError();
}

}  // namespace m3
