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
#include "m3_tc.h"
#include "m3_tc_common.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr int kP = 64, kN = 128, kNH = 64, kRows = 128;
constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_XW = 81920, OFF_H = 98304, OFF_PHI = 114688,
                   OFF_SC = 147456;
constexpr int kScal = 132;  // floats per scalar array
// scalar arrays: dt, lam, a, ac, g, w, sw, eac ; then carry[64], quarter sums[4][64]
constexpr uint32_t kSmemBytes = OFF_SC + (8 * kScal + 64 + 256) * 4 + 64;
constexpr uint32_t TM_G = 0, TM_Y = 128, TM_H = 192, TM_COLS = 256;

__device__ __forceinline__ float bf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <int R>
__device__ __forceinline__ void load_row_group(const __nv_bfloat16* src, bool live, uint32_t (&raw)[4 * R]) {
  if (live) {
    const uint4* q = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const uint4 v = __ldg(q + i);
      raw[4 * i] = v.x; raw[4 * i + 1] = v.y; raw[4 * i + 2] = v.z; raw[4 * i + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4 * R; ++i) raw[i] = 0u;
  }
}
// element i of a packed bf16 register array
template <int NREG>
__device__ __forceinline__ float elem(const uint32_t (&raw)[NREG], int i) {
  return (i & 1) ? bf16_hi(raw[i >> 1]) : bf16_lo(raw[i >> 1]);
}
__device__ __forceinline__ void store_chunk(uint8_t* base, uint32_t off, const float (&v)[8]) {
  uint4 q;
  q.x = pack_bf16(v[0], v[1]); q.y = pack_bf16(v[2], v[3]); q.z = pack_bf16(v[4], v[5]); q.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(base + off) = q;
}

template <int R, bool ROT>
__global__ void __launch_bounds__(256, 1) tc_fwd_kernel(TcFwdParams p) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int LT = kRows / R;  // time steps per tile
  uint8_t* sC = smem + OFF_C;    // C^ operand, later M = G o band
  uint8_t* sB = smem + OFF_B;
  uint8_t* sX = smem + OFF_X;
  uint8_t* sXw = smem + OFF_XW;
  uint8_t* sH = smem + OFF_H;    // bf16 H [p][n]
  float* sPhi = reinterpret_cast<float*>(smem + OFF_PHI);
  float* sc = reinterpret_cast<float*>(smem + OFF_SC);
  float *s_dt = sc, *s_lam = sc + kScal, *s_a = sc + 2 * kScal, *s_ac = sc + 3 * kScal, *s_g = sc + 4 * kScal,
        *s_w = sc + 5 * kScal, *s_sw = sc + 6 * kScal, *s_eac = sc + 7 * kScal;
  float* s_carry = sc + 8 * kScal;       // [64] running angle
  float* s_q = s_carry + 64;             // [4][64]
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_q + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
  const int T = p.T, H = p.H;
  const int ntiles = (T + LT - 1) / LT;
  const float A = -expf(p.a_log[h]);
  const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
  const int quad = warp & 3, ch = warp >> 2;
  const int row = quad * 32 + lane;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
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
      const size_t i0 = ((size_t)b * T) * H + h;
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

  bool failed = false;
  for (int k = 0; k < ntiles; ++k) {
    const int t0 = k * LT;
    // ---- 1. per-token scalars -------------------------------------------------
    if (tid <= LT) {
      const int t = t0 + tid;
      float vdt = 0.0f, vl = 1.0f;
      if (t < T) {
        const size_t i = ((size_t)b * T + t) * H + h;
        vdt = bf(p.dt, i);
        vl = p.disc == 0 ? 1.0f : (p.disc == 1 ? 0.5f : bf(p.lam, i));
      }
      s_dt[tid] = vdt;
      s_lam[tid] = vl;
    }
    __syncthreads();
    if (tid < LT) {
      const int t = t0 + tid;
      float gv = 0.0f, wv = 0.0f, av = 0.0f;
      if (t < T) {
        gv = s_lam[tid] * s_dt[tid];
        const float f = (t + 1 < T) ? (1.0f - s_lam[tid + 1]) * s_dt[tid + 1] : 0.0f;
        wv = gv + f;
        av = s_dt[tid] * A;
      }
      s_g[tid] = gv; s_w[tid] = wv; s_a[tid] = av;
    }
    __syncthreads();
    if (warp == 0) {  // inclusive scan of a over the tile
      constexpr int EPL = LT / 32;
      float loc[EPL];
      float run = 0.0f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) { run += s_a[lane * EPL + i]; loc[i] = run; }
      float tot = run;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, tot, o);
        if (lane >= o) tot += n;
      }
      const float base = tot - run;
#pragma unroll
      for (int i = 0; i < EPL; ++i) s_ac[lane * EPL + i] = base + loc[i];
    }
    __syncthreads();
    if (tid < LT) {
      const float cd = s_ac[LT - 1];
      s_sw[tid] = __expf(fmaxf(cd - s_ac[tid], -60.0f)) * s_w[tid];
      s_eac[tid] = __expf(fmaxf(s_ac[tid], -60.0f));
    }
    // ---- 2. wrapped cumulative angle of the tile ------------------------------
    if (ROT) {
      constexpr int LQ = LT / 4;
      const int q = tid >> 6, m = tid & 63;
      float run = 0.0f;
#pragma unroll 4
      for (int i = 0; i < LQ; ++i) {
        const int l = q * LQ + i, t = t0 + l;
        if (t < T) run += s_dt[l] * bf(p.theta, (((size_t)b * T + t) * H + h) * kNH + m);
        sPhi[l * kNH + m] = run;
      }
      s_q[q * 64 + m] = run;
      __syncthreads();
      float off = s_carry[m];
      for (int qq = 0; qq < q; ++qq) off += s_q[qq * 64 + m];
      for (int i = 0; i < LQ; ++i) {
        const int l = q * LQ + i;
        const float v = sPhi[l * kNH + m] + off;
        const float wv = v - rintf(v * 0.15915494309189535f) * 6.283185307179586f;
        sPhi[l * kNH + m] = wv;
        if (p.angle_out && t0 + l == T - 1) p.angle_out[(size_t)bh * kNH + m] = wv;
      }
      float ncarry = 0.0f;
      if (q == 3) {
        const float v = off + s_q[3 * 64 + m];
        ncarry = v - rintf(v * 0.15915494309189535f) * 6.283185307179586f;
      }
      if (p.ckpt_angle && q == 0) p.ckpt_angle[((size_t)bh * ntiles + k) * kNH + m] = s_carry[m];
      __syncthreads();
      if (q == 3) s_carry[m] = ncarry;
    } else {
      __syncthreads();
    }
    // ---- 3. stage operands ------------------------------------------------------
    {
      const size_t tok0 = ((size_t)b * T + t0) * H + h;  // token-head index of l = 0 (stride H per step)
      if (ROT) {
        for (int it = tid; it < LT * 8; it += 256) {
          const int l = it >> 3, mg = it & 7, m0 = mg * 8;
          const bool live = t0 + l < T;
          float cs[8], sn[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) __sincosf(sPhi[l * kNH + m0 + j], &sn[j], &cs[j]);
          const size_t base = (tok0 + (size_t)l * H) * kN * R;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const __nv_bfloat16* src = which ? p.c : p.b;
            uint8_t* dst = which ? sC : sB;
            uint32_t r1[4 * R], r2[4 * R];
            load_row_group<R>(src + base + (size_t)m0 * R, live, r1);
            load_row_group<R>(src + base + (size_t)(m0 + kNH) * R, live, r2);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              float o1[8], o2[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float v1 = elem(r1, j * R + r), v2 = elem(r2, j * R + r);
                o1[j] = v1 * cs[j] + v2 * sn[j];
                o2[j] = v2 * cs[j] - v1 * sn[j];
              }
              store_chunk(dst, tile_off(l * R + r, m0, kN), o1);
              store_chunk(dst, tile_off(l * R + r, m0 + kNH, kN), o2);
            }
          }
        }
      } else {
        for (int it = tid; it < LT * 16; it += 256) {
          const int l = it >> 4, n0 = (it & 15) * 8;
          const bool live = t0 + l < T;
          const size_t base = (tok0 + (size_t)l * H) * kN * R + (size_t)n0 * R;
#pragma unroll
          for (int which = 0; which < 2; ++which) {
            const __nv_bfloat16* src = which ? p.c : p.b;
            uint8_t* dst = which ? sC : sB;
            uint32_t r1[4 * R];
            load_row_group<R>(src + base, live, r1);
#pragma unroll
            for (int r = 0; r < R; ++r) {
              float o[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = elem(r1, j * R + r);
              store_chunk(dst, tile_off(l * R + r, n0, kN), o);
            }
          }
        }
      }
      for (int it = tid; it < LT * 8; it += 256) {
        const int l = it >> 3, p0 = (it & 7) * 8;
        const bool live = t0 + l < T;
        uint32_t r1[4 * R];
        load_row_group<R>(p.x + (tok0 + (size_t)l * H) * kP * R + (size_t)p0 * R, live, r1);
        const float sw = s_sw[l];
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float o[8], ow[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { o[j] = elem(r1, j * R + r); ow[j] = o[j] * sw; }
          store_chunk(sX, tile_off(l * R + r, p0, kP), o);
          store_chunk(sXw, tile_off(l * R + r, p0, kP), ow);
        }
      }
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- 4. MMA phase 1: Yoff = C^ . H (over n), G = C^ B^^T -------------------------
    if (tid == 0) {
      tc_fence_after();
      const Operand aC = k_major(smem_u32(sC), kN);
      gemm_issue(tm + TM_Y, aC, k_major(smem_u32(sH), kN), make_idesc(64, 0, 0), kN, false);
      gemm_issue(tm + TM_G, aC, k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
      umma_commit(&bars[0]);
    }
    {
      const bool ok = mbar_wait(&bars[0], k & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    // ---- 5. band, decays, checkpoint ---------------------------------------------------
    {
      const int l = row / R;
      const float acl = s_ac[l];
      const int lmax = (quad * 32 + 31) / R;  // last time step held by this warp
#pragma unroll 1
      for (int cc = 0; cc < 4; ++cc) {
        const int c0 = 64 * ch + 16 * cc;
        float m[16];
        if (c0 / R > lmax) {
#pragma unroll
          for (int j = 0; j < 16; ++j) m[j] = 0.0f;
        } else {
          float v[16];
          tmem_ld16(tmem_addr(tm, quad * 32, TM_G + c0), v);
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int s = (c0 + j) / R;
            float r = 0.0f;
            if (s < l) r = v[j] * s_w[s] * __expf(fmaxf(acl - s_ac[s], -60.0f));
            else if (s == l) r = v[j] * s_g[s];
            m[j] = r;
          }
        }
        float lo[8], hi[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) { lo[j] = m[j]; hi[j] = m[8 + j]; }
        store_chunk(sC, tile_off(row, c0, kRows), lo);
        store_chunk(sC, tile_off(row, c0 + 8, kRows), hi);
      }
      const float eac = s_eac[l];
      const float ecd = __expf(fmaxf(s_ac[LT - 1], -60.0f));
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float v[16];
        tmem_ld16(tmem_addr(tm, quad * 32, TM_Y + p0), v);
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= eac;
        tmem_st16(tmem_addr(tm, quad * 32, TM_Y + p0), v);
        // state: lane = n, columns = p
        tmem_ld16(tmem_addr(tm, quad * 32, TM_H + p0), v);
        if (p.ckpt_h) {
          float4* dst = reinterpret_cast<float4*>(p.ckpt_h + (((size_t)bh * ntiles + k) * kN + row) * kP + p0);
#pragma unroll
          for (int j = 0; j < 4; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] *= ecd;
        tmem_st16(tmem_addr(tm, quad * 32, TM_H + p0), v);
      }
      tmem_wait_st();
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    // ---- 6. MMA phase 2: Y += M X~ ; H^T += B^^T (sigma_w X~) ------------------------------
    if (tid == 0) {
      tc_fence_after();
      gemm_issue(tm + TM_Y, k_major(smem_u32(sC), kRows), mn_major(smem_u32(sX), kP), make_idesc(64, 0, 1), kRows, true);
      gemm_issue(tm + TM_H, mn_major(smem_u32(sB), kN), mn_major(smem_u32(sXw), kP), make_idesc(64, 1, 1), kRows, true);
      umma_commit(&bars[1]);
    }
    {
      const bool ok = mbar_wait(&bars[1], k & 1);
      if (__syncthreads_or(!ok)) { failed = true; break; }
    }
    tc_fence_after();
    // ---- 7. outputs -----------------------------------------------------------------------
    {
      const int l = row / R, r = row % R, t = t0 + l;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int p0 = 32 * ch + 16 * cc;
        float v[16];
        tmem_ld16(tmem_addr(tm, quad * 32, TM_Y + p0), v);
        if (p.d_skip) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
            const uint4 q = *reinterpret_cast<const uint4*>(sX + tile_off(row, p0 + 8 * hh, kP));
            const uint32_t w4[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              v[8 * hh + 2 * j] += dsk * bf16_lo(w4[j]);
              v[8 * hh + 2 * j + 1] += dsk * bf16_hi(w4[j]);
            }
          }
        }
        if (t < T) {
          __nv_bfloat16* dst = p.y + (((size_t)b * T + t) * H + h) * kP * R;
          if (R == 1) {
            uint4 q0, q1;
            q0.x = pack_bf16(v[0], v[1]); q0.y = pack_bf16(v[2], v[3]); q0.z = pack_bf16(v[4], v[5]); q0.w = pack_bf16(v[6], v[7]);
            q1.x = pack_bf16(v[8], v[9]); q1.y = pack_bf16(v[10], v[11]); q1.z = pack_bf16(v[12], v[13]); q1.w = pack_bf16(v[14], v[15]);
            reinterpret_cast<uint4*>(dst + p0)[0] = q0;
            reinterpret_cast<uint4*>(dst + p0)[1] = q1;
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) dst[(size_t)(p0 + j) * R + r] = __float2bfloat16_rn(v[j]);
          }
        }
        // refresh the bf16 copy of the state (lane = n = row, columns = p)
        tmem_ld16(tmem_addr(tm, quad * 32, TM_H + p0), v);
#pragma unroll
        for (int j = 0; j < 16; ++j)
          *reinterpret_cast<__nv_bfloat16*>(sH + tile_off(p0 + j, row, kN)) = __float2bfloat16_rn(v[j]);
        if (k == ntiles - 1 && p.h_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) p.h_out[((size_t)bh * kP + p0 + j) * kN + row] = v[j];
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
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  if (failed && tid == 0 && p.err) atomicExch(p.err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

template <int R>
cudaError_t launch_r(cudaStream_t st, const TcFwdParams& p, bool rot) {
  auto kern = rot ? tc_fwd_kernel<R, true> : tc_fwd_kernel<R, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<p.B * p.H, 256, kSmemBytes, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_forward(cudaStream_t st, const TcFwdParams& p, bool rot) {
  switch (p.R) {
    case 1: return launch_r<1>(st, p, rot);
    case 2: return launch_r<2>(st, p, rot);
    case 4: return launch_r<4>(st, p, rot);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace m3
