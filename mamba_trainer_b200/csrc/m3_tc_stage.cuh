// Per-tile preparation shared by the tensor-core kernels: token scalars, the wrapped
// cumulative angle of a tile, and staging of rotated / de-interleaved bf16 operands.
// 256 threads per CTA; LT = 128 / R time steps per tile; head_dim 64, d_state 128.
#pragma once
#include "m3_tc_common.cuh"

namespace m3tc {

constexpr int kP = 64, kN = 128, kNH = 64, kRows = 128;
constexpr int kScal = 132;  // floats per per-token scalar array
constexpr float kInvTwoPi = 0.15915494309189535f, kTwoPiF = 6.283185307179586f;

__device__ __forceinline__ float bf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float wrap2pi(float v) { return v - rintf(v * kInvTwoPi) * kTwoPiF; }
__device__ __forceinline__ float expc(float d) { return __expf(fmaxf(d, -60.0f)); }
__device__ __forceinline__ float inside(float d) { return (d > -60.0f && d < 0.0f) ? 1.0f : 0.0f; }

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
template <int NREG>
__device__ __forceinline__ float elem(const uint32_t (&raw)[NREG], int i) {
  return (i & 1) ? bf16_hi(raw[i >> 1]) : bf16_lo(raw[i >> 1]);
}
__device__ __forceinline__ void store_chunk(uint8_t* base, uint32_t off, const float (&v)[8]) {
  uint4 q;
  q.x = pack_bf16(v[0], v[1]); q.y = pack_bf16(v[2], v[3]); q.z = pack_bf16(v[4], v[5]); q.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(base + off) = q;
}
// 8 consecutive bf16 of an operand buffer as floats
__device__ __forceinline__ void load_chunk(const uint8_t* base, uint32_t off, float (&v)[8]) {
  const uint4 q = *reinterpret_cast<const uint4*>(base + off);
  v[0] = bf16_lo(q.x); v[1] = bf16_hi(q.x); v[2] = bf16_lo(q.y); v[3] = bf16_hi(q.y);
  v[4] = bf16_lo(q.z); v[5] = bf16_hi(q.z); v[6] = bf16_lo(q.w); v[7] = bf16_hi(q.w);
}

// Scalar arrays of one tile, all [kScal] floats in shared memory.
struct TileScalars {
  float *dt, *lam, *a, *ac, *g, *w, *sw, *eac;
};

// dt, lambda (with one step of look-ahead), g, w (shifted add), a = dt A, its inclusive
// cumulative sum ac, sw = exp(cd - ac) w and eac = exp(ac).  Ends with every array visible
// to all threads (the caller's next __syncthreads is still required for sw / eac).
template <int R>
__device__ __forceinline__ void tile_scalars(const TileScalars& s, const __nv_bfloat16* dt, const __nv_bfloat16* lam,
                                             int disc, float A, int b, int h, int H, int T, int t0) {
  constexpr int LT = kRows / R;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid <= LT) {
    const int t = t0 + tid;
    float vdt = 0.0f, vl = 1.0f;
    if (t < T) {
      const size_t i = ((size_t)b * T + t) * H + h;
      vdt = bf(dt, i);
      vl = disc == 0 ? 1.0f : (disc == 1 ? 0.5f : bf(lam, i));
    }
    s.dt[tid] = vdt;
    s.lam[tid] = vl;
  }
  __syncthreads();
  if (tid < LT) {
    const int t = t0 + tid;
    float gv = 0.0f, wv = 0.0f, av = 0.0f;
    if (t < T) {
      gv = s.lam[tid] * s.dt[tid];
      const float f = (t + 1 < T) ? (1.0f - s.lam[tid + 1]) * s.dt[tid + 1] : 0.0f;
      wv = gv + f;
      av = s.dt[tid] * A;
    }
    s.g[tid] = gv; s.w[tid] = wv; s.a[tid] = av;
  }
  __syncthreads();
  if (warp == 0) {
    constexpr int EPL = LT / 32;
    float loc[EPL];
    float run = 0.0f;
#pragma unroll
    for (int i = 0; i < EPL; ++i) { run += s.a[lane * EPL + i]; loc[i] = run; }
    float tot = run;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, tot, o);
      if (lane >= o) tot += n;
    }
    const float base = tot - run;
#pragma unroll
    for (int i = 0; i < EPL; ++i) s.ac[lane * EPL + i] = base + loc[i];
  }
  __syncthreads();
  if (tid < LT) {
    const float cd = s.ac[LT - 1];
    s.sw[tid] = expc(cd - s.ac[tid]) * s.w[tid];
    s.eac[tid] = expc(s.ac[tid]);
  }
}

// phi[l][m] = wrap(carry[m] + sum_{l' <= l} dt_l' theta[t0 + l'][m]) for the tile; returns (to
// threads with q == 3) the wrapped angle leaving the tile.  s_q: [4][64] scratch.  Contains
// one __syncthreads; the caller syncs again before reading phi written by other threads.
template <int R>
__device__ __forceinline__ float tile_angles(float* sPhi, float* s_q, const float* carry, const float* s_dt,
                                             const __nv_bfloat16* theta, int b, int h, int H, int T, int t0,
                                             float* angle_out_bh) {
  constexpr int LT = kRows / R, LQ = LT / 4;
  const int tid = threadIdx.x, q = tid >> 6, m = tid & 63;
  float run = 0.0f;
#pragma unroll 4
  for (int i = 0; i < LQ; ++i) {
    const int l = q * LQ + i, t = t0 + l;
    if (t < T) run += s_dt[l] * bf(theta, (((size_t)b * T + t) * H + h) * kNH + m);
    sPhi[l * kNH + m] = run;
  }
  s_q[q * 64 + m] = run;
  __syncthreads();
  float off = carry[m];
  for (int qq = 0; qq < q; ++qq) off += s_q[qq * 64 + m];
  for (int i = 0; i < LQ; ++i) {
    const int l = q * LQ + i;
    const float wv = wrap2pi(sPhi[l * kNH + m] + off);
    sPhi[l * kNH + m] = wv;
    if (angle_out_bh && t0 + l == T - 1) angle_out_bh[m] = wv;
  }
  return wrap2pi(off + s_q[3 * 64 + m]);  // meaningful for q == 3
}

// Rotated (or plain) B^ / C^ rows of the tile into [128 x 128] operand buffers.
template <int R, bool ROT>
__device__ __forceinline__ void stage_bc(uint8_t* sB, uint8_t* sC, const __nv_bfloat16* gb, const __nv_bfloat16* gc,
                                         const float* sPhi, size_t tok0, int H, int T, int t0) {
  constexpr int LT = kRows / R;
  const int tid = threadIdx.x;
  if (ROT) {
    for (int it = tid; it < LT * 8; it += 256) {
      const int l = it >> 3, m0 = (it & 7) * 8;
      const bool live = t0 + l < T;
      float cs[8], sn[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) __sincosf(sPhi[l * kNH + m0 + j], &sn[j], &cs[j]);
      const size_t base = (tok0 + (size_t)l * H) * kN * R;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const __nv_bfloat16* src = which ? gc : gb;
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
        const __nv_bfloat16* src = which ? gc : gb;
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
}

// A [B,T,H,64,R] tensor's tile as a [128 x 64] operand, plus a copy with row l scaled by scale[l].
template <int R>
__device__ __forceinline__ void stage_px(uint8_t* s_plain, uint8_t* s_scaled, const __nv_bfloat16* g, const float* scale,
                                         size_t tok0, int H, int T, int t0) {
  constexpr int LT = kRows / R;
  for (int it = threadIdx.x; it < LT * 8; it += 256) {
    const int l = it >> 3, p0 = (it & 7) * 8;
    const bool live = t0 + l < T;
    uint32_t r1[4 * R];
    load_row_group<R>(g + (tok0 + (size_t)l * H) * kP * R + (size_t)p0 * R, live, r1);
    const float sv = scale[l];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float o[8], ow[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = elem(r1, j * R + r); ow[j] = o[j] * sv; }
      store_chunk(s_plain, tile_off(l * R + r, p0, kP), o);
      store_chunk(s_scaled, tile_off(l * R + r, p0, kP), ow);
    }
  }
}

// Sum over the 256 threads of the CTA; red: >= 8 floats of shared scratch.  Contains two syncs.
__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += red[i];
  return s;
}

// v[32] per lane -> returns on lane j the sum over the warp's lanes of v[j].
__device__ __forceinline__ float warp_column_sums(float (&v)[32]) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    const bool up = (lane & o) != 0;
#pragma unroll
    for (int i = 0; i < o; ++i) {
      const float send = up ? v[i] : v[i + o];
      const float keep = up ? v[i + o] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
    }
  }
  return v[0];
}

}  // namespace m3tc
