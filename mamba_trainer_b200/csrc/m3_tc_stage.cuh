// Per-tile preparation shared by the tensor-core kernels: token scalars, the wrapped
// cumulative angle of a tile, and staging of rotated / de-interleaved bf16 operands.
// 256 threads per CTA; LT = 128 / R time steps per tile; head_dim 64, d_state 128.
#pragma once
#include <cuda_fp16.h>

#include "m3_tc_common.cuh"

namespace m3tc {

constexpr int kP = 64, kN = 128, kNH = 64, kRows = 128;
constexpr int kScal = 132;  // floats per per-token scalar array (a multiple of 4: 16-byte reads of runs of columns)
constexpr float kInvTwoPi = 0.15915494309189535f, kTwoPiF = 6.283185307179586f;

__device__ __forceinline__ float bf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ float wrap2pi(float v) { return v - rintf(v * kInvTwoPi) * kTwoPiF; }
__device__ __forceinline__ float expc(float d) { return __expf(fmaxf(d, -60.0f)); }
__device__ __forceinline__ float inside(float d) { return (d > -60.0f && d < 0.0f) ? 1.0f : 0.0f; }

// Index of angle (l, m) in a [LT][64] float buffer whose 16-byte chunks are XOR-swizzled by
// l & 7: threads that own different rows read the same plane group without bank conflicts.
__device__ __forceinline__ int phi_idx(int l, int m) { return l * kNH + ((((m >> 2) ^ (l & 7)) << 2) | (m & 3)); }

__device__ __forceinline__ void prefetch_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

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
// Operand stores and the banks.  An operand row is 16 bytes of an 8 x 8 core matrix (128 bytes = all 32
// banks), so the bank group of a 16-byte store is its row & 7, whatever the column.  The conversion's work
// items lie over a warp as 4 steps x 8 column groups, a quarter warp - the unit a 16-byte store is served in -
// as 4 steps x 2 groups; step l holds rows l * R + r.  Were every lane to store rank r at the same time, a
// quarter warp would touch 8 / (2 R) ... 4 distinct bank groups only (rank 2: two-way conflicts, rank 4:
// four-way).  So the lanes go through the ranks in different orders, r = rr ^ rank_rotation(): for rank 2 the
// lanes of odd column groups start with rank 1, for rank 4 the order also depends on the step, and the eight
// rows of a quarter warp's store then fall into eight different bank groups.
template <int R>
__device__ __forceinline__ int rank_rotation() {
  const int lane = threadIdx.x & 31;
  return R == 2 ? ((lane >> 2) & 1) : (R == 4 ? ((((lane & 3) >> 1) << 1) | ((lane >> 2) & 1)) : 0);
}
// Element j of rank r of a rank-interleaved group of 8 R raw values (r may depend on the lane).
template <int R, int NREG>
__device__ __forceinline__ float elem_rank(const uint32_t (&raw)[NREG], int j, int r) {
  if constexpr (R == 1) {
    return elem(raw, j);
  } else if constexpr (R == 2) {
    return __uint_as_float(__byte_perm(raw[j], 0u, (r & 1) ? 0x3244u : 0x1044u));
  } else {
    const uint32_t w = (r & 2) ? raw[2 * j + 1] : raw[2 * j];
    return __uint_as_float(__byte_perm(w, 0u, (r & 1) ? 0x3244u : 0x1044u));
  }
}
__device__ __forceinline__ void store_chunk(uint8_t* base, uint32_t off, const float (&v)[8]) {
  uint4 q;
  q.x = pack_bf16(v[0], v[1]); q.y = pack_bf16(v[2], v[3]); q.z = pack_bf16(v[4], v[5]); q.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(base + off) = q;
}
// 16 consecutive columns of one row of an operand buffer [rows x cols] (col0 a multiple of 8)
__device__ __forceinline__ void store_row16(uint8_t* base, int row, int col0, int cols, const float (&v)[16]) {
  float lo[8], hi[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
  store_chunk(base, tile_off(row, col0, cols), lo);
  store_chunk(base, tile_off(row, col0 + 8, cols), hi);
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
  float *cf;   // cf[s] = exp(ac[e(s)] - ac[s]) <= 1, e(s) = last time step of s's 16-column chunk
};
constexpr int kNumScal = 9;  // arrays in a TileScalars block

// Decay between a row's step l and the columns of one 16-column chunk, factorised so that a
// thread pays ONE exponential per chunk: exp(ac_l - ac_s) = exp(ac_l - ac_e) * cf[s].  The row
// factor exceeds 1 only for rows inside the chunk, where it is bounded by the chunk's own span;
// it is clamped at e^80 (a chunk whose 16 / R steps decay by more than e^80 has no
// representable contribution left) and at e^-87 below.
__device__ __forceinline__ float row_factor(float ac_l, float ac_e) {
  return __expf(fminf(fmaxf(ac_l - ac_e, -87.0f), 80.0f));
}

// dt and lambda of step t0 + i in thread 32 + i (i <= LT: one step of look-ahead), as registers, so
// the loads of the NEXT tile can be in flight while the current one computes.
template <int R>
__device__ __forceinline__ void load_dt_lam(float& vdt, float& vl, const __nv_bfloat16* dt, const __nv_bfloat16* lam,
                                            int disc, int b, int h, int H, int T, int t0, bool rev) {
  constexpr int LT = kRows / R;
  const int tid = (int)threadIdx.x - 32, t = t0 + tid;
  vdt = 0.0f;
  vl = 1.0f;
  if (tid >= 0 && tid <= LT && t >= 0 && t < T) {
    const size_t i = ((size_t)b * T + (rev ? T - 1 - t : t)) * H + h;  // t is a scan position
    vdt = bf(dt, i);
    vl = disc == 0 ? 1.0f : (disc == 1 ? 0.5f : bf(lam, i));
  }
}

// In the direct kernels the per-tile scalars are the work of warps 1-7: warp 0 holds the thread that issues
// the tensor-core products, and that thread is held up by the tensor pipe for as long as the products run, so
// it must not be needed at a barrier meanwhile.  Warps 1-7 meet at named barrier 1 (224 threads); every one
// of their threads must reach each of its uses.
__device__ __forceinline__ void scalar_warps_sync() { asm volatile("bar.sync 1, 224;" ::: "memory"); }

// g, w (shifted add), a = dt A, its inclusive cumulative sum ac, sw = exp(cd - ac) w,
// eac = exp(ac) and the column factors cf, from the (dt, lambda) registers of load_dt_lam.
// The caller's next __syncthreads makes them visible to everyone (warp 0 included).
template <int R>
__device__ __forceinline__ void tile_scalars(const TileScalars& s, float vdt, float vl, float A, int T, int t0) {
  constexpr int LT = kRows / R;
  if (threadIdx.x < 32) return;  // warp 0 takes no part (see scalar_warps_sync)
  const int tid = (int)threadIdx.x - 32, warp = tid >> 5, lane = tid & 31;
  if (tid <= LT) {
    s.dt[tid] = vdt;
    s.lam[tid] = vl;
  }
  scalar_warps_sync();
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
  scalar_warps_sync();
  if (warp == 0) {  // the first of the seven
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
  scalar_warps_sync();
  if (tid < LT) {
    constexpr int SPC = 16 / R;  // time steps per 16-column chunk
    const float cd = s.ac[LT - 1], ac = s.ac[tid];
    s.sw[tid] = expc(cd - ac) * s.w[tid];
    s.eac[tid] = expc(ac);
    s.cf[tid] = __expf(fmaxf(s.ac[(tid / SPC) * SPC + SPC - 1] - ac, -87.0f));
  }
}

// ---------------------------------------------------------------------------------------
// Split staging: `issue_*` puts every global load of a tile in flight (into registers) before
// anything depends on them; `commit_*` converts and stores once the scalars and angles exist.
// Work items are (time step l, 16-byte group) pairs laid over the warp as 4 steps x 8 groups.
// ---------------------------------------------------------------------------------------
template <int GB>
__device__ __forceinline__ void item_coords(int i, int& l, int& grp) {
  // 4 steps x 8 groups per warp: each row contributes a full 128-byte line to a warp's load
  // (half as many lines per instruction as an 8 x 4 split, which measured 3-6 % slower end to
  // end), at the price of 2-way conflicts on the 16-byte operand stores.
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = warp + 8 * i;
  constexpr int GB8 = GB / 2;
  l = (w / GB8) * 4 + (lane & 3);
  grp = (w % GB8) * 8 + (lane >> 2);
}

template <int R, bool ROT>
struct RawBC {
  static constexpr int NIT = (ROT ? 4 : 8) / R;
  static constexpr int NP = ROT ? 2 : 1;
  static constexpr int GB = ROT ? 2 : 4;
  uint32_t v[NIT][2][NP][4 * R];
};

template <int R>
struct RawPX {
  static constexpr int NIT = 4 / R;
  uint32_t v[NIT][4 * R];
};

template <int R>
__device__ __forceinline__ void issue_px(RawPX<R>& raw, const __nv_bfloat16* g, size_t tok0, int H, int T, int t0) {
#pragma unroll
  for (int i = 0; i < RawPX<R>::NIT; ++i) {
    int l, grp;
    item_coords<2>(i, l, grp);
    load_row_group<R>(g + (tok0 + (size_t)l * H) * kP * R + (size_t)grp * 8 * R, t0 + l < T, raw.v[i]);
  }
}

template <int R>
__device__ __forceinline__ void commit_px(const RawPX<R>& raw, uint8_t* s_plain, uint8_t* s_scaled, const float* scale) {
#pragma unroll
  for (int i = 0; i < RawPX<R>::NIT; ++i) {
    int l, grp;
    item_coords<2>(i, l, grp);
    const float sv = scale[l];
    const int rot = rank_rotation<R>();
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
      const int r = rr ^ rot;
      float o[8], ow[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = elem_rank<R>(raw.v[i], j, r); ow[j] = o[j] * sv; }
      store_chunk(s_plain, tile_off(l * R + r, grp * 8, kP), o);
      store_chunk(s_scaled, tile_off(l * R + r, grp * 8, kP), ow);
    }
  }
}

// Per-source scalars of the 16 columns [c0, c0 + 16) of a band chunk: 16 / R distinct time steps.
template <int R>
struct ColScalars {
  static constexpr int NS = 16 / R;
  float cf[NS], w[NS], g[NS];
};
template <int R>
__device__ __forceinline__ void load_col_scalars(ColScalars<R>& c, const TileScalars& ts, int c0) {
  // s0 is a multiple of NS (4, 8 or 16) and every scalar array starts on a 16-byte boundary (kScal is
  // a multiple of 4): 16-byte broadcast reads, a quarter of the instructions of scalar ones
  const int s0 = c0 / R;
  const float4* qc = reinterpret_cast<const float4*>(ts.cf + s0);
  const float4* qw = reinterpret_cast<const float4*>(ts.w + s0);
  const float4* qg = reinterpret_cast<const float4*>(ts.g + s0);
#pragma unroll
  for (int i = 0; i < ColScalars<R>::NS / 4; ++i) {
    const float4 a = qc[i], b = qw[i], d = qg[i];
    c.cf[4 * i] = a.x; c.cf[4 * i + 1] = a.y; c.cf[4 * i + 2] = a.z; c.cf[4 * i + 3] = a.w;
    c.w[4 * i] = b.x; c.w[4 * i + 1] = b.y; c.w[4 * i + 2] = b.z; c.w[4 * i + 3] = b.w;
    c.g[4 * i] = d.x; c.g[4 * i + 1] = d.y; c.g[4 * i + 2] = d.z; c.g[4 * i + 3] = d.w;
  }
}

// ---------------------------------------------------------------------------------------
// Output staging: a thread owns a ROW of an accumulator tile, but the caller's tensors want
// whole rows written by neighbouring lanes.  Rows go to shared memory first ([128][C] bf16,
// 16-byte chunks XOR-swizzled by row & 7 so that both the row-owner writes and the
// row-spanning reads are conflict-free), then leave as coalesced 16-byte stores, with the
// rank de-interleave ((t, r) rows -> [.., C, R] elements) done on the way out.
// ---------------------------------------------------------------------------------------
template <int C>
__device__ __forceinline__ uint32_t stg_off(int row, int chunk) {
  return (uint32_t)(row * (C * 2) + ((chunk ^ (row & 7)) << 4));
}
template <int C>
__device__ __forceinline__ void stage_store16(uint8_t* stg, int row, int col0, const float (&v)[16]) {
  uint4 q0, q1;
  q0.x = pack_bf16(v[0], v[1]); q0.y = pack_bf16(v[2], v[3]); q0.z = pack_bf16(v[4], v[5]); q0.w = pack_bf16(v[6], v[7]);
  q1.x = pack_bf16(v[8], v[9]); q1.y = pack_bf16(v[10], v[11]); q1.z = pack_bf16(v[12], v[13]); q1.w = pack_bf16(v[14], v[15]);
  *reinterpret_cast<uint4*>(stg + stg_off<C>(row, col0 >> 3)) = q0;
  *reinterpret_cast<uint4*>(stg + stg_off<C>(row, (col0 >> 3) + 1)) = q1;
}
// Tile rows (l * R + r) -> g[(tok0 + l * H) * C * R + c * R + r], tokens t0 + l < T only.
// One item per 16 output bytes, consecutive items -> consecutive addresses, so every store
// instruction of a warp writes 512 contiguous bytes whatever the rank.  The ranks are interleaved
// in registers: output word w of a token's chunk holds elements (j, r), (j, r + 1) with
// j = 2w / R, r = 2w % R, i.e. one 16-bit half from each of two neighbouring rank rows.
template <int R, int C>
__device__ __forceinline__ void copy_out(const uint8_t* stg, __nv_bfloat16* g, size_t tok0, int H, int T, int t0) {
  constexpr int LT = kRows / R, CPR = C / 8;  // source chunks per row
#pragma unroll
  for (int i = 0; i < LT * CPR * R / 256; ++i) {
    const int it = threadIdx.x + 256 * i;
    const int o = it % R, c = (it / R) % CPR, l = it / (R * CPR);
    if (t0 + l >= T) continue;
    uint4 q;
    if (R == 1) {
      q = *reinterpret_cast<const uint4*>(stg + stg_off<C>(l, c));
    } else {
      uint32_t w4[4];
#pragma unroll
      for (int wi = 0; wi < 4; ++wi) {
        const int w = 4 * o + wi, j = (2 * w) / R, r = (2 * w) % R;
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(stg + stg_off<C>(l * R + r, c) + ((j >> 1) << 2));
        const uint32_t hi = *reinterpret_cast<const uint32_t*>(stg + stg_off<C>(l * R + r + 1, c) + ((j >> 1) << 2));
        w4[wi] = __byte_perm(lo, hi, (j & 1) ? 0x7632 : 0x5410);
      }
      q = make_uint4(w4[0], w4[1], w4[2], w4[3]);
    }
    *reinterpret_cast<uint4*>(g + (tok0 + (size_t)l * H) * C * R + (size_t)c * 8 * R + (size_t)o * 8) = q;
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
