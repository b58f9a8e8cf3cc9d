// Generic backward, part A: the contraction kernels of the hand-written adjoint.
//
// The reference has no hand adjoint: its backward is the tape walking the ~25
// primitives of src/ssm/scan.rs:116-291 (rules in src/autograd/ops.rs:204-264,
// :1066-1139).  The kernels here compute the same derivatives for the folded form:
// rows rho = (t, r); G = C~ B~^T; band as in src/tensor/ops/fused.rs:2044-2070 with
// the clamp derivative of :2080-2138.
#pragma once
#include "m3_internal.h"

namespace m3 {

// dY~[(l, r), p] of chunk k, straight from the caller's dy [B,T,H,P,R]; zero in the pad.
template <class T>
struct DyRows {
  const T* dy;
  int b, h, k, T_, H, P, R, L, rev;
  __device__ __forceinline__ float operator()(int rho, int p) const {
    const int l = rho / R, r = rho - l * R, t = k * L + l;
    if (t >= T_ || p >= P) return 0.0f;
    const int tm = rev ? T_ - 1 - t : t;  // right-to-left heads: scan position t is time T-1-t
    return ldf(dy, (((size_t)b * T_ + tm) * H + h) * P * R + (size_t)p * R + r);
  }
};

__device__ __forceinline__ float band_at(const float* s_ac, const float* s_g, const float* s_w, int l, int s) {
  if (s < l) return s_w[s] * exp_decay(s_ac[l] - s_ac[s]);
  if (s == l) return s_g[s];
  return 0.0f;
}

// Sum over the 16 lanes that share threadIdx.x >> 4.
__device__ __forceinline__ float half_warp_sum(float v) {
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- row tile of one chunk: dC^ (complete), dBand, d acum from the carry-out term
template <class T>
__global__ void __launch_bounds__(256) kb_rows(Dims d, const T* __restrict__ dy, GenericWs ws, GenericBwdWs bw) {
  extern __shared__ float sm[];
  float* sA = sm;
  float* sB = sm + kGemmBK * kGemmLd;
  float* s_ac = sm + kGemmSmemFloats;
  float* s_g = s_ac + d.L;
  float* s_w = s_g + d.L;
  float* s_rowdot = s_w + d.L;     // [64]
  float* Pt = s_rowdot + 64;       // [64 * 65]
  float* dGb = Pt + 64 * 65;       // [64 * LR]
  const int k = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  const int P = d.P, N = d.N, R = d.R, LR = d.LR, L = d.L;
  const int TL = max(1, 64 / R), CW = TL * R;
  const int l0 = blockIdx.x * TL, l1 = min(L, l0 + TL);
  const int rows = (l1 - l0) * R, row0 = l0 * R, ncols = l1 * R;
  const size_t tb = (size_t)bh * d.Tp + (size_t)k * L;
  for (int l = threadIdx.x; l < L; l += blockDim.x) {
    s_ac[l] = ws.acum[tb + l];
    s_g[l] = ws.g[tb + l];
    s_w[l] = ws.w[tb + l];
  }
  if (threadIdx.x < 64) s_rowdot[threadIdx.x] = 0.0f;
  __syncthreads();
  const float* X = ws.Xh + tb * R * P;
  const float* Bm = ws.Bh + tb * R * N;
  const float* Cm = ws.Ch + tb * R * N;
  const float* Hk = ws.Hs + ((size_t)bh * (d.C + 1) + k) * P * N;
  float* dC = bw.dCh + tb * R * N;
  float* dBand = bw.dBand + ((size_t)bh * d.C + k) * L * L;
  const DyRows<T> dyf{dy, b, h, k, d.T, d.H, P, R, L, h >= d.H - d.rev};
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], acc2[4][4];
  for (int n0 = 0; n0 < ncols; n0 += CW) {
    zero_acc(acc);
    zero_acc(acc2);
    gemm_tile<true, true>(
        acc, 0, n0, 0, N,
        [&](int m, int kk) { return m < rows ? Cm[(size_t)(row0 + m) * N + kk] : 0.0f; },
        [&](int kk, int n) { return n < ncols ? Bm[(size_t)n * N + kk] : 0.0f; }, sA, sB);
    gemm_tile<true, true>(
        acc2, 0, n0, 0, P,
        [&](int m, int kk) { return m < rows ? dyf(row0 + m, kk) : 0.0f; },
        [&](int kk, int n) { return n < ncols ? X[(size_t)n * P + kk] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, cj = tx * 4 + j, col = n0 + cj;
        float prod = 0.0f;
        if (m < rows && cj < CW && col < ncols) {
          const int l = l0 + m / R, s = col / R;
          const float bv = band_at(s_ac, s_g, s_w, l, s);
          dGb[(size_t)m * LR + col] = acc2[i][j] * bv;
          if (s <= l) prod = acc2[i][j] * acc[i][j];
        }
        Pt[m * 65 + cj] = prod;
      }
    __syncthreads();
    for (int e = threadIdx.x; e < TL * TL; e += blockDim.x) {
      const int ll = e / TL, ss = e % TL;
      const int l = l0 + ll, s = n0 / R + ss;
      if (l < l1 && s <= l) {
        float sum = 0.0f;
        for (int i = 0; i < R; ++i)
          for (int j = 0; j < R; ++j) sum += Pt[(ll * R + i) * 65 + ss * R + j];
        dBand[(size_t)l * L + s] = sum;
      }
    }
    __syncthreads();
  }
  for (int n0 = 0; n0 < N; n0 += 64) {
    zero_acc(acc);
    zero_acc(acc2);
    gemm_tile<true, false>(
        acc, 0, n0, 0, ncols,
        [&](int m, int kk) { return m < rows ? dGb[(size_t)m * LR + kk] : 0.0f; },
        [&](int kk, int n) { return n < N ? Bm[(size_t)kk * N + n] : 0.0f; }, sA, sB);
    gemm_tile<true, false>(
        acc2, 0, n0, 0, P,
        [&](int m, int kk) { return m < rows ? dyf(row0 + m, kk) : 0.0f; },
        [&](int kk, int n) { return n < N ? Hk[(size_t)kk * N + n] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = ty * 4 + i;
      float part = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int n = n0 + tx * 4 + j;
        if (m < rows && n < N) {
          const float eac = exp_decay(s_ac[l0 + m / R]);
          dC[(size_t)(row0 + m) * N + n] = acc[i][j] + eac * acc2[i][j];
          part += acc2[i][j] * Cm[(size_t)(row0 + m) * N + n];
        }
      }
      part = half_warp_sum(part);
      if (tx == 0) s_rowdot[m] += part;
    }
  }
  __syncthreads();
  for (int ll = threadIdx.x; ll < l1 - l0; ll += blockDim.x) {
    float sum = 0.0f;
    for (int i = 0; i < R; ++i) sum += s_rowdot[ll * R + i];
    const float ac = s_ac[l0 + ll];
    bw.dac[tb + l0 + ll] = exp_decay(ac) * clamp_inside(ac) * sum;
  }
}

// ---- local dH_k = (exp(acum) dY~)^T C~   [P x N]
template <class T>
__global__ void __launch_bounds__(256) kb_dhloc(Dims d, const T* __restrict__ dy, GenericWs ws, GenericBwdWs bw) {
  extern __shared__ float sm[];
  float* sA = sm;
  float* sB = sm + kGemmBK * kGemmLd;
  float* s_e = sm + kGemmSmemFloats;  // [L]
  const int tiles_n = (d.N + 63) / 64;
  const int p0 = (blockIdx.x / tiles_n) * 64, n0 = (blockIdx.x % tiles_n) * 64;
  const int k = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  const size_t tb = (size_t)bh * d.Tp + (size_t)k * d.L;
  for (int l = threadIdx.x; l < d.L; l += blockDim.x) s_e[l] = exp_decay(ws.acum[tb + l]);
  __syncthreads();
  const float* Cm = ws.Ch + tb * d.R * d.N;
  const int P = d.P, N = d.N, R = d.R;
  const DyRows<T> dyf{dy, b, h, k, d.T, d.H, P, R, d.L, h >= d.H - d.rev};
  float acc[4][4];
  zero_acc(acc);
  gemm_tile<false, false>(
      acc, p0, n0, 0, d.LR,
      [&](int p, int rho) { return s_e[rho / R] * dyf(rho, p); },
      [&](int rho, int n) { return n < N ? Cm[(size_t)rho * N + n] : 0.0f; }, sA, sB);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float* out = bw.dHs + ((size_t)bh * (d.C + 1) + k) * P * N;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (p < P && n < N) out[(size_t)p * N + n] = acc[i][j];
    }
}

// ---- reverse state pass: dS_k = dH_{k+1};  dH_k = exp(cd_k) dH_{k+1} + local_k.
// Slot k of dHs ends up holding dS_k, slot C the gradient of the seed state.
__global__ void kb_state_pass_rev(Dims d, const float* __restrict__ dh, GenericWs ws, GenericBwdWs bw) {
  const int bh = blockIdx.y;
  const int PN = d.P * d.N;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = e < PN;
  const int lane = threadIdx.x & 31;
  float carry = (live && dh) ? dh[(size_t)bh * PN + e] : 0.0f;
  float* dHs = bw.dHs + (size_t)bh * (d.C + 1) * PN;
  for (int k1 = d.C; k1 > 0; k1 -= 32) {
    const int kk = k1 - 1 - lane;  // lane j serves chunk k1-1-j
    const float mine = (kk >= 0) ? exp_decay(ws.acum[(size_t)bh * d.Tp + (size_t)kk * d.L + d.L - 1]) : 1.0f;
    const int cnt = min(32, k1);
    for (int j = 0; j < cnt; ++j) {
      const float ecd = __shfl_sync(0xffffffffu, mine, j);
      if (live) {
        const size_t o = (size_t)(k1 - 1 - j) * PN + e;
        const float loc = dHs[o];
        dHs[o] = carry;
        carry = fmaf(ecd, carry, loc);
      }
    }
  }
  if (live) dHs[(size_t)d.C * PN + e] = carry;
}

// ---- d cd_k = exp(cd_k) <dS_k, H_k> (block k < C); block C: <dH_0, last_u0>
__global__ void __launch_bounds__(256) kb_dcd(Dims d, const float* __restrict__ lu0, GenericWs ws, GenericBwdWs bw) {
  __shared__ float red[8];
  const int k = blockIdx.x, bh = blockIdx.y;
  const int PN = d.P * d.N;
  const float* a = bw.dHs + ((size_t)bh * (d.C + 1) + k) * PN;
  const float* bptr = (k < d.C) ? ws.Hs + ((size_t)bh * (d.C + 1) + k) * PN : lu0 + (size_t)bh * PN;
  if (k == d.C && !lu0) return;
  float s = 0.0f;
  for (int e = threadIdx.x; e < PN; e += 256) s += a[e] * bptr[e];
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) {
    if (k < d.C) {
      const float cd = ws.acum[(size_t)bh * d.Tp + (size_t)k * d.L + d.L - 1];
      bw.dcd[(size_t)bh * d.C + k] = exp_decay(cd) * clamp_inside(cd) * s;
    } else {
      bw.ip0[bh] = s;
    }
  }
}

// ---- column tile of one chunk: dX~ and dB^ (complete), and the chunk-state terms
// of dw and d acum.
template <class T>
__global__ void __launch_bounds__(256) kb_cols(Dims d, const T* __restrict__ dy, GenericWs ws, GenericBwdWs bw) {
  extern __shared__ float sm[];
  float* sA = sm;
  float* sB = sm + kGemmBK * kGemmLd;
  float* s_ac = sm + kGemmSmemFloats;
  float* s_g = s_ac + d.L;
  float* s_w = s_g + d.L;
  float* s_q = s_w + d.L;   // [64]
  float* Wb = s_q + 64;     // [64 * LR]
  const int k = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  const int P = d.P, N = d.N, R = d.R, LR = d.LR, L = d.L;
  const int TL = max(1, 64 / R);
  const int s0 = blockIdx.x * TL, s1 = min(L, s0 + TL);
  const int rows = (s1 - s0) * R, row0 = s0 * R;
  const size_t tb = (size_t)bh * d.Tp + (size_t)k * L;
  for (int l = threadIdx.x; l < L; l += blockDim.x) {
    s_ac[l] = ws.acum[tb + l];
    s_g[l] = ws.g[tb + l];
    s_w[l] = ws.w[tb + l];
  }
  if (threadIdx.x < 64) s_q[threadIdx.x] = 0.0f;
  __syncthreads();
  const float cd = s_ac[L - 1];
  const float* X = ws.Xh + tb * R * P;
  const float* Bm = ws.Bh + tb * R * N;
  const float* Cm = ws.Ch + tb * R * N;
  const float* dS = bw.dHs + ((size_t)bh * (d.C + 1) + k) * P * N;
  float* dX = bw.dXh + tb * R * P;
  float* dB = bw.dBh + tb * R * N;
  const DyRows<T> dyf{dy, b, h, k, d.T, d.H, P, R, L, h >= d.H - d.rev};
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4], acc2[4][4];
  // pass 1: W = (G o band)^T rows of this tile, then dX~
  for (int n0 = row0; n0 < LR; n0 += 64) {
    zero_acc(acc);
    gemm_tile<true, true>(
        acc, 0, n0, 0, N,
        [&](int m, int kk) { return m < rows ? Bm[(size_t)(row0 + m) * N + kk] : 0.0f; },
        [&](int kk, int n) { return n < LR ? Cm[(size_t)n * N + kk] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, rl = n0 + tx * 4 + j;
        if (m < rows && rl < LR)
          Wb[(size_t)m * LR + rl] = acc[i][j] * band_at(s_ac, s_g, s_w, rl / R, s0 + m / R);
      }
  }
  __syncthreads();
  for (int p0 = 0; p0 < P; p0 += 64) {
    zero_acc(acc);
    zero_acc(acc2);
    gemm_tile<true, false>(
        acc, 0, p0, row0, LR,
        [&](int m, int kk) { return m < rows ? Wb[(size_t)m * LR + kk] : 0.0f; },
        [&](int kk, int n) { return dyf(kk, n); }, sA, sB);
    gemm_tile<true, true>(
        acc2, 0, p0, 0, N,
        [&](int m, int kk) { return m < rows ? Bm[(size_t)(row0 + m) * N + kk] : 0.0f; },
        [&](int kk, int n) { return n < P ? dS[(size_t)n * N + kk] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int m = ty * 4 + i;
      float part = 0.0f;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int p = p0 + tx * 4 + j;
        if (m < rows && p < P) {
          const int s = s0 + m / R;
          const float sw = exp_decay(cd - s_ac[s]) * s_w[s];
          dX[(size_t)(row0 + m) * P + p] = acc[i][j] + sw * acc2[i][j];
          part += acc2[i][j] * X[(size_t)(row0 + m) * P + p];
        }
      }
      part = half_warp_sum(part);
      if (tx == 0) s_q[m] += part;
    }
  }
  __syncthreads();
  // pass 2: W = (dM o band)^T rows of this tile, then dB^
  for (int n0 = row0; n0 < LR; n0 += 64) {
    zero_acc(acc);
    gemm_tile<true, true>(
        acc, 0, n0, 0, P,
        [&](int m, int kk) { return m < rows ? X[(size_t)(row0 + m) * P + kk] : 0.0f; },
        [&](int kk, int n) { return n < LR ? dyf(n, kk) : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, rl = n0 + tx * 4 + j;
        if (m < rows && rl < LR)
          Wb[(size_t)m * LR + rl] = acc[i][j] * band_at(s_ac, s_g, s_w, rl / R, s0 + m / R);
      }
  }
  __syncthreads();
  for (int n0 = 0; n0 < N; n0 += 64) {
    zero_acc(acc);
    zero_acc(acc2);
    gemm_tile<true, false>(
        acc, 0, n0, row0, LR,
        [&](int m, int kk) { return m < rows ? Wb[(size_t)m * LR + kk] : 0.0f; },
        [&](int kk, int n) { return n < N ? Cm[(size_t)kk * N + n] : 0.0f; }, sA, sB);
    gemm_tile<true, false>(
        acc2, 0, n0, 0, P,
        [&](int m, int kk) { return m < rows ? X[(size_t)(row0 + m) * P + kk] : 0.0f; },
        [&](int kk, int n) { return n < N ? dS[(size_t)kk * N + n] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, n = n0 + tx * 4 + j;
        if (m < rows && n < N) {
          const int s = s0 + m / R;
          const float sw = exp_decay(cd - s_ac[s]) * s_w[s];
          dB[(size_t)(row0 + m) * N + n] = acc[i][j] + sw * acc2[i][j];
        }
      }
  }
  __syncthreads();
  for (int ss = threadIdx.x; ss < s1 - s0; ss += blockDim.x) {
    float q = 0.0f;
    for (int j = 0; j < R; ++j) q += s_q[ss * R + j];
    const int s = s0 + ss;
    const float raw = cd - s_ac[s];
    const float sg = exp_decay(raw);
    bw.dws[tb + s] = sg * q;
    bw.dast[tb + s] = sg * s_w[s] * q * clamp_inside(raw);
  }
}

}  // namespace m3
