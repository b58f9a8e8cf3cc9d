// Generic backward, part B: per-token scalars, rotation adjoint, layout restore and
// the per-head parameter reductions.
#pragma once
#include "m3_internal.h"

namespace m3 {

// ---- per chunk: d acum (band + carry-out + chunk-state + chunk-decay terms), its
// reverse cumulative sum da, and dw, dg.  Band adjoint: src/tensor/ops/fused.rs:2080-2138.
template <class T>
__global__ void kb_scalars(Dims d, const T* __restrict__ dt, GenericWs ws, GenericBwdWs bw) {
  extern __shared__ float sm[];
  float* s_ac = sm;
  float* s_g = s_ac + d.L;
  float* s_w = s_g + d.L;
  float* s_da = s_w + d.L;
  __shared__ float red[8];
  const int k = blockIdx.x, bh = blockIdx.y, b = bh / d.H, h = bh % d.H;
  const int L = d.L;
  const size_t tb = (size_t)bh * d.Tp + (size_t)k * L;
  for (int l = threadIdx.x; l < L; l += blockDim.x) {
    s_ac[l] = ws.acum[tb + l];
    s_g[l] = ws.g[tb + l];
    s_w[l] = ws.w[tb + l];
  }
  __syncthreads();
  const float* dBand = bw.dBand + ((size_t)bh * d.C + k) * L * L;
  for (int u = threadIdx.x; u < L; u += blockDim.x) {
    const float au = s_ac[u];
    float rows = 0.0f;
    for (int s = 0; s <= u; ++s) {
      const float raw = au - s_ac[s];
      const float band = (s == u ? s_g[s] : s_w[s]) * exp_decay(raw);
      rows += dBand[(size_t)u * L + s] * band * clamp_inside(raw);
    }
    float cols = 0.0f, dwv = 0.0f, dgv = 0.0f;
    for (int t = u; t < L; ++t) {
      const float raw = s_ac[t] - au;
      const float dec = exp_decay(raw);
      const float gr = dBand[(size_t)t * L + u];
      cols += gr * (t == u ? s_g[u] : s_w[u]) * dec * clamp_inside(raw);
      if (t == u) dgv += gr * dec; else dwv += gr * dec;
    }
    s_da[u] = rows - cols + bw.dac[tb + u] - bw.dast[tb + u];
    bw.dw[tb + u] = dwv + bw.dws[tb + u];
    bw.dg[tb + u] = dgv;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float tail = bw.dcd[(size_t)bh * d.C + k];
    for (int s = 0; s < L; ++s) tail += bw.dast[tb + s];
    float run = 0.0f;
    for (int l = L - 1; l >= 0; --l) {
      run += s_da[l] + (l == L - 1 ? tail : 0.0f);
      s_da[l] = run;
    }
  }
  __syncthreads();
  float part = 0.0f;
  for (int l = threadIdx.x; l < L; l += blockDim.x) {
    const int t = k * L + l;
    bw.da[tb + l] = s_da[l];
    if (t < d.T && !d.raw) part += s_da[l] * ldf(dt, tok_index(d, b, t, h));
  }
  part = block_sum_256(part, red);
  if (threadIdx.x == 0) bw.partA[(size_t)bh * d.C + k] = part;
}

// ---- gradient through the returned last_u (scan.rs:621-638), added to the rows of T-1
__global__ void kb_last_u(Dims d, const float* __restrict__ dlu, GenericWs ws, GenericBwdWs bw) {
  const int bh = blockIdx.x;
  const int P = d.P, N = d.N, R = d.R;
  const size_t row = (size_t)bh * d.Tp * R + (size_t)(d.T - 1) * R;
  const float* g = dlu + (size_t)bh * P * N;
  for (int e = threadIdx.x; e < R * P; e += blockDim.x) {
    const int r = e / P, p = e % P;
    float s = 0.0f;
    for (int n = 0; n < N; ++n) s += g[(size_t)p * N + n] * ws.Bh[(row + r) * N + n];
    bw.dXh[(row + r) * P + p] += s;
  }
  for (int e = threadIdx.x; e < R * N; e += blockDim.x) {
    const int r = e / N, n = e % N;
    float s = 0.0f;
    for (int p = 0; p < P; ++p) s += g[(size_t)p * N + n] * ws.Xh[(row + r) * P + p];
    bw.dBh[(row + r) * N + n] += s;
  }
}

// ---- rotate dB^, dC^ back by +phi into the caller's layout and collect d phi
// (src/tensor/ops/fused.rs:627-672).  Real dynamics: a plain layout restore.
template <class T>
__global__ void kb_unrotate(Dims d, GenericWs ws, GenericBwdWs bw, const float* __restrict__ dangle,
                            T* __restrict__ db, T* __restrict__ dc) {
  const int k = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int bh = b * d.H + h;
  const int N = d.N, R = d.R, NH = d.NH, L = d.L;
  const int t0 = k * L;
  if (d.rot) {
    for (int e = threadIdx.x; e < L * NH; e += blockDim.x) {
      const int m = e % NH, l = e / NH, t = t0 + l;
      if (t >= d.T) {
        bw.dphi[((size_t)bh * d.Tp + t) * NH + m] = 0.0f;
        continue;
      }
      float sn, cs;
      sincosf(ws.phi[((size_t)bh * d.Tp + t) * NH + m], &sn, &cs);
      float dphi = 0.0f;
      const size_t ob = tok_index(d, b, t, h) * N * R;
      for (int r = 0; r < R; ++r) {
        const size_t row = ((size_t)bh * d.Tp * R + (size_t)t * R + r) * N;
        {
          const float g1 = bw.dBh[row + m], g2 = bw.dBh[row + m + NH];
          const float o1 = ws.Bh[row + m], o2 = ws.Bh[row + m + NH];
          dphi += g1 * o2 - g2 * o1;
          if (db) {
            stf(db, ob + (size_t)m * R + r, g1 * cs - g2 * sn);
            stf(db, ob + (size_t)(m + NH) * R + r, g1 * sn + g2 * cs);
          }
        }
        {
          const float g1 = bw.dCh[row + m], g2 = bw.dCh[row + m + NH];
          const float o1 = ws.Ch[row + m], o2 = ws.Ch[row + m + NH];
          dphi += g1 * o2 - g2 * o1;
          if (dc) {
            stf(dc, ob + (size_t)m * R + r, g1 * cs - g2 * sn);
            stf(dc, ob + (size_t)(m + NH) * R + r, g1 * sn + g2 * cs);
          }
        }
      }
      if (dangle && t == d.T - 1) dphi += dangle[(size_t)bh * NH + m];
      bw.dphi[((size_t)bh * d.Tp + t) * NH + m] = dphi;
    }
  } else {
    for (int e = threadIdx.x; e < L * N * R; e += blockDim.x) {
      const int r = e % R, n = (e / R) % N, l = e / (R * N), t = t0 + l;
      if (t >= d.T) continue;
      const size_t row = ((size_t)bh * d.Tp * R + (size_t)t * R + r) * N + n;
      const size_t o = tok_index(d, b, t, h) * N * R + (size_t)n * R + r;
      if (db) stf(db, o, bw.dBh[row]);
      if (dc) stf(dc, o, bw.dCh[row]);
    }
  }
}

// ---- reverse cumulative sum of d phi over the whole sequence (adjoint of the
// cumsum at scan.rs:491): chunk sums, suffix over chunks, then within the chunk.
__global__ void kb_dphi_sum(Dims d, GenericBwdWs bw) {
  const int k = blockIdx.x, bh = blockIdx.y;
  for (int m = threadIdx.x; m < d.NH; m += blockDim.x) {
    float s = 0.0f;
    for (int l = 0; l < d.L; ++l) s += bw.dphi[((size_t)bh * d.Tp + (size_t)k * d.L + l) * d.NH + m];
    bw.dpsum[((size_t)bh * d.C + k) * d.NH + m] = s;
  }
}

__global__ void kb_dphi_suffix(Dims d, GenericBwdWs bw, float* __restrict__ dangle0) {
  const int bh = blockIdx.x;
  for (int m = threadIdx.x; m < d.NH; m += blockDim.x) {
    float run = 0.0f;
    for (int k = d.C - 1; k >= 0; --k) {
      const size_t i = ((size_t)bh * d.C + k) * d.NH + m;
      const float s = bw.dpsum[i];
      bw.dpsum[i] = run;   // sum over all later chunks
      run += s;
    }
    if (dangle0) dangle0[(size_t)bh * d.NH + m] = run;
  }
}

template <class T>
__global__ void kb_dstep(Dims d, const T* __restrict__ dt, const T* __restrict__ theta, GenericBwdWs bw,
                         T* __restrict__ dtheta) {
  const int k = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int bh = b * d.H + h;
  const int NH = d.NH, L = d.L, t0 = k * L;
  for (int m = threadIdx.x; m < NH; m += blockDim.x) {
    float run = bw.dpsum[((size_t)bh * d.C + k) * NH + m];
    for (int l = L - 1; l >= 0; --l) {
      const int t = t0 + l;
      const size_t o = ((size_t)bh * d.Tp + t) * NH + m;
      run += bw.dphi[o];
      bw.dphi[o] = run;  // dstep
      if (t < d.T && dtheta) {
        const size_t i = tok_index(d, b, t, h);
        stf(dtheta, i * NH + m, run * ldf(dt, i));
      }
    }
  }
  __syncthreads();
  for (int l = threadIdx.x; l < L; l += blockDim.x) {
    const int t = t0 + l;
    float s = 0.0f;
    if (t < d.T) {
      const size_t i = tok_index(d, b, t, h);
      for (int m = 0; m < NH; ++m) s += bw.dphi[((size_t)bh * d.Tp + t) * NH + m] * ldf(theta, i * NH + m);
    }
    bw.ddt_rot[(size_t)bh * d.Tp + t] = s;
  }
}

// ---- dx = dX~ (layout restore) + D dy ; partial sums of dD = sum dy x (scan.rs:594-597)
template <class T>
__global__ void __launch_bounds__(256) kb_dx(Dims d, const T* __restrict__ x, const T* __restrict__ dy,
                                             const float* __restrict__ d_skip, GenericBwdWs bw,
                                             T* __restrict__ dx) {
  __shared__ float red[8];
  const int k = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int bh = b * d.H + h;
  const int P = d.P, R = d.R, L = d.L, t0 = k * L;
  const float dsk = d_skip ? d_skip[h] : 0.0f;
  float part = 0.0f;
  for (int e = threadIdx.x; e < L * P * R; e += blockDim.x) {
    const int r = e % R, p = (e / R) % P, l = e / (R * P), t = t0 + l;
    if (t >= d.T) continue;
    const size_t o = tok_index(d, b, t, h) * P * R + (size_t)p * R + r;
    float v = bw.dXh[((size_t)bh * d.Tp * R + (size_t)t * R + r) * P + p];
    if (d_skip) {
      const float gy = ldf(dy, o);
      v += dsk * gy;
      part += gy * ldf(x, o);
    }
    if (dx) stf(dx, o, v);
  }
  part = block_sum_256(part, red);
  if (threadIdx.x == 0) bw.partD[(size_t)bh * d.C + k] = part;
}

// ---- per token: d dt and d lambda (trapezoid adjoint, src/autograd/ops.rs:1169-1212 over
// src/tensor/ops/fused.rs:2513-2549; seed-state terms of scan.rs:524-535)
template <class T>
__global__ void kb_final(Dims d, const T* __restrict__ dt, const T* __restrict__ lam,
                         const float* __restrict__ a_log, GenericBwdWs bw, int has_state,
                         T* __restrict__ ddt, T* __restrict__ dlam, T* __restrict__ da_raw, T* __restrict__ dg_raw,
                         T* __restrict__ dw_raw) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t total = (size_t)d.B * d.T * d.H;
  if (i >= total) return;
  const int h = i % d.H;
  const int t = (i / d.H) % d.T;
  const int b = i / ((size_t)d.H * d.T);
  const int bh = b * d.H + h;
  const size_t o = (size_t)bh * d.Tp + t;        // scratch is in scan order: t is the scan position
  const size_t ti = tok_index(d, b, t, h);        // and this is its token in memory
  if (d.raw) {  // the ssd_chunked form: gradients of the caller's a, g, w as they are
    if (da_raw) stf(da_raw, ti, bw.da[o]);
    if (dg_raw) stf(dg_raw, ti, bw.dg[o]);
    if (dw_raw) stf(dw_raw, ti, bw.dw[o]);
    return;
  }
  const float A = -expf(a_log[h]);
  const float vdt = ldf(dt, ti), vl = lambda_at(lam, d.disc, ti);
  const float gw = bw.dg[o] + bw.dw[o];
  const float dwm1 = t > 0 ? bw.dw[o - 1] : 0.0f;
  float vdl = gw * vdt - dwm1 * vdt;
  float vdd = bw.da[o] * A + gw * vl + dwm1 * (1.0f - vl);
  if (d.rot) vdd += bw.ddt_rot[o];
  if (has_state && t == 0) {
    const float ip = bw.ip0[bh];
    vdl -= vdt * ip;
    vdd += (1.0f - vl) * ip;
  }
  if (ddt) stf(ddt, ti, vdd);
  if (dlam) stf(dlam, ti, vdl);
}

// ---- seed-state gradients: dh0 = dH_0, dlast_u0 = (1 - lambda_0) dt_0 dH_0
template <class T>
__global__ void kb_state_grads(Dims d, const T* __restrict__ dt, const T* __restrict__ lam, GenericBwdWs bw,
                               float* __restrict__ dh0, float* __restrict__ dlu0) {
  const int bh = blockIdx.y, b = bh / d.H, h = bh % d.H;
  const int PN = d.P * d.N;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= PN) return;
  const size_t i0 = tok_index(d, b, 0, h);
  const float first = d.raw ? 0.0f : (1.0f - lambda_at(lam, d.disc, i0)) * ldf(dt, i0);
  const float v = bw.dHs[((size_t)bh * (d.C + 1) + d.C) * PN + e];
  if (dh0) dh0[(size_t)bh * PN + e] = v;
  if (dlu0) dlu0[(size_t)bh * PN + e] = first * v;
}

// ---- per head: d a_log = A * sum da dt (A = -exp(a_log), scan.rs:470-475) and dD,
// summed over batch and chunks in a fixed order.
__global__ void kb_reduce_heads(Dims d, const float* __restrict__ a_log, GenericBwdWs bw,
                                float* __restrict__ da_log, float* __restrict__ dd_skip) {
  __shared__ float red[8];
  const int h = blockIdx.x;
  float sa = 0.0f, sd = 0.0f;
  const int n = d.B * d.C;
  for (int e = threadIdx.x; e < n; e += 256) {
    const int b = e / d.C, k = e % d.C;
    const size_t o = ((size_t)b * d.H + h) * d.C + k;
    sa += bw.partA[o];
    if (dd_skip) sd += bw.partD[o];
  }
  sa = block_sum_256(sa, red);
  sd = block_sum_256(sd, red);
  if (threadIdx.x == 0) {
    if (da_log) da_log[h] = -expf(a_log[h]) * sa;
    if (dd_skip) dd_skip[h] = sd;
  }
}

}  // namespace m3
