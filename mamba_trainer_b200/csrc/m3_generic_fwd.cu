// Generic forward of the Mamba-3 SSD scan: CUDA cores, fp32 arithmetic, any shape.
//
// This family serves float32 inputs (whose tolerance tensor cores cannot meet) and
// every shape the tensor-core family does not take.  It follows the reference scan
// (src/ssm/scan.rs:458-618 over :116-291) with two structural changes: the R^2
// one-channel scans are folded into one contraction over rows (t, r), and the
// C x C inter-chunk product (:219-251) is a sequential pass over chunk states.
#include "m3_internal.h"

namespace m3 {

// ---- angle: per-chunk sums of dt * theta (scan.rs:490) ---------------------
template <class T>
__global__ void k_angle_sum(Dims d, const T* __restrict__ dt, const T* __restrict__ theta,
                            float* __restrict__ abase) {
  const int k = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int bh = b * d.H + h;
  for (int m = threadIdx.x; m < d.NH; m += blockDim.x) {
    float s = 0.0f;
    for (int l = 0; l < d.L; ++l) {
      const int t = k * d.L + l;
      if (t >= d.T) break;
      const size_t i = tok_index(d, b, t, h);
      s += ldf(dt, i) * ldf(theta, i * d.NH + m);
    }
    abase[((size_t)bh * d.C + k) * d.NH + m] = s;
  }
}

// ---- angle: exclusive wrapped prefix over chunks (scan.rs:491-497) ---------
__global__ void k_angle_prefix(Dims d, const float* __restrict__ angle0, float* abase) {
  const int bh = blockIdx.x;
  for (int m = threadIdx.x; m < d.NH; m += blockDim.x) {
    float run = angle0 ? angle0[(size_t)bh * d.NH + m] : 0.0f;
    for (int k = 0; k < d.C; ++k) {
      const size_t i = ((size_t)bh * d.C + k) * d.NH + m;
      const float s = abase[i];
      abase[i] = run;
      run = wrap_angle(run + s);
    }
  }
}

// ---- per chunk: weights, cumulative decay, angles, rotated head-major copies
// trapezoid weights: src/autograd/ops.rs:1169-1212; rotation: scan.rs:498-507 over
// src/tensor/ops/fused.rs:588-619; zero padding of the ragged tail: scan.rs:151-158.
template <class T>
__global__ void k_prep(Dims d, const T* __restrict__ x, const T* __restrict__ bm,
                       const T* __restrict__ cm, const T* __restrict__ dt,
                       const T* __restrict__ lam, const T* __restrict__ theta,
                       const float* __restrict__ a_log, const T* __restrict__ a_raw, const T* __restrict__ g_raw,
                       const T* __restrict__ w_raw, GenericWs ws, float* angle_out) {
  extern __shared__ float sm[];
  float* s_dt = sm;                 // [L + 1]
  float* s_lam = sm + d.L + 1;      // [L + 1]
  const int k = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int bh = b * d.H + h;
  const int t0 = k * d.L;
  for (int l = threadIdx.x; l <= d.L; l += blockDim.x) {
    const int t = t0 + l;
    float vdt = 0.0f, vl = 1.0f;
    if (t < d.T && !d.raw) {
      const size_t i = tok_index(d, b, t, h);
      vdt = ldf(dt, i);
      vl = lambda_at(lam, d.disc, i);
    }
    s_dt[l] = vdt;
    s_lam[l] = vl;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const float A = d.raw ? 0.0f : -expf(a_log[h]);
    float run = 0.0f;
    for (int l = 0; l < d.L; ++l) {
      const int t = t0 + l;
      float gv = 0.0f, wv = 0.0f, av = 0.0f;
      if (t < d.T && d.raw) {  // scan.rs:116-126: the caller's own a, g, w
        const size_t i = tok_index(d, b, t, h);
        av = ldf(a_raw, i);
        gv = ldf(g_raw, i);
        wv = ldf(w_raw, i);
      } else if (t < d.T) {
        av = s_dt[l] * A;
        gv = s_lam[l] * s_dt[l];
        const float f = (t + 1 < d.T) ? (1.0f - s_lam[l + 1]) * s_dt[l + 1] : 0.0f;
        wv = gv + f;
      }
      run += av;
      const size_t o = (size_t)bh * d.Tp + t;
      ws.acum[o] = run;
      ws.g[o] = gv;
      ws.w[o] = wv;
    }
  }
  if (d.rot) {
    for (int m = threadIdx.x; m < d.NH; m += blockDim.x) {
      float run = ws.abase[((size_t)bh * d.C + k) * d.NH + m];
      for (int l = 0; l < d.L; ++l) {
        const int t = t0 + l;
        float ph = 0.0f;
        if (t < d.T) {
          const size_t i = tok_index(d, b, t, h);
          run += s_dt[l] * ldf(theta, i * d.NH + m);
          ph = wrap_angle(run);
          if (angle_out && t == d.T - 1) angle_out[(size_t)bh * d.NH + m] = ph;
        }
        ws.phi[((size_t)bh * d.Tp + t) * d.NH + m] = ph;
      }
    }
    __syncthreads();
  }
  // x -> Xh
  const int nx = d.L * d.P * d.R;
  for (int e = threadIdx.x; e < nx; e += blockDim.x) {
    const int r = e % d.R, p = (e / d.R) % d.P, l = e / (d.R * d.P);
    const int t = t0 + l;
    float v = 0.0f;
    if (t < d.T) v = ldf(x, tok_index(d, b, t, h) * d.P * d.R + (size_t)p * d.R + r);
    ws.Xh[((size_t)bh * d.Tp * d.R + (size_t)t * d.R + r) * d.P + p] = v;
  }
  if (d.rot) {
    const int nb = d.L * d.NH * d.R;
    for (int e = threadIdx.x; e < nb; e += blockDim.x) {
      const int r = e % d.R, m = (e / d.R) % d.NH, l = e / (d.R * d.NH);
      const int t = t0 + l;
      float b1 = 0.f, b2 = 0.f, c1 = 0.f, c2 = 0.f;
      if (t < d.T) {
        const size_t base = tok_index(d, b, t, h) * d.N * d.R;
        const float vb1 = ldf(bm, base + (size_t)m * d.R + r);
        const float vb2 = ldf(bm, base + (size_t)(m + d.NH) * d.R + r);
        const float vc1 = ldf(cm, base + (size_t)m * d.R + r);
        const float vc2 = ldf(cm, base + (size_t)(m + d.NH) * d.R + r);
        float sn, cs;
        sincosf(ws.phi[((size_t)bh * d.Tp + t) * d.NH + m], &sn, &cs);
        b1 = vb1 * cs + vb2 * sn;  b2 = vb2 * cs - vb1 * sn;
        c1 = vc1 * cs + vc2 * sn;  c2 = vc2 * cs - vc1 * sn;
      }
      const size_t o = ((size_t)bh * d.Tp * d.R + (size_t)t * d.R + r) * d.N;
      ws.Bh[o + m] = b1;  ws.Bh[o + m + d.NH] = b2;
      ws.Ch[o + m] = c1;  ws.Ch[o + m + d.NH] = c2;
    }
  } else {
    const int nb = d.L * d.N * d.R;
    for (int e = threadIdx.x; e < nb; e += blockDim.x) {
      const int r = e % d.R, n = (e / d.R) % d.N, l = e / (d.R * d.N);
      const int t = t0 + l;
      float vb = 0.f, vc = 0.f;
      if (t < d.T) {
        const size_t i = tok_index(d, b, t, h) * d.N * d.R + (size_t)n * d.R + r;
        vb = ldf(bm, i);
        vc = ldf(cm, i);
      }
      const size_t o = ((size_t)bh * d.Tp * d.R + (size_t)t * d.R + r) * d.N + n;
      ws.Bh[o] = vb;
      ws.Ch[o] = vc;
    }
  }
}

// ---- chunk state S_k = sum_rho sigma_w(rho) X~[rho,:]^T B^[rho,:]  (scan.rs:208-216)
__global__ void __launch_bounds__(256) k_chunk_state(Dims d, GenericWs ws) {
  extern __shared__ float sm[];
  float* sA = sm;
  float* sB = sm + kGemmBK * kGemmLd;
  float* s_sw = sm + kGemmSmemFloats;  // [L]
  const int tiles_n = (d.N + 63) / 64;
  const int p0 = (blockIdx.x / tiles_n) * 64, n0 = (blockIdx.x % tiles_n) * 64;
  const int k = blockIdx.y, bh = blockIdx.z;
  const float* acum = ws.acum + (size_t)bh * d.Tp + (size_t)k * d.L;
  const float* w = ws.w + (size_t)bh * d.Tp + (size_t)k * d.L;
  const float cd = acum[d.L - 1];
  for (int l = threadIdx.x; l < d.L; l += blockDim.x) s_sw[l] = exp_decay(cd - acum[l]) * w[l];
  __syncthreads();
  const float* X = ws.Xh + ((size_t)bh * d.Tp + (size_t)k * d.L) * d.R * d.P;
  const float* Bm = ws.Bh + ((size_t)bh * d.Tp + (size_t)k * d.L) * d.R * d.N;
  const int P = d.P, N = d.N, R = d.R;
  float acc[4][4];
  zero_acc(acc);
  gemm_tile<false, false>(
      acc, p0, n0, 0, d.LR,
      [&](int p, int rho) { return p < P ? s_sw[rho / R] * X[(size_t)rho * P + p] : 0.0f; },
      [&](int rho, int n) { return n < N ? Bm[(size_t)rho * N + n] : 0.0f; }, sA, sB);
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float* out = ws.Hs + ((size_t)bh * (d.C + 1) + k) * P * N;
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + ty * 4 + i, n = n0 + tx * 4 + j;
      if (p < P && n < N) out[(size_t)p * N + n] = acc[i][j];
    }
}

// ---- inter-chunk state pass: H_{k+1} = exp(cd_k) H_k + S_k, sequential over k.
// Lanes own state elements (coalesced); the 32 chunk decays of a stretch are loaded
// by one lane each and handed round by warp shuffle.  Replaces scan.rs:219-251;
// the seed is S = h + (1 - lambda_0) dt_0 last_u (scan.rs:524-535).
template <class T>
__global__ void k_state_pass(Dims d, const T* __restrict__ dt, const T* __restrict__ lam,
                             const float* __restrict__ h0, const float* __restrict__ lu0,
                             GenericWs ws, float* h_out) {
  const int bh = blockIdx.y, b = bh / d.H, h = bh % d.H;
  const int PN = d.P * d.N;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = e < PN;
  const int lane = threadIdx.x & 31;
  float carry = 0.0f;
  if (live && h0) {
    carry = h0[(size_t)bh * PN + e];
    if (lu0) {
      const size_t i0 = tok_index(d, b, 0, h);
      carry += (1.0f - lambda_at(lam, d.disc, i0)) * ldf(dt, i0) * lu0[(size_t)bh * PN + e];
    }
  }
  float* Hs = ws.Hs + (size_t)bh * (d.C + 1) * PN;
  for (int k0 = 0; k0 < d.C; k0 += 32) {
    const int kk = k0 + lane;
    const float mine = (kk < d.C) ? exp_decay(ws.acum[(size_t)bh * d.Tp + (size_t)kk * d.L + d.L - 1]) : 1.0f;
    const int cnt = min(32, d.C - k0);
    for (int j = 0; j < cnt; ++j) {
      const float ecd = __shfl_sync(0xffffffffu, mine, j);
      if (live) {
        const size_t o = (size_t)(k0 + j) * PN + e;
        const float s = Hs[o];
        Hs[o] = carry;
        carry = fmaf(ecd, carry, s);
      }
    }
  }
  if (live) {
    Hs[(size_t)d.C * PN + e] = carry;
    if (h_out) h_out[(size_t)bh * PN + e] = carry;
  }
}

// ---- outputs of one row tile of one chunk (scan.rs:192-205 and :254-268, D skip :594-597)
//   Y = (C~ B~^T o band) X~ + exp(acum) C~ H_k^T + D x
template <class T>
__global__ void __launch_bounds__(256) k_chunk_out(Dims d, const T* __restrict__ x,
                                                   const float* __restrict__ d_skip,
                                                   GenericWs ws, T* __restrict__ y) {
  extern __shared__ float sm[];
  float* sA = sm;
  float* sB = sm + kGemmBK * kGemmLd;
  float* s_ac = sm + kGemmSmemFloats;
  float* s_g = s_ac + d.L;
  float* s_w = s_g + d.L;
  float* Mb = s_w + d.L;  // [64, LR]
  const int k = blockIdx.y, bh = blockIdx.z, b = bh / d.H, h = bh % d.H;
  const int P = d.P, N = d.N, R = d.R, LR = d.LR;
  const int TL = max(1, 64 / R);
  const int l0 = blockIdx.x * TL, l1 = min(d.L, l0 + TL);
  const int rows = (l1 - l0) * R, row0 = l0 * R, ncols = l1 * R;
  const size_t tb = (size_t)bh * d.Tp + (size_t)k * d.L;
  for (int l = threadIdx.x; l < d.L; l += blockDim.x) {
    s_ac[l] = ws.acum[tb + l];
    s_g[l] = ws.g[tb + l];
    s_w[l] = ws.w[tb + l];
  }
  __syncthreads();
  const float* X = ws.Xh + tb * R * P;
  const float* Bm = ws.Bh + tb * R * N;
  const float* Cm = ws.Ch + tb * R * N;
  const float* Hk = ws.Hs + ((size_t)bh * (d.C + 1) + k) * P * N;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc[4][4];
  for (int n0 = 0; n0 < ncols; n0 += 64) {
    zero_acc(acc);
    gemm_tile<true, true>(
        acc, 0, n0, 0, N,
        [&](int m, int kk) { return m < rows ? Cm[(size_t)(row0 + m) * N + kk] : 0.0f; },
        [&](int kk, int n) { return n < ncols ? Bm[(size_t)n * N + kk] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, col = n0 + tx * 4 + j;
        if (m < rows && col < ncols) {
          const int l = l0 + m / R, s = col / R;
          float v = 0.0f;
          if (s < l) v = acc[i][j] * s_w[s] * exp_decay(s_ac[l] - s_ac[s]);
          else if (s == l) v = acc[i][j] * s_g[s];
          Mb[(size_t)m * LR + col] = v;
        }
      }
  }
  __syncthreads();
  const float dsk = d_skip ? d_skip[h] : 0.0f;
  for (int p0 = 0; p0 < P; p0 += 64) {
    zero_acc(acc);
    gemm_tile<true, false>(
        acc, 0, p0, 0, ncols,
        [&](int m, int kk) { return m < rows ? Mb[(size_t)m * LR + kk] : 0.0f; },
        [&](int kk, int n) { return n < P ? X[(size_t)kk * P + n] : 0.0f; }, sA, sB);
    gemm_tile<true, true>(
        acc, 0, p0, 0, N,
        [&](int m, int kk) {
          return m < rows ? Cm[(size_t)(row0 + m) * N + kk] * exp_decay(s_ac[l0 + m / R]) : 0.0f;
        },
        [&](int kk, int n) { return n < P ? Hk[(size_t)n * N + kk] : 0.0f; }, sA, sB);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int m = ty * 4 + i, p = p0 + tx * 4 + j;
        if (m < rows && p < P) {
          const int l = l0 + m / R, r = m % R, t = k * d.L + l;
          if (t < d.T) {
            const size_t o = tok_index(d, b, t, h) * P * R + (size_t)p * R + r;
            float v = acc[i][j];
            if (d_skip) v += dsk * ldf(x, o);
            stf(y, o, v);
          }
        }
      }
  }
}

// ---- last_u = sum_r x_{T-1}^(r) (x) B^_{T-1}^(r)   (scan.rs:621-638)
__global__ void k_last_u(Dims d, GenericWs ws, float* __restrict__ last_u) {
  const int bh = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= d.P * d.N) return;
  const int p = e / d.N, n = e % d.N;
  const size_t row = (size_t)bh * d.Tp * d.R + (size_t)(d.T - 1) * d.R;
  float s = 0.0f;
  for (int r = 0; r < d.R; ++r) s += ws.Xh[(row + r) * d.P + p] * ws.Bh[(row + r) * d.N + n];
  last_u[(size_t)bh * d.P * d.N + e] = s;
}

size_t generic_ws_layout(const Dims& d, GenericWs* ws, char* base) {
  size_t off = 0;
  auto take = [&](size_t nfloat) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += ((nfloat * sizeof(float) + 255) / 256) * 256;
    return p;
  };
  const size_t BH = (size_t)d.B * d.H, rows = (size_t)d.Tp * d.R;
  GenericWs tmp;
  tmp.Xh = take(BH * rows * d.P);
  tmp.Bh = take(BH * rows * d.N);
  tmp.Ch = take(BH * rows * d.N);
  tmp.acum = take(BH * d.Tp);
  tmp.g = take(BH * d.Tp);
  tmp.w = take(BH * d.Tp);
  tmp.phi = take(BH * d.Tp * d.NH);
  tmp.abase = take(BH * d.C * d.NH);
  tmp.Hs = take(BH * (d.C + 1) * d.P * d.N);
  if (ws) *ws = tmp;
  return off;
}

size_t chunk_out_smem(const Dims& d) {
  return sizeof(float) * ((size_t)kGemmSmemFloats + 3 * (size_t)d.L + 64 * (size_t)d.LR);
}

template <class T>
static cudaError_t forward_t(cudaStream_t st, const Dims& d, const m3_scan_desc& desc,
                             const m3_scan_out& out, const GenericWs& ws, uint64_t* launches) {
  const T* x = static_cast<const T*>(desc.x);
  const T* bm = static_cast<const T*>(desc.b);
  const T* cm = static_cast<const T*>(desc.c);
  const T* dt = static_cast<const T*>(desc.dt);
  const T* lam = static_cast<const T*>(desc.lambda);
  const T* th = static_cast<const T*>(desc.theta);
  const dim3 gchunk(d.C, d.H, d.B);
  const int BH = d.B * d.H, PN = d.P * d.N;
  uint64_t n = 0;
  if (d.rot) {
    k_angle_sum<T><<<gchunk, 64, 0, st>>>(d, dt, th, ws.abase);
    k_angle_prefix<<<BH, 64, 0, st>>>(d, desc.angle0, ws.abase);
    n += 2;
  }
  k_prep<T><<<gchunk, 256, sizeof(float) * 2 * (d.L + 1), st>>>(
      d, x, bm, cm, dt, lam, th, desc.a_log, static_cast<const T*>(desc.a_raw), static_cast<const T*>(desc.g_raw),
      static_cast<const T*>(desc.w_raw), ws, desc.want_state ? out.angle : nullptr);
  const int tiles = ((d.P + 63) / 64) * ((d.N + 63) / 64);
  k_chunk_state<<<dim3(tiles, d.C, BH), 256, sizeof(float) * (kGemmSmemFloats + d.L), st>>>(d, ws);
  k_state_pass<T><<<dim3((PN + 255) / 256, BH), 256, 0, st>>>(
      d, dt, lam, desc.h0, d.raw ? nullptr : desc.last_u0, ws, desc.want_state ? out.h : nullptr);
  const size_t smem = chunk_out_smem(d);
  cudaError_t e = cudaFuncSetAttribute(k_chunk_out<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return e;
  const int TL = d.R >= 64 ? 1 : 64 / d.R;
  k_chunk_out<T><<<dim3((d.L + TL - 1) / TL, d.C, BH), 256, smem, st>>>(
      d, x, desc.d_skip, ws, static_cast<T*>(out.y));
  n += 4;
  if (desc.want_state && out.last_u && !d.raw) {
    k_last_u<<<dim3((PN + 255) / 256, BH), 256, 0, st>>>(d, ws, out.last_u);
    n += 1;
  }
  if (launches) *launches += n;
  return cudaGetLastError();
}

cudaError_t generic_forward(cudaStream_t st, const Dims& d, const m3_scan_desc& desc,
                            const m3_scan_out& out, const GenericWs& ws, uint64_t* launches) {
  if (desc.dtype == M3_BF16) return forward_t<__nv_bfloat16>(st, d, desc, out, ws, launches);
  return forward_t<float>(st, d, desc, out, ws, launches);
}

}  // namespace m3
