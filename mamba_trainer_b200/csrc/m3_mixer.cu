// Mixer-side steps either side of the scan, each as one launch instead of the reference's chain of
// primitives (src/models/mamba3.rs:403-461, :475-484):
//   m3_bc_*        B / C: group -> head expansion, per-head bias, RMS norm over d_state, and the
//                  permute to the scan's rank-last layout (:409-436)
//   m3_dt_lambda_* dt = softplus(dt_raw + dt_bias), lambda = sigmoid(lambda_raw) (:440-446)
//   m3_gate_*      y * silu(z) (:475-484, without post_gate_norm)
//   m3_gate_norm_* rms_norm(y) * gain * silu(z) (:475-484 with post_gate_norm; src/nn/norm.rs:95-105)
// All are HBM-bound streaming kernels; inputs may be column bands of a wider row (the input
// projection / the convolution's output), outputs of the forward are dense.
#include <cuda_bf16.h>

#include <initializer_list>
#include <type_traits>

#include "m3_internal.h"

#define M3_CUDA(ctx, call)                                       \
  do {                                                           \
    cudaError_t e_ = (call);                                     \
    if (e_ != cudaSuccess) return m3::cuda_fail(ctx, e_, #call); \
  } while (0)

namespace {

using m3::ldf;
using m3::stf;

constexpr int kBcWarps = 8;      // warps per block
constexpr int kBcTokens = 256;   // tokens per block (32 per warp)
constexpr int kMaxPerLane = 8;   // d_state <= 32 * kMaxPerLane = 256 on the fast path

struct BcDims {
  int B, T, H, G, N, R, PG;      // PG = heads per group
  long long rs;                  // token stride of the raw rows (elements)
  float eps;
  int has_norm;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- B / C forward: one warp per (token, head); lanes stride over d_state ---------------------------
template <class T>
__global__ void __launch_bounds__(kBcWarps * 32)
    k_bc_fwd(BcDims d, const T* __restrict__ raw, const float* __restrict__ bias, const float* __restrict__ gain,
             T* __restrict__ out) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t row = (size_t)blockIdx.x * kBcWarps + warp;  // (b * T + t) * H + h
  if (row >= (size_t)d.B * d.T * d.H) return;
  const int h = row % d.H;
  const size_t bt = row / d.H;
  const int g = h / d.PG;
  const T* src = raw + bt * d.rs + (size_t)g * d.R * d.N;
  T* dst = out + row * d.N * d.R;
  for (int r = 0; r < d.R; ++r) {
    float v[kMaxPerLane];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int n = lane + 32 * j;
      v[j] = 0.0f;
      if (n < d.N) {
        v[j] = ldf(src, (size_t)r * d.N + n) + (bias ? bias[(size_t)h * d.N + n] : 0.0f);
        ss += v[j] * v[j];
      }
    }
    float scale = 1.0f;
    if (d.has_norm) scale = rsqrtf(warp_sum(ss) / (float)d.N + d.eps);
#pragma unroll
    for (int j = 0; j < kMaxPerLane; ++j) {
      const int n = lane + 32 * j;
      if (n < d.N) stf(dst, (size_t)n * d.R + r, v[j] * scale * ((d.has_norm && gain) ? gain[n] : 1.0f));
    }
  }
}

// ---- the same for bf16 with d_state 128 or 256: a lane owns 16 consecutive state columns (two
// 16-byte loads per rank), so a row takes d_state / 16 lanes and a warp works on 2 or 4 rows at once;
// the row's sum of squares is a 3- or 4-step shuffle.  These kernels are bound by instruction
// issue, not by memory, so work per instruction is what counts.
__device__ __forceinline__ void unpack8(const uint4& q, float* v) {
  v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xffff0000u);
  v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xffff0000u);
  v[4] = __uint_as_float(q.z << 16); v[5] = __uint_as_float(q.z & 0xffff0000u);
  v[6] = __uint_as_float(q.w << 16); v[7] = __uint_as_float(q.w & 0xffff0000u);
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void load16f(const float* p, float (&v)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p) + k);
    v[4 * k] = t.x; v[4 * k + 1] = t.y; v[4 * k + 2] = t.z; v[4 * k + 3] = t.w;
  }
}
template <int LPR>
__device__ __forceinline__ float row_sum(float v) {  // over the LPR adjacent lanes of one row
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

template <int R, int N>
__global__ void __launch_bounds__(kBcWarps * 32)
    k_bc_fwd_vec(BcDims d, const __nv_bfloat16* __restrict__ raw, const float* __restrict__ bias,
                 const float* __restrict__ gain, __nv_bfloat16* __restrict__ out) {
  constexpr int LPR = N / 16, RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPR, n0 = 16 * sub;
  const size_t rows = (size_t)d.B * d.T * d.H;
  const size_t row_raw = ((size_t)blockIdx.x * kBcWarps + warp) * RPW + lane / LPR;
  const bool valid = row_raw < rows;
  const size_t row = valid ? row_raw : rows - 1;  // every lane takes part in the shuffles
  const int h = row % d.H;
  const size_t bt = row / d.H;
  const int g = h / d.PG;
  const __nv_bfloat16* src = raw + bt * d.rs + (size_t)g * R * N + n0;
  uint4 q[R][2];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    q[r][0] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * N));
    q[r][1] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * N + 8));
  }
  float bs[16], gn[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { bs[i] = 0.0f; gn[i] = 1.0f; }
  if (bias) load16f(bias + (size_t)h * N + n0, bs);
  if (d.has_norm && gain) load16f(gain + n0, gn);
  float o[16][R];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float v[16];
    unpack8(q[r][0], v);
    unpack8(q[r][1], v + 8);
    float ss = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      v[i] += bs[i];
      ss = fmaf(v[i], v[i], ss);
    }
    const float scale = d.has_norm ? rsqrtf(row_sum<LPR>(ss) * (1.0f / N) + d.eps) : 1.0f;
#pragma unroll
    for (int i = 0; i < 16; ++i) o[i][r] = v[i] * scale * gn[i];
  }
  if (!valid) return;
  const float* flat = &o[0][0];  // (n0 + i, r) in storage order: 16 * R consecutive outputs
  uint4* dp = reinterpret_cast<uint4*>(out + row * N * R + (size_t)n0 * R);
#pragma unroll
  for (int k = 0; k < 2 * R; ++k)
    dp[k] = make_uint4(pack2(flat[8 * k], flat[8 * k + 1]), pack2(flat[8 * k + 2], flat[8 * k + 3]),
                       pack2(flat[8 * k + 4], flat[8 * k + 5]), pack2(flat[8 * k + 6], flat[8 * k + 7]));
}

// ---- B / C backward: a block owns one group and kBcTokens tokens; a warp walks tokens, sums the
// gradient of the raw row over the heads of the group, and keeps private partial sums of the bias
// and gain gradients in shared memory (no atomics: every sum has a fixed order).
template <class T>
__global__ void __launch_bounds__(kBcWarps * 32)
    k_bc_bwd(BcDims d, const T* __restrict__ raw, const float* __restrict__ bias, const float* __restrict__ gain,
             const T* __restrict__ dout, T* __restrict__ draw, float* __restrict__ part) {
  extern __shared__ float sm[];  // [warps][PG + 1][N]: bias partials per head of the group, then gain
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = blockIdx.y;
  const size_t ntok = (size_t)d.B * d.T;
  const size_t tok0 = (size_t)blockIdx.x * kBcTokens;
  float* mine = sm + (size_t)warp * (d.PG + 1) * d.N;
  for (int i = lane; i < (d.PG + 1) * d.N; i += 32) mine[i] = 0.0f;
  __syncwarp();
  for (int it = warp; it < kBcTokens; it += kBcWarps) {
    const size_t bt = tok0 + it;
    if (bt >= ntok) break;
    const T* src = raw + bt * d.rs + (size_t)g * d.R * d.N;
    for (int r = 0; r < d.R; ++r) {
      float acc[kMaxPerLane];
#pragma unroll
      for (int j = 0; j < kMaxPerLane; ++j) acc[j] = 0.0f;
      for (int hg = 0; hg < d.PG; ++hg) {
        const int h = g * d.PG + hg;
        const T* go = dout + (bt * d.H + h) * d.N * d.R;
        float v[kMaxPerLane], dxh[kMaxPerLane];
        float ss = 0.0f, dot = 0.0f;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const int n = lane + 32 * j;
          v[j] = dxh[j] = 0.0f;
          if (n < d.N) {
            v[j] = ldf(src, (size_t)r * d.N + n) + (bias ? bias[(size_t)h * d.N + n] : 0.0f);
            const float gy = ldf(go, (size_t)n * d.R + r);
            dxh[j] = gy * ((d.has_norm && gain) ? gain[n] : 1.0f);
            ss += v[j] * v[j];
            if (!d.has_norm) dxh[j] = gy;
          }
        }
        float rstd = 1.0f, mean_dot = 0.0f;
        if (d.has_norm) {
          rstd = rsqrtf(warp_sum(ss) / (float)d.N + d.eps);
#pragma unroll
          for (int j = 0; j < kMaxPerLane; ++j) dot += dxh[j] * v[j] * rstd;
          mean_dot = warp_sum(dot) / (float)d.N;
        }
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const int n = lane + 32 * j;
          if (n < d.N) {
            const float xh = v[j] * rstd;
            const float dv = d.has_norm ? rstd * (dxh[j] - xh * mean_dot) : dxh[j];
            acc[j] += dv;
            mine[(size_t)hg * d.N + n] += dv;                                          // d bias[h, n]
            if (d.has_norm && gain) mine[(size_t)d.PG * d.N + n] += ldf(go, (size_t)n * d.R + r) * xh;  // d gain[n]
          }
        }
      }
      if (draw) {
        T* dr = draw + bt * d.rs + (size_t)g * d.R * d.N;
#pragma unroll
        for (int j = 0; j < kMaxPerLane; ++j) {
          const int n = lane + 32 * j;
          if (n < d.N) stf(dr, (size_t)r * d.N + n, acc[j]);
        }
      }
    }
  }
  __syncthreads();
  if (!part) return;
  const size_t blk = (size_t)blockIdx.x * gridDim.y + g;
  const int width = (d.PG + 1) * d.N;
  for (int i = threadIdx.x; i < width; i += blockDim.x) {
    float s = 0.0f;
    for (int w = 0; w < kBcWarps; ++w) s += sm[(size_t)w * width + i];
    part[blk * width + i] = s;
  }
}

// The same for bf16, d_state 128 or 256, one head per group: 16 columns per lane as in the forward
// kernel, the bias / gain partial sums in registers across the warp's tokens, then added over the
// warp's rows by shuffles (a fixed tree) and over the block's warps through shared memory.
template <int R, int N>
__global__ void __launch_bounds__(kBcWarps * 32)
    k_bc_bwd_vec(BcDims d, const __nv_bfloat16* __restrict__ raw, const float* __restrict__ bias,
                 const float* __restrict__ gain, const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ draw,
                 float* __restrict__ part) {
  constexpr int LPR = N / 16, RPW = 32 / LPR;
  __shared__ float sm[kBcWarps][2][N];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % LPR, rw = lane / LPR, n0 = 16 * sub;
  const int g = blockIdx.y, h = g;  // PG == 1
  const size_t ntok = (size_t)d.B * d.T;
  const size_t tok0 = (size_t)blockIdx.x * kBcTokens;
  float bs[16], gn[16], pbias[16], pgain[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) { bs[i] = 0.0f; gn[i] = 1.0f; pbias[i] = 0.0f; pgain[i] = 0.0f; }
  if (bias) load16f(bias + (size_t)h * N + n0, bs);
  const bool use_gain = d.has_norm && gain;
  if (use_gain) load16f(gain + n0, gn);
  for (int it = warp * RPW + rw; it < kBcTokens; it += kBcWarps * RPW) {
    const size_t bt_raw = tok0 + it;
    const bool valid = bt_raw < ntok;
    const size_t bt = valid ? bt_raw : ntok - 1;
    const __nv_bfloat16* src = raw + bt * d.rs + (size_t)g * R * N + n0;
    const __nv_bfloat16* go = dout + (bt * d.H + h) * N * R + (size_t)n0 * R;
    uint4 q[R][2], gq[2 * R];
#pragma unroll
    for (int r = 0; r < R; ++r) {
      q[r][0] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * N));
      q[r][1] = __ldg(reinterpret_cast<const uint4*>(src + (size_t)r * N + 8));
    }
#pragma unroll
    for (int k = 0; k < 2 * R; ++k) gq[k] = __ldg(reinterpret_cast<const uint4*>(go) + k);
    float gy[16][R];  // (n0 + i, r), as stored
    {
      float* flat = &gy[0][0];
#pragma unroll
      for (int k = 0; k < 2 * R; ++k) unpack8(gq[k], flat + 8 * k);
    }
    const float live = valid ? 1.0f : 0.0f;
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float v[16], dxh[16];
      unpack8(q[r][0], v);
      unpack8(q[r][1], v + 8);
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        v[i] += bs[i];
        ss = fmaf(v[i], v[i], ss);
        dxh[i] = gy[i][r] * gn[i];
      }
      float rstd = 1.0f, mean_dot = 0.0f;
      if (d.has_norm) {
        rstd = rsqrtf(row_sum<LPR>(ss) * (1.0f / N) + d.eps);
        float dot = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; ++i) dot = fmaf(dxh[i], v[i], dot);
        mean_dot = row_sum<LPR>(dot) * rstd * (1.0f / N);
      }
      float dv[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float xh = v[i] * rstd;
        dv[i] = d.has_norm ? rstd * (dxh[i] - xh * mean_dot) : dxh[i];
        pbias[i] = fmaf(live, dv[i], pbias[i]);
        pgain[i] = fmaf(live * gy[i][r], xh, pgain[i]);
      }
      if (draw && valid) {
        uint4* dr = reinterpret_cast<uint4*>(draw + bt * d.rs + (size_t)g * R * N + (size_t)r * N + n0);
        dr[0] = make_uint4(pack2(dv[0], dv[1]), pack2(dv[2], dv[3]), pack2(dv[4], dv[5]), pack2(dv[6], dv[7]));
        dr[1] = make_uint4(pack2(dv[8], dv[9]), pack2(dv[10], dv[11]), pack2(dv[12], dv[13]), pack2(dv[14], dv[15]));
      }
    }
  }
  // rows of the warp (lanes LPR apart), then warps of the block
#pragma unroll
  for (int i = 0; i < 16; ++i) {
#pragma unroll
    for (int o = LPR; o < 32; o <<= 1) {
      pbias[i] += __shfl_xor_sync(0xffffffffu, pbias[i], o);
      pgain[i] += __shfl_xor_sync(0xffffffffu, pgain[i], o);
    }
  }
  if (rw == 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      sm[warp][0][n0 + i] = pbias[i];
      sm[warp][1][n0 + i] = pgain[i];
    }
  }
  __syncthreads();
  if (!part) return;
  const size_t blk = (size_t)blockIdx.x * gridDim.y + g;
  for (int i = threadIdx.x; i < 2 * N; i += blockDim.x) {
    float s = 0.0f;
#pragma unroll
    for (int w = 0; w < kBcWarps; ++w) s += sm[w][i / N][i % N];
    part[blk * 2 * N + i] = s;   // width = (PG + 1) * N with PG == 1
  }
}

// ---- dt / lambda ---------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus(float v) { return v > 20.0f ? v : log1pf(__expf(v)); }
__device__ __forceinline__ float sigmoid(float v) { return __fdividef(1.0f, 1.0f + __expf(-v)); }

template <class T>
__global__ void k_act_fwd(int ntok, int H, long long stride, const T* __restrict__ dt_raw, const T* __restrict__ lam_raw,
                          const float* __restrict__ dt_bias, T* __restrict__ dt, T* __restrict__ lam) {
  const size_t n = (size_t)ntok * H;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int h = i % H;
    const size_t bt = i / H;
    stf(dt, i, softplus(ldf(dt_raw, bt * stride + h) + (dt_bias ? dt_bias[h] : 0.0f)));
    if (lam_raw && lam) stf(lam, i, sigmoid(ldf(lam_raw, bt * stride + h)));
  }
}

constexpr int kActRun = 8;  // tokens per thread of the backward pass
// Thread (run, head): walks kActRun tokens of one head and leaves that run's partial sum of the bias
// gradient; the runs are added by column_sums.
template <class T>
__global__ void k_act_bwd(int ntok, int H, long long stride, const T* __restrict__ dt_raw, const T* __restrict__ lam_raw,
                          const float* __restrict__ dt_bias, const T* __restrict__ ddt, const T* __restrict__ dlam,
                          T* __restrict__ ddt_raw, T* __restrict__ dlam_raw, float* __restrict__ part) {
  const int nruns = (ntok + kActRun - 1) / kActRun;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)nruns * H) return;
  const int h = i % H, run = i / H;
  const int lo = run * kActRun, hi = min(ntok, lo + kActRun);
  const float bias = dt_bias ? dt_bias[h] : 0.0f;
  float s = 0.0f;
  for (int bt = lo; bt < hi; ++bt) {
    const size_t a = (size_t)bt * H + h, j = (size_t)bt * stride + h;
    const float g = ldf(ddt, a) * sigmoid(ldf(dt_raw, j) + bias);
    if (ddt_raw) stf(ddt_raw, j, g);
    s += g;
    if (lam_raw && dlam && dlam_raw) {
      const float l = sigmoid(ldf(lam_raw, j));
      stf(dlam_raw, j, ldf(dlam, a) * l * (1.0f - l));
    }
  }
  if (part) part[i] = s;
}

// ---- gate -----------------------------------------------------------------------------------------------
__device__ __forceinline__ float silu(float v) { return v * sigmoid(v); }
__device__ __forceinline__ float silu_grad(float v) {
  const float s = sigmoid(v);
  return s * (1.0f + v * (1.0f - s));
}

// 8 elements per thread step when everything is 16-byte aligned (VEC), else one.
template <class T, bool VEC>
__global__ void k_gate_fwd(size_t ntok, int Cn, long long zs, const T* __restrict__ y, const T* __restrict__ z,
                           T* __restrict__ out) {
  constexpr int V = VEC ? (int)(16 / sizeof(T)) : 1;
  const int per_row = Cn / V;
  const size_t n = ntok * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t bt = i / per_row;
    const int c = (int)(i % per_row) * V;
    if (VEC) {
      const uint4 qy = __ldg(reinterpret_cast<const uint4*>(y + bt * Cn + c));
      const uint4 qz = __ldg(reinterpret_cast<const uint4*>(z + bt * zs + c));
      uint4 qo;
      const T* py = reinterpret_cast<const T*>(&qy);
      const T* pz = reinterpret_cast<const T*>(&qz);
      T* po = reinterpret_cast<T*>(&qo);
#pragma unroll
      for (int k = 0; k < V; ++k) stf(po, k, ldf(py, k) * silu(ldf(pz, k)));
      *reinterpret_cast<uint4*>(out + bt * Cn + c) = qo;
    } else {
      stf(out, bt * Cn + c, ldf(y, bt * Cn + c) * silu(ldf(z, bt * zs + c)));
    }
  }
}

template <class T, bool VEC>
__global__ void k_gate_bwd(size_t ntok, int Cn, long long zs, const T* __restrict__ y, const T* __restrict__ z,
                           const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz) {
  constexpr int V = VEC ? (int)(16 / sizeof(T)) : 1;
  const int per_row = Cn / V;
  const size_t n = ntok * per_row;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const size_t bt = i / per_row;
    const int c = (int)(i % per_row) * V;
    if (VEC) {
      const uint4 qy = __ldg(reinterpret_cast<const uint4*>(y + bt * Cn + c));
      const uint4 qz = __ldg(reinterpret_cast<const uint4*>(z + bt * zs + c));
      const uint4 qg = __ldg(reinterpret_cast<const uint4*>(dout + bt * Cn + c));
      uint4 o1, o2;
      const T* py = reinterpret_cast<const T*>(&qy);
      const T* pz = reinterpret_cast<const T*>(&qz);
      const T* pg = reinterpret_cast<const T*>(&qg);
      T* p1 = reinterpret_cast<T*>(&o1);
      T* p2 = reinterpret_cast<T*>(&o2);
#pragma unroll
      for (int k = 0; k < V; ++k) {
        const float zv = ldf(pz, k), gv = ldf(pg, k);
        stf(p1, k, gv * silu(zv));
        stf(p2, k, gv * ldf(py, k) * silu_grad(zv));
      }
      if (dy) *reinterpret_cast<uint4*>(dy + bt * Cn + c) = o1;
      if (dz) *reinterpret_cast<uint4*>(dz + bt * zs + c) = o2;
    } else {
      const float zv = ldf(z, bt * zs + c), gv = ldf(dout, bt * Cn + c);
      if (dy) stf(dy, bt * Cn + c, gv * silu(zv));
      if (dz) stf(dz, bt * zs + c, gv * ldf(y, bt * Cn + c) * silu_grad(zv));
    }
  }
}

int bc_dims(m3_ctx* ctx, const m3_bc_desc* s, BcDims* d) {
  if (!ctx || !s) return M3_ERR_NULL;
  if (s->batch <= 0 || s->seq < 0 || s->heads <= 0 || s->groups <= 0 || s->d_state <= 0 || s->rank <= 0)
    return m3::fail(ctx, M3_ERR_SHAPE, "B/C prologue: extents must be positive");
  if (s->heads % s->groups) return m3::fail(ctx, M3_ERR_CONFIG, "heads %d not a multiple of groups %d", s->heads, s->groups);
  if (s->d_state > 32 * kMaxPerLane) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "d_state %d > %d", s->d_state, 32 * kMaxPerLane);
  if (s->dtype != M3_F32 && s->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s->dtype);
  if (!s->b_raw || !s->c_raw) return m3::fail(ctx, M3_ERR_NULL, "b_raw and c_raw are required");
  d->B = s->batch; d->T = s->seq; d->H = s->heads; d->G = s->groups; d->N = s->d_state; d->R = s->rank;
  d->PG = s->heads / s->groups;
  const long long dense = (long long)s->groups * s->rank * s->d_state;
  d->rs = s->raw_stride ? s->raw_stride : dense;
  if (d->rs < dense) return m3::fail(ctx, M3_ERR_SHAPE, "raw_stride below groups * rank * d_state");
  d->eps = s->eps;
  d->has_norm = s->has_norm ? 1 : 0;
  return M3_OK;
}

// ---- the gate behind a post-gate RMS norm: out = y * rsqrt(mean_c y^2 + eps) * gain * silu(z) -------
// One block per token row, rows grid-strided; thread t owns channels t, t + kGnThreads, ... (coalesced),
// so a block's per-channel sums for d gain stay in registers over all of its rows.
constexpr int kGnThreads = 256, kGnMaxPer = 32;  // channels <= kGnThreads * kGnMaxPer

__device__ __forceinline__ float gn_block_sum(float v, float* red) {
  v = warp_sum(v);
  __syncthreads();  // the previous sum's readers are done with red
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.0f;
#pragma unroll
  for (int i = 0; i < kGnThreads / 32; ++i) t += red[i];  // the same order in every thread
  return t;
}

template <class T>
__global__ void __launch_bounds__(kGnThreads)
k_gate_norm_fwd(size_t ntok, int Cn, long long zs, float eps, const T* __restrict__ y, const T* __restrict__ z,
                const float* __restrict__ gain, T* __restrict__ out) {
  __shared__ float red[kGnThreads / 32];
  for (size_t bt = blockIdx.x; bt < ntok; bt += gridDim.x) {
    float v[kGnMaxPer];
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < kGnMaxPer; ++j) {
      const int c = threadIdx.x + j * kGnThreads;
      v[j] = c < Cn ? ldf(y, bt * Cn + c) : 0.0f;
      ss += v[j] * v[j];
    }
    const float r = rsqrtf(gn_block_sum(ss, red) / (float)Cn + eps);
#pragma unroll
    for (int j = 0; j < kGnMaxPer; ++j) {
      const int c = threadIdx.x + j * kGnThreads;
      if (c < Cn) stf(out, bt * Cn + c, v[j] * r * (gain ? gain[c] : 1.0f) * silu(ldf(z, bt * zs + c)));
    }
  }
}

// With n = y r gain and u = gain * dout * silu(z):  dy = r u - y r^3 mean_c(u y),  dz = dout n silu'(z),
// d gain[c] = sum over rows of dout silu(z) y r  (per-block partial sums, added in a fixed order afterwards).
template <class T>
__global__ void __launch_bounds__(kGnThreads)
k_gate_norm_bwd(size_t ntok, int Cn, long long zs, float eps, const T* __restrict__ y, const T* __restrict__ z,
                const float* __restrict__ gain, const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz,
                float* __restrict__ part) {
  __shared__ float red[kGnThreads / 32];
  float accg[kGnMaxPer];
#pragma unroll
  for (int j = 0; j < kGnMaxPer; ++j) accg[j] = 0.0f;
  for (size_t bt = blockIdx.x; bt < ntok; bt += gridDim.x) {
    float yv[kGnMaxPer], dn[kGnMaxPer], w[kGnMaxPer];
    float ss = 0.0f, dot = 0.0f;
#pragma unroll
    for (int j = 0; j < kGnMaxPer; ++j) {
      const int c = threadIdx.x + j * kGnThreads;
      yv[j] = dn[j] = w[j] = 0.0f;
      if (c < Cn) {
        const float g = gain ? gain[c] : 1.0f;
        const float zv = ldf(z, bt * zs + c), gv = ldf(dout, bt * Cn + c);
        yv[j] = ldf(y, bt * Cn + c);
        dn[j] = gv * silu(zv);
        w[j] = gv * silu_grad(zv) * g;
        ss += yv[j] * yv[j];
        dot += dn[j] * g * yv[j];
      }
    }
    const float r = rsqrtf(gn_block_sum(ss, red) / (float)Cn + eps);
    const float md = gn_block_sum(dot, red) / (float)Cn;
#pragma unroll
    for (int j = 0; j < kGnMaxPer; ++j) {
      const int c = threadIdx.x + j * kGnThreads;
      if (c < Cn) {
        const float g = gain ? gain[c] : 1.0f;
        if (dy) stf(dy, bt * Cn + c, r * (dn[j] * g - yv[j] * r * r * md));
        if (dz) stf(dz, bt * zs + c, w[j] * yv[j] * r);
        accg[j] += dn[j] * yv[j] * r;
      }
    }
  }
  if (part) {
#pragma unroll
    for (int j = 0; j < kGnMaxPer; ++j) {
      const int c = threadIdx.x + j * kGnThreads;
      if (c < Cn) part[(size_t)blockIdx.x * Cn + c] = accg[j];
    }
  }
}

// Vector form of the two kernels above (16-byte accesses, rows and strides aligned): a row belongs to a
// group of GS threads - a warp (eight rows per block, sums by shuffles, no block barrier) while a row has at
// most 32 * kGnVec vectors, else the whole block - and thread gl of the group owns vectors gl, gl + GS, ...
// of every row it meets, raw in registers between the two passes over the row.
constexpr int kGnVec = 8;  // vectors per thread, at most (the kernels are built for 1, 2, 4 and 8)

template <int GS>
__device__ __forceinline__ float gn_group_sum(float v, float* red) {
  if (GS == 32) return warp_sum(v);
  return gn_block_sum(v, red);
}

template <class T, int GS, int NV>
__global__ void __launch_bounds__(kGnThreads)
k_gate_norm_fwd_vec(size_t ntok, int Cn, long long zs, float eps, const T* __restrict__ y, const T* __restrict__ z,
                    const float* __restrict__ gain, T* __restrict__ out) {
  constexpr int V = (int)(16 / sizeof(T)), RPB = kGnThreads / GS;
  __shared__ float red[kGnThreads / 32];
  const int gl = threadIdx.x % GS, gr = threadIdx.x / GS, nvec = Cn / V;
  for (size_t bt = (size_t)blockIdx.x * RPB + gr; bt < ntok; bt += (size_t)gridDim.x * RPB) {
    uint4 qy[NV], qz[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = gl + j * GS;
      if (v < nvec) {
        qy[j] = __ldg(reinterpret_cast<const uint4*>(y + bt * Cn + (size_t)v * V));
        qz[j] = __ldg(reinterpret_cast<const uint4*>(z + bt * zs + (size_t)v * V));
      }
    }
    float ss = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if (gl + j * GS < nvec) {
        const T* py = reinterpret_cast<const T*>(&qy[j]);
#pragma unroll
        for (int k = 0; k < V; ++k) ss += ldf(py, k) * ldf(py, k);
      }
    const float r = rsqrtf(gn_group_sum<GS>(ss, red) / (float)Cn + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = gl + j * GS;
      if (v < nvec) {
        const T* py = reinterpret_cast<const T*>(&qy[j]);
        const T* pz = reinterpret_cast<const T*>(&qz[j]);
        uint4 qo;
        T* po = reinterpret_cast<T*>(&qo);
#pragma unroll
        for (int k = 0; k < V; ++k) stf(po, k, ldf(py, k) * r * (gain ? __ldg(gain + v * V + k) : 1.0f) * silu(ldf(pz, k)));
        *reinterpret_cast<uint4*>(out + bt * Cn + (size_t)v * V) = qo;
      }
    }
  }
}

template <class T, int GS, int NV>
__global__ void __launch_bounds__(kGnThreads)
k_gate_norm_bwd_vec(size_t ntok, int Cn, long long zs, float eps, const T* __restrict__ y, const T* __restrict__ z,
                    const float* __restrict__ gain, const T* __restrict__ dout, T* __restrict__ dy, T* __restrict__ dz,
                    float* __restrict__ part) {
  constexpr int V = (int)(16 / sizeof(T)), RPB = kGnThreads / GS;
  __shared__ float red[kGnThreads / 32];
  extern __shared__ float s_acc[];  // [Cn] when GS == 32 and d gain is wanted: the block's eight rows' sums
  const int gl = threadIdx.x % GS, gr = threadIdx.x / GS, nvec = Cn / V;
  float accg[NV * V];
#pragma unroll
  for (int i = 0; i < NV * V; ++i) accg[i] = 0.0f;
  for (size_t bt = (size_t)blockIdx.x * RPB + gr; bt < ntok; bt += (size_t)gridDim.x * RPB) {
    uint4 qy[NV], qz[NV], qg[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = gl + j * GS;
      if (v < nvec) {
        qy[j] = __ldg(reinterpret_cast<const uint4*>(y + bt * Cn + (size_t)v * V));
        qz[j] = __ldg(reinterpret_cast<const uint4*>(z + bt * zs + (size_t)v * V));
        qg[j] = __ldg(reinterpret_cast<const uint4*>(dout + bt * Cn + (size_t)v * V));
      }
    }
    float ss = 0.0f, dot = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = gl + j * GS;
      if (v < nvec) {
        const T* py = reinterpret_cast<const T*>(&qy[j]);
        const T* pz = reinterpret_cast<const T*>(&qz[j]);
        const T* pg = reinterpret_cast<const T*>(&qg[j]);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float yv = ldf(py, k);
          ss += yv * yv;
          dot += ldf(pg, k) * silu(ldf(pz, k)) * (gain ? __ldg(gain + v * V + k) : 1.0f) * yv;
        }
      }
    }
    const float r = rsqrtf(gn_group_sum<GS>(ss, red) / (float)Cn + eps);
    const float md = gn_group_sum<GS>(dot, red) / (float)Cn;
    const float r2md = r * r * md;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int v = gl + j * GS;
      if (v < nvec) {
        const T* py = reinterpret_cast<const T*>(&qy[j]);
        const T* pz = reinterpret_cast<const T*>(&qz[j]);
        const T* pg = reinterpret_cast<const T*>(&qg[j]);
        uint4 o1, o2;
        T* p1 = reinterpret_cast<T*>(&o1);
        T* p2 = reinterpret_cast<T*>(&o2);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          const float g = gain ? __ldg(gain + v * V + k) : 1.0f;
          const float yv = ldf(py, k), zv = ldf(pz, k), gv = ldf(pg, k);
          const float sg = sigmoid(zv);
          const float dn = gv * zv * sg;
          stf(p1, k, r * (dn * g - yv * r2md));
          stf(p2, k, gv * sg * (1.0f + zv * (1.0f - sg)) * g * yv * r);
          accg[j * V + k] += dn * yv * r;
        }
        if (dy) *reinterpret_cast<uint4*>(dy + bt * Cn + (size_t)v * V) = o1;
        if (dz) *reinterpret_cast<uint4*>(dz + bt * zs + (size_t)v * V) = o2;
      }
    }
  }
  if (part) {
    if (GS == 32) {  // the eight warps' sums, added warp after warp: one order whatever the scheduling
      for (int w = 0; w < RPB; ++w) {
        if (gr == w) {
#pragma unroll
          for (int j = 0; j < NV; ++j) {
            const int v = gl + j * GS;
            if (v < nvec)
#pragma unroll
              for (int k = 0; k < V; ++k) s_acc[v * V + k] = (w ? s_acc[v * V + k] : 0.0f) + accg[j * V + k];
          }
        }
        __syncthreads();
      }
      for (int c = threadIdx.x; c < Cn; c += kGnThreads) part[(size_t)blockIdx.x * Cn + c] = s_acc[c];
    } else {
#pragma unroll
      for (int j = 0; j < NV; ++j) {
        const int v = gl + j * GS;
        if (v < nvec)
#pragma unroll
          for (int k = 0; k < V; ++k) part[(size_t)blockIdx.x * Cn + v * V + k] = accg[j * V + k];
      }
    }
  }
}

// Calls f(integral_constant<GS>, integral_constant<NV>) with the smallest NV of 1, 2, 4, 8 that covers the row.
template <class F>
static void gate_norm_dispatch(int gs, int nvec, F&& f) {
  const int per = (nvec + gs - 1) / gs;
  auto with_gs = [&](auto G) {
    if (per <= 1) f(G, std::integral_constant<int, 1>{});
    else if (per <= 2) f(G, std::integral_constant<int, 2>{});
    else if (per <= 4) f(G, std::integral_constant<int, 4>{});
    else f(G, std::integral_constant<int, 8>{});
  };
  if (gs == 32) with_gs(std::integral_constant<int, 32>{});
  else with_gs(std::integral_constant<int, 256>{});
}

}  // namespace

extern "C" {

int m3_bc_forward(m3_ctx* ctx, const m3_bc_desc* s, void* b, void* c) {
  BcDims d;
  const int rc = bc_dims(ctx, s, &d);
  if (rc != M3_OK) return rc;
  if (!b || !c) return m3::fail(ctx, M3_ERR_NULL, "b and c are required");
  if (d.T == 0) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t rows = (size_t)d.B * d.T * d.H;
  const unsigned grid = (unsigned)((rows + kBcWarps - 1) / kBcWarps);
  const bool aligned = !(d.rs % 8) && !(reinterpret_cast<uintptr_t>(s->b_raw) % 16) && !(reinterpret_cast<uintptr_t>(s->c_raw) % 16) &&
                       !(reinterpret_cast<uintptr_t>(b) % 16) && !(reinterpret_cast<uintptr_t>(c) % 16) &&
                       !(reinterpret_cast<uintptr_t>(s->b_bias) % 16) && !(reinterpret_cast<uintptr_t>(s->c_bias) % 16) &&
                       !(reinterpret_cast<uintptr_t>(s->norm_weight) % 16);
  if (s->dtype == M3_BF16 && aligned && (d.N == 128 || d.N == 256) && (d.R == 1 || d.R == 2 || d.R == 4)) {
    using T = __nv_bfloat16;
    for (int which = 0; which < 2; ++which) {
      const T* raw = static_cast<const T*>(which ? s->c_raw : s->b_raw);
      const float* bias = which ? s->c_bias : s->b_bias;
      T* out = static_cast<T*>(which ? c : b);
#define M3_BC_FWD(RR, NN)                                                                       \
  k_bc_fwd_vec<RR, NN><<<(unsigned)((rows + kBcWarps * (512 / NN) - 1) / (kBcWarps * (512 / NN))), \
                         kBcWarps * 32, 0, ctx->stream>>>(d, raw, bias, s->norm_weight, out)
      if (d.N == 128) {
        if (d.R == 1) M3_BC_FWD(1, 128); else if (d.R == 2) M3_BC_FWD(2, 128); else M3_BC_FWD(4, 128);
      } else {
        if (d.R == 1) M3_BC_FWD(1, 256); else if (d.R == 2) M3_BC_FWD(2, 256); else M3_BC_FWD(4, 256);
      }
#undef M3_BC_FWD
    }
  } else if (s->dtype == M3_BF16) {
    using T = __nv_bfloat16;
    k_bc_fwd<T><<<grid, kBcWarps * 32, 0, ctx->stream>>>(d, static_cast<const T*>(s->b_raw), s->b_bias, s->norm_weight, static_cast<T*>(b));
    k_bc_fwd<T><<<grid, kBcWarps * 32, 0, ctx->stream>>>(d, static_cast<const T*>(s->c_raw), s->c_bias, s->norm_weight, static_cast<T*>(c));
  } else {
    k_bc_fwd<float><<<grid, kBcWarps * 32, 0, ctx->stream>>>(d, static_cast<const float*>(s->b_raw), s->b_bias, s->norm_weight, static_cast<float*>(b));
    k_bc_fwd<float><<<grid, kBcWarps * 32, 0, ctx->stream>>>(d, static_cast<const float*>(s->c_raw), s->c_bias, s->norm_weight, static_cast<float*>(c));
  }
  M3_CUDA(ctx, cudaGetLastError());
  ctx->launches += 2;
  return M3_OK;
}

int m3_bc_backward(m3_ctx* ctx, const m3_bc_desc* s, const void* db, const void* dc, void* db_raw, void* dc_raw,
                   float* db_bias, float* dc_bias, float* dnorm_weight) {
  BcDims d;
  const int rc = bc_dims(ctx, s, &d);
  if (rc != M3_OK) return rc;
  if (!db || !dc) return m3::fail(ctx, M3_ERR_NULL, "db and dc are required");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t nb = (size_t)d.H * d.N * sizeof(float);
  if (d.T == 0) {
    if (db_bias) M3_CUDA(ctx, cudaMemsetAsync(db_bias, 0, nb, ctx->stream));
    if (dc_bias) M3_CUDA(ctx, cudaMemsetAsync(dc_bias, 0, nb, ctx->stream));
    if (dnorm_weight) M3_CUDA(ctx, cudaMemsetAsync(dnorm_weight, 0, d.N * sizeof(float), ctx->stream));
    return M3_OK;
  }
  const int nblk_tok = (int)(((size_t)d.B * d.T + kBcTokens - 1) / kBcTokens);
  const int width = (d.PG + 1) * d.N;
  const size_t smem = (size_t)kBcWarps * width * sizeof(float);
  if (smem > 200 * 1024) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "heads per group %d x d_state %d needs %zu bytes of shared memory", d.PG, d.N, smem);
  float* part = nullptr;
  M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&part), (size_t)nblk_tok * d.G * width * sizeof(float), ctx->stream));
  const dim3 grid(nblk_tok, d.G);
  cudaError_t e = cudaSuccess;
  for (int which = 0; which < 2 && e == cudaSuccess; ++which) {
    const void* raw = which ? s->c_raw : s->b_raw;
    const float* bias = which ? s->c_bias : s->b_bias;
    const void* go = which ? dc : db;
    void* draw = which ? dc_raw : db_raw;
    float* dbias = bias ? (which ? dc_bias : db_bias) : nullptr;
    const bool aligned = !(d.rs % 8) && !(reinterpret_cast<uintptr_t>(raw) % 16) && !(reinterpret_cast<uintptr_t>(go) % 16) &&
                         !(reinterpret_cast<uintptr_t>(draw) % 16) && !(reinterpret_cast<uintptr_t>(bias) % 16) &&
                         !(reinterpret_cast<uintptr_t>(s->norm_weight) % 16);
    if (s->dtype == M3_BF16 && aligned && d.PG == 1 && (d.N == 128 || d.N == 256) && (d.R == 1 || d.R == 2 || d.R == 4)) {
      using T = __nv_bfloat16;
#define M3_BC_BWD(RR, NN)                                                                                       \
  k_bc_bwd_vec<RR, NN><<<grid, kBcWarps * 32, 0, ctx->stream>>>(d, static_cast<const T*>(raw), bias, s->norm_weight, \
                                                                static_cast<const T*>(go), static_cast<T*>(draw), part)
      if (d.N == 128) {
        if (d.R == 1) M3_BC_BWD(1, 128); else if (d.R == 2) M3_BC_BWD(2, 128); else M3_BC_BWD(4, 128);
      } else {
        if (d.R == 1) M3_BC_BWD(1, 256); else if (d.R == 2) M3_BC_BWD(2, 256); else M3_BC_BWD(4, 256);
      }
#undef M3_BC_BWD
    } else if (s->dtype == M3_BF16) {
      using T = __nv_bfloat16;
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_bc_bwd<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        k_bc_bwd<T><<<grid, kBcWarps * 32, smem, ctx->stream>>>(d, static_cast<const T*>(raw), bias, s->norm_weight,
                                                                 static_cast<const T*>(go), static_cast<T*>(draw), part);
    } else {
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(k_bc_bwd<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        k_bc_bwd<float><<<grid, kBcWarps * 32, smem, ctx->stream>>>(d, static_cast<const float*>(raw), bias, s->norm_weight,
                                                                     static_cast<const float*>(go), static_cast<float*>(draw), part);
    }
    if (e == cudaSuccess) e = cudaGetLastError();
    if (e == cudaSuccess && dbias)  // d bias[g * PG + hg, n]: the first PG * N columns of group g's partials
      e = m3::column_sums(ctx->stream, part, nblk_tok, (size_t)d.G * width, d.PG * d.N, dbias, false, d.G, width,
                          (size_t)d.PG * d.N);
    // the gain is shared by B and C (one bc_norm module): the second pass adds to the first
    if (e == cudaSuccess && d.has_norm && s->norm_weight && dnorm_weight)
      e = m3::column_sums(ctx->stream, part + (size_t)d.PG * d.N, nblk_tok * d.G, width, d.N, dnorm_weight, which == 1);
    ctx->launches += 3;
  }
  cudaError_t e2 = cudaFreeAsync(part, ctx->stream);
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "B/C prologue backward");
  if (e2 != cudaSuccess) return m3::cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

int m3_dt_lambda_forward(m3_ctx* ctx, const m3_act_desc* s, void* dt, void* lambda) {
  if (!ctx || !s) return M3_ERR_NULL;
  if (s->batch <= 0 || s->seq < 0 || s->heads <= 0) return m3::fail(ctx, M3_ERR_SHAPE, "dt / lambda: extents must be positive");
  if (s->dtype != M3_F32 && s->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s->dtype);
  if (!s->dt_raw || !dt) return m3::fail(ctx, M3_ERR_NULL, "dt_raw and dt are required");
  if (s->seq == 0) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const int ntok = s->batch * s->seq;
  const long long st = s->stride ? s->stride : s->heads;
  const size_t n = (size_t)ntok * s->heads;
  const unsigned grid = (unsigned)((n + 255) / 256 < 2048 ? (n + 255) / 256 : 2048);
  if (s->dtype == M3_BF16) {
    using T = __nv_bfloat16;
    k_act_fwd<T><<<grid, 256, 0, ctx->stream>>>(ntok, s->heads, st, static_cast<const T*>(s->dt_raw),
                                                 static_cast<const T*>(s->lambda_raw), s->dt_bias, static_cast<T*>(dt), static_cast<T*>(lambda));
  } else {
    k_act_fwd<float><<<grid, 256, 0, ctx->stream>>>(ntok, s->heads, st, static_cast<const float*>(s->dt_raw),
                                                     static_cast<const float*>(s->lambda_raw), s->dt_bias, static_cast<float*>(dt), static_cast<float*>(lambda));
  }
  M3_CUDA(ctx, cudaGetLastError());
  ctx->launches += 1;
  return M3_OK;
}

int m3_dt_lambda_backward(m3_ctx* ctx, const m3_act_desc* s, const void* ddt, const void* dlambda, void* ddt_raw,
                          void* dlambda_raw, float* ddt_bias) {
  if (!ctx || !s) return M3_ERR_NULL;
  if (s->batch <= 0 || s->seq < 0 || s->heads <= 0) return m3::fail(ctx, M3_ERR_SHAPE, "dt / lambda: extents must be positive");
  if (s->dtype != M3_F32 && s->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s->dtype);
  if (!s->dt_raw || !ddt) return m3::fail(ctx, M3_ERR_NULL, "dt_raw and ddt are required");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  if (s->seq == 0) {
    if (ddt_bias) M3_CUDA(ctx, cudaMemsetAsync(ddt_bias, 0, s->heads * sizeof(float), ctx->stream));
    return M3_OK;
  }
  const int ntok = s->batch * s->seq;
  const long long st = s->stride ? s->stride : s->heads;
  const int nruns = (ntok + kActRun - 1) / kActRun;
  float* part = nullptr;
  const bool want_bias = ddt_bias && s->dt_bias;
  if (want_bias) M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&part), (size_t)nruns * s->heads * sizeof(float), ctx->stream));
  const size_t nthreads = (size_t)nruns * s->heads;
  const unsigned grid = (unsigned)((nthreads + 127) / 128);
  if (s->dtype == M3_BF16) {
    using T = __nv_bfloat16;
    k_act_bwd<T><<<grid, 128, 0, ctx->stream>>>(ntok, s->heads, st, static_cast<const T*>(s->dt_raw), static_cast<const T*>(s->lambda_raw),
                                                 s->dt_bias, static_cast<const T*>(ddt), static_cast<const T*>(dlambda),
                                                 static_cast<T*>(ddt_raw), static_cast<T*>(dlambda_raw), part);
  } else {
    k_act_bwd<float><<<grid, 128, 0, ctx->stream>>>(ntok, s->heads, st, static_cast<const float*>(s->dt_raw),
                                                     static_cast<const float*>(s->lambda_raw), s->dt_bias, static_cast<const float*>(ddt),
                                                     static_cast<const float*>(dlambda), static_cast<float*>(ddt_raw),
                                                     static_cast<float*>(dlambda_raw), part);
  }
  cudaError_t e = cudaGetLastError();
  ctx->launches += 1;
  if (e == cudaSuccess && want_bias) {
    e = m3::column_sums(ctx->stream, part, nruns, s->heads, s->heads, ddt_bias);
    ctx->launches += 1;
  }
  cudaError_t e2 = part ? cudaFreeAsync(part, ctx->stream) : cudaSuccess;
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "dt / lambda backward");
  if (e2 != cudaSuccess) return m3::cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

static bool gate_vec(const m3_gate_desc* s, int es, long long zs, std::initializer_list<const void*> ptrs) {
  const int V = 16 / es;
  if (s->channels % V || zs % V) return false;
  for (const void* p : ptrs)
    if (p && (reinterpret_cast<uintptr_t>(p) % 16)) return false;
  return true;
}

static int gate_check(m3_ctx* ctx, const m3_gate_desc* s) {
  if (!ctx || !s) return M3_ERR_NULL;
  if (s->batch <= 0 || s->seq < 0 || s->channels <= 0) return m3::fail(ctx, M3_ERR_SHAPE, "gate: extents must be positive");
  if (s->dtype != M3_F32 && s->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s->dtype);
  if (!s->y || !s->z) return m3::fail(ctx, M3_ERR_NULL, "y and z are required");
  if (s->z_stride && s->z_stride < s->channels) return m3::fail(ctx, M3_ERR_SHAPE, "z_stride below the channel count");
  return M3_OK;
}

int m3_gate_forward(m3_ctx* ctx, const m3_gate_desc* s, void* out) {
  const int rc = gate_check(ctx, s);
  if (rc != M3_OK) return rc;
  if (!out) return m3::fail(ctx, M3_ERR_NULL, "out is required");
  if (s->seq == 0) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t ntok = (size_t)s->batch * s->seq;
  const long long zs = s->z_stride ? s->z_stride : s->channels;
  const int es = s->dtype == M3_BF16 ? 2 : 4;
  const bool vec = gate_vec(s, es, zs, {s->y, s->z, out});
  const size_t items = ntok * (s->channels / (vec ? 16 / es : 1));
  const unsigned grid = (unsigned)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
  if (s->dtype == M3_BF16) {
    using T = __nv_bfloat16;
    if (vec) k_gate_fwd<T, true><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const T*>(s->y), static_cast<const T*>(s->z), static_cast<T*>(out));
    else k_gate_fwd<T, false><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const T*>(s->y), static_cast<const T*>(s->z), static_cast<T*>(out));
  } else {
    if (vec) k_gate_fwd<float, true><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const float*>(s->y), static_cast<const float*>(s->z), static_cast<float*>(out));
    else k_gate_fwd<float, false><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const float*>(s->y), static_cast<const float*>(s->z), static_cast<float*>(out));
  }
  M3_CUDA(ctx, cudaGetLastError());
  ctx->launches += 1;
  return M3_OK;
}

int m3_gate_backward(m3_ctx* ctx, const m3_gate_desc* s, const void* dout, void* dy, void* dz) {
  const int rc = gate_check(ctx, s);
  if (rc != M3_OK) return rc;
  if (!dout) return m3::fail(ctx, M3_ERR_NULL, "dout is required");
  if (s->seq == 0) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t ntok = (size_t)s->batch * s->seq;
  const long long zs = s->z_stride ? s->z_stride : s->channels;
  const int es = s->dtype == M3_BF16 ? 2 : 4;
  const bool vec = gate_vec(s, es, zs, {s->y, s->z, dout, dy, dz});
  const size_t items = ntok * (s->channels / (vec ? 16 / es : 1));
  const unsigned grid = (unsigned)((items + 255) / 256 < 148 * 16 ? (items + 255) / 256 : 148 * 16);
  if (s->dtype == M3_BF16) {
    using T = __nv_bfloat16;
    if (vec) k_gate_bwd<T, true><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const T*>(s->y), static_cast<const T*>(s->z), static_cast<const T*>(dout), static_cast<T*>(dy), static_cast<T*>(dz));
    else k_gate_bwd<T, false><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const T*>(s->y), static_cast<const T*>(s->z), static_cast<const T*>(dout), static_cast<T*>(dy), static_cast<T*>(dz));
  } else {
    if (vec) k_gate_bwd<float, true><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const float*>(s->y), static_cast<const float*>(s->z), static_cast<const float*>(dout), static_cast<float*>(dy), static_cast<float*>(dz));
    else k_gate_bwd<float, false><<<grid, 256, 0, ctx->stream>>>(ntok, s->channels, zs, static_cast<const float*>(s->y), static_cast<const float*>(s->z), static_cast<const float*>(dout), static_cast<float*>(dy), static_cast<float*>(dz));
  }
  M3_CUDA(ctx, cudaGetLastError());
  ctx->launches += 1;
  return M3_OK;
}

// Threads per row of the vector kernels (32 or 256), or 0 for the element-wise kernels (rows that are not
// whole 16-byte vectors, or a pointer off a 16-byte boundary).
static int gate_norm_group(const m3_gate_norm_desc* s, long long zs, std::initializer_list<const void*> ptrs) {
  const int V = s->dtype == M3_BF16 ? 8 : 4;
  if (s->channels % V || zs % V) return 0;
  for (const void* p : ptrs)
    if (p && (reinterpret_cast<uintptr_t>(p) % 16)) return 0;
  const int nvec = s->channels / V;
  return nvec <= 32 * kGnVec ? 32 : (nvec <= kGnThreads * kGnVec ? 256 : 0);
}

static int gate_norm_check(m3_ctx* ctx, const m3_gate_norm_desc* s) {
  if (!ctx || !s) return M3_ERR_NULL;
  if (s->batch <= 0 || s->seq < 0 || s->channels <= 0) return m3::fail(ctx, M3_ERR_SHAPE, "gate: extents must be positive");
  if (s->channels > kGnThreads * kGnMaxPer)
    return m3::fail(ctx, M3_ERR_UNSUPPORTED, "post-gate norm over %d channels (at most %d)", s->channels, kGnThreads * kGnMaxPer);
  if (s->dtype != M3_F32 && s->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s->dtype);
  if (!s->y || !s->z) return m3::fail(ctx, M3_ERR_NULL, "y and z are required");
  if (s->z_stride && s->z_stride < s->channels) return m3::fail(ctx, M3_ERR_SHAPE, "z_stride below the channel count");
  if (!(s->eps >= 0.0f)) return m3::fail(ctx, M3_ERR_CONFIG, "eps must not be negative");
  return M3_OK;
}

int m3_gate_norm_forward(m3_ctx* ctx, const m3_gate_norm_desc* s, void* out) {
  const int rc = gate_norm_check(ctx, s);
  if (rc != M3_OK) return rc;
  if (!out) return m3::fail(ctx, M3_ERR_NULL, "out is required");
  if (s->seq == 0) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t ntok = (size_t)s->batch * s->seq;
  const long long zs = s->z_stride ? s->z_stride : s->channels;
  const int gs = gate_norm_group(s, zs, {s->y, s->z, out});
  const size_t nblk = gs ? (ntok + kGnThreads / gs - 1) / (kGnThreads / gs) : ntok;
  const unsigned grid = (unsigned)(nblk < 148u * 8u ? nblk : 148u * 8u);
  auto launch = [&](auto tag) {
    using T = decltype(tag);
    const T *y = static_cast<const T*>(s->y), *z = static_cast<const T*>(s->z);
    T* o = static_cast<T*>(out);
    if (gs)
      gate_norm_dispatch(gs, s->channels / (int)(16 / sizeof(T)), [&](auto G, auto N) {
        k_gate_norm_fwd_vec<T, decltype(G)::value, decltype(N)::value><<<grid, kGnThreads, 0, ctx->stream>>>(
            ntok, s->channels, zs, s->eps, y, z, s->weight, o);
      });
    else k_gate_norm_fwd<T><<<grid, kGnThreads, 0, ctx->stream>>>(ntok, s->channels, zs, s->eps, y, z, s->weight, o);
  };
  if (s->dtype == M3_BF16) launch(__nv_bfloat16{}); else launch(float{});
  M3_CUDA(ctx, cudaGetLastError());
  ctx->launches += 1;
  return M3_OK;
}

int m3_gate_norm_backward(m3_ctx* ctx, const m3_gate_norm_desc* s, const void* dout, void* dy, void* dz, float* dweight) {
  const int rc = gate_norm_check(ctx, s);
  if (rc != M3_OK) return rc;
  if (!dout) return m3::fail(ctx, M3_ERR_NULL, "dout is required");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const bool want_w = dweight && s->weight;
  if (s->seq == 0) {
    if (want_w) M3_CUDA(ctx, cudaMemsetAsync(dweight, 0, s->channels * sizeof(float), ctx->stream));
    return M3_OK;
  }
  const size_t ntok = (size_t)s->batch * s->seq;
  const long long zs = s->z_stride ? s->z_stride : s->channels;
  const int gs = gate_norm_group(s, zs, {s->y, s->z, dout, dy, dz});
  const size_t nblk = gs ? (ntok + kGnThreads / gs - 1) / (kGnThreads / gs) : ntok;
  const unsigned grid = (unsigned)(nblk < 148u * 4u ? nblk : 148u * 4u);
  float* part = nullptr;
  if (want_w) M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&part), (size_t)grid * s->channels * sizeof(float), ctx->stream));
  auto launch = [&](auto tag) {
    using T = decltype(tag);
    const T *y = static_cast<const T*>(s->y), *z = static_cast<const T*>(s->z), *g = static_cast<const T*>(dout);
    T *py = static_cast<T*>(dy), *pz = static_cast<T*>(dz);
    const size_t sm = part ? (size_t)s->channels * sizeof(float) : 0;
    if (gs)
      gate_norm_dispatch(gs, s->channels / (int)(16 / sizeof(T)), [&](auto G, auto N) {
        k_gate_norm_bwd_vec<T, decltype(G)::value, decltype(N)::value><<<grid, kGnThreads, gs == 32 ? sm : 0, ctx->stream>>>(
            ntok, s->channels, zs, s->eps, y, z, s->weight, g, py, pz, part);
      });
    else k_gate_norm_bwd<T><<<grid, kGnThreads, 0, ctx->stream>>>(ntok, s->channels, zs, s->eps, y, z, s->weight, g, py, pz, part);
  };
  if (s->dtype == M3_BF16) launch(__nv_bfloat16{}); else launch(float{});
  cudaError_t e = cudaGetLastError();
  ctx->launches += 1;
  if (e == cudaSuccess && want_w) {
    e = m3::column_sums(ctx->stream, part, (int)grid, s->channels, s->channels, dweight);
    ctx->launches += 1;
  }
  cudaError_t e2 = part ? cudaFreeAsync(part, ctx->stream) : cudaSuccess;
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "gate + norm backward");
  if (e2 != cudaSuccess) return m3::cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

}  // extern "C"
