// Depthwise causal convolution over time followed by SiLU: the step in front of the scan
// (CausalConv1d, src/nn/conv.rs:143-213, kernels src/tensor/ops/fused.rs:780-1200; the mixer
// applies SiLU to its result, src/models/mamba3.rs:401).
//
//   pre[b,t,c] = bias[c] + sum_{delay < K} w[K-1-delay, c] * x[b, t-delay, c]      (x[t<0] = history or 0)
//   y = silu(pre)  (or pre)
//
// HBM-bound: x is read once and y written once.  A thread owns one 16-byte vector of channels
// and walks a run of time steps with the K-1 previous inputs in registers; the 32 lanes of a
// warp cover 512 contiguous bytes of a row.  Rows may be strided (x is a column band of the
// mixer's input projection).  The backward pass recomputes pre from x, so nothing is saved.
#include <cuda_bf16.h>

#include <initializer_list>

#include "m3_internal.h"

#define M3_CUDA(ctx, call)                                       \
  do {                                                           \
    cudaError_t e_ = (call);                                     \
    if (e_ != cudaSuccess) return m3::cuda_fail(ctx, e_, #call); \
  } while (0)

namespace {

constexpr int kMaxTaps = 8;
constexpr int kRunFwd = 4;   // time steps per thread, forward
constexpr int kRunBwd = 8;   // and backward (its look-ahead recomputes K-1 steps per run)
constexpr int kLanesT = 8;   // threads of a block along time
constexpr int kLanesC = 32;  // threads of a block along channel vectors

template <class T, int V>
struct Vec;
template <>
struct Vec<__nv_bfloat16, 8> {
  using raw_t = uint4;
  static __device__ __forceinline__ raw_t load_raw(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
  static __device__ __forceinline__ raw_t zero_raw() { return make_uint4(0u, 0u, 0u, 0u); }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) { unpack(load_raw(p), v); }
  static __device__ __forceinline__ void unpack(const raw_t& q, float (&v)[8]) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 q;
    uint32_t* w = reinterpret_cast<uint32_t*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = q;
  }
};
template <>
struct Vec<__nv_bfloat16, 4> {  // 8-byte vectors: half the registers per thread, for the backward pass
  using raw_t = uint2;
  static __device__ __forceinline__ raw_t load_raw(const __nv_bfloat16* p) { return __ldg(reinterpret_cast<const uint2*>(p)); }
  static __device__ __forceinline__ raw_t zero_raw() { return make_uint2(0u, 0u); }
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) { unpack(load_raw(p), v); }
  static __device__ __forceinline__ void unpack(const raw_t& q, float (&v)[4]) {
    v[0] = __uint_as_float(q.x << 16); v[1] = __uint_as_float(q.x & 0xffff0000u);
    v[2] = __uint_as_float(q.y << 16); v[3] = __uint_as_float(q.y & 0xffff0000u);
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    uint2 q;
    q.x = *reinterpret_cast<uint32_t*>(&a);
    q.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = q;
  }
};
template <>
struct Vec<float, 4> {
  using raw_t = float4;
  static __device__ __forceinline__ raw_t load_raw(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
  static __device__ __forceinline__ raw_t zero_raw() { return make_float4(0.f, 0.f, 0.f, 0.f); }
  static __device__ __forceinline__ void load(const float* p, float (&v)[4]) { unpack(load_raw(p), v); }
  static __device__ __forceinline__ void unpack(const raw_t& q, float (&v)[4]) {
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <class T>
struct Vec<T, 1> {
  using raw_t = float;
  static __device__ __forceinline__ raw_t load_raw(const T* p) { return m3::ldf(p, 0); }
  static __device__ __forceinline__ raw_t zero_raw() { return 0.0f; }
  static __device__ __forceinline__ void unpack(const raw_t& q, float (&v)[1]) { v[0] = q; }
  static __device__ __forceinline__ void load(const T* p, float (&v)[1]) { v[0] = m3::ldf(p, 0); }
  static __device__ __forceinline__ void store(T* p, const float (&v)[1]) { m3::stf(p, 0, v[0]); }
};

struct ConvDims {
  int B, T, C, K;
  long long xs, ys;  // elements between consecutive time steps of x (and dx) / of y (and dy)
  int act;
  int split;         // channels >= split live in a second output tensor (0: none)
  long long y2s;     // its row stride
  int nrev;          // channel ranges convolved right to left (the backward direction of a
  int rev_lo[4];     // bidirectional mixer): position s of such a channel is time T-1-s
  int rev_hi[4];
};

__device__ __forceinline__ bool walks_backwards(const ConvDims& d, int c0) {
  bool r = false;
#pragma unroll
  for (int i = 0; i < 4; ++i) r = r || (i < d.nrev && c0 >= d.rev_lo[i] && c0 < d.rev_hi[i]);
  return r;
}
// Time of position s for a channel of the given direction.
__device__ __forceinline__ int at_time(const ConvDims& d, bool rev, int s) { return rev ? d.T - 1 - s : s; }

// Where channel vector c0 of the output (or of its gradient) lives: the first tensor, or the
// second one for channels at and beyond the split.
template <class T>
__device__ __forceinline__ T* out_band(const ConvDims& d, T* y, T* y2, int c0, long long* stride) {
  if (d.split > 0 && c0 >= d.split) {
    *stride = d.y2s;
    return y2 + (c0 - d.split);
  }
  *stride = d.ys;
  return y + c0;
}

// Fast-math division (2 ulp): the kernels are bound by instruction issue, and an IEEE division
// costs about as much as the rest of a tap loop.
__device__ __forceinline__ float silu(float v) { return __fdividef(v, 1.0f + __expf(-v)); }
__device__ __forceinline__ float silu_grad(float v) {
  const float s = __fdividef(1.0f, 1.0f + __expf(-v));
  return s * (1.0f + v * (1.0f - s));
}

// x of (b, t, channel vector c0): the sequence, the carried history for t < 0, or zero.
template <class T, int V>
__device__ __forceinline__ typename Vec<T, V>::raw_t load_x(const ConvDims& d, const T* x, const T* hist, int b, int t,
                                                            int c0, bool rev = false) {
  if (t >= 0 && t < d.T) return Vec<T, V>::load_raw(x + ((size_t)b * d.T + at_time(d, rev, t)) * d.xs + c0);
  if (t < 0 && hist && t + (d.K - 1) >= 0)
    return Vec<T, V>::load_raw(hist + ((size_t)b * (d.K - 1) + (t + d.K - 1)) * d.C + c0);
  return Vec<T, V>::zero_raw();
}

// The kernels are compiled for KT in {2, 4, 8} taps; a K-tap convolution runs as the KT-tap one
// whose first KT-K taps are zero, so every loop over taps is static.
// acc[i] += a[i] * b[i] over a thread's V channels, two channels per instruction (packed fp32 pairs) when
// V is even: these kernels are bound by instruction issue.
template <int V>
__device__ __forceinline__ void fma_vec(const float (&a)[V], const float (&b)[V], float (&acc)[V]) {
  if constexpr (V % 2 == 0) {
#pragma unroll
    for (int i = 0; i < V; i += 2) {
      const float2 r = __ffma2_rn(make_float2(a[i], a[i + 1]), make_float2(b[i], b[i + 1]), make_float2(acc[i], acc[i + 1]));
      acc[i] = r.x;
      acc[i + 1] = r.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = fmaf(a[i], b[i], acc[i]);
  }
}

template <class T, int V, int KT>
__global__ void __launch_bounds__(kLanesT* kLanesC)
    k_conv_fwd(ConvDims d, const T* __restrict__ x, const T* __restrict__ hist, const float* __restrict__ w,
               const float* __restrict__ bias, T* __restrict__ y, T* __restrict__ y2) {
  const int c0 = (blockIdx.x * kLanesC + threadIdx.x) * V;
  const int b = blockIdx.z;
  const int t0 = (blockIdx.y * kLanesT + threadIdx.y) * kRunFwd;
  if (c0 >= d.C || t0 >= d.T) return;
  long long ys;
  T* yb = out_band<T>(d, y, y2, c0, &ys);
  const bool rev = walks_backwards(d, c0);
  const int pad = KT - d.K;
  float wt[KT][V], bs[V], win[KT][V];  // win[k] pairs with tap k: x[t - (KT-1-k)]
#pragma unroll
  for (int k = 0; k < KT; ++k)
#pragma unroll
    for (int i = 0; i < V; ++i) wt[k][i] = (k >= pad) ? w[(size_t)(k - pad) * d.C + c0 + i] : 0.0f;
#pragma unroll
  for (int i = 0; i < V; ++i) bs[i] = bias ? bias[c0 + i] : 0.0f;
  // Every row this thread needs is requested before the first one is used.
  typename Vec<T, V>::raw_t raw[kRunFwd + KT - 1];  // raw[j] = x[t0 - (KT-1) + j]
#pragma unroll
  for (int j = 0; j < kRunFwd + KT - 1; ++j) raw[j] = load_x<T, V>(d, x, hist, b, t0 - (KT - 1) + j, c0, rev);
#pragma unroll
  for (int k = 0; k < KT - 1; ++k) Vec<T, V>::unpack(raw[k], win[k + 1]);
  const int t1 = min(t0 + kRunFwd, d.T);
#pragma unroll
  for (int it = 0; it < kRunFwd; ++it) {
    const int t = t0 + it;
#pragma unroll
    for (int k = 0; k < KT - 1; ++k)
#pragma unroll
      for (int i = 0; i < V; ++i) win[k][i] = win[k + 1][i];
    Vec<T, V>::unpack(raw[KT - 1 + it], win[KT - 1]);
    float acc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = bs[i];
#pragma unroll
    for (int k = 0; k < KT; ++k) fma_vec<V>(wt[k], win[k], acc);
    if (d.act) {
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] = silu(acc[i]);
    }
    if (t < t1) Vec<T, V>::store(yb + ((size_t)b * d.T + at_time(d, rev, t)) * ys, acc);
  }
}

// The K-1 inputs a later window continues from (causal_conv1d_history): the tail of [history; x].
template <class T>
__global__ void k_conv_history(ConvDims d, const T* __restrict__ x, const T* __restrict__ hist, T* __restrict__ out) {
  const size_t n = (size_t)d.B * (d.K - 1) * d.C;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = i % d.C, j = (i / d.C) % (d.K - 1), b = i / ((size_t)d.C * (d.K - 1));
    const int t = d.T - (d.K - 1) + j;
    float v = 0.0f;
    if (t >= 0) v = m3::ldf(x, ((size_t)b * d.T + t) * d.xs + c);
    else if (hist && t + (d.K - 1) >= 0) v = m3::ldf(hist, ((size_t)b * (d.K - 1) + (t + d.K - 1)) * d.C + c);
    m3::stf(out, i, v);
  }
}

// Backward: g = dy * act'(pre) with pre recomputed; dx[t] = sum_delay w[K-1-delay] g[t+delay];
// per-block partial sums of dw[k] = sum g[t] x[t-(K-1-k)] and dbias = sum g[t].
template <class T, int V, int KT>
// two blocks per SM: the kernel is bound by instruction issue and needs the warps
__global__ void __launch_bounds__(kLanesT* kLanesC, 2)
    k_conv_bwd(ConvDims d, const T* __restrict__ x, const T* __restrict__ hist, const float* __restrict__ w,
               const float* __restrict__ bias, const T* __restrict__ dy, const T* __restrict__ dy2, T* __restrict__ dx,
               T* __restrict__ dhist, float* __restrict__ part) {
  __shared__ float red[kLanesT][V][kLanesC + 1];  // [time lane][element of the vector][channel lane]: conflict-free
  const int c0 = (blockIdx.x * kLanesC + threadIdx.x) * V;
  const int b = blockIdx.z;
  const int t0 = (blockIdx.y * kLanesT + threadIdx.y) * kRunBwd;
  const bool active = c0 < d.C && t0 < d.T;
  const int pad = KT - d.K;
  float pw[KT][V], pb[V];
#pragma unroll
  for (int k = 0; k < KT; ++k)
#pragma unroll
    for (int i = 0; i < V; ++i) pw[k][i] = 0.0f;
#pragma unroll
  for (int i = 0; i < V; ++i) pb[i] = 0.0f;
  if (active) {
    float wt[KT][V], bs[V], win[KT][V], gw[KT][V];  // gw[j] = g[s - (KT-1) + j] after step s
#pragma unroll
    for (int k = 0; k < KT; ++k)
#pragma unroll
      for (int i = 0; i < V; ++i) {
        wt[k][i] = (k >= pad) ? w[(size_t)(k - pad) * d.C + c0 + i] : 0.0f;
        gw[k][i] = 0.0f;
      }
#pragma unroll
    for (int i = 0; i < V; ++i) bs[i] = bias ? bias[c0 + i] : 0.0f;
    // Every row this thread needs (its run, KT-1 steps behind for the taps and KT-1 ahead for the
    // look-ahead of dx) is requested before the first one is used.
    long long ys;
    const T* gb = out_band<const T>(d, dy, dy2, c0, &ys);
    const bool rev = walks_backwards(d, c0);
    typename Vec<T, V>::raw_t rx[kRunBwd + 2 * (KT - 1)], rg[kRunBwd + KT - 1];  // rx[j] = x[t0-(KT-1)+j], rg[j] = dy[t0+j]
#pragma unroll
    for (int j = 0; j < kRunBwd + 2 * (KT - 1); ++j) rx[j] = load_x<T, V>(d, x, hist, b, t0 - (KT - 1) + j, c0, rev);
#pragma unroll
    for (int j = 0; j < kRunBwd + KT - 1; ++j)
      rg[j] = (t0 + j < d.T) ? Vec<T, V>::load_raw(gb + ((size_t)b * d.T + at_time(d, rev, t0 + j)) * ys) : Vec<T, V>::zero_raw();
#pragma unroll
    for (int k = 0; k < KT - 1; ++k) Vec<T, V>::unpack(rx[k], win[k + 1]);
    const int t1 = min(t0 + kRunBwd, d.T);
    // s walks the run plus KT-1 steps of look-ahead; dx[s-(KT-1)] is complete once g[s] is known.
    const int emit_from = (t0 == 0 && dhist) ? -(d.K - 1) : t0;
#pragma unroll
    for (int it = 0; it < kRunBwd + KT - 1; ++it) {
      const int s = t0 + it;
#pragma unroll
      for (int k = 0; k < KT - 1; ++k)
#pragma unroll
        for (int i = 0; i < V; ++i) {
          win[k][i] = win[k + 1][i];
          gw[k][i] = gw[k + 1][i];
        }
      {
        float gy[V], acc[V];
        Vec<T, V>::unpack(rx[KT - 1 + it], win[KT - 1]);
        Vec<T, V>::unpack(rg[it], gy);
        const bool valid = s < d.T;
        const float own = s < t1 ? 1.0f : 0.0f;  // own steps feed the parameter gradients, each exactly once
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] = bs[i];
#pragma unroll
        for (int k = 0; k < KT; ++k) fma_vec<V>(wt[k], win[k], acc);
#pragma unroll
        for (int i = 0; i < V; ++i) gw[KT - 1][i] = valid ? (d.act ? gy[i] * silu_grad(acc[i]) : gy[i]) : 0.0f;
        float og[V];
#pragma unroll
        for (int i = 0; i < V; ++i) og[i] = own * gw[KT - 1][i];
#pragma unroll
        for (int k = 0; k < KT; ++k) fma_vec<V>(og, win[k], pw[k]);
#pragma unroll
        for (int i = 0; i < V; ++i) pb[i] += og[i];
      }
      const int te = s - (KT - 1);  // dx[te] = sum_delay w[KT-1-delay] g[te+delay] = sum_j w[KT-1-j] gw[j]
      if (te >= emit_from && te < t1) {
        float o[V];
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] = 0.0f;
#pragma unroll
        for (int j = 0; j < KT; ++j) fma_vec<V>(wt[KT - 1 - j], gw[j], o);
        if (te >= 0) {
          if (dx) Vec<T, V>::store(dx + ((size_t)b * d.T + at_time(d, rev, te)) * d.xs + c0, o);
        } else {
          Vec<T, V>::store(dhist + ((size_t)b * (d.K - 1) + (te + d.K - 1)) * d.C + c0, o);
        }
      }
    }
  }
  if (!part) return;
  // Block partials: sum the kLanesT time lanes in a fixed order, one (tap | bias) slice at a time.
  const size_t blk = (size_t)blockIdx.z * gridDim.y + blockIdx.y;
#pragma unroll
  for (int k = 0; k <= KT; ++k) {
    if (k < pad) continue;  // a padding tap has no gradient
    __syncthreads();
#pragma unroll
    for (int i = 0; i < V; ++i) red[threadIdx.y][i][threadIdx.x] = (k == KT) ? pb[i] : pw[k < KT ? k : 0][i];
    __syncthreads();
    if (threadIdx.y == 0 && c0 < d.C) {
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float s = 0.0f;
#pragma unroll
        for (int ty = 0; ty < kLanesT; ++ty) s += red[ty][i][threadIdx.x];
        part[(blk * (d.K + 1) + (k - pad)) * d.C + c0 + i] = s;
      }
    }
  }
}

int check(m3_ctx* ctx, const m3_conv_desc* c, ConvDims* d) {
  if (!ctx || !c) return M3_ERR_NULL;
  if (c->batch <= 0 || c->seq < 0 || c->channels <= 0)
    return m3::fail(ctx, M3_ERR_SHAPE, "conv extents must be positive (batch %d seq %d channels %d)", c->batch, c->seq, c->channels);
  if (c->kernel_size < 1 || c->kernel_size > kMaxTaps)
    return m3::fail(ctx, M3_ERR_UNSUPPORTED, "kernel_size %d outside [1, %d]", c->kernel_size, kMaxTaps);
  if (c->dtype != M3_F32 && c->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", c->dtype);
  if (!c->x || !c->weight) return m3::fail(ctx, M3_ERR_NULL, "x and weight are required");
  d->B = c->batch; d->T = c->seq; d->C = c->channels; d->K = c->kernel_size;
  d->xs = c->x_stride ? c->x_stride : c->channels;
  d->ys = c->y_stride ? c->y_stride : c->channels;
  if (d->xs < c->channels || d->ys < (c->split > 0 ? c->split : c->channels))
    return m3::fail(ctx, M3_ERR_SHAPE, "row strides below the channel count");
  d->act = c->activation ? 1 : 0;
  d->nrev = c->n_reversed;
  if (c->n_reversed < 0 || c->n_reversed > 4) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "at most 4 reversed channel ranges");
  for (int i = 0; i < 4; ++i) {
    d->rev_lo[i] = i < c->n_reversed ? c->reversed_lo[i] : 0;
    d->rev_hi[i] = i < c->n_reversed ? c->reversed_hi[i] : 0;
    if (i < c->n_reversed && (d->rev_lo[i] < 0 || d->rev_hi[i] > c->channels || d->rev_lo[i] > d->rev_hi[i]))
      return m3::fail(ctx, M3_ERR_SHAPE, "reversed channel range %d outside [0, channels]", i);
  }
  if (c->n_reversed > 0 && c->history) return m3::fail(ctx, M3_ERR_CONFIG, "a right-to-left channel has no history to continue from");
  d->split = c->split;
  d->y2s = 0;
  if (c->split < 0 || c->split >= c->channels) return m3::fail(ctx, M3_ERR_SHAPE, "split %d outside [0, channels)", c->split);
  if (c->split > 0) {
    d->y2s = c->y2_stride ? c->y2_stride : c->channels - c->split;
    if (d->y2s < c->channels - c->split) return m3::fail(ctx, M3_ERR_SHAPE, "y2_stride below the second band's width");
  }
  return M3_OK;
}

bool vector_ok(const ConvDims& d, int V, int es, std::initializer_list<const void*> ptrs) {
  if (d.C % V || d.xs % V || d.ys % V || d.split % V || d.y2s % V) return false;
  for (int i = 0; i < d.nrev; ++i)
    if (d.rev_lo[i] % V || d.rev_hi[i] % V) return false;  // a vector must not straddle a direction change
  for (const void* p : ptrs)
    if (p && (reinterpret_cast<uintptr_t>(p) % (size_t)(V * es))) return false;
  return true;
}

template <class T, int V>
cudaError_t fwd_launch(cudaStream_t st, const ConvDims& d, const m3_conv_desc& c, void* y) {
  T* y2 = static_cast<T*>(c.y2);
  const dim3 block(kLanesC, kLanesT);
  const dim3 grid((d.C / V + kLanesC - 1) / kLanesC, (d.T + kLanesT * kRunFwd - 1) / (kLanesT * kRunFwd), d.B);
  const T* x = static_cast<const T*>(c.x);
  const T* h = static_cast<const T*>(c.history);
  if (d.K <= 2) k_conv_fwd<T, V, 2><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<T*>(y), y2);
  else if (d.K <= 4) k_conv_fwd<T, V, 4><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<T*>(y), y2);
  else k_conv_fwd<T, V, kMaxTaps><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<T*>(y), y2);
  return cudaGetLastError();
}

template <class T, int V>
cudaError_t bwd_launch(cudaStream_t st, const ConvDims& d, const m3_conv_desc& c, const void* dy, void* dx, void* dhist,
                       float* part, dim3* grid_out) {
  const dim3 block(kLanesC, kLanesT);
  const dim3 grid((d.C / V + kLanesC - 1) / kLanesC, (d.T + kLanesT * kRunBwd - 1) / (kLanesT * kRunBwd), d.B);
  *grid_out = grid;
  const T* x = static_cast<const T*>(c.x);
  const T* h = static_cast<const T*>(c.history);
  if (d.K <= 2)
    k_conv_bwd<T, V, 2><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<const T*>(dy), static_cast<const T*>(c.dy2), static_cast<T*>(dx),
                                                 static_cast<T*>(dhist), part);
  else if (d.K <= 4)
    k_conv_bwd<T, V, 4><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<const T*>(dy), static_cast<const T*>(c.dy2), static_cast<T*>(dx),
                                                 static_cast<T*>(dhist), part);
  else
    k_conv_bwd<T, V, kMaxTaps><<<grid, block, 0, st>>>(d, x, h, c.weight, c.bias, static_cast<const T*>(dy),
                                                        static_cast<const T*>(c.dy2), static_cast<T*>(dx), static_cast<T*>(dhist), part);
  return cudaGetLastError();
}

}  // namespace

extern "C" {

int m3_conv_forward(m3_ctx* ctx, const m3_conv_desc* c, void* y, void* new_history) {
  ConvDims d;
  const int rc = check(ctx, c, &d);
  if (rc != M3_OK) return rc;
  if (!y) return m3::fail(ctx, M3_ERR_NULL, "y is required");
  if (c->split > 0 && !c->y2) return m3::fail(ctx, M3_ERR_NULL, "split needs y2");
  if (c->n_reversed > 0 && new_history) return m3::fail(ctx, M3_ERR_CONFIG, "a right-to-left channel carries no history");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  cudaError_t e = cudaSuccess;
  if (d.T > 0) {
    if (c->dtype == M3_BF16) {
      e = vector_ok(d, 4, 2, {c->x, c->history, y, c->y2}) ? fwd_launch<__nv_bfloat16, 4>(ctx->stream, d, *c, y)
                                                     : fwd_launch<__nv_bfloat16, 1>(ctx->stream, d, *c, y);
    } else {
      e = vector_ok(d, 4, 4, {c->x, c->history, y, c->y2}) ? fwd_launch<float, 4>(ctx->stream, d, *c, y)
                                                     : fwd_launch<float, 1>(ctx->stream, d, *c, y);
    }
    if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "conv forward");
    ctx->launches += 1;
  }
  if (new_history && d.K > 1) {
    const size_t n = (size_t)d.B * (d.K - 1) * d.C;
    const int blocks = (int)((n + 255) / 256 < 1024 ? (n + 255) / 256 : 1024);
    if (c->dtype == M3_BF16)
      k_conv_history<__nv_bfloat16><<<blocks, 256, 0, ctx->stream>>>(d, static_cast<const __nv_bfloat16*>(c->x),
                                                                      static_cast<const __nv_bfloat16*>(c->history),
                                                                      static_cast<__nv_bfloat16*>(new_history));
    else
      k_conv_history<float><<<blocks, 256, 0, ctx->stream>>>(d, static_cast<const float*>(c->x),
                                                              static_cast<const float*>(c->history),
                                                              static_cast<float*>(new_history));
    M3_CUDA(ctx, cudaGetLastError());
    ctx->launches += 1;
  }
  return M3_OK;
}

int m3_conv_backward(m3_ctx* ctx, const m3_conv_desc* c, const void* dy, void* dx, float* dweight, float* dbias,
                     void* dhistory) {
  ConvDims d;
  const int rc = check(ctx, c, &d);
  if (rc != M3_OK) return rc;
  if (!dy) return m3::fail(ctx, M3_ERR_NULL, "dy is required");
  if (c->split > 0 && !c->dy2) return m3::fail(ctx, M3_ERR_NULL, "split needs dy2");
  if (dhistory && !c->history) return m3::fail(ctx, M3_ERR_NULL, "dhistory without a history");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const bool want_par = dweight || (dbias && c->bias);
  if (d.T == 0) {
    if (dweight) M3_CUDA(ctx, cudaMemsetAsync(dweight, 0, (size_t)d.K * d.C * sizeof(float), ctx->stream));
    if (dbias) M3_CUDA(ctx, cudaMemsetAsync(dbias, 0, (size_t)d.C * sizeof(float), ctx->stream));
    if (dhistory) M3_CUDA(ctx, cudaMemsetAsync(dhistory, 0, (size_t)d.B * (d.K - 1) * d.C * (c->dtype == M3_BF16 ? 2 : 4), ctx->stream));
    return M3_OK;
  }
  const int nblk = d.B * ((d.T + kLanesT * kRunBwd - 1) / (kLanesT * kRunBwd));
  float* part = nullptr;
  if (want_par)
    M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&part), (size_t)nblk * (d.K + 1) * d.C * sizeof(float), ctx->stream));
  dim3 grid;
  cudaError_t e;
  if (c->dtype == M3_BF16) {
    e = vector_ok(d, 4, 2, {c->x, c->history, dy, c->dy2, dx, dhistory})
            ? bwd_launch<__nv_bfloat16, 4>(ctx->stream, d, *c, dy, dx, dhistory, part, &grid)
            : bwd_launch<__nv_bfloat16, 1>(ctx->stream, d, *c, dy, dx, dhistory, part, &grid);
  } else {
    e = vector_ok(d, 4, 4, {c->x, c->history, dy, c->dy2, dx, dhistory})
            ? bwd_launch<float, 4>(ctx->stream, d, *c, dy, dx, dhistory, part, &grid)
            : bwd_launch<float, 1>(ctx->stream, d, *c, dy, dx, dhistory, part, &grid);
  }
  ctx->launches += 1;
  if (e == cudaSuccess && want_par) {
    const size_t n = (size_t)(d.K + 1) * d.C;  // a block's partial: K taps of C channels, then the bias
    if (dweight) e = m3::column_sums(ctx->stream, part, nblk, n, d.K * d.C, dweight);
    if (e == cudaSuccess && dbias && c->bias) e = m3::column_sums(ctx->stream, part + (size_t)d.K * d.C, nblk, n, d.C, dbias);
  }
  // a convolution without a bias has no bias gradient: the buffer, if one was passed, reads zero (as it
  // does for an empty sequence) rather than whatever it held
  if (e == cudaSuccess && dbias && !c->bias) e = cudaMemsetAsync(dbias, 0, (size_t)d.C * sizeof(float), ctx->stream);
  if (e == cudaSuccess && want_par) {
    ctx->launches += (dweight ? 1 : 0) + ((dbias && c->bias) ? 1 : 0);
  }
  cudaError_t e2 = part ? cudaFreeAsync(part, ctx->stream) : cudaSuccess;
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "conv backward");
  if (e2 != cudaSuccess) return m3::cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

}  // extern "C"
