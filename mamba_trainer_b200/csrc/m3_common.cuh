// Shared device helpers of the generic (CUDA-core, fp32) kernel family.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace m3 {

constexpr float kLogDecayFloor = -60.0f;   // LOG_DECAY_FLOOR, src/ssm/scan.rs:54-57
constexpr float kTwoPi = 6.283185307179586f;

// Extents of one scan call.  L is the chunk actually used, C the number of chunks,
// Tp = C * L the padded length, NH = N / 2 planes when rotational (else 0).
struct Dims {
  int B, T, H, P, N, R, L, C, Tp, NH;
  int disc;      // m3_discretization
  int rot;       // 1 when rotational
  int LR;        // L * R rows per chunk
  int raw;       // 1: a, g, w come from the caller (the ssd_chunked form)
  int rev;       // the last `rev` heads walk time right to left (bidirectional mixer)
};

// Token-head index (row of a [B, T, H, ...] tensor) of scan position t of head h: heads that
// walk right to left (src/models/mamba3.rs:352-370, :548-556) see position t at time T-1-t.
__host__ __device__ __forceinline__ size_t tok_index(const Dims& d, int b, int t, int h) {
  const int tm = (h >= d.H - d.rev) ? d.T - 1 - t : t;
  return ((size_t)b * d.T + tm) * d.H + h;
}

__device__ __forceinline__ float ldf(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, size_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// exp(clamp(d, floor, 0)) - every log-decay difference goes through this.
__device__ __forceinline__ float exp_decay(float d) {
  return expf(fminf(fmaxf(d, kLogDecayFloor), 0.0f));
}
// Derivative of the clamp: one strictly inside (floor, 0), zero elsewhere
// (src/tensor/ops/fused.rs:2080-2138).
__device__ __forceinline__ float clamp_inside(float d) {
  return (d > kLogDecayFloor && d < 0.0f) ? 1.0f : 0.0f;
}
// x - round(x / 2pi) * 2pi, src/tensor/ops/elemwise.rs:347-349.
__device__ __forceinline__ float wrap_angle(float x) {
  return x - rintf(x / kTwoPi) * kTwoPi;
}

// lambda of a token: the tensor when learned, else the constant of
// Discretization::fixed_lambda (src/ssm/config.rs:30-36).
template <class TIn>
__device__ __forceinline__ float lambda_at(const TIn* lam, int disc, size_t i) {
  if (disc == 0) return 1.0f;
  if (disc == 1) return 0.5f;
  return ldf(lam, i);
}

// ---------------------------------------------------------------------------
// 64x64 block GEMM on CUDA cores, 256 threads, 4x4 outputs per thread.
//   acc[i][j] += sum_{k in [k_begin, k_end)} A(m0 + ty*4+i, k) * B(k, n0 + tx*4+j)
// fa(m, k) / fb(k, n) are callables returning float and must themselves return 0
// outside the operand's extents.  AKF / BKF say whether the operand is contiguous
// along k (true) or along m / n (false); it only picks the load order.
// sA, sB: shared scratch of 16 * 68 floats each.
// ---------------------------------------------------------------------------
constexpr int kGemmTile = 64;
constexpr int kGemmBK = 16;
constexpr int kGemmLd = 68;
constexpr int kGemmSmemFloats = 2 * kGemmBK * kGemmLd;

template <bool AKF, bool BKF, class FA, class FB>
__device__ __forceinline__ void gemm_tile(float (&acc)[4][4], int m0, int n0, int k_begin,
                                          int k_end, FA fa, FB fb, float* sA, float* sB) {
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  for (int k0 = k_begin; k0 < k_end; k0 += kGemmBK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int e = tid + i * 256;
      int m, k;
      if (AKF) { k = e & 15; m = e >> 4; } else { m = e & 63; k = e >> 6; }
      const int kk = k0 + k;
      sA[k * kGemmLd + m] = (kk < k_end) ? fa(m0 + m, kk) : 0.0f;
      int n, k2;
      if (BKF) { k2 = e & 15; n = e >> 4; } else { n = e & 63; k2 = e >> 6; }
      const int kk2 = k0 + k2;
      sB[k2 * kGemmLd + n] = (kk2 < k_end) ? fb(kk2, n0 + n) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < kGemmBK; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&sA[k * kGemmLd + ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&sB[k * kGemmLd + tx * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
      const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
}

__device__ __forceinline__ void zero_acc(float (&acc)[4][4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
}

// Sum over the 256 threads of a block; red: 8 floats of shared scratch.
__device__ __forceinline__ float block_sum_256(float v, float* red) {
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

}  // namespace m3
