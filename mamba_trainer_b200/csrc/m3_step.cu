// One decoding step of the Mamba-3 recurrence (the reference's mamba3_step,
// src/ssm/scan.rs:649-712, with its three fused helpers ssm_coefficients / ssm_angle /
// ssm_state_update, src/tensor/ops/fused.rs:1338-1806, folded into one launch):
//   alpha = exp(dt A), beta = (1 - lambda) dt alpha, gamma = lambda dt
//   phi   = wrap(angle + dt theta);  B^, C^ = B, C rotated by -phi
//   u     = sum_r x^(r) (x) B^^(r);  h' = alpha h + beta last_u + gamma u
//   y^(r) = C^^(r) . h' (over d_state) + D x^(r)
// One CTA per (batch, head); the fp32 state streams through once (read h and last_u, write h'
// and u), which is all the traffic that matters: the step is HBM bound.
#include "m3_internal.h"

namespace m3 {

constexpr int kStepMaxRank = 8;

template <class T>
__global__ void __launch_bounds__(256) k_step(m3_step_desc d, m3_step_out o) {
  extern __shared__ float sm[];
  const int P = d.head_dim, N = d.d_state, R = d.rank, NH = N / 2;
  float* s_b = sm;               // [R][N] rotated B
  float* s_c = s_b + R * N;      // [R][N] rotated C
  float* s_x = s_c + R * N;      // [R][P]
  const int bh = blockIdx.x, h = bh % d.heads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* x = static_cast<const T*>(d.x) + (size_t)bh * P * R;
  const T* bm = static_cast<const T*>(d.b) + (size_t)bh * N * R;
  const T* cm = static_cast<const T*>(d.c) + (size_t)bh * N * R;
  const float dt = ldf(static_cast<const T*>(d.dt), bh);
  const float lam = lambda_at(static_cast<const T*>(d.lambda), d.discretization, bh);
  const float alpha = expf(dt * -expf(d.a_log[h]));
  const float beta = (1.0f - lam) * dt * alpha, gamma = lam * dt;
  const bool rot = d.dynamics == M3_ROTATIONAL;
  if (rot) {
    const T* th = static_cast<const T*>(d.theta) + (size_t)bh * NH;
    for (int m = tid; m < NH; m += 256) {
      const float a0 = d.angle ? d.angle[(size_t)bh * NH + m] : 0.0f;
      const float ph = wrap_angle(a0 + dt * ldf(th, m));
      if (o.angle) o.angle[(size_t)bh * NH + m] = ph;
      float sn, cs;
      sincosf(ph, &sn, &cs);
      for (int r = 0; r < R; ++r) {
        const float b1 = ldf(bm, (size_t)m * R + r), b2 = ldf(bm, (size_t)(m + NH) * R + r);
        const float c1 = ldf(cm, (size_t)m * R + r), c2 = ldf(cm, (size_t)(m + NH) * R + r);
        s_b[r * N + m] = b1 * cs + b2 * sn;  s_b[r * N + m + NH] = b2 * cs - b1 * sn;
        s_c[r * N + m] = c1 * cs + c2 * sn;  s_c[r * N + m + NH] = c2 * cs - c1 * sn;
      }
    }
  } else {
    for (int e = tid; e < N * R; e += 256) {
      const int n = e / R, r = e % R;
      s_b[r * N + n] = ldf(bm, e);
      s_c[r * N + n] = ldf(cm, e);
    }
  }
  for (int e = tid; e < P * R; e += 256) s_x[(e % R) * P + e / R] = ldf(x, e);
  __syncthreads();
  const float dsk = d.d_skip ? d.d_skip[h] : 0.0f;
  const float* hin = d.h + (size_t)bh * P * N;
  const float* uin = d.last_u + (size_t)bh * P * N;
  float* hout = o.h + (size_t)bh * P * N;
  float* uout = o.last_u + (size_t)bh * P * N;
  T* y = static_cast<T*>(o.y) + (size_t)bh * P * R;
  // 128-bit path: each lane owns 4 consecutive state columns per pass; it needs rows of whole float4s
  // and 16-byte aligned state tensors (a caller may hand over an offset view), else the scalar loop
  const bool vec4 = (N & 3) == 0 &&
                    !((reinterpret_cast<uintptr_t>(d.h) | reinterpret_cast<uintptr_t>(d.last_u) |
                       reinterpret_cast<uintptr_t>(o.h) | reinterpret_cast<uintptr_t>(o.last_u)) & 15);
  if (vec4) {
    for (int p = warp; p < P; p += 8) {
      float acc[kStepMaxRank];
#pragma unroll
      for (int r = 0; r < kStepMaxRank; ++r) acc[r] = 0.0f;
      for (int n = 4 * lane; n < N; n += 128) {
        const size_t i = (size_t)p * N + n;
        const float4 hv = __ldg(reinterpret_cast<const float4*>(hin + i));
        const float4 uv = __ldg(reinterpret_cast<const float4*>(uin + i));
        float u[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int r = 0; r < R; ++r) {
          const float xv = s_x[r * P + p];
          const float4 bv = *reinterpret_cast<const float4*>(&s_b[r * N + n]);
          u[0] += xv * bv.x; u[1] += xv * bv.y; u[2] += xv * bv.z; u[3] += xv * bv.w;
        }
        float4 hn;
        hn.x = alpha * hv.x + beta * uv.x + gamma * u[0];
        hn.y = alpha * hv.y + beta * uv.y + gamma * u[1];
        hn.z = alpha * hv.z + beta * uv.z + gamma * u[2];
        hn.w = alpha * hv.w + beta * uv.w + gamma * u[3];
        *reinterpret_cast<float4*>(hout + i) = hn;
        *reinterpret_cast<float4*>(uout + i) = make_float4(u[0], u[1], u[2], u[3]);
#pragma unroll
        for (int r = 0; r < kStepMaxRank; ++r)
          if (r < R) {
            const float4 cv = *reinterpret_cast<const float4*>(&s_c[r * N + n]);
            acc[r] += cv.x * hn.x + cv.y * hn.y + cv.z * hn.z + cv.w * hn.w;
          }
      }
#pragma unroll
      for (int r = 0; r < kStepMaxRank; ++r) {
        if (r < R) {
          float v = acc[r];
#pragma unroll
          for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
          if (lane == 0) stf(y, (size_t)p * R + r, v + dsk * s_x[r * P + p]);
        }
      }
    }
    return;
  }
  for (int p = warp; p < P; p += 8) {
    float acc[kStepMaxRank];
#pragma unroll
    for (int r = 0; r < kStepMaxRank; ++r) acc[r] = 0.0f;
    for (int n = lane; n < N; n += 32) {
      float u = 0.0f;
      for (int r = 0; r < R; ++r) u += s_x[r * P + p] * s_b[r * N + n];
      const size_t i = (size_t)p * N + n;
      const float hn = alpha * hin[i] + beta * uin[i] + gamma * u;
      hout[i] = hn;
      uout[i] = u;
#pragma unroll
      for (int r = 0; r < kStepMaxRank; ++r)
        if (r < R) acc[r] += s_c[r * N + n] * hn;
    }
#pragma unroll
    for (int r = 0; r < kStepMaxRank; ++r) {
      if (r < R) {
        float v = acc[r];
#pragma unroll
        for (int s = 16; s > 0; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
        if (lane == 0) stf(y, (size_t)p * R + r, v + dsk * s_x[r * P + p]);
      }
    }
  }
}

}  // namespace m3

extern "C" int m3_step_forward(m3_ctx* ctx, const m3_step_desc* d, const m3_step_out* o) {
  if (!ctx) return M3_ERR_NULL;
  if (!d || !o) return m3::fail(ctx, M3_ERR_NULL, "descriptor and outputs are required");
  if (d->batch <= 0 || d->heads <= 0 || d->head_dim <= 0 || d->d_state <= 0 || d->rank <= 0)
    return m3::fail(ctx, M3_ERR_SHAPE, "extents must be positive");
  if (d->rank > m3::kStepMaxRank) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "rank %d > %d in the decode step", d->rank, m3::kStepMaxRank);
  if (d->dtype != M3_F32 && d->dtype != M3_BF16) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", d->dtype);
  if (d->dynamics == M3_ROTATIONAL && (d->d_state % 2)) return m3::fail(ctx, M3_ERR_CONFIG, "rotational dynamics require an even d_state");
  if (!d->x || !d->b || !d->c || !d->dt || !d->a_log || !d->h || !d->last_u || !o->y || !o->h || !o->last_u)
    return m3::fail(ctx, M3_ERR_NULL, "x, b, c, dt, a_log, the state and the outputs are required");
  if (d->discretization == M3_LEARNED_TRAPEZOID && !d->lambda) return m3::fail(ctx, M3_ERR_NULL, "learned trapezoid needs lambda");
  if (d->dynamics == M3_ROTATIONAL && !d->theta) return m3::fail(ctx, M3_ERR_NULL, "rotational dynamics need theta");
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "cudaSetDevice");
  const size_t smem = sizeof(float) * ((size_t)2 * d->rank * d->d_state + (size_t)d->rank * d->head_dim);
  if (smem > 200 * 1024) return m3::fail(ctx, M3_ERR_UNSUPPORTED, "decode step: rank * (2 d_state + head_dim) too large");
  const int grid = d->batch * d->heads;
  if (d->dtype == M3_BF16) {
    e = cudaFuncSetAttribute(m3::k_step<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) m3::k_step<__nv_bfloat16><<<grid, 256, smem, ctx->stream>>>(*d, *o);
  } else {
    e = cudaFuncSetAttribute(m3::k_step<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) m3::k_step<float><<<grid, 256, smem, ctx->stream>>>(*d, *o);
  }
  if (e == cudaSuccess) e = cudaGetLastError();
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "decode step");
  ctx->launches += 1;
  return M3_OK;
}
