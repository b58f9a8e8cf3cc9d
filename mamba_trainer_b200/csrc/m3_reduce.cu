// Deterministic column sums of per-block partial results: out[c] (+)= sum_t part[t * stride + c].
// Used by every backward pass that produces parameter gradients: the terms of a column are cut into
// 32 interleaved runs, each run is summed serially and the 32 run totals are added in run order, so
// the result does not depend on scheduling (no atomics).
#include "m3_internal.h"

namespace m3 {
namespace {

__global__ void __launch_bounds__(1024) k_column_sums(const float* __restrict__ part, int nterms, size_t stride, int ncols,
                                                     float* __restrict__ out, int accumulate, size_t part_group_stride,
                                                     size_t out_group_stride) {
  __shared__ float red[32][33];
  const int c = blockIdx.x * 32 + threadIdx.x;
  const float* p = part + (size_t)blockIdx.y * part_group_stride;
  float s = 0.0f;
  if (c < ncols)
    for (int t = threadIdx.y; t < nterms; t += 32) s += p[(size_t)t * stride + c];
  red[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && c < ncols) {
    float* o = out + (size_t)blockIdx.y * out_group_stride + c;
    float tot = accumulate ? *o : 0.0f;
#pragma unroll
    for (int i = 0; i < 32; ++i) tot += red[i][threadIdx.x];
    *o = tot;
  }
}

}  // namespace

cudaError_t column_sums(cudaStream_t st, const float* part, int nterms, size_t stride, int ncols, float* out,
                        bool accumulate, int groups, size_t part_group_stride, size_t out_group_stride) {
  if (ncols <= 0 || groups <= 0) return cudaSuccess;
  const dim3 grid((ncols + 31) / 32, groups), block(32, 32);
  k_column_sums<<<grid, block, 0, st>>>(part, nterms, stride, ncols, out, accumulate ? 1 : 0, part_group_stride,
                                        out_group_stride);
  return cudaGetLastError();
}

}  // namespace m3
