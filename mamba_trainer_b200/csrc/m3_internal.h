// Host-side declarations shared by the translation units of libm3scan.
#pragma once
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/m3scan.h"
#include "m3_common.cuh"

// A context: one device, one stream, a launch counter and the last error message.
struct m3_ctx {
  int device = 0;
  cudaStream_t stream = nullptr;
  bool own_stream = false;
  uint64_t launches = 0;
  // Flag raised by a kernel whose bounded wait gave up.  One int of page-locked host memory mapped
  // into the device's address space: kernels store through `dev_err`, the host reads `err_host`
  // without a copy - at m3_sync and on entry to every scan call.
  int* dev_err = nullptr;
  volatile int* err_host = nullptr;
  uint32_t wait_limit = 0;          // iteration limit of the kernels' bounded waits; 0 = the default
  cudaMemPool_t pool = nullptr;     // this context's own scratch pool (freed memory is kept for reuse)
  bool no_scratch = false;          // set for the span of a call that must not allocate
  char err[512] = {0};
};

namespace m3 {
// Scratch for a call, from the context's own stream-ordered pool, ordered on `st`.
inline cudaError_t scratch_alloc(m3_ctx* ctx, void** out, size_t bytes, cudaStream_t st) {
  return ctx->pool ? cudaMallocFromPoolAsync(out, bytes, ctx->pool, st) : cudaMallocAsync(out, bytes, st);
}
// Report (and clear) a wait that gave up in an earlier call; M3_OK if none did.
int take_device_flag(m3_ctx* ctx, const char* when);
}  // namespace m3

namespace m3 {

// Record a failure message on the context (if any) and return `code`.
int fail(m3_ctx* ctx, int code, const char* fmt, ...);
int cuda_fail(m3_ctx* ctx, cudaError_t e, const char* what);
// Validate a descriptor and derive the extents the kernels use.
int make_dims(m3_ctx* ctx, const m3_scan_desc& s, Dims* out);

// Scratch of the generic family, all float, head-major (bh = b * H + h) so that the
// rows of one chunk are contiguous.  Row rho = t * R + r.
struct GenericWs {
  float* Xh;     // [BH, Tp*R, P]   x, ranks as rows
  float* Bh;     // [BH, Tp*R, N]   rotated B
  float* Ch;     // [BH, Tp*R, N]   rotated C
  float* acum;   // [BH, Tp]        in-chunk cumulative log decay
  float* g;      // [BH, Tp]        diagonal weight
  float* w;      // [BH, Tp]        off-diagonal weight
  float* phi;    // [BH, Tp, NH]    wrapped cumulative angle
  float* abase;  // [BH, C, NH]     angle entering each chunk
  float* Hs;     // [BH, C+1, P, N] state entering chunk k; slot C = final state
};

// Extra scratch of the generic backward.
struct GenericBwdWs {
  float* dXh;    // [BH, Tp*R, P]
  float* dBh;    // [BH, Tp*R, N]
  float* dCh;    // [BH, Tp*R, N]
  float* dHs;    // [BH, C, P, N]   local dH, then dS_k in place
  float* dBand;  // [BH, C, L, L]
  float* dcd;    // [BH, C]
  float* dac;    // [BH, Tp]  d acum partial from the carry-out term
  float* dws;    // [BH, Tp]  dw from the chunk-state term
  float* dast;   // [BH, Tp]  d acum from the chunk-state term (sigma w q inside)
  float* da;     // [BH, Tp]
  float* dg;     // [BH, Tp]
  float* dw;     // [BH, Tp]
  float* dphi;   // [BH, Tp, NH]  then dstep in place
  float* dpsum;  // [BH, C, NH]
  float* ddt_rot;// [BH, Tp]
  float* partA;  // [BH, C]   partial sums for d a_log
  float* partD;  // [BH, C]   partial sums for d d_skip
  float* ip0;    // [BH]      <dH_0, last_u0>
};

size_t generic_ws_layout(const Dims& d, GenericWs* ws, char* base);
size_t generic_bwd_ws_layout(const Dims& d, GenericBwdWs* ws, char* base);

cudaError_t generic_forward(cudaStream_t st, const Dims& d, const m3_scan_desc& desc,
                            const m3_scan_out& out, const GenericWs& ws, uint64_t* launches);
cudaError_t generic_backward(cudaStream_t st, const Dims& d, const m3_scan_desc& desc,
                             const GenericWs& ws, const GenericBwdWs& bw,
                             const m3_scan_bwd_in& in, uint32_t mask,
                             const m3_scan_grads& grads, uint64_t* launches);

cudaError_t finalize_scalars(cudaStream_t st, const Dims& d, const m3_scan_desc& desc, const GenericBwdWs& bw,
                             void* ddt, void* dlam, float* dalog, float* ddsk, uint64_t* launches);

// out[g][c] (+)= sum_{t < nterms} part[g * part_group_stride + t * stride + c] for c < ncols, g < groups;
// fixed summation order (see m3_reduce.cu).
cudaError_t column_sums(cudaStream_t st, const float* part, int nterms, size_t stride, int ncols, float* out,
                        bool accumulate = false, int groups = 1, size_t part_group_stride = 0,
                        size_t out_group_stride = 0);

}  // namespace m3
