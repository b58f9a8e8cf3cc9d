// Generic backward of the Mamba-3 SSD scan: launch sequence of the hand adjoint.
#include "m3_generic_bwd_a.cuh"
#include "m3_generic_bwd_b.cuh"

namespace m3 {

size_t generic_bwd_ws_layout(const Dims& d, GenericBwdWs* ws, char* base) {
  size_t off = 0;
  auto take = [&](size_t nfloat) {
    float* p = base ? reinterpret_cast<float*>(base + off) : nullptr;
    off += ((nfloat * sizeof(float) + 255) / 256) * 256;
    return p;
  };
  const size_t BH = (size_t)d.B * d.H, rows = (size_t)d.Tp * d.R;
  GenericBwdWs t;
  t.dXh = take(BH * rows * d.P);
  t.dBh = take(BH * rows * d.N);
  t.dCh = take(BH * rows * d.N);
  t.dHs = take(BH * (d.C + 1) * d.P * d.N);
  t.dBand = take(BH * d.C * d.L * d.L);
  t.dcd = take(BH * d.C);
  t.dac = take(BH * d.Tp);
  t.dws = take(BH * d.Tp);
  t.dast = take(BH * d.Tp);
  t.da = take(BH * d.Tp);
  t.dg = take(BH * d.Tp);
  t.dw = take(BH * d.Tp);
  t.dphi = take(BH * d.Tp * d.NH);
  t.dpsum = take(BH * d.C * d.NH);
  t.ddt_rot = take(BH * d.Tp);
  t.partA = take(BH * d.C);
  t.partD = take(BH * d.C);
  t.ip0 = take(BH);
  if (ws) *ws = t;
  return off;
}

template <class T>
static cudaError_t backward_t(cudaStream_t st, const Dims& d, const m3_scan_desc& desc, const GenericWs& ws,
                              const GenericBwdWs& bw, const m3_scan_bwd_in& in, uint32_t mask,
                              const m3_scan_grads& g, uint64_t* launches) {
  const T* x = static_cast<const T*>(desc.x);
  const T* dt = static_cast<const T*>(desc.dt);
  const T* lam = static_cast<const T*>(desc.lambda);
  const T* th = static_cast<const T*>(desc.theta);
  const T* dy = static_cast<const T*>(in.dy);
  auto want = [&](uint32_t bit, const void* p) { return (mask & bit) && p; };
  T* dx = want(M3_GRAD_X, g.dx) ? static_cast<T*>(g.dx) : nullptr;
  T* db = want(M3_GRAD_B, g.db) ? static_cast<T*>(g.db) : nullptr;
  T* dc = want(M3_GRAD_C, g.dc) ? static_cast<T*>(g.dc) : nullptr;
  T* ddt = want(M3_GRAD_DT, g.ddt) ? static_cast<T*>(g.ddt) : nullptr;
  T* dlam = (want(M3_GRAD_LAMBDA, g.dlambda) && d.disc == M3_LEARNED_TRAPEZOID) ? static_cast<T*>(g.dlambda) : nullptr;
  T* dth = (want(M3_GRAD_THETA, g.dtheta) && d.rot) ? static_cast<T*>(g.dtheta) : nullptr;
  float* dalog = (want(M3_GRAD_A_LOG, g.da_log) && !d.raw) ? g.da_log : nullptr;
  float* ddsk = (want(M3_GRAD_D_SKIP, g.dd_skip) && desc.d_skip) ? g.dd_skip : nullptr;
  const bool has_state = desc.h0 != nullptr;
  float* dh0 = (has_state && want(M3_GRAD_H0, g.dh0)) ? g.dh0 : nullptr;
  float* dlu0 = (has_state && !d.raw && want(M3_GRAD_LAST_U0, g.dlast_u0)) ? g.dlast_u0 : nullptr;
  float* dang0 = (d.rot && desc.angle0 && want(M3_GRAD_ANGLE0, g.dangle0)) ? g.dangle0 : nullptr;

  const int BH = d.B * d.H, PN = d.P * d.N;
  const dim3 gchunk(d.C, d.H, d.B);
  const int TL = d.R >= 64 ? 1 : 64 / d.R;
  const int tiles_l = (d.L + TL - 1) / TL;
  const int tiles_pn = ((d.P + 63) / 64) * ((d.N + 63) / 64);
  uint64_t n = 0;
  cudaError_t e;

  const size_t sm_rows = sizeof(float) * ((size_t)kGemmSmemFloats + 3 * d.L + 64 + 64 * 65 + 64 * (size_t)d.LR);
  e = cudaFuncSetAttribute(kb_rows<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_rows);
  if (e != cudaSuccess) return e;
  kb_rows<T><<<dim3(tiles_l, d.C, BH), 256, sm_rows, st>>>(d, dy, ws, bw);
  kb_dhloc<T><<<dim3(tiles_pn, d.C, BH), 256, sizeof(float) * (kGemmSmemFloats + d.L), st>>>(d, dy, ws, bw);
  kb_state_pass_rev<<<dim3((PN + 255) / 256, BH), 256, 0, st>>>(d, in.dh, ws, bw);
  kb_dcd<<<dim3(d.C + 1, BH), 256, 0, st>>>(d, d.raw ? nullptr : desc.last_u0, ws, bw);
  const size_t sm_cols = sizeof(float) * ((size_t)kGemmSmemFloats + 3 * d.L + 64 + 64 * (size_t)d.LR);
  e = cudaFuncSetAttribute(kb_cols<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sm_cols);
  if (e != cudaSuccess) return e;
  kb_cols<T><<<dim3(tiles_l, d.C, BH), 256, sm_cols, st>>>(d, dy, ws, bw);
  kb_scalars<T><<<dim3(d.C, BH), 256, sizeof(float) * 4 * d.L, st>>>(d, dt, ws, bw);
  n += 6;
  if (in.dlast_u) {
    kb_last_u<<<BH, 256, 0, st>>>(d, in.dlast_u, ws, bw);
    n += 1;
  }
  if (d.rot || db || dc) {
    kb_unrotate<T><<<gchunk, 256, 0, st>>>(d, ws, bw, in.dangle, db, dc);
    n += 1;
  }
  if (d.rot) {
    kb_dphi_sum<<<dim3(d.C, BH), 64, 0, st>>>(d, bw);
    kb_dphi_suffix<<<BH, 64, 0, st>>>(d, bw, dang0);
    kb_dstep<T><<<gchunk, 64, 0, st>>>(d, dt, th, bw, dth);
    n += 3;
  }
  kb_dx<T><<<gchunk, 256, 0, st>>>(d, x, dy, desc.d_skip, bw, dx);
  const size_t total = (size_t)d.B * d.T * d.H;
  kb_final<T><<<(unsigned)((total + 255) / 256), 256, 0, st>>>(
      d, dt, lam, desc.a_log, bw, (has_state && !d.raw) ? 1 : 0, ddt, dlam, static_cast<T*>(g.da_raw),
      static_cast<T*>(g.dg_raw), static_cast<T*>(g.dw_raw));
  n += 2;
  if (dh0 || dlu0) {
    kb_state_grads<T><<<dim3((PN + 255) / 256, BH), 256, 0, st>>>(d, dt, lam, bw, dh0, dlu0);
    n += 1;
  }
  if (dalog || ddsk) {
    kb_reduce_heads<<<d.H, 256, 0, st>>>(d, desc.a_log, bw, dalog, ddsk);
    n += 1;
  }
  if (launches) *launches += n;
  return cudaGetLastError();
}

// The last two launches of any backward: per-token d dt / d lambda from (da, dg, dw, the
// rotation term, the seed-state term) and the per-head reductions.  `d.Tp` and `d.C` give the
// pitch of the per-token arrays and the number of partial sums per (batch, head).
cudaError_t finalize_scalars(cudaStream_t st, const Dims& d, const m3_scan_desc& desc, const GenericBwdWs& bw,
                             void* ddt, void* dlam, float* dalog, float* ddsk, uint64_t* launches) {
  const size_t total = (size_t)d.B * d.T * d.H;
  const unsigned grid = (unsigned)((total + 255) / 256);
  const int has_state = desc.h0 ? 1 : 0;
  if (desc.dtype == M3_BF16) {
    using T = __nv_bfloat16;
    kb_final<T><<<grid, 256, 0, st>>>(d, static_cast<const T*>(desc.dt), static_cast<const T*>(desc.lambda), desc.a_log,
                                      bw, has_state, static_cast<T*>(ddt), static_cast<T*>(dlam), nullptr, nullptr, nullptr);
  } else {
    kb_final<float><<<grid, 256, 0, st>>>(d, static_cast<const float*>(desc.dt), static_cast<const float*>(desc.lambda),
                                          desc.a_log, bw, has_state, static_cast<float*>(ddt), static_cast<float*>(dlam),
                                          nullptr, nullptr, nullptr);
  }
  uint64_t n = 1;
  if (dalog || ddsk) {
    kb_reduce_heads<<<d.H, 256, 0, st>>>(d, desc.a_log, bw, dalog, ddsk);
    n += 1;
  }
  if (launches) *launches += n;
  return cudaGetLastError();
}

cudaError_t generic_backward(cudaStream_t st, const Dims& d, const m3_scan_desc& desc, const GenericWs& ws,
                             const GenericBwdWs& bw, const m3_scan_bwd_in& in, uint32_t mask,
                             const m3_scan_grads& grads, uint64_t* launches) {
  if (desc.dtype == M3_BF16) return backward_t<__nv_bfloat16>(st, d, desc, ws, bw, in, mask, grads, launches);
  return backward_t<float>(st, d, desc, ws, bw, in, mask, grads, launches);
}

}  // namespace m3
