// C ABI of libm3scan: contexts, device buffers, and the forward / backward entry
// points that validate a descriptor, lay out scratch and enqueue a kernel family.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>

#include "m3_internal.h"
#include "m3_tc.h"

struct m3_saved {
  m3_scan_desc desc;
  m3::Dims dims;
  int path = M3_PATH_GENERIC;
  char* ws_base = nullptr;
  size_t ws_bytes = 0;
  m3::GenericWs gws;
  __nv_bfloat16* tc_ckpt_h = nullptr;  // tensor-core family: bf16 state entering each tile
  float* tc_ckpt_angle = nullptr;  // and the angle entering each tile
  bool tc_direct = false;          // the forward ran the direct form: so does the backward (same tile maps)
  cudaStream_t stream = nullptr;   // the stream the forward ran on: the scratch is freed in its order
};

namespace m3 {

int fail(m3_ctx* ctx, int code, const char* fmt, ...) {
  if (ctx) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ctx->err, sizeof(ctx->err), fmt, ap);
    va_end(ap);
  }
  return code;
}

int cuda_fail(m3_ctx* ctx, cudaError_t e, const char* what) {
  return fail(ctx, M3_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

int take_device_flag(m3_ctx* ctx, const char* when) {
  if (!ctx->err_host || !*ctx->err_host) return M3_OK;
  *ctx->err_host = 0;
  return fail(ctx, M3_ERR_TIMEOUT, "a bounded device-side wait gave up (%s); results of the affected call are invalid", when);
}

}  // namespace m3

using m3::cuda_fail;
using m3::fail;
using m3::make_dims;

namespace m3 {

#define M3_CUDA(ctx, call)                                   \
  do {                                                       \
    cudaError_t e_ = (call);                                 \
    if (e_ != cudaSuccess) return cuda_fail(ctx, e_, #call); \
  } while (0)

// Largest number of rows (chunk length x rank) one chunk of the generic family may
// have: its band tile lives in shared memory.  The scan's result does not depend on
// the chunk length (only terms below exp(-60) move), so a longer requested chunk is
// split; src/ssm/scan.rs:146 clamps the request in the same spirit.
constexpr int kGenericMaxRows = 512;

int make_dims(m3_ctx* ctx, const m3_scan_desc& s, m3::Dims* out) {
  if (s.batch <= 0 || s.heads <= 0 || s.head_dim <= 0 || s.d_state <= 0 || s.rank <= 0 || s.seq < 0)
    return fail(ctx, M3_ERR_SHAPE, "extents must be positive (batch %d seq %d heads %d head_dim %d d_state %d rank %d)",
                s.batch, s.seq, s.heads, s.head_dim, s.d_state, s.rank);
  if (s.dtype != M3_F32 && s.dtype != M3_BF16) return fail(ctx, M3_ERR_UNSUPPORTED, "dtype %d", s.dtype);
  if (s.discretization < M3_EULER || s.discretization > M3_LEARNED_TRAPEZOID)
    return fail(ctx, M3_ERR_CONFIG, "discretization %d", s.discretization);
  if (s.dynamics != M3_REAL && s.dynamics != M3_ROTATIONAL) return fail(ctx, M3_ERR_CONFIG, "dynamics %d", s.dynamics);
  if (s.dynamics == M3_ROTATIONAL && (s.d_state % 2))
    return fail(ctx, M3_ERR_CONFIG, "rotational dynamics require an even d_state");
  if (s.rank > 64) return fail(ctx, M3_ERR_UNSUPPORTED, "rank %d > 64", s.rank);
  if (s.reverse_heads < 0 || s.reverse_heads > s.heads)
    return fail(ctx, M3_ERR_CONFIG, "reverse_heads %d outside [0, heads = %d]", s.reverse_heads, s.heads);
  const bool raw = s.a_raw != nullptr;
  if (raw) {
    if (!s.g_raw || !s.w_raw) return fail(ctx, M3_ERR_NULL, "a_raw needs g_raw and w_raw");
    if (s.dynamics != M3_REAL || s.theta) return fail(ctx, M3_ERR_CONFIG, "the a/g/w form has no rotation");
    if (!s.x || !s.b || !s.c) return fail(ctx, M3_ERR_NULL, "x, b and c are required");
  } else {
    if (!s.x || !s.b || !s.c || !s.dt || !s.a_log) return fail(ctx, M3_ERR_NULL, "x, b, c, dt and a_log are required");
    if (s.discretization == M3_LEARNED_TRAPEZOID && !s.lambda) return fail(ctx, M3_ERR_NULL, "learned trapezoid needs lambda");
    if ((s.h0 == nullptr) != (s.last_u0 == nullptr)) return fail(ctx, M3_ERR_NULL, "a carried state needs both h and last_u");
  }
  if (s.dynamics == M3_ROTATIONAL && !s.theta) return fail(ctx, M3_ERR_NULL, "rotational dynamics need theta");
  if ((size_t)s.batch * s.heads > 65535u) return fail(ctx, M3_ERR_UNSUPPORTED, "batch * heads > 65535");
  m3::Dims d;
  d.B = s.batch; d.T = s.seq; d.H = s.heads; d.P = s.head_dim; d.N = s.d_state; d.R = s.rank;
  int L = s.chunk < 1 ? 1 : s.chunk;
  if (s.seq > 0 && L > s.seq) L = s.seq;
  const int cap = kGenericMaxRows / s.rank > 0 ? kGenericMaxRows / s.rank : 1;
  if (L > cap) L = cap;
  d.L = L;
  d.C = (s.seq + L - 1) / L;
  d.Tp = d.C * L;
  d.rot = s.dynamics == M3_ROTATIONAL;
  d.NH = d.rot ? s.d_state / 2 : 0;
  d.disc = s.discretization;
  d.LR = L * s.rank;
  d.raw = raw ? 1 : 0;
  d.rev = s.reverse_heads;
  *out = d;
  return M3_OK;
}

}  // namespace m3

namespace {

// Launches whose CTAs wait on one another (stripes cut into segments) must not share the GPU with another such
// launch: each could hold SMs the other's unscheduled CTAs are waited for on, and both would sit out their
// bounded waits.  Within this process they are therefore chained across streams: a launch waits for the event
// the previous one of the device recorded behind itself.  (They fill every SM anyway, so nothing is lost; launches
// that wait on nobody - whole stripes, other libraries' kernels - finish on their own and need no such care.)
// Streams under capture are left alone: a captured graph replays alone on its stream.
struct SplitChain {
  std::mutex mu;
  cudaEvent_t ev[64] = {};
  bool recorded[64] = {};
};
SplitChain& split_chain() {
  static SplitChain c;
  return c;
}
cudaError_t split_chain_enter(m3_ctx* ctx) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return cudaSuccess;
  }
  const int dev = ctx->device;
  if (dev < 0 || dev >= 64) return cudaSuccess;
  SplitChain& c = split_chain();
  std::lock_guard<std::mutex> lock(c.mu);
  return c.recorded[dev] ? cudaStreamWaitEvent(ctx->stream, c.ev[dev], 0) : cudaSuccess;
}
void split_chain_leave(m3_ctx* ctx) {
  cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
  if (cudaStreamIsCapturing(ctx->stream, &cs) != cudaSuccess || cs != cudaStreamCaptureStatusNone) {
    cudaGetLastError();
    return;
  }
  const int dev = ctx->device;
  if (dev < 0 || dev >= 64) return;
  SplitChain& c = split_chain();
  std::lock_guard<std::mutex> lock(c.mu);
  if (!c.ev[dev] && cudaEventCreateWithFlags(&c.ev[dev], cudaEventDisableTiming) != cudaSuccess) {
    c.ev[dev] = nullptr;
    cudaGetLastError();
    return;
  }
  if (cudaEventRecord(c.ev[dev], ctx->stream) == cudaSuccess) c.recorded[dev] = true;
  else cudaGetLastError();
}

// Time segments of the stripes for one launch of the role-split kernels: the plan, and - when a stripe is
// cut - the hand-over scratch (state, angle, flags; the flags zeroed on the stream).  `*scratch` is null
// when nothing is handed over; the caller frees it on the stream after the launch.
template <class Params>
cudaError_t plan_segments(m3_ctx* ctx, Params& p, int tiles, bool allow_split, char** scratch) {
  *scratch = nullptr;
  size_t bytes = 0;
  m3::tc_segment_plan(p.B * p.H, tiles, allow_split, &p.nseg, &p.tps, &p.grid, &bytes);
  if (p.nseg == 1) return cudaSuccess;
  cudaError_t e = m3::scratch_alloc(ctx, reinterpret_cast<void**>(scratch), bytes, ctx->stream);
  if (e != cudaSuccess) return e;
  const size_t items = (size_t)p.B * p.H * p.nseg;
  p.seg_state = reinterpret_cast<float*>(*scratch);
  p.seg_angle = p.seg_state + items * 64 * 128;
  p.seg_flag = reinterpret_cast<int*>(p.seg_angle + items * 64);
  e = cudaMemsetAsync(p.seg_flag, 0, items * sizeof(int), ctx->stream);
  if (e == cudaSuccess) e = split_chain_enter(ctx);
  return e;
}

// Backward of a forward that ran the tensor-core family: one stripe kernel, then the shared
// per-token / per-head finalisation.
int tc_backward_call(m3_ctx* ctx, const m3_saved* saved, const m3_scan_bwd_in* in, uint32_t mask,
                     const m3_scan_grads* g) {
  const m3_scan_desc& desc = saved->desc;
  m3::Dims d = saved->dims;
  const int steps = m3::tc_tile_steps(d.R), tiles = m3::tc_tiles(d.T, d.R);
  d.L = steps; d.C = tiles; d.Tp = tiles * steps; d.LR = 128;
  const size_t BH = (size_t)d.B * d.H;
  const size_t per_tok = BH * d.Tp, per_tile = BH * tiles;
  const size_t nfloat = 4 * per_tok + 2 * per_tile + BH;
  float* base = nullptr;
  M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&base), nfloat * sizeof(float), ctx->stream));
  m3::GenericBwdWs bw{};
  bw.da = base; bw.dg = base + per_tok; bw.dw = base + 2 * per_tok; bw.ddt_rot = base + 3 * per_tok;
  bw.partA = base + 4 * per_tok; bw.partD = bw.partA + per_tile; bw.ip0 = bw.partD + per_tile;
  auto want = [&](uint32_t bit, const void* p) { return (mask & bit) && p; };
  using bf16 = __nv_bfloat16;
  m3::TcBwdParams p{};
  p.x = static_cast<const bf16*>(desc.x); p.b = static_cast<const bf16*>(desc.b); p.c = static_cast<const bf16*>(desc.c);
  p.dt = static_cast<const bf16*>(desc.dt); p.lam = static_cast<const bf16*>(desc.lambda);
  p.theta = static_cast<const bf16*>(desc.theta); p.dy = static_cast<const bf16*>(in->dy);
  p.a_log = desc.a_log; p.d_skip = desc.d_skip; p.h0 = desc.h0; p.lu0 = desc.last_u0;
  p.dh = in->dh; p.dlu = in->dlast_u; p.dangle = d.rot ? in->dangle : nullptr;
  p.ckpt_h = saved->tc_ckpt_h; p.ckpt_angle = saved->tc_ckpt_angle;
  p.dx = want(M3_GRAD_X, g->dx) ? static_cast<bf16*>(g->dx) : nullptr;
  p.db = want(M3_GRAD_B, g->db) ? static_cast<bf16*>(g->db) : nullptr;
  p.dc = want(M3_GRAD_C, g->dc) ? static_cast<bf16*>(g->dc) : nullptr;
  p.dtheta = (want(M3_GRAD_THETA, g->dtheta) && d.rot) ? static_cast<bf16*>(g->dtheta) : nullptr;
  p.da = bw.da; p.dg = bw.dg; p.dw = bw.dw; p.ddt_rot = bw.ddt_rot; p.partA = bw.partA; p.partD = bw.partD; p.ip0 = bw.ip0;
  const bool has_state = desc.h0 != nullptr;
  p.dh0 = (has_state && want(M3_GRAD_H0, g->dh0)) ? g->dh0 : nullptr;
  p.dlu0 = (has_state && want(M3_GRAD_LAST_U0, g->dlast_u0)) ? g->dlast_u0 : nullptr;
  p.dangle0 = (d.rot && desc.angle0 && want(M3_GRAD_ANGLE0, g->dangle0)) ? g->dangle0 : nullptr;
  p.err = ctx->dev_err;
  p.B = d.B; p.T = d.T; p.H = d.H; p.R = d.R; p.disc = d.disc; p.rev = d.rev;
  p.wait_limit = ctx->wait_limit ? ctx->wait_limit : (1u << 18);
  if (!m3::tc_aligned(p.dy) || !m3::tc_aligned(p.dx) || !m3::tc_aligned(p.db) || !m3::tc_aligned(p.dc) ||
      !m3::tc_aligned(p.dtheta)) {
    cudaFreeAsync(base, ctx->stream);
    return fail(ctx, M3_ERR_UNSUPPORTED, "the tensor-core family needs 16-byte aligned dy and gradient buffers");
  }
  p.use_tma = (saved->tc_direct && d.R == 1 && !d.rot && d.rev == 0 && d.T % 8 == 0 && !(reinterpret_cast<uintptr_t>(p.ckpt_h) & 15) &&
               m3::tc_make_tile_map(&p.tm_b, p.b, d.B, d.T, d.H, 128) && m3::tc_make_tile_map(&p.tm_c, p.c, d.B, d.T, d.H, 128)) ? 1 : 0;
  if (saved->tc_direct && !p.use_tma) {
    cudaFreeAsync(base, ctx->stream);
    return fail(ctx, M3_ERR_UNSUPPORTED, "the forward pass ran the direct form; its backward pass cannot be set up");
  }
  if (!p.use_tma) {
    if (!m3::tc_make_row_map(&p.tm_b, p.b, d.B, d.T, d.H, 128 * d.R, steps, true) ||
        !m3::tc_make_row_map(&p.tm_c, p.c, d.B, d.T, d.H, 128 * d.R, steps, true) ||
        !m3::tc_make_row_map(&p.tm_x, p.x, d.B, d.T, d.H, 64 * d.R, steps, true) ||
        !m3::tc_make_row_map(&p.tm_dy, p.dy, d.B, d.T, d.H, 64 * d.R, steps, true) ||
        (d.rot && !m3::tc_make_row_map(&p.tm_th, p.theta, d.B, d.T, d.H, 64, steps, false))) {
      cudaFreeAsync(base, ctx->stream);
      return fail(ctx, M3_ERR_UNSUPPORTED, "the tensor-core family needs 16-byte aligned b, c, x, dy and theta");
    }
    // the gradients asked for leave by bulk tensor stores where they can; by plain stores otherwise
    p.out_maps = ((!p.dx || m3::tc_make_row_map(&p.tm_dx, p.dx, d.B, d.T, d.H, 64 * d.R, steps, true)) &&
                  (!p.db || m3::tc_make_row_map(&p.tm_db, p.db, d.B, d.T, d.H, 128 * d.R, steps, true)) &&
                  (!p.dc || m3::tc_make_row_map(&p.tm_dc, p.dc, d.B, d.T, d.H, 128 * d.R, steps, true))) ? 1 : 0;
  }
  char* seg = nullptr;
  cudaError_t e = plan_segments(ctx, p, tiles, !p.use_tma, &seg);
  if (e == cudaSuccess) e = m3::tc_backward(ctx->stream, p, d.rot != 0);
  if (seg) {
    split_chain_leave(ctx);
    cudaFreeAsync(seg, ctx->stream);
  }
  if (e == cudaSuccess) {
    ctx->launches += 1;
    void* ddt = want(M3_GRAD_DT, g->ddt) ? g->ddt : nullptr;
    void* dlam = (want(M3_GRAD_LAMBDA, g->dlambda) && d.disc == M3_LEARNED_TRAPEZOID) ? g->dlambda : nullptr;
    float* dalog = want(M3_GRAD_A_LOG, g->da_log) ? g->da_log : nullptr;
    float* ddsk = (want(M3_GRAD_D_SKIP, g->dd_skip) && desc.d_skip) ? g->dd_skip : nullptr;
    e = m3::finalize_scalars(ctx->stream, d, desc, bw, ddt, dlam, dalog, ddsk, &ctx->launches);
  }
  cudaError_t e2 = cudaFreeAsync(base, ctx->stream);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "tensor-core backward");
  if (e2 != cudaSuccess) return cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

}  // namespace

extern "C" {

const char* m3_version(void) { return "0.1.0"; }

int m3_ctx_create(int device, m3_ctx** out) {
  if (!out) return M3_ERR_NULL;
  *out = nullptr;
  m3_ctx* ctx = new (std::nothrow) m3_ctx();
  if (!ctx) return M3_ERR_CUDA;
  ctx->device = device;
  cudaError_t e = cudaSetDevice(device);
  if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    delete ctx;
    return M3_ERR_CUDA;
  }
  ctx->own_stream = true;
  int* flag = nullptr;
  if (cudaHostAlloc(reinterpret_cast<void**>(&flag), sizeof(int), cudaHostAllocMapped) != cudaSuccess ||
      cudaHostGetDevicePointer(reinterpret_cast<void**>(&ctx->dev_err), flag, 0) != cudaSuccess) {
    if (flag) cudaFreeHost(flag);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return M3_ERR_CUDA;
  }
  *flag = 0;
  ctx->err_host = flag;
  // Scratch comes from a pool of this context's own, which keeps freed memory for the next call
  // (steady-state calls then do not allocate) and gives it back when the context is destroyed; the
  // device's default pool and its settings are left alone.  Where the driver refuses a pool, calls
  // fall back to the default pool as it is.
  cudaMemPoolProps props{};
  props.allocType = cudaMemAllocationTypePinned;
  props.handleTypes = cudaMemHandleTypeNone;
  props.location.type = cudaMemLocationTypeDevice;
  props.location.id = device;
  if (cudaMemPoolCreate(&ctx->pool, &props) == cudaSuccess) {
    uint64_t keep = UINT64_MAX;
    cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep);
  } else {
    ctx->pool = nullptr;
    cudaGetLastError();
  }
  *out = ctx;
  return M3_OK;
}

int m3_ctx_destroy(m3_ctx* ctx) {
  if (!ctx) return M3_OK;
  cudaSetDevice(ctx->device);
  if (ctx->own_stream && ctx->stream) {
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
  }
  cudaDeviceSynchronize();  // scratch freed on other streams (a saved handle's) must be back in the pool
  if (ctx->pool) cudaMemPoolDestroy(ctx->pool);
  if (ctx->err_host) cudaFreeHost(const_cast<int*>(ctx->err_host));
  delete ctx;
  return M3_OK;
}

int m3_ctx_set_stream(m3_ctx* ctx, void* cuda_stream) {
  if (!ctx) return M3_ERR_NULL;
  if (ctx->own_stream && ctx->stream) {
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaStreamDestroy(ctx->stream);
  }
  ctx->stream = static_cast<cudaStream_t>(cuda_stream);
  ctx->own_stream = false;
  return M3_OK;
}

int m3_sync(m3_ctx* ctx) {
  if (!ctx) return M3_ERR_NULL;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  M3_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return m3::take_device_flag(ctx, "seen at m3_sync");
}

int m3_ctx_set_wait_limit(m3_ctx* ctx, uint32_t iterations) {
  if (!ctx) return M3_ERR_NULL;
  ctx->wait_limit = iterations;
  return M3_OK;
}

const char* m3_last_error(const m3_ctx* ctx) { return ctx ? ctx->err : "null context"; }

uint64_t m3_launch_count(const m3_ctx* ctx) { return ctx ? ctx->launches : 0; }

int m3_alloc(m3_ctx* ctx, size_t bytes, void** out) {
  if (!ctx || !out) return M3_ERR_NULL;
  *out = nullptr;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  M3_CUDA(ctx, cudaMalloc(out, bytes ? bytes : 1));
  return M3_OK;
}

int m3_free(m3_ctx* ctx, void* ptr) {
  if (!ctx) return M3_ERR_NULL;
  if (!ptr) return M3_OK;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  M3_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  M3_CUDA(ctx, cudaFree(ptr));
  return M3_OK;
}

int m3_upload(m3_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx || (bytes && (!dst || !src))) return M3_ERR_NULL;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  M3_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
  return M3_OK;
}

int m3_download(m3_ctx* ctx, void* dst, const void* src, size_t bytes) {
  if (!ctx || (bytes && (!dst || !src))) return M3_ERR_NULL;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  M3_CUDA(ctx, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
  M3_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return M3_OK;
}

size_t m3_scan_scratch_bytes(const m3_scan_desc* desc, int for_backward) {
  if (!desc) return 0;
  m3::Dims d;
  m3_scan_desc s = *desc;
  // Only the extents matter here: stand in for pointers the caller may not have yet.
  static const float dummy = 0.0f;
  s.x = s.b = s.c = s.dt = &dummy; s.a_log = &dummy;
  if (s.discretization == M3_LEARNED_TRAPEZOID) s.lambda = &dummy;
  if (s.dynamics == M3_ROTATIONAL) s.theta = &dummy;
  s.h0 = s.last_u0 = nullptr;
  if (s.a_raw) s.a_raw = s.g_raw = s.w_raw = &dummy;
  if (make_dims(nullptr, s, &d) != M3_OK || d.T == 0) return 0;
  size_t n = m3::generic_ws_layout(d, nullptr, nullptr);
  if (for_backward) n += m3::generic_bwd_ws_layout(d, nullptr, nullptr);
  return n;
}

int m3_scan_forward(m3_ctx* ctx, const m3_scan_desc* desc, const m3_scan_out* out, m3_saved** saved) {
  if (saved) *saved = nullptr;
  if (!ctx) return M3_ERR_NULL;
  if (!desc || !out) return fail(ctx, M3_ERR_NULL, "descriptor and outputs are required");
  int rc = m3::take_device_flag(ctx, "in an earlier call, seen on entry to m3_scan_forward");
  if (rc != M3_OK) return rc;
  m3::Dims d;
  rc = make_dims(ctx, *desc, &d);
  if (rc != M3_OK) return rc;
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const size_t PN = (size_t)d.P * d.N, BH = (size_t)d.B * d.H;
  if (d.T == 0) {
    // Nothing to scan (scan.rs:134-144): the carried state passes through.
    if (desc->want_state) {
      if (out->h) {
        if (desc->h0) M3_CUDA(ctx, cudaMemcpyAsync(out->h, desc->h0, BH * PN * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        else M3_CUDA(ctx, cudaMemsetAsync(out->h, 0, BH * PN * 4, ctx->stream));
      }
      if (out->last_u) {
        if (desc->last_u0) M3_CUDA(ctx, cudaMemcpyAsync(out->last_u, desc->last_u0, BH * PN * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        else M3_CUDA(ctx, cudaMemsetAsync(out->last_u, 0, BH * PN * 4, ctx->stream));
      }
      if (out->angle && d.rot) {
        if (desc->angle0) M3_CUDA(ctx, cudaMemcpyAsync(out->angle, desc->angle0, BH * d.NH * 4, cudaMemcpyDeviceToDevice, ctx->stream));
        else M3_CUDA(ctx, cudaMemsetAsync(out->angle, 0, BH * d.NH * 4, ctx->stream));
      }
    }
    return M3_OK;
  }
  if (!out->y) return fail(ctx, M3_ERR_NULL, "y is required");
  const bool tc_ok = m3::tc_supported(*desc) && !d.raw && m3::tc_aligned(out->y);
  if (desc->path == M3_PATH_TENSOR && !tc_ok)
    return fail(ctx, M3_ERR_UNSUPPORTED, "the tensor-core family does not take this shape");
  if (tc_ok && desc->path != M3_PATH_GENERIC) {
    m3::TcFwdParams p{};
    p.x = static_cast<const __nv_bfloat16*>(desc->x); p.b = static_cast<const __nv_bfloat16*>(desc->b);
    p.c = static_cast<const __nv_bfloat16*>(desc->c); p.dt = static_cast<const __nv_bfloat16*>(desc->dt);
    p.lam = static_cast<const __nv_bfloat16*>(desc->lambda); p.theta = static_cast<const __nv_bfloat16*>(desc->theta);
    p.a_log = desc->a_log; p.d_skip = desc->d_skip; p.h0 = desc->h0; p.lu0 = desc->last_u0; p.angle0 = desc->angle0;
    p.y = static_cast<__nv_bfloat16*>(out->y);
    p.h_out = desc->want_state ? out->h : nullptr;
    p.lu_out = desc->want_state ? out->last_u : nullptr;
    p.angle_out = (desc->want_state && d.rot) ? out->angle : nullptr;
    p.err = ctx->dev_err;
    p.B = d.B; p.T = d.T; p.H = d.H; p.R = d.R; p.disc = d.disc; p.rev = d.rev;
    p.wait_limit = ctx->wait_limit ? ctx->wait_limit : (1u << 18);
    // Rank 1 with real dynamics needs no conversion of its rows: bulk tensor copies land them in
    // operand layout (every head left to right, T a multiple of 8, 16-byte aligned tensors).
    p.use_tma = (d.R == 1 && !d.rot && d.rev == 0 && d.T % 8 == 0 &&
                 m3::tc_make_tile_map(&p.tm_b, p.b, d.B, d.T, d.H, 128) && m3::tc_make_tile_map(&p.tm_c, p.c, d.B, d.T, d.H, 128) &&
                 m3::tc_make_tile_map(&p.tm_x, p.x, d.B, d.T, d.H, 64)) ? 1 : 0;
    if (!p.use_tma) {
      // every other shape: the raw rows of b and c are fetched by bulk tensor copies, a tile at a time
      const int steps = m3::tc_tile_steps(d.R);
      if (!m3::tc_make_row_map(&p.tm_b, p.b, d.B, d.T, d.H, 128 * d.R, steps, true) ||
          !m3::tc_make_row_map(&p.tm_c, p.c, d.B, d.T, d.H, 128 * d.R, steps, true))
        return fail(ctx, M3_ERR_UNSUPPORTED, "the tensor-core family needs 16-byte aligned b and c");
      if (d.rot && !m3::tc_make_row_map(&p.tm_th, p.theta, d.B, d.T, d.H, 64, steps, false))
        return fail(ctx, M3_ERR_UNSUPPORTED, "the tensor-core family needs a 16-byte aligned theta");
      // y leaves by bulk tensor stores where it can (a 16-byte aligned tensor); by plain stores otherwise
      p.out_maps = m3::tc_make_row_map(&p.tm_y, p.y, d.B, d.T, d.H, 64 * d.R, steps, true) ? 1 : 0;
    }
    char* base = nullptr;
    size_t bytes = 0;
    if (saved) {  // the backward pass needs the state and the angle entering every tile
      const size_t tiles = (size_t)m3::tc_tiles(d.T, d.R);
      const size_t nh = BH * tiles * 128 * 64, na = BH * tiles * 64;
      bytes = nh * sizeof(__nv_bfloat16) + na * sizeof(float);
      M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&base), bytes, ctx->stream));
      p.ckpt_h = reinterpret_cast<__nv_bfloat16*>(base);
      p.ckpt_angle = reinterpret_cast<float*>(base + nh * sizeof(__nv_bfloat16));
    }
    // a caller that must not allocate gets whole stripes: cutting them needs hand-over scratch
    char* seg = nullptr;
    cudaError_t te = plan_segments(ctx, p, m3::tc_tiles(d.T, d.R), !p.use_tma && !ctx->no_scratch, &seg);
    if (te == cudaSuccess) te = m3::tc_forward(ctx->stream, p, d.rot != 0);
    if (seg) {
      split_chain_leave(ctx);
      cudaFreeAsync(seg, ctx->stream);
    }
    if (te != cudaSuccess) {
      if (base) cudaFreeAsync(base, ctx->stream);
      return cuda_fail(ctx, te, "tensor-core forward");
    }
    ctx->launches += 1;
    if (saved) {
      m3_saved* sv = new (std::nothrow) m3_saved();
      if (!sv) {
        cudaFreeAsync(base, ctx->stream);
        return fail(ctx, M3_ERR_CUDA, "out of host memory");
      }
      sv->desc = *desc;
      sv->dims = d;
      sv->path = M3_PATH_TENSOR;
      sv->ws_base = base;
      sv->ws_bytes = bytes;
      sv->tc_ckpt_h = p.ckpt_h;
      sv->tc_ckpt_angle = p.ckpt_angle;
      sv->tc_direct = p.use_tma != 0;
      sv->stream = ctx->stream;
      *saved = sv;
    }
    return M3_OK;
  }
  const size_t bytes = m3::generic_ws_layout(d, nullptr, nullptr);
  char* base = nullptr;
  M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&base), bytes, ctx->stream));
  m3::GenericWs ws;
  m3::generic_ws_layout(d, &ws, base);
  cudaError_t e = m3::generic_forward(ctx->stream, d, *desc, *out, ws, &ctx->launches);
  if (e != cudaSuccess) {
    cudaFreeAsync(base, ctx->stream);
    return cuda_fail(ctx, e, "generic forward");
  }
  if (saved) {
    m3_saved* sv = new (std::nothrow) m3_saved();
    if (!sv) {
      cudaFreeAsync(base, ctx->stream);
      return fail(ctx, M3_ERR_CUDA, "out of host memory");
    }
    sv->desc = *desc;
    sv->dims = d;
    sv->path = M3_PATH_GENERIC;
    sv->ws_base = base;
    sv->ws_bytes = bytes;
    sv->gws = ws;
    sv->stream = ctx->stream;
    *saved = sv;
  } else {
    M3_CUDA(ctx, cudaFreeAsync(base, ctx->stream));
  }
  return M3_OK;
}

int m3_scan_backward(m3_ctx* ctx, const m3_saved* saved, const m3_scan_bwd_in* in, uint32_t grad_mask,
                     const m3_scan_grads* grads) {
  if (!ctx) return M3_ERR_NULL;
  if (!saved || !in || !grads) return fail(ctx, M3_ERR_NULL, "saved context, upstream gradients and outputs are required");
  if (!in->dy) return fail(ctx, M3_ERR_NULL, "dy is required");
  {
    const int rc = m3::take_device_flag(ctx, "in an earlier call, seen on entry to m3_scan_backward");
    if (rc != M3_OK) return rc;
  }
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  if (saved->path == M3_PATH_TENSOR) return tc_backward_call(ctx, saved, in, grad_mask, grads);
  const m3::Dims& d = saved->dims;
  const size_t bytes = m3::generic_bwd_ws_layout(d, nullptr, nullptr);
  char* base = nullptr;
  M3_CUDA(ctx, m3::scratch_alloc(ctx, reinterpret_cast<void**>(&base), bytes, ctx->stream));
  m3::GenericBwdWs bw;
  m3::generic_bwd_ws_layout(d, &bw, base);
  cudaError_t e = m3::generic_backward(ctx->stream, d, saved->desc, saved->gws, bw, *in, grad_mask, *grads,
                                       &ctx->launches);
  cudaError_t e2 = cudaFreeAsync(base, ctx->stream);
  if (e != cudaSuccess) return cuda_fail(ctx, e, "generic backward");
  if (e2 != cudaSuccess) return cuda_fail(ctx, e2, "cudaFreeAsync");
  return M3_OK;
}

int m3_saved_free(m3_ctx* ctx, m3_saved* saved) {
  if (!ctx) return M3_ERR_NULL;
  if (!saved) return M3_OK;
  cudaSetDevice(ctx->device);
  // Freed in the order of the stream the forward (and, by the tape's order, the backward) ran on: the
  // context may have been rebound to another stream since, and the pool must not hand this block
  // to a later allocation while kernels of the old stream still read it.
  cudaError_t e = saved->ws_base ? cudaFreeAsync(saved->ws_base, saved->stream ? saved->stream : ctx->stream) : cudaSuccess;
  delete saved;
  if (e != cudaSuccess) return cuda_fail(ctx, e, "cudaFreeAsync");
  return M3_OK;
}

}  // extern "C"
