// Forward + backward of the scan for callers whose tensors live in HOST memory.
//
// Every batch row is an independent recurrence, so a call is cut into batch slices that go
// through three stages on three streams: host-to-device copy (copy stream), forward + backward
// (the context's stream), device-to-host copy (a second copy stream).  The staging buffers and
// the device result buffers exist twice, so slice i+1 is copied in and slice i-1 copied out while
// slice i computes; the same ordering carries across consecutive runs, so a stream of runs keeps
// both PCIe directions busy.  Results equal one call on the whole batch; the per-head parameter
// gradients are summed over the slices in a fixed order by a small kernel.
#include <new>
#include <vector>

#include "m3_internal.h"

#define M3_CUDA(ctx, call)                                       \
  do {                                                           \
    cudaError_t e_ = (call);                                     \
    if (e_ != cudaSuccess) return m3::cuda_fail(ctx, e_, #call); \
  } while (0)
#define M3_TRY(call)           \
  do {                         \
    int rc_ = (call);          \
    if (rc_ != M3_OK) return rc_; \
  } while (0)

namespace {

constexpr int kSets = 3;    // staging / result buffer sets: one copying in, one computing, one copying out
constexpr int kTickets = 8; // completion events kept for m3_host_pipe_wait

struct DevSet {
  void *x = nullptr, *b = nullptr, *c = nullptr, *dt = nullptr, *lam = nullptr, *theta = nullptr, *dy = nullptr;
  void *y = nullptr, *dx = nullptr, *db = nullptr, *dc = nullptr, *ddt = nullptr, *dlam = nullptr, *dtheta = nullptr;
  cudaEvent_t in_ready = nullptr, computed = nullptr, out_done = nullptr;
  bool used = false;
};

// out[h] = sum over slices of part[s][h], in slice order.
__global__ void k_sum_slices(const float* __restrict__ part, float* __restrict__ out, int slices, int heads) {
  const int h = blockIdx.x * blockDim.x + threadIdx.x;
  if (h >= heads) return;
  float s = 0.0f;
  for (int i = 0; i < slices; ++i) s += part[(size_t)i * heads + h];
  out[h] = s;
}

}  // namespace

struct m3_host_pipe {
  m3_ctx* ctx = nullptr;
  m3_scan_desc shape{};
  int slices = 0, width = 0;
  std::vector<int> bounds;
  size_t row_x = 0, row_bc = 0, row_tok = 0, row_theta = 0;  // bytes of one batch row
  DevSet set[kSets];
  float *part_alog = nullptr, *part_dskip = nullptr;  // [slices][heads]
  float *sum_alog = nullptr, *sum_dskip = nullptr;    // [heads]
  cudaStream_t s_in = nullptr, s_out = nullptr;
  cudaEvent_t sums_ready = nullptr, sums_out = nullptr;
  bool sums_used = false;
  cudaEvent_t ticket[kTickets] = {};
  uint64_t runs = 0, slices_done = 0;
};

namespace {

int free_pipe(m3_host_pipe* p) {
  if (!p) return M3_OK;
  cudaSetDevice(p->ctx->device);
  if (p->s_in) cudaStreamSynchronize(p->s_in);
  if (p->s_out) cudaStreamSynchronize(p->s_out);
  cudaStreamSynchronize(p->ctx->stream);
  for (DevSet& s : p->set) {
    void* bufs[] = {s.x, s.b, s.c, s.dt, s.lam, s.theta, s.dy, s.y, s.dx, s.db, s.dc, s.ddt, s.dlam, s.dtheta};
    for (void* q : bufs)
      if (q) cudaFree(q);
    cudaEvent_t evs[] = {s.in_ready, s.computed, s.out_done};
    for (cudaEvent_t e : evs)
      if (e) cudaEventDestroy(e);
  }
  float* fb[] = {p->part_alog, p->part_dskip, p->sum_alog, p->sum_dskip};
  for (float* q : fb)
    if (q) cudaFree(q);
  if (p->sums_ready) cudaEventDestroy(p->sums_ready);
  if (p->sums_out) cudaEventDestroy(p->sums_out);
  for (cudaEvent_t e : p->ticket)
    if (e) cudaEventDestroy(e);
  if (p->s_in) cudaStreamDestroy(p->s_in);
  if (p->s_out) cudaStreamDestroy(p->s_out);
  delete p;
  return M3_OK;
}

int build_pipe(m3_host_pipe* p) {
  m3_ctx* ctx = p->ctx;
  const m3_scan_desc& s = p->shape;
  const size_t es = s.dtype == M3_BF16 ? 2 : 4;
  const size_t th = (size_t)s.seq * s.heads;
  p->row_x = th * s.head_dim * s.rank * es;
  p->row_bc = th * s.d_state * s.rank * es;
  p->row_tok = th * es;
  p->row_theta = th * (s.d_state / 2) * es;
  const bool learned = s.discretization == M3_LEARNED_TRAPEZOID, rot = s.dynamics == M3_ROTATIONAL;
  const size_t w = (size_t)p->width;
  M3_CUDA(ctx, cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking));
  M3_CUDA(ctx, cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
  for (DevSet& d : p->set) {
    M3_CUDA(ctx, cudaMalloc(&d.x, w * p->row_x));
    M3_CUDA(ctx, cudaMalloc(&d.b, w * p->row_bc));
    M3_CUDA(ctx, cudaMalloc(&d.c, w * p->row_bc));
    M3_CUDA(ctx, cudaMalloc(&d.dt, w * p->row_tok));
    M3_CUDA(ctx, cudaMalloc(&d.dy, w * p->row_x));
    M3_CUDA(ctx, cudaMalloc(&d.y, w * p->row_x));
    M3_CUDA(ctx, cudaMalloc(&d.dx, w * p->row_x));
    M3_CUDA(ctx, cudaMalloc(&d.db, w * p->row_bc));
    M3_CUDA(ctx, cudaMalloc(&d.dc, w * p->row_bc));
    M3_CUDA(ctx, cudaMalloc(&d.ddt, w * p->row_tok));
    if (learned) {
      M3_CUDA(ctx, cudaMalloc(&d.lam, w * p->row_tok));
      M3_CUDA(ctx, cudaMalloc(&d.dlam, w * p->row_tok));
    }
    if (rot) {
      M3_CUDA(ctx, cudaMalloc(&d.theta, w * p->row_theta));
      M3_CUDA(ctx, cudaMalloc(&d.dtheta, w * p->row_theta));
    }
    M3_CUDA(ctx, cudaEventCreateWithFlags(&d.in_ready, cudaEventDisableTiming));
    M3_CUDA(ctx, cudaEventCreateWithFlags(&d.computed, cudaEventDisableTiming));
    M3_CUDA(ctx, cudaEventCreateWithFlags(&d.out_done, cudaEventDisableTiming));
  }
  const size_t ph = (size_t)p->slices * s.heads * sizeof(float);
  M3_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&p->part_alog), ph));
  M3_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&p->part_dskip), ph));
  M3_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&p->sum_alog), s.heads * sizeof(float)));
  M3_CUDA(ctx, cudaMalloc(reinterpret_cast<void**>(&p->sum_dskip), s.heads * sizeof(float)));
  M3_CUDA(ctx, cudaEventCreateWithFlags(&p->sums_ready, cudaEventDisableTiming));
  M3_CUDA(ctx, cudaEventCreateWithFlags(&p->sums_out, cudaEventDisableTiming));
  for (cudaEvent_t& e : p->ticket) M3_CUDA(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  return M3_OK;
}

}  // namespace

extern "C" {

int m3_host_alloc(size_t bytes, void** out) {
  if (!out) return M3_ERR_NULL;
  return cudaHostAlloc(out, bytes ? bytes : 1, cudaHostAllocDefault) == cudaSuccess ? M3_OK : M3_ERR_CUDA;
}

int m3_host_free(void* ptr) {
  if (!ptr) return M3_OK;
  return cudaFreeHost(ptr) == cudaSuccess ? M3_OK : M3_ERR_CUDA;
}

int m3_host_pipe_create(m3_ctx* ctx, const m3_scan_desc* shape, int slices, m3_host_pipe** out) {
  if (!ctx || !shape || !out) return M3_ERR_NULL;
  *out = nullptr;
  m3::Dims d;
  m3_scan_desc probe = *shape;
  probe.h0 = probe.last_u0 = probe.angle0 = nullptr;
  probe.a_raw = probe.g_raw = probe.w_raw = nullptr;
  probe.want_state = 0;
  {  // validate the extents with placeholder pointers: only a_log / d_skip are read from `shape`
    m3_scan_desc v = probe;
    const void* any = shape->a_log;
    v.x = v.b = v.c = v.dt = any;
    v.lambda = shape->discretization == M3_LEARNED_TRAPEZOID ? any : nullptr;
    v.theta = shape->dynamics == M3_ROTATIONAL ? any : nullptr;
    M3_TRY(m3::make_dims(ctx, v, &d));
  }
  if (!shape->a_log) return m3::fail(ctx, M3_ERR_NULL, "m3_host_pipe_create: a_log is required");
  if (shape->batch < 1 || shape->seq < 1) return m3::fail(ctx, M3_ERR_SHAPE, "m3_host_pipe_create: empty batch or sequence");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  m3_host_pipe* p = new (std::nothrow) m3_host_pipe();
  if (!p) return m3::fail(ctx, M3_ERR_CUDA, "out of host memory");
  p->ctx = ctx;
  p->shape = probe;
  p->slices = slices < 1 ? 1 : (slices > shape->batch ? shape->batch : slices);
  p->bounds.resize(p->slices + 1);
  for (int i = 0; i <= p->slices; ++i) p->bounds[i] = (int)(((long long)i * shape->batch + p->slices / 2) / p->slices);
  p->bounds[0] = 0;
  p->bounds[p->slices] = shape->batch;
  for (int i = 0; i < p->slices; ++i) p->width = p->bounds[i + 1] - p->bounds[i] > p->width ? p->bounds[i + 1] - p->bounds[i] : p->width;
  const int rc = build_pipe(p);
  if (rc != M3_OK) {
    free_pipe(p);
    return rc;
  }
  *out = p;
  return M3_OK;
}

int m3_host_pipe_destroy(m3_host_pipe* pipe) { return free_pipe(pipe); }

int m3_host_pipe_run(m3_host_pipe* p, const m3_host_in* in, const m3_host_out* out, uint64_t* ticket) {
  if (!p || !in || !out) return M3_ERR_NULL;
  m3_ctx* ctx = p->ctx;
  const m3_scan_desc& s = p->shape;
  const bool learned = s.discretization == M3_LEARNED_TRAPEZOID, rot = s.dynamics == M3_ROTATIONAL;
  if (!in->x || !in->b || !in->c || !in->dt || !in->dy || (learned && !in->lambda) || (rot && !in->theta))
    return m3::fail(ctx, M3_ERR_NULL, "m3_host_pipe_run: a required host input is NULL");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  const cudaStream_t main = ctx->stream;
  auto at = [](const void* base, size_t off) { return static_cast<const char*>(base) + off; };
  auto at_w = [](void* base, size_t off) { return static_cast<char*>(base) + off; };
  for (int i = 0; i < p->slices; ++i) {
    DevSet& d = p->set[p->slices_done % kSets];
    const size_t lo = (size_t)p->bounds[i], n = (size_t)(p->bounds[i + 1] - p->bounds[i]);
    // ---- stage 1: host -> device, once the slice that used these buffers has computed -------------
    if (d.used) M3_CUDA(ctx, cudaStreamWaitEvent(p->s_in, d.computed, 0));
    M3_CUDA(ctx, cudaMemcpyAsync(d.x, at(in->x, lo * p->row_x), n * p->row_x, cudaMemcpyHostToDevice, p->s_in));
    M3_CUDA(ctx, cudaMemcpyAsync(d.b, at(in->b, lo * p->row_bc), n * p->row_bc, cudaMemcpyHostToDevice, p->s_in));
    M3_CUDA(ctx, cudaMemcpyAsync(d.c, at(in->c, lo * p->row_bc), n * p->row_bc, cudaMemcpyHostToDevice, p->s_in));
    M3_CUDA(ctx, cudaMemcpyAsync(d.dt, at(in->dt, lo * p->row_tok), n * p->row_tok, cudaMemcpyHostToDevice, p->s_in));
    if (learned)
      M3_CUDA(ctx, cudaMemcpyAsync(d.lam, at(in->lambda, lo * p->row_tok), n * p->row_tok, cudaMemcpyHostToDevice, p->s_in));
    if (rot)
      M3_CUDA(ctx, cudaMemcpyAsync(d.theta, at(in->theta, lo * p->row_theta), n * p->row_theta, cudaMemcpyHostToDevice, p->s_in));
    M3_CUDA(ctx, cudaMemcpyAsync(d.dy, at(in->dy, lo * p->row_x), n * p->row_x, cudaMemcpyHostToDevice, p->s_in));
    M3_CUDA(ctx, cudaEventRecord(d.in_ready, p->s_in));
    // ---- stage 2: forward + backward, once the inputs are in and the old results are out -----------
    M3_CUDA(ctx, cudaStreamWaitEvent(main, d.in_ready, 0));
    if (d.used) M3_CUDA(ctx, cudaStreamWaitEvent(main, d.out_done, 0));
    m3_scan_desc sd = s;
    sd.batch = (int32_t)n;
    sd.x = d.x; sd.b = d.b; sd.c = d.c; sd.dt = d.dt; sd.lambda = d.lam; sd.theta = d.theta;
    m3_scan_out so{};
    so.y = d.y;
    m3_saved* saved = nullptr;
    M3_TRY(m3_scan_forward(ctx, &sd, &so, &saved));
    m3_scan_bwd_in bi{};
    bi.dy = d.dy;
    m3_scan_grads g{};
    uint32_t mask = M3_GRAD_X | M3_GRAD_B | M3_GRAD_C | M3_GRAD_DT | M3_GRAD_A_LOG;
    g.dx = d.dx; g.db = d.db; g.dc = d.dc; g.ddt = d.ddt;
    g.da_log = p->part_alog + (size_t)i * s.heads;
    if (learned) { g.dlambda = d.dlam; mask |= M3_GRAD_LAMBDA; }
    if (rot) { g.dtheta = d.dtheta; mask |= M3_GRAD_THETA; }
    if (s.d_skip) { g.dd_skip = p->part_dskip + (size_t)i * s.heads; mask |= M3_GRAD_D_SKIP; }
    const int rb = m3_scan_backward(ctx, saved, &bi, mask, &g);
    const int rf = m3_saved_free(ctx, saved);
    M3_TRY(rb);
    M3_TRY(rf);
    M3_CUDA(ctx, cudaEventRecord(d.computed, main));
    // ---- stage 3: device -> host ------------------------------------------------------------------
    M3_CUDA(ctx, cudaStreamWaitEvent(p->s_out, d.computed, 0));
    if (out->y) M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->y, lo * p->row_x), d.y, n * p->row_x, cudaMemcpyDeviceToHost, p->s_out));
    if (out->dx) M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->dx, lo * p->row_x), d.dx, n * p->row_x, cudaMemcpyDeviceToHost, p->s_out));
    if (out->db) M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->db, lo * p->row_bc), d.db, n * p->row_bc, cudaMemcpyDeviceToHost, p->s_out));
    if (out->dc) M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->dc, lo * p->row_bc), d.dc, n * p->row_bc, cudaMemcpyDeviceToHost, p->s_out));
    if (out->ddt) M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->ddt, lo * p->row_tok), d.ddt, n * p->row_tok, cudaMemcpyDeviceToHost, p->s_out));
    if (learned && out->dlambda)
      M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->dlambda, lo * p->row_tok), d.dlam, n * p->row_tok, cudaMemcpyDeviceToHost, p->s_out));
    if (rot && out->dtheta)
      M3_CUDA(ctx, cudaMemcpyAsync(at_w(out->dtheta, lo * p->row_theta), d.dtheta, n * p->row_theta, cudaMemcpyDeviceToHost, p->s_out));
    M3_CUDA(ctx, cudaEventRecord(d.out_done, p->s_out));
    d.used = true;
    ++p->slices_done;
  }
  // ---- per-head parameter gradients: fixed-order sum over the slices, then out ------------------------
  if (p->sums_used) M3_CUDA(ctx, cudaStreamWaitEvent(main, p->sums_out, 0));
  const int blocks = (s.heads + 127) / 128;
  k_sum_slices<<<blocks, 128, 0, main>>>(p->part_alog, p->sum_alog, p->slices, s.heads);
  ++ctx->launches;
  if (s.d_skip) {
    k_sum_slices<<<blocks, 128, 0, main>>>(p->part_dskip, p->sum_dskip, p->slices, s.heads);
    ++ctx->launches;
  }
  M3_CUDA(ctx, cudaGetLastError());
  M3_CUDA(ctx, cudaEventRecord(p->sums_ready, main));
  M3_CUDA(ctx, cudaStreamWaitEvent(p->s_out, p->sums_ready, 0));
  if (out->da_log)
    M3_CUDA(ctx, cudaMemcpyAsync(out->da_log, p->sum_alog, s.heads * sizeof(float), cudaMemcpyDeviceToHost, p->s_out));
  if (s.d_skip && out->dd_skip)
    M3_CUDA(ctx, cudaMemcpyAsync(out->dd_skip, p->sum_dskip, s.heads * sizeof(float), cudaMemcpyDeviceToHost, p->s_out));
  M3_CUDA(ctx, cudaEventRecord(p->sums_out, p->s_out));
  p->sums_used = true;
  M3_CUDA(ctx, cudaEventRecord(p->ticket[p->runs % kTickets], p->s_out));
  if (ticket) *ticket = p->runs;
  ++p->runs;
  return M3_OK;
}

int m3_host_pipe_wait(m3_host_pipe* p, uint64_t ticket) {
  if (!p) return M3_ERR_NULL;
  m3_ctx* ctx = p->ctx;
  if (ticket >= p->runs) return m3::fail(ctx, M3_ERR_CONFIG, "m3_host_pipe_wait: no such run");
  M3_CUDA(ctx, cudaSetDevice(ctx->device));
  // A slot reused by a later run waits for that later run, which finishes after this one.
  M3_CUDA(ctx, cudaEventSynchronize(p->ticket[ticket % kTickets]));
  {
    const int rc = m3::take_device_flag(ctx, "in a run of the host pipeline that has finished by now");
    if (rc != M3_OK) return rc;
  }
  return M3_OK;
}

}  // extern "C"
