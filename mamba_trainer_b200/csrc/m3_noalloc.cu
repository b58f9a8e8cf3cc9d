// m3_scan_forward_noalloc: the forward scan for callers that must not allocate.
//
// Some hosts of this library cannot ask the driver for device memory while they run:
// a serving process that handed the whole GPU to its own arena at start-up and treats
// any later driver allocation as a fault; a latency-bound decode loop for which the
// implicit synchronisation of an allocation is unacceptable; code running inside a
// region where allocation calls are simply not permitted.  m3_scan_forward takes its
// scratch (head-major copies, chunk states) from the stream-ordered pool, which such a
// caller cannot afford.  This entry point runs the same kernels on a fixed block of
// device memory that is part of the library image instead.
//
// The price: every GPU that loads the library holds M3_NOALLOC_SCRATCH_BYTES until the
// process exits, requests needing more are refused, and all calls share the block.
#include <mutex>

#include "m3_internal.h"
#include "m3_tc.h"

namespace {

// The scratch itself.  In host code this name is only a handle for the runtime's symbol
// table, never a device address: the address is looked up once per device below.
static __device__ __align__(256) unsigned char g_noalloc_scratch[M3_NOALLOC_SCRATCH_BYTES];

// Device code may name the array directly.  This kernel is never launched; it exists so
// that the array is referenced from device code and stays in the image.
__global__ void k_noalloc_anchor(unsigned char* out) { out[0] = g_noalloc_scratch[0]; }

constexpr int kMaxDevices = 64;
std::mutex g_mu;
char* g_scratch_addr[kMaxDevices] = {nullptr};

// Device address of the scratch on `device`, which must be the current device.
cudaError_t scratch_address(int device, char** out) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (!g_scratch_addr[device]) {
    void* p = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[device] = static_cast<char*>(p);
  }
  *out = g_scratch_addr[device];
  return cudaSuccess;
}

}  // namespace

extern "C" int m3_scan_forward_noalloc(m3_ctx* ctx, const m3_scan_desc* desc, const m3_scan_out* out) {
  if (!ctx) return M3_ERR_NULL;
  if (!desc || !out) return m3::fail(ctx, M3_ERR_NULL, "descriptor and outputs are required");
  m3::Dims d;
  int rc = m3::make_dims(ctx, *desc, &d);
  if (rc != M3_OK) return rc;
  if (d.T == 0) return m3_scan_forward(ctx, desc, out, nullptr);  // that branch only copies the state
  if (!out->y) return m3::fail(ctx, M3_ERR_NULL, "y is required");
  // Shapes the tensor-core family serves need no scratch at all when nothing is kept for a backward
  // pass: that call allocates nothing either, and is the fast one.
  if (m3::tc_supported(*desc) && !d.raw && desc->path != M3_PATH_GENERIC) {
    ctx->no_scratch = true;  // whole stripes: no hand-over scratch between time segments
    const int rc = m3_scan_forward(ctx, desc, out, nullptr);
    ctx->no_scratch = false;
    return rc;
  }
  if (ctx->device < 0 || ctx->device >= kMaxDevices)
    return m3::fail(ctx, M3_ERR_UNSUPPORTED, "device ordinal %d outside the table of %d", ctx->device, kMaxDevices);
  const size_t need = m3::generic_ws_layout(d, nullptr, nullptr);
  if (need > (size_t)M3_NOALLOC_SCRATCH_BYTES)
    return m3::fail(ctx, M3_ERR_UNSUPPORTED,
                    "this scan needs %zu bytes of scratch; the built-in block holds %zu - use m3_scan_forward",
                    need, (size_t)M3_NOALLOC_SCRATCH_BYTES);
  cudaError_t e = cudaSetDevice(ctx->device);
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "cudaSetDevice");
  char* base = nullptr;
  e = scratch_address(ctx->device, &base);
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "cudaGetSymbolAddress");
  m3::GenericWs ws;
  m3::generic_ws_layout(d, &ws, base);
  // Every scratch region is written in full before it is read (padded rows are stored
  // as zeros, every chunk-state slot is produced by the chunk kernels), so nothing left
  // behind by the previous call needs clearing.
  e = m3::generic_forward(ctx->stream, d, *desc, *out, ws, &ctx->launches);
  if (e != cudaSuccess) return m3::cuda_fail(ctx, e, "forward on built-in scratch");
  return M3_OK;
}
