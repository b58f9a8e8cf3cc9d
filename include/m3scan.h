/*
 * m3scan - C ABI of the fused Mamba-3 SSD scan for NVIDIA B200 (sm_100a).
 *
 * One fused operator (forward + hand-written adjoint) replaces the scan that the
 * mamba3 crate composes from differentiable primitives.  Every entry point below
 * names the reference interface it stands in for (paths are relative to the
 * mamba3 crate root).  All pointers in descriptors are DEVICE pointers unless
 * stated otherwise; tensors are dense row-major in the reference's own layouts;
 * the library never writes to an input buffer.
 *
 * Threading: an m3_ctx is bound to one device and one stream and must be used by
 * one host thread at a time; different contexts are independent.  All work is
 * enqueued on the context's stream and returns without waiting; only
 * m3_download and m3_sync block (the reference's only blocking call is
 * Tensor::to_data, src/tensor/base.rs:92-96).
 *
 * Errors: every call returns an m3_status; nothing aborts or throws across the
 * boundary.  m3_last_error gives the message of the last failure on a context.
 * The codes mirror the reference's Error enum (src/error.rs:9-48).
 */
#ifndef M3SCAN_H
#define M3SCAN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct m3_ctx m3_ctx;     /* device + stream + caches            */
typedef struct m3_saved m3_saved; /* what forward keeps for the adjoint  */

typedef enum {
  M3_OK = 0,
  M3_ERR_SHAPE = 1,       /* Error::Shape  - inconsistent extents              */
  M3_ERR_RANK = 2,        /* Error::Rank   - kept for the host mirror          */
  M3_ERR_CONFIG = 3,      /* Error::Config - e.g. odd d_state with rotation    */
  M3_ERR_UNSUPPORTED = 4, /* Error::Unsupported                                */
  M3_ERR_CUDA = 5,        /* a CUDA runtime call failed                        */
  M3_ERR_TIMEOUT = 6,     /* a bounded device-side wait gave up                */
  M3_ERR_NULL = 7         /* a required pointer was NULL                       */
} m3_status;

/* Element type of x, b, c, dt, lambda, theta, y and their gradients
 * (FloatElem, src/backend.rs; f32 and bf16 are the two the build serves).
 * a_log, d_skip, the carried state and their gradients are always float. */
typedef enum { M3_F32 = 0, M3_BF16 = 1 } m3_dtype;

/* Discretization, src/ssm/config.rs:18-42.  Euler and Trapezoid use the constant
 * lambda of fixed_lambda() (:30-36) and ignore desc.lambda (it may be NULL). */
typedef enum { M3_EULER = 0, M3_TRAPEZOID = 1, M3_LEARNED_TRAPEZOID = 2 } m3_discretization;

/* StateDynamics, src/ssm/config.rs:45-56.  Rotational needs theta and even d_state. */
typedef enum { M3_REAL = 0, M3_ROTATIONAL = 1 } m3_dynamics;

/* Which kernel family runs.  AUTO picks the tensor-core family when the shape is
 * one it serves and the generic family otherwise. */
typedef enum { M3_PATH_AUTO = 0, M3_PATH_GENERIC = 1, M3_PATH_TENSOR = 2 } m3_path;

/* ScanInputs, src/ssm/scan.rs:361-385.  rank is SsmMode::rank() (config.rs:74-79). */
typedef struct {
  int32_t batch, seq, heads, head_dim, d_state, rank;
  int32_t chunk;          /* ScanInputs::chunk_size; clamped to [1, seq] (scan.rs:146) */
  int32_t dtype;          /* m3_dtype */
  int32_t discretization; /* m3_discretization */
  int32_t dynamics;       /* m3_dynamics */
  int32_t want_state;     /* ScanInputs::want_state */
  int32_t path;           /* m3_path */
  int32_t reverse_heads;  /* the LAST reverse_heads heads walk time right to left: the fused form of
                           * the bidirectional mixer (src/models/mamba3.rs:97-112), which reverses the
                           * backward half of x, B, C, dt, lambda, theta in time before the scan
                           * (:352-370) and the backward heads' y after it (:548-556).  Here those
                           * heads read and write their tokens in reverse order instead; inputs,
                           * outputs and gradients all stay in ordinary time.  0 = none; heads/2 for
                           * the bidirectional mixer.  The carried state of such a head enters at the
                           * last token and the returned one is the state after token 0. */
  int32_t reserved0;      /* must be 0 */
  const void *x;          /* [batch, seq, heads, head_dim, rank] */
  const void *b;          /* [batch, seq, heads, d_state, rank]  */
  const void *c;          /* [batch, seq, heads, d_state, rank]  */
  const void *dt;         /* [batch, seq, heads], positive       */
  const void *lambda;     /* [batch, seq, heads] in [0,1]; NULL unless learned */
  const void *theta;      /* [batch, seq, heads, d_state/2]; NULL for real dynamics */
  const float *a_log;     /* [heads], A = -exp(a_log)            */
  const float *d_skip;    /* [heads] or NULL                     */
  const float *h0;        /* SsmState::h      [batch, heads, head_dim, d_state] or NULL */
  const float *last_u0;   /* SsmState::last_u [batch, heads, head_dim, d_state] or NULL */
  const float *angle0;    /* SsmState::angle  [batch, heads, d_state/2] or NULL */
  /* ssd_chunked, src/ssm/scan.rs:116-126: the caller supplies the log decay a = dt*A and the
   * diagonal / off-diagonal weights g, w themselves, all [batch, seq, heads].  When a_raw is
   * set (then g_raw and w_raw must be too) dt, lambda and a_log are not read, theta must be
   * NULL, h0 alone is the boundary value carried in (last_u0 is not read) and no last_u is
   * produced.  The generic kernel family serves this form. */
  const void *a_raw, *g_raw, *w_raw;
} m3_scan_desc;

/* ScanOutput, src/ssm/scan.rs:446-452.  Caller-allocated.  The three state
 * buffers are written only when want_state is set (NULL skips that one). */
typedef struct {
  void *y;        /* [batch, seq, heads, head_dim, rank], desc.dtype */
  float *h;       /* [batch, heads, head_dim, d_state] */
  float *last_u;  /* [batch, heads, head_dim, d_state] */
  float *angle;   /* [batch, heads, d_state/2] (rotational only) */
} m3_scan_out;

/* Upstream gradients handed to the adjoint: the argument of the BackwardRule
 * (src/autograd/graph.rs:61-62) for y, plus the optional gradients that reach the
 * returned SsmState (states are Vars in the reference, scan.rs:294-302). */
typedef struct {
  const void *dy;        /* like y */
  const float *dh;       /* like h, or NULL */
  const float *dlast_u;  /* like last_u, or NULL */
  const float *dangle;   /* like angle, or NULL */
} m3_scan_bwd_in;

/* Bits of grad_mask: the `wanted` slice of Var::record_with_mask
 * (src/autograd/var.rs:169-204).  A cleared bit (or a NULL pointer) skips the store. */
enum {
  M3_GRAD_X = 1u << 0, M3_GRAD_B = 1u << 1, M3_GRAD_C = 1u << 2, M3_GRAD_DT = 1u << 3,
  M3_GRAD_A_LOG = 1u << 4, M3_GRAD_LAMBDA = 1u << 5, M3_GRAD_THETA = 1u << 6,
  M3_GRAD_D_SKIP = 1u << 7, M3_GRAD_H0 = 1u << 8, M3_GRAD_LAST_U0 = 1u << 9,
  M3_GRAD_ANGLE0 = 1u << 10, M3_GRAD_ALL = 0x7ffu
};

/* Caller-allocated gradient buffers, shaped like the corresponding inputs. */
typedef struct {
  void *dx, *db, *dc, *ddt, *dlambda, *dtheta;   /* desc.dtype */
  float *da_log, *dd_skip;                        /* [heads]    */
  float *dh0, *dlast_u0, *dangle0;                /* float      */
  void *da_raw, *dg_raw, *dw_raw;                 /* desc.dtype; written instead of ddt / dlambda /
                                                     da_log when the forward used a_raw, g_raw, w_raw */
} m3_scan_grads;

/* Library version string "major.minor.patch". */
const char *m3_version(void);

/* Device<R>::default() / Device::new, src/backend.rs: bind a context to a device
 * ordinal.  The context starts on a stream of its own. */
int m3_ctx_create(int device, m3_ctx **out);
int m3_ctx_destroy(m3_ctx *ctx);
/* Run on a caller-owned cudaStream_t instead (NULL = the legacy default stream). */
int m3_ctx_set_stream(m3_ctx *ctx, void *cuda_stream);
/* Block until everything enqueued on the context has finished.  Returns M3_ERR_TIMEOUT
 * (and clears the condition) if a kernel's bounded wait gave up since the last report:
 * every device-side wait of the library has an iteration limit, after which the kernel
 * raises a flag and returns instead of spinning.  The flag lives in host memory mapped
 * into the device, so m3_scan_forward / m3_scan_backward / m3_host_pipe_wait also look
 * at it on entry, at no cost, and report a wait that gave up in an EARLIER call the same
 * way (the reference has no counterpart: its kernels never wait on one another). */
int m3_sync(m3_ctx *ctx);
/* Iteration limit of those bounded waits for calls made through this context; 0 restores
 * the default (2^18: a wait polls its mbarrier at most limit - 1 times, far beyond any
 * healthy wait).  Diagnostic: a limit of 1 makes every wait of the tensor-core kernels
 * give up at once, which is how the failure path is exercised without a fault.  No
 * counterpart in the reference. */
int m3_ctx_set_wait_limit(m3_ctx *ctx, uint32_t iterations);
/* Message of the last failure on this context ("" if none).  Never NULL. */
const char *m3_last_error(const m3_ctx *ctx);
/* Kernels launched through this context so far (the reference's launch_count(),
 * src/backend.rs:231-281). */
uint64_t m3_launch_count(const m3_ctx *ctx);

/* Device buffers owned by the library: Tensor::zeros / from_f32 / to_data,
 * src/tensor/base.rs:21-199. */
int m3_alloc(m3_ctx *ctx, size_t bytes, void **out);
int m3_free(m3_ctx *ctx, void *ptr);
int m3_upload(m3_ctx *ctx, void *dst_device, const void *src_host, size_t bytes);
int m3_download(m3_ctx *ctx, void *dst_host, const void *src_device, size_t bytes);

/* mamba3_scan, src/ssm/scan.rs:458-618 (with ssd_chunked :116-291 folded in).
 * `saved` may be NULL (inference, no rule is built: var.rs:174-180); otherwise it
 * receives a handle the caller frees with m3_saved_free after the last backward.
 * The saved context refers to the input buffers of `desc`: keep them alive and
 * unchanged until then (the reference's closure holds clones, var.rs:210-216).
 * The tensor-core kernel family moves rows as 16-byte vectors: with M3_PATH_AUTO a call whose
 * x, b, c, theta or y is not 16-byte aligned runs the generic family instead (M3_PATH_TENSOR
 * refuses it), and the backward of a forward that ran the tensor-core family needs 16-byte
 * aligned dy, dx, db, dc and dtheta (M3_ERR_UNSUPPORTED otherwise). */
int m3_scan_forward(m3_ctx *ctx, const m3_scan_desc *desc, const m3_scan_out *out,
                    m3_saved **saved);

/* The BackwardRule of the fused node (src/autograd/graph.rs:61-62).  It does not
 * consume `saved`, so it may run again (backward_retain, var.rs:218-221). */
int m3_scan_backward(m3_ctx *ctx, const m3_saved *saved, const m3_scan_bwd_in *in,
                     uint32_t grad_mask, const m3_scan_grads *grads);

int m3_saved_free(m3_ctx *ctx, m3_saved *saved);

/* mamba3_step, src/ssm/scan.rs:649-712: one decoding step.  Shapes are ScanInputs' with seq = 1
 * and no time axis: x [batch, heads, head_dim, rank]; b, c [batch, heads, d_state, rank]; dt,
 * lambda [batch, heads]; theta [batch, heads, d_state/2]; the state is read from (h, last_u,
 * angle) and the new one written to m3_step_out (distinct buffers: inputs are never written). */
typedef struct {
  int32_t batch, heads, head_dim, d_state, rank;
  int32_t dtype, discretization, dynamics;
  const void *x, *b, *c, *dt, *lambda, *theta;
  const float *a_log, *d_skip;
  const float *h, *last_u, *angle;   /* angle may be NULL (zero) */
} m3_step_desc;
typedef struct {
  void *y;                            /* [batch, heads, head_dim, rank], desc.dtype */
  float *h, *last_u, *angle;          /* the state after the step */
} m3_step_out;
int m3_step_forward(m3_ctx *ctx, const m3_step_desc *desc, const m3_step_out *out);

/* No counterpart in the reference.  The forward scan (inference form: no saved
 * context) for hosts that must not allocate device memory while they run - a server
 * that gave the whole GPU to its own arena at start-up, a latency-bound decode loop
 * that cannot take an allocation's implicit synchronisation, any region where
 * allocation calls are off limits.  It calls no cudaMalloc / cudaFree and no
 * allocating library routine: the scratch m3_scan_forward would take from the
 * stream-ordered pool is a block of M3_NOALLOC_SCRATCH_BYTES built into the library
 * image (so every GPU that loads the library holds that much until the process
 * exits).  Inputs and outputs are still the caller's.  Descriptors whose scratch
 * (m3_scan_scratch_bytes(desc, 0)) exceeds the block are refused with
 * M3_ERR_UNSUPPORTED.  Shapes the tensor-core family serves run there unless
 * desc->path says M3_PATH_GENERIC: with nothing kept for a backward pass that family
 * needs no scratch at all; everything else runs the generic family on the block.
 * The first call on each device looks up the block's device address (with that
 * device current), and - CUDA loads a library's kernels and file-scope device arrays
 * when they are first touched - it is also the call during which the driver maps the
 * block and the kernels it launches: make one warm-up call per device and element type
 * at start-up, before the arena is sized and before any stream capture; from the
 * second call on nothing is allocated by anyone.  All calls on a device share the
 * block and it keeps the previous call's contents (nothing in it needs to start at
 * zero): two calls whose kernels overlap on the GPU race - keep them on one stream or
 * order them yourself. */
#define M3_NOALLOC_SCRATCH_BYTES (16u << 20)
int m3_scan_forward_noalloc(m3_ctx *ctx, const m3_scan_desc *desc, const m3_scan_out *out);

/* Forward + backward for tensors that live in HOST memory: the reference's
 * Tensor::from_f32 ... mamba3_scan ... backward ... to_data sequence
 * (src/tensor/base.rs:21-199 around src/ssm/scan.rs:458-618) for a caller that owns
 * host buffers only.  The call is cut into `slices` contiguous batch slices (every
 * batch row is an independent recurrence) that move through three stages on three
 * streams - host-to-device copy, forward + backward on the context's stream,
 * device-to-host copy - with two sets of device buffers, so the copies of one slice
 * hide behind the kernels and the opposite-direction copies of its neighbours, within
 * a run and across consecutive runs.  Results equal one call on the whole batch; the
 * per-head gradients are summed over the slices in slice order.
 *
 * m3_host_in / m3_host_out hold HOST pointers, shaped like the corresponding fields of
 * m3_scan_desc / m3_scan_out / m3_scan_grads; they should be page-locked
 * (m3_host_alloc, or any cudaHostAlloc / cudaHostRegister memory) or the copies do not
 * overlap.  `shape` gives the extents, dtype, discretization, dynamics, chunk and path
 * and the DEVICE pointers a_log and d_skip (d_skip may be NULL); its other pointers are
 * ignored.  lambda / theta (and their gradients) are used only by the learned
 * trapezoid / rotational dynamics.  A NULL field of m3_host_out skips that copy. */
typedef struct m3_host_pipe m3_host_pipe;
typedef struct {
  const void *x, *b, *c, *dt, *lambda, *theta, *dy;
} m3_host_in;
typedef struct {
  void *y, *dx, *db, *dc, *ddt, *dlambda, *dtheta; /* desc.dtype */
  float *da_log, *dd_skip;                         /* [heads]    */
} m3_host_out;
int m3_host_alloc(size_t bytes, void **out_host);
int m3_host_free(void *host_ptr);
int m3_host_pipe_create(m3_ctx *ctx, const m3_scan_desc *shape, int slices, m3_host_pipe **out);
/* Enqueue one run and return at once.  Inputs must stay unchanged, and outputs must not
 * be read, until m3_host_pipe_wait returns for the ticket written to *ticket (may be
 * NULL).  Runs complete in order. */
int m3_host_pipe_run(m3_host_pipe *pipe, const m3_host_in *in, const m3_host_out *out, uint64_t *ticket);
/* Block until the run with this ticket has delivered its outputs to host memory. */
int m3_host_pipe_wait(m3_host_pipe *pipe, uint64_t ticket);
int m3_host_pipe_destroy(m3_host_pipe *pipe);

/* CausalConv1d::apply / apply_with_history (src/nn/conv.rs:143-213; kernels
 * src/tensor/ops/fused.rs:780-1200) fused with the SiLU the mixer applies to its result
 * (src/models/mamba3.rs:401): the step in front of the scan.
 *   y[b,t,c] = act(bias[c] + sum_{delay < K} weight[K-1-delay, c] * x[b, t-delay, c])
 * with x[t < 0] taken from `history` (the last K-1 inputs of the previous window) or zero.
 * Rows may be strided: x is usually a column band of the input projection. */
typedef struct {
  int32_t batch, seq, channels;
  int32_t kernel_size;   /* taps K, 1..8 */
  int32_t dtype;         /* m3_dtype of x, history, y and their gradients */
  int32_t activation;    /* 0 = none (the bare convolution), 1 = SiLU */
  int64_t x_stride;      /* elements between consecutive time steps of x and dx; 0 = channels */
  int64_t y_stride;      /* the same for y and dy; 0 = channels */
  const void *x;         /* [batch, seq, channels] with row stride x_stride */
  const void *history;   /* [batch, K-1, channels] dense, or NULL (zeros) */
  const float *weight;   /* [K, channels] */
  const float *bias;     /* [channels] or NULL */
  /* Optional second output: channels [split, channels) go to y2 (the forward's second result,
   * row stride y2_stride, 0 = channels - split) instead of y, and the backward reads their
   * gradient from dy2 - the mixer's x | B C cut (src/models/mamba3.rs:403-406) without a copy.
   * split = 0: everything in y / dy. */
  int32_t split, reserved0;
  int64_t y2_stride;
  void *y2;
  const void *dy2;
  /* Channel ranges [lo, hi) that are convolved right to left: the backward direction of a
   * bidirectional mixer, whose x, B and C halves the reference reverses in time before the
   * convolution (src/models/mamba3.rs:352-370).  Inputs, outputs and gradients stay in ordinary
   * time; such channels take no history.  n_reversed = 0: none. */
  int32_t n_reversed;
  int32_t reversed_lo[4], reversed_hi[4];
  int32_t reserved1;
} m3_conv_desc;
/* new_history (causal_conv1d_history): [batch, K-1, channels], the inputs the next window
 * continues from; NULL skips it. */
int m3_conv_forward(m3_ctx *ctx, const m3_conv_desc *desc, void *y, void *new_history);
/* The adjoint; it recomputes the pre-activation from x, so the forward saves nothing.
 * dx has x's strides; dweight [K, channels], dbias [channels] (float) and dhistory
 * (like history) may each be NULL.  The parameter gradients are summed in a fixed order;
 * dbias of a convolution without a bias is written as zeros. */
int m3_conv_backward(m3_ctx *ctx, const m3_conv_desc *desc, const void *dy, void *dx,
                     float *dweight, float *dbias, void *dhistory);

/* B and C on their way from the convolution to the scan (src/models/mamba3.rs:409-436): expand
 * groups to heads, add the per-head bias, RMS-normalise over d_state (RmsNorm, src/nn/norm.rs:95-105)
 * and permute to the scan's rank-last layout - one launch per tensor instead of about six.
 *   v = raw[b, t, h / (heads/groups), r, :] + bias[h, :];   out[b, t, h, :, r] = v * rsqrt(mean(v^2) + eps) * weight */
typedef struct {
  int32_t batch, seq, heads, groups, d_state, rank;
  int32_t dtype;              /* m3_dtype of the raw rows, b, c and their gradients */
  int32_t has_norm;           /* 0: no bc_norm (bias only) */
  float eps;                  /* RmsNorm eps */
  int32_t reserved0;
  int64_t raw_stride;         /* elements between consecutive tokens of b_raw / c_raw; 0 = groups*rank*d_state */
  const void *b_raw, *c_raw;  /* [batch, seq, groups, rank, d_state] with token stride raw_stride */
  const float *b_bias, *c_bias; /* [heads, d_state] or NULL */
  const float *norm_weight;   /* [d_state] or NULL (no gain) */
} m3_bc_desc;
/* b, c: [batch, seq, heads, d_state, rank], the layout m3_scan_desc wants. */
int m3_bc_forward(m3_ctx *ctx, const m3_bc_desc *desc, void *b, void *c);
/* db_raw / dc_raw have the raw rows' strides (the gradient of a group sums its heads); db_bias,
 * dc_bias [heads, d_state] and dnorm_weight [d_state] (one gain shared by B and C) are float and
 * may be NULL.  Sums run in a fixed order. */
int m3_bc_backward(m3_ctx *ctx, const m3_bc_desc *desc, const void *db, const void *dc,
                   void *db_raw, void *dc_raw, float *db_bias, float *dc_bias, float *dnorm_weight);

/* dt = softplus(dt_raw + dt_bias[h]), lambda = sigmoid(lambda_raw) (src/models/mamba3.rs:440-446). */
typedef struct {
  int32_t batch, seq, heads;
  int32_t dtype;
  int64_t stride;             /* elements between consecutive tokens of dt_raw / lambda_raw; 0 = heads */
  const void *dt_raw;         /* [batch, seq, heads] with token stride `stride` */
  const void *lambda_raw;     /* likewise, or NULL */
  const float *dt_bias;       /* [heads] or NULL */
} m3_act_desc;
int m3_dt_lambda_forward(m3_ctx *ctx, const m3_act_desc *desc, void *dt, void *lambda);
int m3_dt_lambda_backward(m3_ctx *ctx, const m3_act_desc *desc, const void *ddt, const void *dlambda,
                          void *ddt_raw, void *dlambda_raw, float *ddt_bias);

/* The gate behind the scan: out = y * silu(z) (Mamba3Mixer::finish without post_gate_norm,
 * src/models/mamba3.rs:475-484).  y, out, dout, dy are dense [batch, seq, channels]; z and dz
 * may be column bands of the input projection (row stride z_stride, 0 = channels). */
typedef struct {
  int32_t batch, seq, channels;
  int32_t dtype;
  int64_t z_stride;
  const void *y, *z;
} m3_gate_desc;
int m3_gate_forward(m3_ctx *ctx, const m3_gate_desc *desc, void *out);
int m3_gate_backward(m3_ctx *ctx, const m3_gate_desc *desc, const void *dout, void *dy, void *dz);

/* The same gate behind the optional post-gate norm (SsmConfig::post_gate_norm, src/ssm/config.rs:113;
 * Mamba3Mixer::finish, src/models/mamba3.rs:475-484; RmsNorm::apply, src/nn/norm.rs:95-105):
 * out = y * rsqrt(mean over channels of y^2 + eps) * weight * silu(z), one launch.  weight is the norm's
 * gain [channels] in float32, or NULL for a norm without gain.  The backward pass returns dy, dz (either may
 * be NULL) and, when both weight and dweight are given, dweight [channels] (zeroed for seq == 0), summed over
 * the rows in a fixed order.  channels is at most 8192 (M3_ERR_UNSUPPORTED beyond). */
typedef struct {
  int32_t batch, seq, channels;
  int32_t dtype;
  int64_t z_stride;
  const void *y, *z;
  const float *weight;
  float eps;
} m3_gate_norm_desc;
int m3_gate_norm_forward(m3_ctx *ctx, const m3_gate_norm_desc *desc, void *out);
int m3_gate_norm_backward(m3_ctx *ctx, const m3_gate_norm_desc *desc, const void *dout, void *dy, void *dz,
                          float *dweight);

/* Bytes of device scratch a forward with this descriptor allocates (kept until
 * m3_saved_free when `saved` is requested). */
size_t m3_scan_scratch_bytes(const m3_scan_desc *desc, int for_backward);

#ifdef __cplusplus
}
#endif
#endif /* M3SCAN_H */
