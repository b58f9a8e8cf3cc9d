//! Raw `extern "C"` declarations of libm3scan.so, field for field and symbol for symbol what
//! `include/m3scan.h` declares.  NOT COMPILED in this repository's build image (it has no Rust
//! toolchain); the executable twin of this file is the ctypes binding `mamba_trainer_b200/_ffi.py`,
//! which the GPU tests drive.  Each item names the reference interface it stands in for.
#![allow(non_camel_case_types, non_upper_case_globals)]

use std::os::raw::{c_char, c_int, c_void};

/// Device + stream + caches.  Opaque.
#[repr(C)]
pub struct m3_ctx {
    _private: [u8; 0],
}
/// What a forward pass keeps for its adjoint.  Opaque.
#[repr(C)]
pub struct m3_saved {
    _private: [u8; 0],
}
/// A host-buffer pipeline for one problem shape.  Opaque.
#[repr(C)]
pub struct m3_host_pipe {
    _private: [u8; 0],
}

// m3_status: the reference's Error variants (src/error.rs) plus the CUDA-side ones.
pub const M3_OK: c_int = 0;
pub const M3_ERR_SHAPE: c_int = 1; // Error::Shape
pub const M3_ERR_RANK: c_int = 2; // Error::Rank
pub const M3_ERR_CONFIG: c_int = 3; // Error::Config
pub const M3_ERR_UNSUPPORTED: c_int = 4; // Error::Unsupported
pub const M3_ERR_CUDA: c_int = 5;
pub const M3_ERR_TIMEOUT: c_int = 6; // a bounded device-side wait gave up
pub const M3_ERR_NULL: c_int = 7;

// m3_dtype
pub const M3_F32: i32 = 0;
pub const M3_BF16: i32 = 1;
// m3_discretization: ssm::config::Discretization (src/ssm/config.rs)
pub const M3_EULER: i32 = 0;
pub const M3_TRAPEZOID: i32 = 1;
pub const M3_LEARNED_TRAPEZOID: i32 = 2;
// m3_dynamics: ssm::config::StateDynamics
pub const M3_REAL: i32 = 0;
pub const M3_ROTATIONAL: i32 = 1;
// m3_path
pub const M3_PATH_AUTO: i32 = 0;
pub const M3_PATH_GENERIC: i32 = 1;
pub const M3_PATH_TENSOR: i32 = 2;

// grad_mask bits: the `wanted` slice of Var::record_with_mask (src/autograd/var.rs:169-204)
pub const M3_GRAD_X: u32 = 1 << 0;
pub const M3_GRAD_B: u32 = 1 << 1;
pub const M3_GRAD_C: u32 = 1 << 2;
pub const M3_GRAD_DT: u32 = 1 << 3;
pub const M3_GRAD_A_LOG: u32 = 1 << 4;
pub const M3_GRAD_LAMBDA: u32 = 1 << 5;
pub const M3_GRAD_THETA: u32 = 1 << 6;
pub const M3_GRAD_D_SKIP: u32 = 1 << 7;
pub const M3_GRAD_H0: u32 = 1 << 8;
pub const M3_GRAD_LAST_U0: u32 = 1 << 9;
pub const M3_GRAD_ANGLE0: u32 = 1 << 10;
pub const M3_GRAD_ALL: u32 = 0x7ff;

pub const M3_NOALLOC_SCRATCH_BYTES: usize = 16 << 20;

/// ScanInputs (src/ssm/scan.rs:361-385); `a_raw/g_raw/w_raw` give the `ssd_chunked` form (:116-126).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_scan_desc {
    pub batch: i32,
    pub seq: i32,
    pub heads: i32,
    pub head_dim: i32,
    pub d_state: i32,
    pub rank: i32,
    pub chunk: i32,
    pub dtype: i32,
    pub discretization: i32,
    pub dynamics: i32,
    pub want_state: i32,
    pub path: i32,
    /// the last `reverse_heads` heads walk time right to left (bidirectional mixer, models/mamba3.rs:97-112)
    pub reverse_heads: i32,
    pub reserved0: i32,
    pub x: *const c_void,
    pub b: *const c_void,
    pub c: *const c_void,
    pub dt: *const c_void,
    pub lambda: *const c_void,
    pub theta: *const c_void,
    pub a_log: *const f32,
    pub d_skip: *const f32,
    pub h0: *const f32,
    pub last_u0: *const f32,
    pub angle0: *const f32,
    pub a_raw: *const c_void,
    pub g_raw: *const c_void,
    pub w_raw: *const c_void,
}

/// ScanOutput (src/ssm/scan.rs:446-452), caller-allocated.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_scan_out {
    pub y: *mut c_void,
    pub h: *mut f32,
    pub last_u: *mut f32,
    pub angle: *mut f32,
}

/// Upstream gradients: the argument of the BackwardRule (src/autograd/graph.rs:61-62) plus those of the state.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_scan_bwd_in {
    pub dy: *const c_void,
    pub dh: *const f32,
    pub dlast_u: *const f32,
    pub dangle: *const f32,
}

#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_scan_grads {
    pub dx: *mut c_void,
    pub db: *mut c_void,
    pub dc: *mut c_void,
    pub ddt: *mut c_void,
    pub dlambda: *mut c_void,
    pub dtheta: *mut c_void,
    pub da_log: *mut f32,
    pub dd_skip: *mut f32,
    pub dh0: *mut f32,
    pub dlast_u0: *mut f32,
    pub dangle0: *mut f32,
    pub da_raw: *mut c_void,
    pub dg_raw: *mut c_void,
    pub dw_raw: *mut c_void,
}

/// mamba3_step (src/ssm/scan.rs:649-712): one decoding step.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_step_desc {
    pub batch: i32,
    pub heads: i32,
    pub head_dim: i32,
    pub d_state: i32,
    pub rank: i32,
    pub dtype: i32,
    pub discretization: i32,
    pub dynamics: i32,
    pub x: *const c_void,
    pub b: *const c_void,
    pub c: *const c_void,
    pub dt: *const c_void,
    pub lambda: *const c_void,
    pub theta: *const c_void,
    pub a_log: *const f32,
    pub d_skip: *const f32,
    pub h: *const f32,
    pub last_u: *const f32,
    pub angle: *const f32,
}
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_step_out {
    pub y: *mut c_void,
    pub h: *mut f32,
    pub last_u: *mut f32,
    pub angle: *mut f32,
}

/// Host pointers of one pipeline run (Tensor::from_f32 ... to_data, src/tensor/base.rs:21-199).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_host_in {
    pub x: *const c_void,
    pub b: *const c_void,
    pub c: *const c_void,
    pub dt: *const c_void,
    pub lambda: *const c_void,
    pub theta: *const c_void,
    pub dy: *const c_void,
}
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_host_out {
    pub y: *mut c_void,
    pub dx: *mut c_void,
    pub db: *mut c_void,
    pub dc: *mut c_void,
    pub ddt: *mut c_void,
    pub dlambda: *mut c_void,
    pub dtheta: *mut c_void,
    pub da_log: *mut f32,
    pub dd_skip: *mut f32,
}

/// CausalConv1d::apply / apply_with_history (src/nn/conv.rs:143-213) with the mixer's SiLU.
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_conv_desc {
    pub batch: i32,
    pub seq: i32,
    pub channels: i32,
    pub kernel_size: i32,
    pub dtype: i32,
    pub activation: i32,
    pub x_stride: i64,
    pub y_stride: i64,
    pub x: *const c_void,
    pub history: *const c_void,
    pub weight: *const f32,
    pub bias: *const f32,
    pub split: i32,
    pub reserved0: i32,
    pub y2_stride: i64,
    pub y2: *mut c_void,
    pub dy2: *const c_void,
    pub n_reversed: i32,
    pub reversed_lo: [i32; 4],
    pub reversed_hi: [i32; 4],
    pub reserved1: i32,
}

/// B and C from the convolution to the scan (src/models/mamba3.rs:409-436).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_bc_desc {
    pub batch: i32,
    pub seq: i32,
    pub heads: i32,
    pub groups: i32,
    pub d_state: i32,
    pub rank: i32,
    pub dtype: i32,
    pub has_norm: i32,
    pub eps: f32,
    pub reserved0: i32,
    pub raw_stride: i64,
    pub b_raw: *const c_void,
    pub c_raw: *const c_void,
    pub b_bias: *const f32,
    pub c_bias: *const f32,
    pub norm_weight: *const f32,
}

/// dt = softplus(dt_raw + dt_bias), lambda = sigmoid(lambda_raw) (src/models/mamba3.rs:440-446).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_act_desc {
    pub batch: i32,
    pub seq: i32,
    pub heads: i32,
    pub dtype: i32,
    pub stride: i64,
    pub dt_raw: *const c_void,
    pub lambda_raw: *const c_void,
    pub dt_bias: *const f32,
}

/// out = y * silu(z) (Mamba3Mixer::finish, src/models/mamba3.rs:475-484).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_gate_desc {
    pub batch: i32,
    pub seq: i32,
    pub channels: i32,
    pub dtype: i32,
    pub z_stride: i64,
    pub y: *const c_void,
    pub z: *const c_void,
}

/// out = rms_norm(y) * weight * silu(z): the gate behind SsmConfig::post_gate_norm
/// (src/models/mamba3.rs:475-484, src/nn/norm.rs:95-105).
#[repr(C)]
#[derive(Clone, Copy)]
pub struct m3_gate_norm_desc {
    pub batch: i32,
    pub seq: i32,
    pub channels: i32,
    pub dtype: i32,
    pub z_stride: i64,
    pub y: *const c_void,
    pub z: *const c_void,
    pub weight: *const f32,
    pub eps: f32,
}

extern "C" {
    pub fn m3_version() -> *const c_char;

    pub fn m3_ctx_create(device: c_int, out: *mut *mut m3_ctx) -> c_int;
    pub fn m3_ctx_destroy(ctx: *mut m3_ctx) -> c_int;
    pub fn m3_ctx_set_stream(ctx: *mut m3_ctx, cuda_stream: *mut c_void) -> c_int;
    /// Waits for the context's stream and reports a device-side wait that gave up (M3_ERR_TIMEOUT).
    pub fn m3_sync(ctx: *mut m3_ctx) -> c_int;
    /// Iteration limit of the kernels' bounded waits; 0 restores the default.
    pub fn m3_ctx_set_wait_limit(ctx: *mut m3_ctx, iterations: u32) -> c_int;
    pub fn m3_last_error(ctx: *const m3_ctx) -> *const c_char;
    /// Kernels launched through this context so far (launch_count(), src/backend.rs:231-281).
    pub fn m3_launch_count(ctx: *const m3_ctx) -> u64;

    // Tensor::from_f32 / to_data for callers without their own device allocator (src/tensor/base.rs)
    pub fn m3_alloc(ctx: *mut m3_ctx, bytes: usize, out: *mut *mut c_void) -> c_int;
    pub fn m3_free(ctx: *mut m3_ctx, ptr: *mut c_void) -> c_int;
    pub fn m3_upload(ctx: *mut m3_ctx, dst_device: *mut c_void, src_host: *const c_void, bytes: usize) -> c_int;
    pub fn m3_download(ctx: *mut m3_ctx, dst_host: *mut c_void, src_device: *const c_void, bytes: usize) -> c_int;

    /// ssm::mamba3_scan / ssm::ssd_chunked (src/ssm/scan.rs:458-618, :116-291).  `saved` NULL: inference form.
    pub fn m3_scan_forward(ctx: *mut m3_ctx, desc: *const m3_scan_desc, out: *const m3_scan_out,
                           saved: *mut *mut m3_saved) -> c_int;
    /// The node's backward rule; may run more than once per saved handle (backward_retain).
    pub fn m3_scan_backward(ctx: *mut m3_ctx, saved: *const m3_saved, input: *const m3_scan_bwd_in, grad_mask: u32,
                            grads: *const m3_scan_grads) -> c_int;
    pub fn m3_saved_free(ctx: *mut m3_ctx, saved: *mut m3_saved) -> c_int;
    pub fn m3_scan_scratch_bytes(desc: *const m3_scan_desc, for_backward: c_int) -> usize;

    /// ssm::mamba3_step (src/ssm/scan.rs:649-712).
    pub fn m3_step_forward(ctx: *mut m3_ctx, desc: *const m3_step_desc, out: *const m3_step_out) -> c_int;

    /// No counterpart in the reference: the forward scan for hosts that must not allocate while running.
    pub fn m3_scan_forward_noalloc(ctx: *mut m3_ctx, desc: *const m3_scan_desc, out: *const m3_scan_out) -> c_int;

    pub fn m3_host_alloc(bytes: usize, out_host: *mut *mut c_void) -> c_int;
    pub fn m3_host_free(host_ptr: *mut c_void) -> c_int;
    pub fn m3_host_pipe_create(ctx: *mut m3_ctx, shape: *const m3_scan_desc, slices: c_int,
                               out: *mut *mut m3_host_pipe) -> c_int;
    pub fn m3_host_pipe_run(pipe: *mut m3_host_pipe, input: *const m3_host_in, out: *const m3_host_out,
                            ticket: *mut u64) -> c_int;
    pub fn m3_host_pipe_wait(pipe: *mut m3_host_pipe, ticket: u64) -> c_int;
    pub fn m3_host_pipe_destroy(pipe: *mut m3_host_pipe) -> c_int;

    pub fn m3_conv_forward(ctx: *mut m3_ctx, desc: *const m3_conv_desc, y: *mut c_void, new_history: *mut c_void) -> c_int;
    pub fn m3_conv_backward(ctx: *mut m3_ctx, desc: *const m3_conv_desc, dy: *const c_void, dx: *mut c_void,
                            dweight: *mut f32, dbias: *mut f32, dhistory: *mut c_void) -> c_int;
    pub fn m3_bc_forward(ctx: *mut m3_ctx, desc: *const m3_bc_desc, b: *mut c_void, c: *mut c_void) -> c_int;
    pub fn m3_bc_backward(ctx: *mut m3_ctx, desc: *const m3_bc_desc, db: *const c_void, dc: *const c_void,
                          db_raw: *mut c_void, dc_raw: *mut c_void, db_bias: *mut f32, dc_bias: *mut f32,
                          dnorm_weight: *mut f32) -> c_int;
    pub fn m3_dt_lambda_forward(ctx: *mut m3_ctx, desc: *const m3_act_desc, dt: *mut c_void, lambda: *mut c_void) -> c_int;
    pub fn m3_dt_lambda_backward(ctx: *mut m3_ctx, desc: *const m3_act_desc, ddt: *const c_void, dlambda: *const c_void,
                                 ddt_raw: *mut c_void, dlambda_raw: *mut c_void, ddt_bias: *mut f32) -> c_int;
    pub fn m3_gate_forward(ctx: *mut m3_ctx, desc: *const m3_gate_desc, out: *mut c_void) -> c_int;
    pub fn m3_gate_backward(ctx: *mut m3_ctx, desc: *const m3_gate_desc, dout: *const c_void, dy: *mut c_void,
                            dz: *mut c_void) -> c_int;
    pub fn m3_gate_norm_forward(ctx: *mut m3_ctx, desc: *const m3_gate_norm_desc, out: *mut c_void) -> c_int;
    pub fn m3_gate_norm_backward(ctx: *mut m3_ctx, desc: *const m3_gate_norm_desc, dout: *const c_void, dy: *mut c_void,
                                 dz: *mut c_void, dweight: *mut f32) -> c_int;
}
