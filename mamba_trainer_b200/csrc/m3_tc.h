// Host-side interface of the tensor-core kernel family.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/m3scan.h"

namespace m3 {

// Shapes the family serves: bf16, head_dim 64, d_state 128, rank 1, 2 or 4.
// 16-byte alignment: the kernels move rows as 16-byte vectors and bulk tensor copies.
inline bool tc_aligned(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool tc_supported(const m3_scan_desc& s) {
  return s.dtype == M3_BF16 && s.head_dim == 64 && s.d_state == 128 && (s.rank == 1 || s.rank == 2 || s.rank == 4) &&
         s.seq > 0 && tc_aligned(s.x) && tc_aligned(s.b) && tc_aligned(s.c) && tc_aligned(s.theta);
}
// Time steps per 128-row tile and tiles per stripe.
inline int tc_tile_steps(int rank) { return 128 / rank; }
inline int tc_tiles(int seq, int rank) { return (seq + tc_tile_steps(rank) - 1) / tc_tile_steps(rank); }

// A tensor map that lands a [128 tokens x cols] bf16 tile of a dense [B, T, H, cols] tensor directly in
// the kernels' operand layout (8 x 8 core matrices tiled [rows/8][cols/8]): dimensions
// (8 elements, 8 tokens, H*cols/8 column groups, B*T/8 token groups), box (8, 8, cols/8, 16), so the
// tile of (batch b, head h, first token t0) is the box at (0, 0, h*cols/8, (b*T + t0)/8).  Needs T % 8 == 0
// and a 16-byte aligned base.  Returns false when the driver refuses (the caller then takes the
// register path).
bool tc_make_tile_map(CUtensorMap* map, const void* base, int B, int T, int H, int cols);

// A tensor map over the rows of a dense [B, T, H, cols] bf16 tensor as the caller stores them:
// dimensions (cols, H, T, B), box (64, 1, steps, 1), so 64 columns of `steps` consecutive time steps of
// one (batch, head) land as a dense [steps][128 bytes] panel (one request per 64 columns), rows past
// either end of the sequence arriving as zeros.  With `swizzle` the 16-byte chunks of a panel row are
// XOR-swizzled by row & 7 (the 128-byte swizzle; the panel must then start on a 1024-byte boundary).
// cols a multiple of 64; needs a 16-byte aligned base.
bool tc_make_row_map(CUtensorMap* map, const void* base, int B, int T, int H, int cols, int steps, bool swizzle);

struct TcFwdParams {
  alignas(64) CUtensorMap tm_b, tm_c, tm_x;   // tile maps of the direct form when use_tma, else row maps of b and c
  alignas(64) CUtensorMap tm_th;              // row map of theta (rotational dynamics, role-split kernel)
  alignas(64) CUtensorMap tm_y;               // row map of y: its tiles leave by bulk tensor stores when out_maps
  int out_maps;
  int use_tma;        // rank 1, real dynamics, T % 8 == 0, no right-to-left heads
  const __nv_bfloat16 *x, *b, *c, *dt, *lam, *theta;
  const float *a_log, *d_skip, *h0, *lu0, *angle0;
  __nv_bfloat16* y;
  float *h_out, *lu_out, *angle_out;
  __nv_bfloat16* ckpt_h;  // [BH, tiles, 64 x 128 operand tile] bf16 state entering each tile, or NULL
  float* ckpt_angle;  // [BH, tiles, 64] angle entering each tile, or NULL
  int* err;           // device flag set when a bounded wait gave up
  int B, T, H, R, disc;
  int rev;            // the last `rev` heads walk time right to left
  uint32_t wait_limit; // iteration limit of the bounded waits (m3_ctx_set_wait_limit)
  // time segments of a stripe (role-split kernel; work distribution in m3_tc_roles.cuh): nseg == 1 hands nothing over
  int nseg, tps, grid;
  float *seg_state, *seg_angle;
  int* seg_flag;
};

// How a launch of the role-split kernels cuts its stripes in time: enough items to keep every SM busy to
// the end (about six per SM), segments of at least four tiles.  Returns segments per stripe, tiles per
// segment and the grid; bytes of hand-over scratch (state, angle, flags) through *scratch_bytes.
void tc_segment_plan(int BH, int tiles, bool allow_split, int* nseg, int* tps, int* grid, size_t* scratch_bytes);

cudaError_t tc_forward(cudaStream_t st, const TcFwdParams& p, bool rotational);
// The direct form (rank 1, real dynamics, use_tma): m3_tc_fwd_direct.cu.
cudaError_t tc_forward_direct(cudaStream_t st, const TcFwdParams& p);

struct TcBwdParams {
  alignas(64) CUtensorMap tm_b, tm_c;   // tile maps of the direct form when use_tma, else row maps of b and c
  alignas(64) CUtensorMap tm_x, tm_dy, tm_th;  // row maps of x, dy and theta (role-split kernel)
  alignas(64) CUtensorMap tm_dx, tm_db, tm_dc; // row maps of the gradients asked for: their tiles leave by bulk tensor stores when out_maps
  int out_maps;
  int use_tma;
  const __nv_bfloat16 *x, *b, *c, *dt, *lam, *theta, *dy;
  const float *a_log, *d_skip, *h0, *lu0;
  const float *dh, *dlu, *dangle;        // gradients reaching the returned state, or NULL
  const __nv_bfloat16* ckpt_h;           // written by the forward pass
  const float* ckpt_angle;
  __nv_bfloat16 *dx, *db, *dc, *dtheta;  // NULL skips the store
  float *da, *dg, *dw, *ddt_rot;         // [BH, tiles * steps] per-token scalars for the final pass
  float *partA, *partD;                  // [BH, tiles] partial sums of d a_log / d d_skip
  float *ip0;                            // [BH] <dH_0, last_u0>
  float *dh0, *dlu0, *dangle0;           // NULL skips the store
  int* err;
  int B, T, H, R, disc;
  int rev;            // the last `rev` heads walk time right to left
  uint32_t wait_limit;
  int nseg, tps, grid;   // as in TcFwdParams; the gradient of the state and the running sum of d phi are handed over
  float *seg_state, *seg_angle;
  int* seg_flag;
};

cudaError_t tc_backward(cudaStream_t st, const TcBwdParams& p, bool rotational);
// The direct form (rank 1, real dynamics, use_tma): m3_tc_bwd_direct.cu.
cudaError_t tc_backward_direct(cudaStream_t st, const TcBwdParams& p);

}  // namespace m3
