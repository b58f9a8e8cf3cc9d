// Tensor-core backward of the Mamba-3 SSD scan (sm_100a: tcgen05 MMA, TMEM accumulators, bulk copies).
//
// The hand-written adjoint of the folded scan: a CTA walks the 128-row tiles of a (batch, head) stripe -
// or of a time segment of one - in REVERSE with the gradient of the state, dH^T [d_state x head_dim]
// fp32, resident in TMEM.  The reference derives this pass from its tape (rules in
// src/autograd/ops.rs:204-264, :1066-1139, kernels src/tensor/ops/fused.rs:627-672,
// :2080-2138, :2513-2549); here it is two MMA phases per tile:
//   A:  G = C^ B^^T,  dM = dY~ X~^T,  T1 = dY~ H_k
//       regs: M = G o band, dG = dM o band, band adjoint sums, dC^ base = exp(acum) T1,
//             dS = dH (bf16 operand), d cd = exp(cd) <dH, H_k>, dH *= exp(cd)
//   B:  dX~ = M^T dY~ (+ sw . B^ dS^T),  dB^ = dG^T C^ + (sw X~) dS,  dC^ += dG B^,
//       dH^T += C^^T (exp(acum) dY~)
//       regs: un-rotate dB^, dC^ by +phi, collect d phi, reverse-scan it, per-token scalars.
// Warp roles (m3_tc_roles.cuh): the issuer warp issues both phases, the look-ahead warp computes the next
// tile's per-token scalars, the copy warp requests the next tile's raw rows of B, C, x, dy and theta (bulk
// tensor copies) and its state checkpoint (a plain bulk copy) as soon as this tile has let go of the
// buffers, and sends this tile's staged gradients d x, d B, d C off by bulk tensor stores.  Shared memory
// has no room for staging beside the operands (a tile's operands alone take 208 KB), so the rows of B and C
// land IN their operand buffers and are converted in place - every epilogue warp reads its share into
// registers, one barrier, then the rotated / de-interleaved operands overwrite them - those of x and dy
// land in dG's buffer, which is idle between two band epilogues, and the gradients are staged in buffers
// the tile has finished with (d x over dS, d B over the scaled copies, d C over dG).
// The (cos, sin) table of the tile's angles is computed once, used for the rotation, and kept in 64
// TMEM columns for the un-rotation of the gradients (its shared-memory buffer becomes M in between).
// Rank 1 with real dynamics has a second form (m3_tc_bwd_direct.cu).
#include "m3_tc.h"
#include "m3_tc_roles.cuh"

namespace m3 {
using namespace m3tc;

namespace {

constexpr uint32_t OFF_C = 0, OFF_B = 32768, OFF_X = 65536, OFF_DY = 81920, OFF_XW = 98304, OFF_DYE = 114688,
                   OFF_M = 131072, OFF_DG = 163840, OFF_HS = 196608, OFF_SC = 212992;
constexpr int kScalFloats = 2 * kNumScal * kScal + 256 * 4 + 512 + 256 + 132 + 132 + 16 + 64 + 256;
static_assert(OFF_SC + kScalFloats * 4 + 64 <= 232448, "backward shared memory exceeds the 227 KB a CTA can have");
constexpr uint32_t kSmemBytes = OFF_SC + kScalFloats * 4 + 64;
constexpr uint32_t TM_G = 0, TM_DM = 128, TM_T1 = 256, TM_DH = 384, TM_TAB = 448, TM_COLS = 512;
// phase B reuse: dB^ accumulates over G's columns, dX~ and U over dM's.
constexpr uint32_t TM_DB = 0, TM_DX = 128, TM_U = 192;

template <int R, bool ROT, bool SPLIT>
__global__ void __launch_bounds__(kCtaThreads, 1) tc_bwd_kernel(const __grid_constant__ TcBwdParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int LT = kRows / R;
  using RT = RawTile<R>;
  uint8_t *sC = smem + OFF_C, *sB = smem + OFF_B, *sX = smem + OFF_X, *sXw = smem + OFF_XW, *sDY = smem + OFF_DY,
          *sDYe = smem + OFF_DYE, *sM = smem + OFF_M, *sDG = smem + OFF_DG, *sHS = smem + OFF_HS;
  float* sTab = reinterpret_cast<float*>(smem + OFF_M);    // theta rows, then the angle table, until M is written
  float* sDphi = reinterpret_cast<float*>(smem + OFF_X);   // d phi of the tile, once X~ and dY~ are spent (up to 32 KB)
  // dG's buffer is free from the copy-out of dC to the next band epilogue: the raw rows of x and dy land there
  uint8_t *rawX = smem + OFF_DG, *rawDY = smem + OFF_DG + RT::bytes(kP);
  float* sc = reinterpret_cast<float*>(smem + OFF_SC);
  // Two sets of per-token scalars: the look-ahead warp fills the next tile's while this tile is worked on.
  auto scal_set = [&](int i) {
    float* q = sc + i * kNumScal * kScal;
    return TileScalars{q, q + kScal, q + 2 * kScal, q + 3 * kScal, q + 4 * kScal, q + 5 * kScal, q + 6 * kScal,
                       q + 7 * kScal, q + 8 * kScal};
  };
  float* part_row = sc + 2 * kNumScal * kScal;   // [2][128]
  float* part_t1 = part_row + 256;    // [2][128]
  float* part_q = part_t1 + 256;      // [2][128]
  float* part_dg = part_q + 256;      // [2][128]
  float* part_col = part_dg + 256;    // [4][128]
  float* part_rot = part_col + 512;   // [2][128]
  float* s_dacum = part_rot + 256;    // [132]
  float* s_dast = s_dacum + 132;      // [132]
  float* s_red = s_dast + 132;        // [16]
  float* s_dcar = s_red + 16;         // [64] sum of d phi over later tiles
  float* s_q = s_dcar + 64;           // [4][64]
  // [0]: phase A; [1]: the first three products of phase B, [4]: the rest of it; [2]: arrival of a tile's raw
  // rows; [3]: of its state checkpoint
  uint64_t* bars = reinterpret_cast<uint64_t*>(s_q + 256);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 5);
  int* s_ok = reinterpret_cast<int*>(tmem_slot + 1);  // outcome of a hand-over wait, for the epilogue warps

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int T = p.T, H = p.H;
  const int ntiles = (T + LT - 1) / LT;
  // Every role walks the same sequence of tiles: those of this CTA's items, each item's from its last tile
  // to its first, the items of the last segment first - as two nested loops, so that what belongs to the
  // item (stripe, head, direction) is invariant where the tiles are walked; `it` counts the tiles this CTA
  // has gone through and picks barrier phases and scalar sets.  Right-to-left heads: scan position s is
  // time T-1-s, reached with a negative token stride.
  // SPLIT: stripes cut in time, a grid of at most one CTA per SM that works through its items.  Otherwise
  // one CTA per stripe, whose single item is known without a decode and whose loops run once.
  const int nseg = SPLIT ? p.nseg : 1;
  const int BH = p.B * H, nitems = BH * nseg;
  auto item_of = [&](int item) {
    if (SPLIT) return decode_item(item, BH, H, ntiles, nseg, p.tps, 1);
    ItemInfo r;
    r.bh = item; r.b = item / H; r.h = item - r.b * H; r.seg = 0; r.k_lo = 0; r.k_hi = ntiles;
    return r;
  };
  const int Tp = ntiles * LT;
  const uint32_t wait_limit = p.wait_limit;

  if (tid == 0) {
    mbar_init(&bars[0], 1);
    mbar_init(&bars[1], 1);
    mbar_init(&bars[2], 2);
    mbar_init(&bars[3], 1);
    mbar_init(&bars[4], 1);
  }
  if (warp == 0) tmem_alloc(tmem_slot, TM_COLS);
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tm = *tmem_slot;

  if (warp == kCopyWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Copy warp.  Tile kk's raw rows land in the operand buffers themselves (one request per lane), its
    // theta rows where the angle table will be, its checkpoint where H_k is read from.
    // --------------------------------------------------------------------------------------------
    // bars[2] counts two arrivals per tile: the rows of B, C and theta, then those of x and dy
    constexpr uint32_t kBcBytes = 2u * RT::bytes(kN) + (ROT ? (uint32_t)LT * kNH * 2u : 0u), kXdyBytes = 2u * RT::bytes(kP);
    auto request_bc = [&](int b, int h, bool rev, int kk) {
      if (lane == 0) mbar_expect_tx(&bars[2], kBcBytes);
      __syncwarp();
      const int t0 = kk * LT;
      int l0 = request_raw_tile<R>(0, sC, &p.tm_c, &bars[2], kN, b, h, T, t0, rev);
      l0 += request_raw_tile<R>(l0, sB, &p.tm_b, &bars[2], kN, b, h, T, t0, rev);
      if (ROT && lane == l0) tma_load_rows(sTab, &p.tm_th, &bars[2], 0, h, rev ? T - t0 - LT : t0, b);
      __syncwarp();
    };
    auto request_ckpt = [&](int bh, int kk) {
      if (lane == 0) {
        mbar_expect_tx(&bars[3], kN * kP * 2);
        bulk_load(sHS, p.ckpt_h + ((size_t)bh * ntiles + kk) * kN * kP, kN * kP * 2, &bars[3]);
      }
      __syncwarp();
    };
    auto request_xdy = [&](int b, int h, bool rev, int kk) {
      if (lane == 0) mbar_expect_tx(&bars[2], kXdyBytes);
      __syncwarp();
      const int t0 = kk * LT;
      const int l0 = request_raw_tile<R>(0, rawX, &p.tm_x, &bars[2], kP, b, h, T, t0, rev);
      request_raw_tile<R>(l0, rawDY, &p.tm_dy, &bars[2], kP, b, h, T, t0, rev);
      __syncwarp();
    };
    // The staged gradients of a finished tile leave by bulk tensor stores, one box per lane: d x from the
    // checkpoint's buffer, d B from that of the scaled copies, d C from dG's.
    auto store_tile = [&](int b, int h, bool rev, int kk) {
      const int t0 = kk * LT;
      if (!tile_leaves_by_map<R>(p.out_maps, rev, T, t0)) return;
      int l0 = 0;
      if (p.dx) l0 += store_out_tile<R>(l0, sHS, &p.tm_dx, kP, b, h, T, t0, rev);
      if (p.db) l0 += store_out_tile<R>(l0, sXw, &p.tm_db, kN, b, h, T, t0, rev);
      if (p.dc) l0 += store_out_tile<R>(l0, sDG, &p.tm_dc, kN, b, h, T, t0, rev);
      bulk_commit();
    };
    int it = 0, requested = 0;
    int pb = 0, ph = 0, pk = 0;  // the tile before the current one
    bool prev = false;
    bool copies_ok = true;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo im = item_of(item);
      const int b = im.b, h = im.h;
      const bool rev = h >= H - p.rev;
      for (int k = im.k_hi - 1; k >= im.k_lo; --k, ++it) {
        if (it > 0) {
          // the tile before this one: every operand and table word has been read and its gradients are staged
          bar_sync(BAR_TAIL, kPairCount);
          store_tile(pb, ph, prev, pk);
          // its copies have landed unless the epilogue warps gave up on them: a barrier is armed again only
          // once its current phase is complete
          if (copies_ok) copies_ok = warp_all(mbar_wait(&bars[2], (it - 1) & 1) && mbar_wait(&bars[3], (it - 1) & 1));
        }
        if (copies_ok) request_bc(b, h, rev, k);  // into the operand buffers and the table's: no staged gradient there
        if (it > 0) bulk_wait_read();             // the stores have read the staging buffers, which now take:
        if (copies_ok) {
          request_ckpt(im.bh, k);                 // the checkpoint, where d x was staged
          request_xdy(b, h, rev, k);              // x and dy, where d C was staged (d B's buffer is the epilogue's)
          ++requested;
        }
        pb = b; ph = h; prev = rev; pk = k;
      }
    }
    if (it > 0) {  // the last tile
      bar_sync(BAR_TAIL, kPairCount);
      store_tile(pb, ph, prev, pk);
    }
    // no copy of this CTA may be in flight when it lets go of its shared memory
    bulk_wait_all();
    if (requested > 0) {
      mbar_wait(&bars[2], (requested - 1) & 1);
      mbar_wait(&bars[3], (requested - 1) & 1);
    }
  } else if (warp == kScalarWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Look-ahead warp: the scalars of the g-th tile this CTA goes through land in set g & 1 as soon as the
    // epilogue warps have let go of it.
    // --------------------------------------------------------------------------------------------
    ScalarLoads<R> ld;
    int it = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo im = item_of(item);
      const int b = im.b, h = im.h;
      const bool rev = h >= H - p.rev;
      const float A = -expf(p.a_log[h]);
      lookahead_load<R>(ld, p.dt, p.lam, p.disc, b, h, H, T, (im.k_hi - 1) * LT, rev);
      for (int k = im.k_hi - 1; k >= im.k_lo; --k, ++it) {
        if (it > 0) bar_sync(BAR_FREE, kPairCount);
        lookahead_scalars<R>(scal_set(it & 1), ld, A, T, k * LT);
        bar_arrive(bar_ahead(it), kPairCount);
        if (k > im.k_lo) lookahead_load<R>(ld, p.dt, p.lam, p.disc, b, h, H, T, (k - 1) * LT, rev);
      }
    }
  } else if (warp > kIssuerWarp) {
    regs_for_helpers();  // the idle warp of the helpers' group
  } else if (warp == kIssuerWarp) {
    regs_for_helpers();
    // --------------------------------------------------------------------------------------------
    // Issuer: both phases of every tile.
    // --------------------------------------------------------------------------------------------
    bool ckpt_ok = true;
    int total = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo im = item_of(item);
      total += im.k_hi - im.k_lo;
    }
    for (int it = 0; it < total; ++it) {
      bar_sync(BAR_OPS0, kPairCount);  // X~ and dY~ staged: the two products that need nothing else start now
      if (ckpt_ok) ckpt_ok = warp_all(mbar_wait(&bars[3], it & 1));  // H_k has landed (long ago, as a rule)
      if (lane == 0) {
        if (!ckpt_ok && p.err) raise_flag(p.err);
        tc_fence_after();
        gemm_issue(tm + TM_DM, k_major(smem_u32(sDY), kP), k_major(smem_u32(sX), kP), make_idesc(128, 0, 0), kP, false);
        gemm_issue(tm + TM_T1, k_major(smem_u32(sDY), kP), k_major(smem_u32(sHS), kP), make_idesc(128, 0, 0), kP, false);
      }
      __syncwarp();
      bar_sync(BAR_OPS, kPairCount);  // C^ and B^ staged
      if (lane == 0) {
        tc_fence_after();
        gemm_issue(tm + TM_G, k_major(smem_u32(sC), kN), k_major(smem_u32(sB), kN), make_idesc(128, 0, 0), kN, false);
        umma_commit(&bars[0]);
      }
      __syncwarp();
      bar_sync(BAR_MID, kPairCount);  // M, dG and dS staged
      if (lane == 0) {
        tc_fence_after();
        const uint32_t aM = smem_u32(sM), aDG = smem_u32(sDG), aC = smem_u32(sC), aB = smem_u32(sB), aHS = smem_u32(sHS);
        gemm_issue(tm + TM_DX, mn_major(aM, kRows), mn_major(smem_u32(sDY), kP), make_idesc(64, 1, 1), kRows, false);
        gemm_issue(tm + TM_U, k_major(aB, kN), mn_major(aHS, kP), make_idesc(64, 0, 1), kN, false);
        gemm_issue(tm + TM_DB, k_major(smem_u32(sXw), kP), k_major(aHS, kP), make_idesc(128, 0, 0), kP, false);
        // every product that reads dS is in this first group: the dx epilogue, which runs while the other
        // three products do, stages its result in dS's buffer
        umma_commit(&bars[1]);
        gemm_issue(tm + TM_DB, mn_major(aDG, kRows), mn_major(aC, kN), make_idesc(128, 1, 1), kRows, true);
        gemm_issue(tm + TM_T1, k_major(aDG, kRows), mn_major(aB, kN), make_idesc(128, 0, 1), kRows, true);
        gemm_issue(tm + TM_DH, mn_major(aC, kN), mn_major(smem_u32(sDYe), kP), make_idesc(64, 1, 1), kRows, true);
        umma_commit(&bars[4]);
      }
      __syncwarp();
    }
    // Nothing of this CTA may be in flight when it lets go of its shared memory and TMEM.
    if (total > 0) {
      mbar_wait(&bars[0], (total - 1) & 1);
      mbar_wait(&bars[1], (total - 1) & 1);
      mbar_wait(&bars[4], (total - 1) & 1);
    }
  } else {
    regs_for_epilogue();
    // --------------------------------------------------------------------------------------------
    // Epilogue warps.
    // --------------------------------------------------------------------------------------------
    const int quad = warp & 3, ch = warp >> 2;
    const int row = quad * 32 + lane;
    const int rl = row / R, rr = row % R;  // time step within the tile and rank of this thread's row
    int total = 0;  // tiles this CTA goes through in all
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo im = item_of(item);
      total += im.k_hi - im.k_lo;
    }

    bool dead = false;  // a bounded wait of this warp gave up: it keeps the barriers going, nothing else
    int it = 0;
    for (int item = blockIdx.x; SPLIT ? item < nitems : item == (int)blockIdx.x; item += SPLIT ? (int)gridDim.x : 1) {
      const ItemInfo im = item_of(item);
      const int bh = im.bh, b = im.b, h = im.h, seg = im.seg, k_lo = im.k_lo, k_hi = im.k_hi;
      const bool rev = h >= H - p.rev;
      const int Hs = rev ? -H : H;
      auto tok_at = [&](int s) { return ((size_t)b * T + (rev ? T - 1 - s : s)) * H + h; };
      const float dsk = p.d_skip ? p.d_skip[h] : 0.0f;
      {
        // dH^T <- gradient reaching the returned h (or zero) for the stripe's last segment, else what the
        // segment after this one handed over (bounded wait for its flag); likewise the running sum of d phi
        const bool seeded = seg + 1 < nseg;
        if (seeded) {
          if (tid == 0) *s_ok = wait_flag(p.seg_flag + (size_t)bh * nseg + seg + 1, wait_limit << 4) ? 1 : 0;
          epi_sync();
          if (!*s_ok) dead = true;
        }
        const float* src = seeded ? p.seg_state + ((size_t)bh * nseg + seg + 1) * kP * kN
                                  : (p.dh ? p.dh + (size_t)bh * kP * kN : nullptr);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int p0 = 32 * ch + 16 * cc;
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = src ? __ldcg(src + (size_t)(p0 + j) * kN + row) : 0.0f;
          tmem_st16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
        }
        tmem_wait_st();
        if (tid < kNH) s_dcar[tid] = seeded ? __ldcg(p.seg_angle + ((size_t)bh * nseg + seg + 1) * kNH + tid) : 0.0f;
        epi_sync();
      }
      for (int k = k_hi - 1; k >= k_lo; --k, ++it) {
      const int t0 = k * LT;
      const size_t tok0 = tok_at(t0);
      const bool last_tile = (k == ntiles - 1);
      const int l_end = T - 1 - t0;  // row of the final token when last_tile
      const TileScalars ts = scal_set(it & 1);
      bar_sync(bar_ahead(it), kPairCount);  // the tile's scalars
      if (it == 0 && total > 1) epi_signal(BAR_FREE, kPairCount, dead);  // the other set has never been used
      // ---- 1. the tile's rows have been landing since the previous tile let go of the buffers --------
      if (!dead) dead = !warp_all(mbar_wait(&bars[2], it & 1, wait_limit));
      if (ROT) {
        if (!dead)
          epi_angle_table<R>(sTab, s_q, p.ckpt_angle + ((size_t)bh * ntiles + k) * kNH, nullptr, ts.dt, T, t0, rev,
                             nullptr, nullptr);
        else
          epi_sync();  // the pass's own barrier
      }
      // ---- 2. operands, converted in place --------------------------------------------------------
      {
        RawBC<R, ROT> raw_bc;
        if (!dead) {
          {  // x and dy have staging of their own: plain conversion, with the scaled copies sigma_w X~ and exp(acum) dY~
            RawPX<R> raw_p;
            load_px_staged<R>(raw_p, rawX, rev);
            store_px<R>(raw_p, sX, sXw, ts.sw);
            load_px_staged<R>(raw_p, rawDY, rev);
            store_px<R>(raw_p, sDY, sDYe, ts.eac);
          }
        }
        fence_async_smem();
        tc_fence_before();
        epi_signal(BAR_OPS0, kPairCount, dead);
        if (!dead) load_bc_staged<R, ROT>(raw_bc, sB, sC, rev);
        epi_sync();  // every warp holds its share of the rows of B and C (and the angle table is complete)
        if (!dead) store_bc<R, ROT>(raw_bc, sB, sC, sTab);
      }
      fence_async_smem();
      tc_fence_before();
      epi_signal(BAR_OPS, kPairCount, dead);
      if (ROT) {
        // This row's (cos, sin) words go into TMEM, for the un-rotation after phase B, while C^ B^^T runs: the
        // product does not read them.  The table lies where the first 128 / R rows of M are about to be
        // written, so the warps that write those rows (the lower quadrants, the ones with time to spare in
        // epilogue A) wait until every warp has its words; the others only report.
        if (!dead) {
#pragma unroll
          for (int c4 = 0; c4 < 4; ++c4) {
            float v[16];
#pragma unroll
            for (int j4 = 0; j4 < 4; ++j4) {
              const float4 q4 = *reinterpret_cast<const float4*>(&sTab[phi_idx(rl, 16 * c4 + 4 * j4)]);
              v[4 * j4] = q4.x; v[4 * j4 + 1] = q4.y; v[4 * j4 + 2] = q4.z; v[4 * j4 + 3] = q4.w;
            }
            tmem_st16(tmem_addr(tm, quad * 32, TM_TAB + 16 * c4), v);
          }
          tmem_wait_st();
        }
        if (quad * 32 < kRows / R) bar_sync(BAR_TABLE, kEpiThreads); else bar_arrive(BAR_TABLE, kEpiThreads);
      }
      if (!dead) dead = !warp_all(mbar_wait(&bars[0], it & 1, wait_limit));
      // ---- 3. epilogue A -------------------------------------------------------------------------
      const float acl = ts.ac[rl];
      const float cd = ts.ac[LT - 1];
      const float ecd = expc(cd);
      float dcd_part = 0.0f;
      if (!dead) {
        tc_fence_after();
        const int lmax = (quad * 32 + 31) / R;
        float rowE = 0.0f, dgp = 0.0f;
#pragma unroll 1
        for (int cb = 0; cb < 2; ++cb) {
          const int c0 = 64 * ch + 32 * cb;
          float dbd[32];
          if (c0 / R > lmax) {
            const float z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
            for (int q8 = 0; q8 < 4; ++q8) {
              store_chunk(sM, tile_off(row, c0 + 8 * q8, kRows), z);
              store_chunk(sDG, tile_off(row, c0 + 8 * q8, kRows), z);
            }
            part_col[quad * 128 + c0 + lane] = 0.0f;
            continue;
          }
          float gq[2][16], dmq[2][16];
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_G + c0 + 16 * hb), gq[hb]);
            tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DM + c0 + 16 * hb), dmq[hb]);
          }
          tmem_wait_ld();
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) { tmem_ld_fence(gq[hb]); tmem_ld_fence(dmq[hb]); }
#pragma unroll
          for (int hb = 0; hb < 2; ++hb) {
            const float (&g)[16] = gq[hb];
            const float (&dm)[16] = dmq[hb];
            float mv[16], dgv[16];
            ColScalars<R> cs;
            load_col_scalars<R>(cs, ts, c0 + 16 * hb);
            const int s0 = (c0 + 16 * hb) / R;
            const float rf = row_factor(acl, ts.ac[s0 + 16 / R - 1]);  // one exponential per chunk
            // A chunk whose last step precedes the first row of this warp lies strictly below the
            // diagonal for all 32 rows (the case of most chunks of the lower rows): no selects needed.
            if (s0 + 16 / R - 1 < (quad * 32) / R) {
              // two columns per instruction (packed fp32 pairs): the epilogues are bound by instruction issue
              const float2 rf2 = make_float2(rf, rf);
              float2 rowE2 = make_float2(0.0f, 0.0f);
#pragma unroll
              for (int j = 0; j < 16; j += 2) {
                const int sa = j / R, sb = (j + 1) / R;
                const float2 w2 = make_float2(cs.w[sa], cs.w[sb]);
                const float2 dec = __fmul2_rn(rf2, make_float2(cs.cf[sa], cs.cf[sb]));
                const float2 wgt = __fmul2_rn(w2, dec);
                const float2 g2 = make_float2(g[j], g[j + 1]), dm2 = make_float2(dm[j], dm[j + 1]);
                const float2 d2 = __fmul2_rn(dm2, __fmul2_rn(g2, dec));
                const float2 m2 = __fmul2_rn(g2, wgt), dg2 = __fmul2_rn(dm2, wgt);
                rowE2 = __ffma2_rn(d2, w2, rowE2);
                mv[j] = m2.x; mv[j + 1] = m2.y;
                dgv[j] = dg2.x; dgv[j + 1] = dg2.y;
                dbd[16 * hb + j] = d2.x; dbd[16 * hb + j + 1] = d2.y;
              }
              rowE += rowE2.x + rowE2.y;
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {  // branch-free selects: below / on / above the diagonal
                const int si = j / R, s = s0 + si;
                const bool below = s < rl, on = s == rl;
                const float dec = rf * cs.cf[si];
                const float wgt = below ? cs.w[si] * dec : (on ? cs.g[si] : 0.0f);
                const float gd = g[j] * dec;
                const float d_ = below ? dm[j] * gd : 0.0f;
                mv[j] = g[j] * wgt;
                dgv[j] = dm[j] * wgt;
                rowE += d_ * cs.w[si];
                dgp += on ? dm[j] * g[j] : 0.0f;
                dbd[16 * hb + j] = d_;
              }
            }
            float lo[8], hi[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { lo[j] = mv[j]; hi[j] = mv[8 + j]; }
            store_chunk(sM, tile_off(row, c0 + 16 * hb, kRows), lo);
            store_chunk(sM, tile_off(row, c0 + 16 * hb + 8, kRows), hi);
#pragma unroll
            for (int j = 0; j < 8; ++j) { lo[j] = dgv[j]; hi[j] = dgv[8 + j]; }
            store_chunk(sDG, tile_off(row, c0 + 16 * hb, kRows), lo);
            store_chunk(sDG, tile_off(row, c0 + 16 * hb + 8, kRows), hi);
          }
          const float colsum = warp_column_sums(dbd);
          part_col[quad * 128 + c0 + lane] = colsum;
        }
        part_row[ch * 128 + row] = rowE;
        part_dg[ch * 128 + row] = dgp;
        // carry-out term: T1 = dY~ H_k ; d acum += exp(acum) <T1, C^> ; dC^ base = exp(acum) T1
        float t1[4][16], dhv[2][16];
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_T1 + 64 * ch + 16 * cc), t1[cc]);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DH + 32 * ch + 16 * cc), dhv[cc]);
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) tmem_ld_fence(t1[cc]);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) tmem_ld_fence(dhv[cc]);
        const float eac = ts.eac[rl];
        const float2 eac2 = make_float2(eac, eac);
        float2 dot2 = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          const int n0 = 64 * ch + 16 * cc;
          float c1[8], c2[8];
          load_chunk(sC, tile_off(row, n0, kN), c1);
          load_chunk(sC, tile_off(row, n0 + 8, kN), c2);
#pragma unroll
          for (int j = 0; j < 8; j += 2) {
            dot2 = __ffma2_rn(make_float2(t1[cc][j], t1[cc][j + 1]), make_float2(c1[j], c1[j + 1]), dot2);
            dot2 = __ffma2_rn(make_float2(t1[cc][8 + j], t1[cc][9 + j]), make_float2(c2[j], c2[j + 1]), dot2);
          }
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float2 v = __fmul2_rn(make_float2(t1[cc][j], t1[cc][j + 1]), eac2);
            t1[cc][j] = v.x; t1[cc][j + 1] = v.y;
          }
          tmem_st16(tmem_addr(tm, quad * 32, TM_T1 + n0), t1[cc]);
        }
        part_t1[ch * 128 + row] = dot2.x + dot2.y;
        // state gradient: lanes are n, columns p; H_k and dS_k are kept [n][p], so a thread's 16 columns are
        // two 16-byte pieces of its own row
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int p0 = 32 * ch + 16 * cc;
          float hk[16];
          load_chunk(sHS, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&hk[0]));
          load_chunk(sHS, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&hk[8]));
#pragma unroll
          for (int j = 0; j < 16; ++j) dcd_part += dhv[cc][j] * hk[j];  // <dH, H_k>
          store_row16(sHS, row, p0, kP, dhv[cc]);                        // dS_k replaces H_k
#pragma unroll
          for (int j = 0; j < 16; j += 2) {
            const float2 v = __fmul2_rn(make_float2(dhv[cc][j], dhv[cc][j + 1]), make_float2(ecd, ecd));
            dhv[cc][j] = v.x; dhv[cc][j + 1] = v.y;
          }
          tmem_st16(tmem_addr(tm, quad * 32, TM_DH + p0), dhv[cc]);
        }
        tmem_wait_st();
      }
      fence_async_smem();
      tc_fence_before();
      epi_signal(BAR_MID, kPairCount, dead);
      // (the sum behind d cd is wanted by the tile's last step only: it is taken while phase B runs)
      const float dcd = ecd * inside(cd) * epi_sum(dcd_part, s_red);
      // ---- 4. epilogue B -------------------------------------------------------------------------
      if (!dead) dead = !warp_all(mbar_wait(&bars[1], it & 1, wait_limit));
      const int t = t0 + rl;
      const bool live = t < T;
      const bool at_end = last_tile && rl == l_end;
      // Column blocks of this thread in a [128 x 128] gradient tile: with rotation the pairs
      // (m, m + 64) must sit in one thread, so it takes [32ch, 32ch+32) and [64+32ch, 64+32ch+32).
      auto gcol = [&](int q4) { return ROT ? ((q4 >> 1) * kNH + 32 * ch + 16 * (q4 & 1)) : (64 * ch + 16 * q4); };
      float dD_part = 0.0f;
      float dphi[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) dphi[j] = 0.0f;
      if (!dead) {
        tc_fence_after();
        float acc[2][16], u[2][16];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DX + 32 * ch + 16 * cc), acc[cc]);
          tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_U + 32 * ch + 16 * cc), u[cc]);
        }
        tmem_wait_ld();
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) { tmem_ld_fence(acc[cc]); tmem_ld_fence(u[cc]); }
        {  // dx = M^T dY~ + sw (B^ dS^T) + D dy ; q = <U, x>
          const float sw = ts.sw[rl];
          const float2 sw2 = make_float2(sw, sw), dsk2 = make_float2(dsk, dsk);
          float2 qp2 = make_float2(0.0f, 0.0f), dD2 = make_float2(0.0f, 0.0f);
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int p0 = 32 * ch + 16 * cc;
            float xv[16], dyv[16];
            load_chunk(sX, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&xv[0]));
            load_chunk(sX, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&xv[8]));
            load_chunk(sDY, tile_off(row, p0, kP), *reinterpret_cast<float(*)[8]>(&dyv[0]));
            load_chunk(sDY, tile_off(row, p0 + 8, kP), *reinterpret_cast<float(*)[8]>(&dyv[8]));
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
              const float2 u2 = make_float2(u[cc][j], u[cc][j + 1]), x2 = make_float2(xv[j], xv[j + 1]);
              const float2 dy2 = make_float2(dyv[j], dyv[j + 1]);
              qp2 = __ffma2_rn(u2, x2, qp2);
              dD2 = __ffma2_rn(dy2, x2, dD2);
              const float2 a2 = __ffma2_rn(sw2, u2, __ffma2_rn(dsk2, dy2, make_float2(acc[cc][j], acc[cc][j + 1])));
              acc[cc][j] = a2.x; acc[cc][j + 1] = a2.y;
            }
            if (at_end && p.dlu) {  // gradient through last_u = sum_r x (x) B^ at the final token
#pragma unroll 1
              for (int j = 0; j < 16; ++j) {
                const float* gl = p.dlu + ((size_t)bh * kP + p0 + j) * kN;
                float s_ = 0.0f;
                for (int n = 0; n < kN; ++n)
                  s_ += gl[n] * __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sB + tile_off(row, n, kN)));
                float add[16];
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) add[jj] = (jj == j) ? s_ : 0.0f;
#pragma unroll
                for (int jj = 0; jj < 16; ++jj) acc[cc][jj] += add[jj];
              }
            }
            if constexpr (R != 2) stage_out16<R>(sHS, row, p0, acc[cc], rev);  // dS is spent: its buffer stages dx
          }
          if constexpr (R == 2) stage_out32<R>(sHS, row, 32 * ch, acc[0], acc[1], rev);  // rank 2: both halves at once
          part_q[ch * 128 + row] = qp2.x + qp2.y;
          dD_part = dD2.x + dD2.y;
        }
      }
      if (!dead) dead = !warp_all(mbar_wait(&bars[4], it & 1, wait_limit));  // the other four products
      if (!dead) {
        tc_fence_after();
        {  // dB^ (TM_DB, operand sB, out db) then dC^ (TM_T1, operand sC, out dc)
          float gq[4][16], tabv[2][16];
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_DB + gcol(q4)), gq[q4]);
          if (ROT) {
#pragma unroll
            for (int mc = 0; mc < 2; ++mc) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_TAB + 32 * ch + 16 * mc), tabv[mc]);
          }
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) tmem_ld_fence(gq[q4]);
          if (ROT) { tmem_ld_fence(tabv[0]); tmem_ld_fence(tabv[1]); }
          auto finish = [&](float (&g)[4][16], const uint8_t* sop, uint8_t* stg, bool is_b) {
            if (is_b && at_end && p.dlu) {  // d last_u reaches B^ of the final token: += dlu^T x
#pragma unroll 1
              for (int q4 = 0; q4 < 4; ++q4)
#pragma unroll 1
                for (int j = 0; j < 16; ++j) {
                  const int n = gcol(q4) + j;
                  float s_ = 0.0f;
                  for (int pp = 0; pp < kP; ++pp)
                    s_ += p.dlu[((size_t)bh * kP + pp) * kN + n] *
                          __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(sX + tile_off(row, pp, kP)));
#pragma unroll
                  for (int a4 = 0; a4 < 4; ++a4)
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) g[a4][jj] += (a4 == q4 && jj == j) ? s_ : 0.0f;
                }
            }
            if (ROT) {
#pragma unroll
              for (int mc = 0; mc < 2; ++mc) {
                const int m0 = 32 * ch + 16 * mc;
                float (&g1)[16] = g[mc];
                float (&g2)[16] = g[2 + mc];
                float o1[16], o2[16];
                load_chunk(sop, tile_off(row, m0, kN), *reinterpret_cast<float(*)[8]>(&o1[0]));
                load_chunk(sop, tile_off(row, m0 + 8, kN), *reinterpret_cast<float(*)[8]>(&o1[8]));
                load_chunk(sop, tile_off(row, kNH + m0, kN), *reinterpret_cast<float(*)[8]>(&o2[0]));
                load_chunk(sop, tile_off(row, kNH + m0 + 8, kN), *reinterpret_cast<float(*)[8]>(&o2[8]));
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  dphi[16 * mc + j] += g1[j] * o2[j] - g2[j] * o1[j];
                  const uint32_t cw = __float_as_uint(tabv[mc][j]);
                  const float2 csn = __half22float2(*reinterpret_cast<const __half2*>(&cw));
                  const float cs = csn.x, sn = csn.y;
                  const float u1 = g1[j] * cs - g2[j] * sn, u2 = g1[j] * sn + g2[j] * cs;
                  g1[j] = u1; g2[j] = u2;
                }
              }
            }
            if constexpr (R == 2) {
#pragma unroll
              for (int q4 = 0; q4 < 4; q4 += 2) stage_out32<R>(stg, row, gcol(q4), g[q4], g[q4 + 1], rev);
            } else {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) stage_out16<R>(stg, row, gcol(q4), g[q4], rev);
            }
          };
          finish(gq, sB, sXw, true);     // sigma_w X~ and exp(acum) dY~ are spent: 32 KB to stage dB
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) tmem_ld16_issue(tmem_addr(tm, quad * 32, TM_T1 + gcol(q4)), gq[q4]);
          tmem_wait_ld();
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) tmem_ld_fence(gq[q4]);
          finish(gq, sC, sDG, false);    // dG is spent: its buffer stages dC
        }
      }
      fence_async_smem();  // the staged gradients, for the stores that read them
      epi_sync();
      if (!tile_leaves_by_map<R>(p.out_maps, rev, T, t0)) {
        if (!dead) {
          if (p.dx) copy_out_rows<R>(sHS, p.dx, kP, tok0, Hs, T, t0, rev);
          if (p.db) copy_out_rows<R>(sXw, p.db, kN, tok0, Hs, T, t0, rev);
          if (p.dc) copy_out_rows<R>(sDG, p.dc, kN, tok0, Hs, T, t0, rev);
        }
        epi_sync();
      }
      // every operand and table word of this tile has been read and its gradients are staged (or gone): the
      // copy warp sends them off and lets the next tile's rows, theta rows and checkpoint land
      epi_signal(BAR_TAIL, kPairCount, dead);
      if (ROT) {
        // d phi of a time step sums its R rows (adjacent lanes); it then takes the buffers of X~ and dY~,
        // which the phase-B products and the epilogue have finished reading.
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          float v = dphi[j];
#pragma unroll
          for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          dphi[j] = v;
        }
        // Ranks 1 and 4 store four planes (16 bytes) at a time - the buffer's swizzle moves whole 16-byte pieces -
        // and keep the scan's running sums in registers; on rank 2 both measured slower (backward + 1.8 % on the
        // scaling workload: the kernel's timing follows its code layout more than its instruction count), so
        // rank 2 keeps the plane-by-plane stores and the second pass over shared memory.
        if constexpr (R == 2) {
          if (rr == 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              float v = live ? dphi[j] : 0.0f;
              if (at_end && p.dangle) v += p.dangle[(size_t)bh * kNH + 32 * ch + j];
              sDphi[phi_idx(rl, 32 * ch + j)] = v;
            }
          }
        } else if (rr == 0) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float v[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              v[c] = live ? dphi[j + c] : 0.0f;
              if (at_end && p.dangle) v[c] += p.dangle[(size_t)bh * kNH + 32 * ch + j + c];
            }
            *reinterpret_cast<float4*>(&sDphi[phi_idx(rl, 32 * ch + j)]) = make_float4(v[0], v[1], v[2], v[3]);
          }
        }
      }
      const float dD_tile = epi_sum(dD_part, s_red);  // also orders part_* and sDphi for what follows
      if (tid == 0) p.partD[(size_t)bh * ntiles + k] = dD_tile;
      // ---- 5. reverse cumulative sum of d phi over time -> d theta, and the dt term -----------------
      if (ROT) {
        constexpr int LQ = LT / 4, NV = 4 / R;  // NV: (time step, 8-plane group) items per thread
        const int q = tid >> 6, m = tid & 63;
        uint4 thq[NV];  // theta of this thread's items of the vector pass below, requested early
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int iv = tid + 256 * i, l = iv >> 3, mg = iv & 7;
          thq[i] = (t0 + l < T) ? __ldg(reinterpret_cast<const uint4*>(p.theta + (tok0 + (size_t)l * Hs) * kNH + mg * 8))
                                : make_uint4(0u, 0u, 0u, 0u);
        }
        float run = 0.0f, loc[R == 2 ? 1 : LQ];  // (not rank 2:) the quarter's running sums wait in registers
#pragma unroll
        for (int i = LQ - 1; i >= 0; --i) {
          run += sDphi[phi_idx(q * LQ + i, m)];
          if constexpr (R == 2) sDphi[phi_idx(q * LQ + i, m)] = run;
          else loc[i] = run;
        }
        s_q[q * 64 + m] = run;
        epi_sync();
        float off = s_dcar[m];
        for (int qq = 3; qq > q; --qq) off += s_q[qq * 64 + m];
#pragma unroll
        for (int i = 0; i < LQ; ++i) {  // d step: sum of d phi from here on
          if constexpr (R == 2) sDphi[phi_idx(q * LQ + i, m)] += off;
          else sDphi[phi_idx(q * LQ + i, m)] = loc[i] + off;
        }
        const float total = off + s_q[0 * 64 + m];  // for q == 0: carry + all four quarters
        epi_sync();
        if (q == 0) {
          s_dcar[m] = total;
          if (k == 0 && p.dangle0) p.dangle0[(size_t)bh * kNH + m] = total;
        }
        // vector pass: d theta = d step * dt (16-byte stores) and the rotation's share of d dt
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int iv = tid + 256 * i, l = iv >> 3, mg = iv & 7;
          const float4 d0 = *reinterpret_cast<const float4*>(&sDphi[phi_idx(l, mg * 8)]);
          const float4 d1 = *reinterpret_cast<const float4*>(&sDphi[phi_idx(l, mg * 8 + 4)]);
          const float ds[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
          const uint32_t tw[4] = {thq[i].x, thq[i].y, thq[i].z, thq[i].w};
          const float dtl = ts.dt[l];
          float prod = 0.0f, o[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            prod += ds[2 * j] * bf16_lo(tw[j]) + ds[2 * j + 1] * bf16_hi(tw[j]);
            o[2 * j] = ds[2 * j] * dtl;
            o[2 * j + 1] = ds[2 * j + 1] * dtl;
          }
          if (t0 + l < T && p.dtheta) {
            uint4 qv;
            qv.x = pack_bf16(o[0], o[1]); qv.y = pack_bf16(o[2], o[3]); qv.z = pack_bf16(o[4], o[5]); qv.w = pack_bf16(o[6], o[7]);
            *reinterpret_cast<uint4*>(p.dtheta + (tok0 + (size_t)l * Hs) * kNH + mg * 8) = qv;
          }
#pragma unroll
          for (int o_ = 1; o_ < 8; o_ <<= 1) prod += __shfl_xor_sync(0xffffffffu, prod, o_);
          if (mg == 0) part_rot[l] = prod;
        }
        epi_sync();
      }
      // ---- 6. per-token scalars of the tile ---------------------------------------------------------
      if (tid < LT) {
        const int l = tid;
        float rows = 0.0f, t1 = 0.0f, q = 0.0f, dgv = 0.0f, col = 0.0f;
#pragma unroll
        for (int r = 0; r < R; ++r) {
          const int ro = l * R + r;
          rows += part_row[ro] + part_row[128 + ro];
          t1 += part_t1[ro] + part_t1[128 + ro];
          q += part_q[ro] + part_q[128 + ro];
          dgv += part_dg[ro] + part_dg[128 + ro];
          col += part_col[ro] + part_col[128 + ro] + part_col[256 + ro] + part_col[384 + ro];
        }
        const float ac = ts.ac[l], w = ts.w[l];
        const float raw = cd - ac;
        const float sg = expc(raw);
        const float dast = sg * w * q * inside(raw);
        const float dac = ts.eac[l] * inside(ac) * t1;
        s_dacum[l] = rows - w * col + dac - dast;
        s_dast[l] = dast;
        const size_t o = (size_t)bh * Tp + t0 + l;
        p.dw[o] = col + sg * q;
        p.dg[o] = dgv;
        if (ROT) p.ddt_rot[o] = part_rot[l];
      }
      epi_sync();
      if (warp == 0) {  // reverse inclusive scan of d acum (+ the chunk-decay terms on the last step)
        constexpr int EPL = LT / 32;
        float tail = 0.0f;
        for (int i = lane; i < LT; i += 32) tail += s_dast[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tail += __shfl_xor_sync(0xffffffffu, tail, o);
        tail += dcd;
        float loc[EPL];
        float run = 0.0f;
#pragma unroll
        for (int i = EPL - 1; i >= 0; --i) {
          const int l = lane * EPL + i;
          run += s_dacum[l] + (l == LT - 1 ? tail : 0.0f);
          loc[i] = run;
        }
        float tot = run;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float n = __shfl_down_sync(0xffffffffu, tot, o);
          if (lane + o < 32) tot += n;
        }
        const float base = tot - run;
        float pa = 0.0f;
#pragma unroll
        for (int i = 0; i < EPL; ++i) {
          const int l = lane * EPL + i;
          const float da = base + loc[i];
          p.da[(size_t)bh * Tp + t0 + l] = da;
          pa += da * ts.dt[l];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pa += __shfl_xor_sync(0xffffffffu, pa, o);
        if (lane == 0) p.partA[(size_t)bh * ntiles + k] = pa;
      }
      // this tile's scalars are spent: the look-ahead warp may overwrite their set
      if (it + 2 < total) epi_signal(BAR_FREE, kPairCount, dead);
      epi_sync();
      }
      {
        // ---- the item's first tile is done: the gradient of the seed state, or the hand-over to the
        //      segment before this one ------------------------------------------------------------------
        const bool hand_over = seg > 0;
        float first = 0.0f;
        if (!hand_over && p.h0) {
          const size_t i0 = tok_at(0);
          const float l0 = p.disc == 0 ? 1.0f : (p.disc == 1 ? 0.5f : bf(p.lam, i0));
          first = (1.0f - l0) * bf(p.dt, i0);
        }
        float ip = 0.0f;
        if (!dead) {
          tc_fence_after();
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            const int p0 = 32 * ch + 16 * cc;
            float v[16];
            tmem_ld16(tmem_addr(tm, quad * 32, TM_DH + p0), v);
            if (hand_over) {
              float* dst = p.seg_state + ((size_t)bh * nseg + seg) * kP * kN;
#pragma unroll
              for (int j = 0; j < 16; ++j) __stcg(dst + (size_t)(p0 + j) * kN + row, v[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const size_t o = ((size_t)bh * kP + p0 + j) * kN + row;
                if (p.dh0) p.dh0[o] = v[j];
                if (p.dlu0) p.dlu0[o] = first * v[j];
                if (p.lu0) ip += v[j] * p.lu0[o];
              }
            }
          }
        }
        if (hand_over) {
          if (tid < kNH) __stcg(p.seg_angle + ((size_t)bh * nseg + seg) * kNH + tid, s_dcar[tid]);
          __threadfence();
          epi_sync();
          // raised even by a CTA that gave up, so that nobody waits in vain: the error flag tells the host
          if (tid == 0) raise_handover(p.seg_flag + (size_t)bh * nseg + seg);
        } else {
          const float tot = epi_sum(ip, s_red);
          if (tid == 0) p.ip0[bh] = tot;
        }
      }
    }
    if (dead && lane == 0 && p.err) raise_flag(p.err);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tm, TM_COLS);
}

template <int R>
cudaError_t launch_r(cudaStream_t st, const TcBwdParams& p, bool rot) {
  auto kern = p.nseg > 1 ? (rot ? tc_bwd_kernel<R, true, true> : tc_bwd_kernel<R, false, true>) : (rot ? tc_bwd_kernel<R, true, false> : tc_bwd_kernel<R, false, false>);
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  if (e != cudaSuccess) return e;
  kern<<<p.grid, kCtaThreads, kSmemBytes, st>>>(p);
  return cudaGetLastError();
}

}  // namespace

cudaError_t tc_backward(cudaStream_t st, const TcBwdParams& p, bool rot) {
  if (p.use_tma && p.R == 1 && !rot) return tc_backward_direct(st, p);
  switch (p.R) {
    case 1: return launch_r<1>(st, p, rot);
    case 2: return launch_r<2>(st, p, rot);
    case 4: return launch_r<4>(st, p, rot);
    default: return cudaErrorInvalidValue;
  }
}

}  // namespace m3
