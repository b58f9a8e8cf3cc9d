// Warp roles of the tensor-core stripe kernels (384 threads per CTA):
//   warps 0-7   epilogue warps: stage the operands of a tile, run the TMEM epilogues, write outputs;
//   warp 8      issuer: every tcgen05.mma / tcgen05.commit of the CTA, and the state checkpoint's bulk
//               copy, so that no epilogue warp is held by the tensor pipe while products are issued;
//   warp 9      look-ahead warp: the per-token scalars of the NEXT tile (dt and lambda of the tile after
//               that wait in its registers), while the epilogue warps work on this one;
//   warp 10     copy warp: the bulk tensor copy requests of the next tile's raw rows.  A request holds
//               its thread until the copy engine accepts it, and the engine is slow to drain while the
//               tensor pipe and the epilogues keep shared memory busy (about 6.5 B per cycle measured
//               inside these kernels against 25-40 alone), so no warp with other duties issues them;
//   warp 11     idle.  It exists because a warp's registers come from its scheduler's file of 16 K (a
//               ninth warp alone would be a third warp on scheduler 0 and cap every thread at 168) and
//               because budgets move between warps only per group of four (setmaxnreg): warps 8-11 give
//               registers back, the eight epilogue warps take them.
// The groups meet at named barriers (one side arrives, the other syncs); every barrier operation is
// executed unconditionally, tile after tile, so a warp that gave up a bounded wait keeps the protocol
// alive and nobody is left waiting at a barrier.  The helpers' work is kept off every critical path by
// a whole tile of lead time: a warp that runs a little code once per tile finds it evicted from the
// instruction caches by the epilogues' long straight-line bodies (60-160 KB per kernel) and pays a fetch
// from L2 for every cache line of it - 200 instructions took most of a tile period - whether it is a
// helper warp or one epilogue warp taking a branch of its own (the scalars on an epilogue warp inside
// the wait for the first products made every tile 2.4 K cycles longer).
#pragma once
#include "m3_tc_stage.cuh"

namespace m3tc {

constexpr int kEpiThreads = 256, kCtaThreads = 384, kPairCount = kEpiThreads + 32;
constexpr int kIssuerWarp = 8, kScalarWarp = 9, kCopyWarp = 10;  // warp 11 idles

// Named barriers (0 is __syncthreads).
enum : int {
  BAR_EPI = 1,    // 256: the epilogue warps among themselves
  BAR_OPS = 2,    // 320: operands of a tile are staged (epilogue warps arrive; issuer and copy warp sync)
  BAR_MID = 3,    // 288: the second group of operands is staged (epilogue warps arrive; issuer syncs)
  BAR_AHEAD = 4,  // 288: scalars of a tile are ready (look-ahead warp arrives; epilogue warps sync); even tiles
  BAR_AHEAD_ODD = 7,  // the same for odd tiles: the look-ahead warp may finish a tile before its predecessor's
                      // scalars have been picked up, and a barrier holds one pending phase only
  BAR_FREE = 5,   // 288: a set of scalars is free again (epilogue warps arrive; look-ahead warp syncs)
  BAR_TAIL = 6,   // 288: a tile's gradients are staged, its operands spent (epilogue warps arrive; copy warp syncs)
  BAR_TABLE = 8,  // 256: (backward) every epilogue warp has copied its angle-table words out of the buffer M takes over
  BAR_OPS0 = 9,   // 288: the x / dy operands of a tile are staged, ahead of B and C (epilogue warps arrive; issuer syncs)
};

__device__ __forceinline__ void bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(int id, int count) {
  asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory");
}
__device__ __forceinline__ void epi_sync() { bar_sync(BAR_EPI, kEpiThreads); }
__device__ __forceinline__ int bar_ahead(int tile_index) { return (tile_index & 1) ? BAR_AHEAD_ODD : BAR_AHEAD; }
// An epilogue warp's side of a barrier a helper warp syncs on: arrive and go on - unless the warp has
// given up a bounded wait and only keeps the protocol alive: then it waits for the helper like everyone,
// so that it cannot run tiles ahead of a helper that is still inside a (bounded, but long) wait and pile
// a second phase of arrivals onto a barrier that holds one.
__device__ __forceinline__ void epi_signal(int id, int count, bool dead) {
  if (dead) bar_sync(id, count); else bar_arrive(id, count);
}

// Register budget per role.  The CTA's 384 threads start with 168 each and budgets only move inside that
// allocation: 256 x 232 + 128 x 40 = 384 x 168.  A request for more than the CTA owns never returns.
__device__ __forceinline__ void regs_for_epilogue() { asm volatile("setmaxnreg.inc.sync.aligned.u32 232;"); }
__device__ __forceinline__ void regs_for_helpers() { asm volatile("setmaxnreg.dec.sync.aligned.u32 40;"); }

// ---------------------------------------------------------------------------------------
// Work distribution.  A stripe (one batch row x head) is cut in time into `nseg` segments of `tps` tiles;
// an item is one segment of one stripe, numbered segment-major (all first segments, then all second ones
// ...; the backward pass starts from the last segment), and CTA c works through the items c, c + grid,
// c + 2 grid ... in that order.  A segment takes the state its predecessor left in global memory (fp32
// state, running angle; in the backward pass the state's gradient and the running sum of d phi) once that
// predecessor has raised its flag.  Items are handed out in dependency order and every CTA takes its own
// in increasing order, so the item a CTA waits for was always started before the one that waits; the wait
// is bounded all the same.  With one segment per stripe nothing is handed over at all.
// ---------------------------------------------------------------------------------------
// What an item number stands for.  Kept out of line: it runs once per item and role and divides twice
// (the kernels' code size is what their instruction fetch pays for).
struct ItemInfo {
  int bh, b, h, seg, k_lo, k_hi;
};
static __device__ __noinline__ ItemInfo decode_item(int item, int BH, int H, int ntiles, int nseg, int tps, int backward) {
  ItemInfo r;
  const int s = item / BH;
  r.seg = backward ? nseg - 1 - s : s;
  r.bh = item - s * BH;
  r.b = r.bh / H;
  r.h = r.bh - r.b * H;
  r.k_lo = r.seg * tps;
  r.k_hi = min(ntiles, r.k_lo + tps);
  return r;
}

// One thread's bounded wait for a hand-over flag (with back-off: the producer is another CTA).
__device__ __forceinline__ bool wait_flag(const int* flag, uint32_t limit) {
  for (uint32_t it = 1; it < limit; ++it) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v) return true;
    __nanosleep(it < 64 ? 100 : 1000);
  }
  return false;
}
__device__ __forceinline__ void raise_handover(int* flag) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(1) : "memory");
}

// true if every lane's wait succeeded (tcgen05.ld is warp-collective, so a warp gives up as one)
__device__ __forceinline__ bool warp_all(bool ok) { return __all_sync(0xffffffffu, ok); }

// ---------------------------------------------------------------------------------------
// Per-token scalars of one tile, by ONE warp (the arithmetic of tile_scalars): g, w (shifted add),
// a = dt A, inclusive cumulative sum ac, sw = exp(cd - ac) w, eac = exp(ac), column factors cf.
// Lane i owns the EPL consecutive steps i*EPL .. i*EPL + EPL - 1.
// ---------------------------------------------------------------------------------------
template <int R>
struct ScalarLoads {
  static constexpr int EPL = (kRows / R) / 32;
  float dt[EPL + 1], lam[EPL + 1];
};
// dt and lambda of the steps lane * EPL .. lane * EPL + EPL of the tile at t0 (one step of look-ahead),
// requested a whole tile before they are used: the loads are few but each is a sector of its own.
template <int R>
__device__ __forceinline__ void lookahead_load(ScalarLoads<R>& v, const __nv_bfloat16* dt, const __nv_bfloat16* lam,
                                               int disc, int b, int h, int H, int T, int t0, bool rev) {
  constexpr int EPL = ScalarLoads<R>::EPL;
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int i = 0; i <= EPL; ++i) {
    const int t = t0 + lane * EPL + i;
    v.dt[i] = 0.0f;
    v.lam[i] = 1.0f;
    if (t < T) {
      const size_t idx = ((size_t)b * T + (rev ? T - 1 - t : t)) * H + h;
      v.dt[i] = bf(dt, idx);
      v.lam[i] = disc == 0 ? 1.0f : (disc == 1 ? 0.5f : bf(lam, idx));
    }
  }
}
template <int R>
__device__ __forceinline__ void lookahead_scalars(const TileScalars& s, const ScalarLoads<R>& v, float A, int T, int t0) {
  constexpr int LT = kRows / R, EPL = LT / 32, SPC = 16 / R;
  const int lane = threadIdx.x & 31;
  float loc[EPL], wv[EPL];
  float run = 0.0f;
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int l = lane * EPL + i, t = t0 + l;
    float gv = 0.0f, w = 0.0f, av = 0.0f;
    if (t < T) {
      gv = v.lam[i] * v.dt[i];
      const float f = (t + 1 < T) ? (1.0f - v.lam[i + 1]) * v.dt[i + 1] : 0.0f;
      w = gv + f;
      av = v.dt[i] * A;
    }
    s.dt[l] = v.dt[i]; s.lam[l] = v.lam[i]; s.g[l] = gv; s.w[l] = w; s.a[l] = av;
    wv[i] = w;
    run += av;
    loc[i] = run;
  }
  if (lane == 31) { s.dt[LT] = v.dt[EPL]; s.lam[LT] = v.lam[EPL]; }
  float tot = run;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, tot, o);
    if (lane >= o) tot += n;
  }
  const float base = tot - run;
  const float cd = __shfl_sync(0xffffffffu, tot, 31);
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    loc[i] += base;
    s.ac[lane * EPL + i] = loc[i];
  }
  __syncwarp();
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int l = lane * EPL + i;
    s.sw[l] = expc(cd - loc[i]) * wv[i];
    s.eac[l] = expc(loc[i]);
    s.cf[l] = __expf(fmaxf(s.ac[(l / SPC) * SPC + SPC - 1] - loc[i], -87.0f));
  }
}

// Wrapped cumulative angle of one tile as a table of half2(cos phi, sin phi) words, [LT][64] at
// phi_idx(l, m), by the 256 threads of the epilogue warps: thread (q, m) owns plane m over the quarter q
// of the tile's steps.  The tile's raw theta rows ([LT][64] bf16, landed by a bulk tensor copy; for a head
// that walks right to left in memory order, i.e. step l in row LT - 1 - l) sit at the start of the table's
// own buffer and are consumed before any table word is written (one barrier separates the passes).
// `carry_in` [64] holds the angle entering the tile (shared or global memory), `carry_out` (may be NULL,
// may alias carry_in) receives the wrapped angle leaving it; `s_q` is [4][64] floats of exchange space; dt
// comes from the tile's scalars.  sin / cos come from the
// special-function unit (the argument is wrapped into [-pi, pi] first, where its error is far below the
// half-precision table's).  Contains one barrier of the epilogue warps; the caller's next one publishes
// the table.
template <int R>
__device__ __forceinline__ void epi_angle_table(float* tab, float* s_q, const float* carry_in, float* carry_out,
                                                const float* s_dt, int T, int t0, bool rev, float* ckpt_slot,
                                                float* angle_out_bh) {
  constexpr int LT = kRows / R, LQ = LT / 4;
  const __nv_bfloat16* raw = reinterpret_cast<const __nv_bfloat16*>(tab);
  const int tid = threadIdx.x, q = tid >> 6, m = tid & 63;
  float loc[LQ];
  float run = 0.0f;
#pragma unroll
  for (int i = 0; i < LQ; ++i) {
    const int l = q * LQ + i;
    run = fmaf(s_dt[l], __bfloat162float(raw[(rev ? LT - 1 - l : l) * kNH + m]), run);
    loc[i] = run;
  }
  s_q[q * 64 + m] = run;
  const float cin = carry_in[m];
  if (ckpt_slot && q == 0) ckpt_slot[m] = cin;
  epi_sync();
  float off = cin;
  for (int qq = 0; qq < q; ++qq) off += s_q[qq * 64 + m];
  if (carry_out && q == 3) carry_out[m] = wrap2pi(off + run);
#pragma unroll
  for (int i = 0; i < LQ; ++i) {
    const int l = q * LQ + i;
    const float wv = wrap2pi(loc[i] + off);
    const __half2 h2 = __floats2half2_rn(__cosf(wv), __sinf(wv));
    tab[phi_idx(l, m)] = __uint_as_float(*reinterpret_cast<const uint32_t*>(&h2));
    if (angle_out_bh && t0 + l == T - 1) angle_out_bh[m] = wv;
  }
}

// (cos, sin) of the eight planes [m0, m0 + 8) of step l from the table (m0 a multiple of 8).
__device__ __forceinline__ void table_cos_sin(const float* tab, int l, int m0, float (&cs)[8], float (&sn)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(&tab[phi_idx(l, m0)]);
  const float4 b = *reinterpret_cast<const float4*>(&tab[phi_idx(l, m0 + 4)]);
  const uint32_t w[8] = {__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w),
                         __float_as_uint(b.x), __float_as_uint(b.y), __float_as_uint(b.z), __float_as_uint(b.w)};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
    cs[j] = f.x;
    sn[j] = f.y;
  }
}

// ---------------------------------------------------------------------------------------
// Raw rows of a tile as the caller stores them, [step][col * R + r], landed by bulk tensor copies of a
// row map (tc_make_row_map): panels of [LT][<= 256 elements], one per 256 columns.  Heads that walk right
// to left receive the tile's time range in memory order, so scan step l sits in row LT - 1 - l.
// Work items are (step, 16-byte group) pairs (convert_coords).
// ---------------------------------------------------------------------------------------
template <int R>
struct RawTile {
  static constexpr int LT = kRows / R;
  static constexpr uint32_t kPanelBytes = (uint32_t)LT * 128u;   // [LT][64 elements], 16-byte chunks XOR-swizzled by row & 7
  static constexpr uint32_t panels(int cols) { return (uint32_t)(cols * R) / 64u; }
  static constexpr uint32_t bytes(int cols) { return panels(cols) * kPanelBytes; }
  // byte offset of the 16-byte piece holding elements [e, e + 8) of scan step l (e a multiple of 8)
  static __device__ __forceinline__ uint32_t piece(int l, uint32_t e, bool rev) {
    const uint32_t rowi = (uint32_t)(rev ? LT - 1 - l : l);
    return (e >> 6) * kPanelBytes + rowi * 128u + ((((e >> 3) & 7u) ^ (rowi & 7u)) << 4);
  }
};
// Requests for one tile's rows of one tensor, by the lanes [lane0, lane0 + panels) of a warp, one panel
// each (a request occupies its thread for hundreds of cycles; side by side they cost one): first scan
// step t0, head h, batch b.  `dst` is 1024-byte aligned (the swizzle pattern repeats every eight rows of
// 128 bytes).  Returns the number of lanes used.
template <int R>
__device__ __forceinline__ int request_raw_tile(int lane0, uint8_t* dst, const void* map, uint64_t* bar, int cols, int b,
                                                int h, int T, int t0, bool rev) {
  using RT = RawTile<R>;
  const int t = rev ? T - t0 - RT::LT : t0;
  const int pn = (int)(threadIdx.x & 31) - lane0;
  if (pn >= 0 && pn < (int)RT::panels(cols))
    tma_load_rows(dst + (uint32_t)pn * RT::kPanelBytes, map, bar, pn * 64, h, t, b);
  return (int)RT::panels(cols);
}

// ---------------------------------------------------------------------------------------
// Results on their way out.  A thread owns a folded row (l, r) of an accumulator tile; the caller's tensor
// wants rows [step][col * R + r].  The tile is staged in shared memory exactly as a bulk tensor copy of a
// row map would have landed it (the layout of RawTile), and leaves by bulk tensor stores, one box per 64
// elements of a row, issued side by side by the lanes of one warp: no thread carries the bytes.  The ranks
// of a step sit in neighbouring lanes, so the interleave is an exchange of registers (rank 2), not a pass
// over shared memory.  A tile whose box would start before the tensor (the ragged last tile of a head that
// walks right to left) leaves by plain 16-byte stores instead.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void st_shared16(uint8_t* dst, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  *reinterpret_cast<uint4*>(dst) = make_uint4(a, b, c, d);
}
// 16 consecutive columns [col0, col0 + 16) of folded row `row` (col0 a multiple of 16).  Whole warps only.
template <int R>
__device__ __forceinline__ void stage_out16(uint8_t* stg, int row, int col0, const float (&v)[16], bool rev) {
  using RT = RawTile<R>;
  const int l = row / R;
  if constexpr (R == 4) {  // no exchange for rank 4: element by element
    const int r = row % R;
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const uint32_t e = (uint32_t)(col0 + j) * R + r;
      *reinterpret_cast<__nv_bfloat16*>(stg + RT::piece(l, e & ~7u, rev) + (e & 7u) * 2u) = __float2bfloat16_rn(v[j]);
    }
  } else {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
    if constexpr (R == 1) {
      st_shared16(stg + RT::piece(l, (uint32_t)col0, rev), w[0], w[1], w[2], w[3]);
      st_shared16(stg + RT::piece(l, (uint32_t)col0 + 8u, rev), w[4], w[5], w[6], w[7]);
    } else {
      // lanes (2i, 2i + 1) hold ranks 0 and 1 of one step: the even lane takes columns [col0, col0 + 8) of
      // both ranks, the odd one [col0 + 8, col0 + 16)
      const bool odd = row & 1;
      uint32_t mine[4], theirs[4], o[8];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        mine[i] = odd ? w[4 + i] : w[i];
        theirs[i] = __shfl_xor_sync(0xffffffffu, odd ? w[i] : w[4 + i], 1);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t r0 = odd ? theirs[k >> 1] : mine[k >> 1], r1 = odd ? mine[k >> 1] : theirs[k >> 1];
        o[k] = __byte_perm(r0, r1, (k & 1) ? 0x7632 : 0x5410);
      }
      const uint32_t e0 = (uint32_t)(col0 + (odd ? 8 : 0)) * 2u;
      st_shared16(stg + RT::piece(l, e0, rev), o[0], o[1], o[2], o[3]);
      st_shared16(stg + RT::piece(l, e0 + 8u, rev), o[4], o[5], o[6], o[7]);
    }
  }
}
// 32 consecutive columns [col0, col0 + 32) of folded row `row` (col0 a multiple of 32).  Whole warps only.
// For rank 2 the two lanes of a step split the 32 columns between them - the even lane takes the first 16 of
// both ranks, the odd lane the last 16 - so that a quarter warp (4 steps x 2 lanes) writes into both 64-byte
// halves of its rows at once and its eight 16-byte stores fall into eight bank groups; with 16 columns at a
// time (stage_out16) both lanes of a step write into the same half and every store is served twice.
template <int R>
__device__ __forceinline__ void stage_out32(uint8_t* stg, int row, int col0, const float (&va)[16], const float (&vb)[16],
                                            bool rev) {
  if constexpr (R != 2) {
    stage_out16<R>(stg, row, col0, va, rev);
    stage_out16<R>(stg, row, col0 + 16, vb, rev);
  } else {
    using RT = RawTile<R>;
    const int l = row / R;
    const bool odd = row & 1;
    uint32_t wa[8], wb[8], other[8], o[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      wa[i] = pack_bf16(va[2 * i], va[2 * i + 1]);
      wb[i] = pack_bf16(vb[2 * i], vb[2 * i + 1]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) other[i] = __shfl_xor_sync(0xffffffffu, odd ? wa[i] : wb[i], 1);
#pragma unroll
    for (int k = 0; k < 16; ++k) {
      // even lane: ranks (mine, theirs) of the first 16 columns; odd lane: (theirs, mine) of the last 16
      const uint32_t r0 = odd ? other[k >> 1] : wa[k >> 1], r1 = odd ? wb[k >> 1] : other[k >> 1];
      o[k] = __byte_perm(r0, r1, (k & 1) ? 0x7632 : 0x5410);
    }
    const uint32_t e0 = (uint32_t)(col0 + (odd ? 16 : 0)) * 2u;
#pragma unroll
    for (int q = 0; q < 4; ++q) st_shared16(stg + RT::piece(l, e0 + 8u * q, rev), o[4 * q], o[4 * q + 1], o[4 * q + 2], o[4 * q + 3]);
  }
}
// May the tile at scan step t0 leave by bulk tensor stores?
template <int R>
__device__ __forceinline__ bool tile_leaves_by_map(int has_maps, bool rev, int T, int t0) {
  return has_maps && !(rev && T - t0 - kRows / R < 0);
}
// The stores of one staged tile of one tensor (`cols` columns per rank), by the lanes [lane0, lane0 + panels)
// of a warp.  The caller commits and waits for the group.  Returns the number of lanes used.
template <int R>
__device__ __forceinline__ int store_out_tile(int lane0, const uint8_t* src, const void* map, int cols, int b, int h, int T,
                                              int t0, bool rev) {
  using RT = RawTile<R>;
  const int pn = (int)(threadIdx.x & 31) - lane0;
  if (pn >= 0 && pn < (int)RT::panels(cols))
    tma_store_rows(map, src + (uint32_t)pn * RT::kPanelBytes, pn * 64, h, rev ? T - t0 - RT::LT : t0, b);
  return (int)RT::panels(cols);
}
// The same tile by plain stores of the 256 epilogue threads: g[(tok0 + l * Hs) * cols * R + e], steps
// t0 + l < T only.
template <int R>
__device__ __forceinline__ void copy_out_rows(const uint8_t* stg, __nv_bfloat16* g, int cols, size_t tok0, int Hs, int T, int t0,
                                             bool rev) {
  constexpr int LT = kRows / R;
  const int E = cols * R, per_row = E / 8;
  for (int it = threadIdx.x; it < LT * per_row; it += kEpiThreads) {
    const int l = it / per_row, c = it - l * per_row;
    if (t0 + l >= T) continue;
    const uint4 q = *reinterpret_cast<const uint4*>(stg + RawTile<R>::piece(l, (uint32_t)c * 8u, rev));
    *reinterpret_cast<uint4*>(g + (tok0 + (size_t)((ptrdiff_t)l * Hs)) * E + (size_t)c * 8) = q;
  }
}

// R consecutive 16-byte pieces of a staged row, starting at element e, as 4 R words.
template <int R>
__device__ __forceinline__ void load_raw_pieces(const uint8_t* base, int l, uint32_t e, bool rev, uint32_t (&raw)[4 * R]) {
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const uint4 v = *reinterpret_cast<const uint4*>(base + RawTile<R>::piece(l, e + 8u * i, rev));
    raw[4 * i] = v.x; raw[4 * i + 1] = v.y; raw[4 * i + 2] = v.z; raw[4 * i + 3] = v.w;
  }
}

// The work items of a tile's conversion: (time step l, 16-byte column group grp) pairs.  Ranks 2 and 4: 4 steps
// x 8 groups per warp as in item_coords, with the bits of the group index permuted so that the two groups a
// quarter warp touches lie 4 / R apart: its eight lanes (4 steps x 2 groups) then read eight different
// 16-byte columns of the swizzled staging rows (a group is R pieces wide; the swizzle XORs the column with
// step & 7), and rank_rotation spreads their operand stores over the bank groups.  Rank 1 has no rank to
// rotate, so its warp covers 8 steps x 4 groups instead: a quarter warp is eight consecutive steps of one
// group - eight different rows & 7 for the operand stores, eight different swizzled columns for the reads.
template <int GB, int R>
__device__ __forceinline__ void convert_coords(int i, int& l, int& grp) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int w = warp + 8 * i;
  constexpr int GB8 = GB / 2;
  const int g3 = lane >> 2;
  if constexpr (R == 1) {
    l = (w / (2 * GB8)) * 8 + (lane & 3) + 4 * (g3 & 1);
    grp = (w % (2 * GB8)) * 4 + (g3 >> 1);
  } else {
    const int gp = R == 4 ? g3 : (((g3 & 1) << 1) | ((g3 >> 1) & 1) | (g3 & 4));
    l = (w / GB8) * 4 + (lane & 3);
    grp = (w % GB8) * 8 + gp;
  }
}

// Staged raw rows -> rotated (by -phi, from the table), rank-de-interleaved bf16 operands B^, C^.
template <int R, bool ROT>
__device__ __forceinline__ void convert_bc(const uint8_t* rawB, const uint8_t* rawC, uint8_t* sB, uint8_t* sC,
                                           const float* tab, bool rev) {
  using RB = RawBC<R, ROT>;
#pragma unroll
  for (int i = 0; i < RB::NIT; ++i) {
    int l, grp;
    convert_coords<RB::GB, R>(i, l, grp);
    const int n0 = grp * 8;
    const int rot = rank_rotation<R>();  // the order of the ranks differs by lane: see rank_rotation
    float cs[8], sn[8];
    if (ROT) table_cos_sin(tab, l, n0, cs, sn);
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      const uint8_t* src = which ? rawC : rawB;
      uint8_t* dst = which ? sC : sB;
      uint32_t v[RB::NP][4 * R];
#pragma unroll
      for (int part = 0; part < RB::NP; ++part)
        load_raw_pieces<R>(src, l, (uint32_t)(n0 + part * kNH) * R, rev, v[part]);
#pragma unroll
      for (int rr = 0; rr < R; ++rr) {
        const int r = rr ^ rot;
        if (ROT) {
          float o1[8], o2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float v1 = elem_rank<R>(v[0], j, r), v2 = elem_rank<R>(v[RB::NP - 1], j, r);
            o1[j] = v1 * cs[j] + v2 * sn[j];
            o2[j] = v2 * cs[j] - v1 * sn[j];
          }
          store_chunk(dst, tile_off(l * R + r, n0, kN), o1);
          store_chunk(dst, tile_off(l * R + r, n0 + kNH, kN), o2);
        } else {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = elem_rank<R>(v[0], j, r);
          store_chunk(dst, tile_off(l * R + r, n0, kN), o);
        }
      }
    }
  }
}


// x-like rows ([step][p * R + r], head_dim 64) of a staged tile into registers and back out as the
// rank-de-interleaved operand plus a copy scaled per time step; same work items as convert_bc, so a
// tile converted IN PLACE (operand written over the staging rows) needs one barrier of the epilogue
// warps between the two calls.
template <int R>
__device__ __forceinline__ void load_px_staged(RawPX<R>& raw, const uint8_t* src, bool rev) {
#pragma unroll
  for (int i = 0; i < RawPX<R>::NIT; ++i) {
    int l, grp;
    convert_coords<2, R>(i, l, grp);
    load_raw_pieces<R>(src, l, (uint32_t)(grp * 8) * R, rev, raw.v[i]);
  }
}
template <int R>
__device__ __forceinline__ void store_px(const RawPX<R>& raw, uint8_t* s_plain, uint8_t* s_scaled, const float* scale) {
#pragma unroll
  for (int i = 0; i < RawPX<R>::NIT; ++i) {
    int l, grp;
    convert_coords<2, R>(i, l, grp);
    const float sv = scale[l];
    const int rot = rank_rotation<R>();
#pragma unroll
    for (int rr = 0; rr < R; ++rr) {
      const int r = rr ^ rot;
      float o[8], ow[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) { o[j] = elem_rank<R>(raw.v[i], j, r); ow[j] = o[j] * sv; }
      store_chunk(s_plain, tile_off(l * R + r, grp * 8, kP), o);
      store_chunk(s_scaled, tile_off(l * R + r, grp * 8, kP), ow);
    }
  }
}
// The two halves of convert_bc for a tile converted in place.
template <int R, bool ROT>
__device__ __forceinline__ void load_bc_staged(RawBC<R, ROT>& raw, const uint8_t* rawB, const uint8_t* rawC, bool rev) {
  using RB = RawBC<R, ROT>;
#pragma unroll
  for (int i = 0; i < RB::NIT; ++i) {
    int l, grp;
    convert_coords<RB::GB, R>(i, l, grp);
#pragma unroll
    for (int which = 0; which < 2; ++which)
#pragma unroll
      for (int part = 0; part < RB::NP; ++part)
        load_raw_pieces<R>(which ? rawC : rawB, l, (uint32_t)(grp * 8 + part * kNH) * R, rev, raw.v[i][which][part]);
  }
}
template <int R, bool ROT>
__device__ __forceinline__ void store_bc(const RawBC<R, ROT>& raw, uint8_t* sB, uint8_t* sC, const float* tab) {
  using RB = RawBC<R, ROT>;
#pragma unroll
  for (int i = 0; i < RB::NIT; ++i) {
    int l, grp;
    convert_coords<RB::GB, R>(i, l, grp);
    const int n0 = grp * 8;
    const int rot = rank_rotation<R>();  // the order of the ranks differs by lane: see rank_rotation
    float cs[8], sn[8];
    if (ROT) table_cos_sin(tab, l, n0, cs, sn);
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      uint8_t* dst = which ? sC : sB;
#pragma unroll
      for (int rr = 0; rr < R; ++rr) {
        const int r = rr ^ rot;
        if (ROT) {
          float o1[8], o2[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float v1 = elem_rank<R>(raw.v[i][which][0], j, r), v2 = elem_rank<R>(raw.v[i][which][RB::NP - 1], j, r);
            o1[j] = v1 * cs[j] + v2 * sn[j];
            o2[j] = v2 * cs[j] - v1 * sn[j];
          }
          store_chunk(dst, tile_off(l * R + r, n0, kN), o1);
          store_chunk(dst, tile_off(l * R + r, n0 + kNH, kN), o2);
        } else {
          float o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) o[j] = elem_rank<R>(raw.v[i][which][0], j, r);
          store_chunk(dst, tile_off(l * R + r, n0, kN), o);
        }
      }
    }
  }
}

// Sum over the 256 threads of the epilogue warps; red: >= 8 floats of shared scratch.  Contains two of
// their barriers.
__device__ __forceinline__ float epi_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  epi_sync();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  epi_sync();
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += red[i];
  return s;
}

}  // namespace m3tc
