// Blackwell (sm_100a) building blocks of the tensor-core kernel family: tcgen05 MMA with
// TMEM accumulators, shared-memory operand descriptors, bounded mbarrier waits.
//
// Operand format used throughout: a [rows x cols] bf16 matrix is stored as 8x8 "core
// matrices" of 128 contiguous bytes (8 rows of 16 bytes), tiled [rows/8][cols/8]:
//     offset(r, c) = ((r/8) * (cols/8) + c/8) * 128 + (r%8) * 16 + (c%8) * 2   bytes.
// The same buffer is a K-major operand when the contraction runs along `cols`
// (LBO = 128, SBO = (cols/8)*128) and an MN-major operand when it runs along `rows`
// (SBO = 128, LBO = (cols/8)*128); no swizzle.  Verified against exact integer-valued
// products on a B200 before any kernel was built on it.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace m3tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint32_t tile_off(int r, int c, int cols) {
  return (uint32_t)((((r >> 3) * (cols >> 3) + (c >> 3)) << 7) + ((r & 7) << 4) + ((c & 7) << 1));
}

// Shared-memory matrix descriptor, no swizzle, version 1 (Blackwell).
__device__ __forceinline__ uint64_t make_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;
  return d;
}

// Instruction descriptor: bf16 x bf16 -> f32, M = 128, given N and operand majors.
__host__ __device__ constexpr uint32_t make_idesc(int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One operand of a GEMM whose K extent is `k_total`: base address and strides.
struct Operand {
  uint32_t addr, lbo, sbo, kstep;
};
// Buffer [rows x cols] used with K along cols.
__device__ __forceinline__ Operand k_major(uint32_t addr, int cols) {
  return Operand{addr, 128u, (uint32_t)(cols >> 3) << 7, 256u};
}
// Buffer [rows x cols] used with K along rows (M/N along cols).
__device__ __forceinline__ Operand mn_major(uint32_t addr, int cols) {
  return Operand{addr, (uint32_t)(cols >> 3) << 7, 128u, (uint32_t)(cols >> 3) << 8};
}

// D[128 x n] (+)= A * B over k_total (multiple of 16); issued by ONE thread.  The descriptors of
// step k differ from those of step 0 only in the start address (low 14 bits, in 16-byte units,
// which cannot carry out of the field for shared-memory addresses), so they are built once and
// advanced by an add: the issuing thread is on the critical path of every tile.
__device__ __forceinline__ void gemm_issue(uint32_t tmem_d, Operand a, Operand b, uint32_t idesc, int k_total,
                                           bool accumulate_first) {
  uint64_t da = make_desc(a.addr, a.lbo, a.sbo), db = make_desc(b.addr, b.lbo, b.sbo);
  const uint64_t sa = a.kstep >> 4, sb = b.kstep >> 4;
#pragma unroll 4
  for (int k = 0; k < k_total / 16; ++k) {
    umma(tmem_d, da, db, idesc, (accumulate_first || k > 0) ? 1u : 0u);
    da += sa;
    db += sb;
  }
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

// Wait for a phase of an mbarrier with an iteration limit: at most limit - 1 polls (each poll may itself
// block for a hardware-defined time), so a limit of 1 gives up at once.  Returns false if it gave up; the
// caller reports that through an error flag and stops working - it never spins without bound.
constexpr uint32_t kWaitLimit = 1u << 18;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint32_t limit = kWaitLimit) {
  const uint32_t a = smem_u32(bar);
  for (uint32_t it = 1; it < limit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}\n"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}

// Report a wait that gave up: the flag is one int of host memory mapped into this GPU's address
// space (the host reads it without a copy), so a plain store and a system-wide fence.
__device__ __forceinline__ void raise_flag(int* flag) {
  *reinterpret_cast<volatile int*>(flag) = 1;
  __threadfence_system();
}

// Bulk tensor copies (TMA) of this GPU's own memory into this CTA's shared memory, completion
// counted in bytes on an mbarrier.  expect_tx arms the barrier for one phase.
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One box of a 4-D tiled tensor map whose two inner coordinates are zero (see tc_make_tile_map).
__device__ __forceinline__ void tma_load_tile(void* dst, const void* tensor_map, uint64_t* bar, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tensor_map), "r"(smem_u32(bar)), "r"(0), "r"(0), "r"(c2), "r"(c3)
      : "memory");
}

// One box of a row map (tc_make_row_map): columns from `col`, head h, time steps from t (may be negative
// or run past the end: those rows arrive as zeros), batch b.
__device__ __forceinline__ void tma_load_rows(void* dst, const void* tensor_map, uint64_t* bar, int col, int h, int t, int b) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(tensor_map), "r"(smem_u32(bar)), "r"(col), "r"(h), "r"(t), "r"(b)
      : "memory");
}

// The reverse direction: one box of a row map leaves shared memory (laid out as tma_load_rows would have
// landed it) for the tensor; rows past the tensor's end are dropped.  `t` must not be negative.  The copy
// joins the issuing thread's current bulk group (bulk_commit / bulk_wait_read / bulk_wait_all).
__device__ __forceinline__ void tma_store_rows(const void* tensor_map, const void* src, int col, int h, int t, int b) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(tensor_map),
               "r"(smem_u32(src)), "r"(col), "r"(h), "r"(t), "r"(b)
               : "memory");
}

// A contiguous block (16-byte aligned, a multiple of 16 bytes) of this GPU's memory into shared memory.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// The reverse direction: a contiguous block of shared memory leaves for global memory (both 16-byte
// aligned, a multiple of 16 bytes).  The issuing thread closes a group; bulk_wait_read returns once
// its groups have finished READING shared memory, bulk_wait_all once they are written out.
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Whole-warp calls.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}

// TMEM address of (lane, column) relative to an allocation base.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
  return base + ((uint32_t)lane << 16) + (uint32_t)col;
}

// 16 consecutive columns of this thread's lane (warp-collective; lane field = warp's quadrant base).
__device__ __forceinline__ void tmem_ld16(uint32_t addr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(addr)
      : "memory");
  tmem_wait_ld();
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// The same load without the wait: issue several, then tmem_wait_ld() once, then pass every
// destination array through tmem_ld_fence() before the first use (it pins the uses behind the
// wait; it emits no instruction).
__device__ __forceinline__ void tmem_ld16_issue(uint32_t addr, float (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=f"(v[0]), "=f"(v[1]), "=f"(v[2]), "=f"(v[3]), "=f"(v[4]), "=f"(v[5]), "=f"(v[6]), "=f"(v[7]), "=f"(v[8]),
        "=f"(v[9]), "=f"(v[10]), "=f"(v[11]), "=f"(v[12]), "=f"(v[13]), "=f"(v[14]), "=f"(v[15])
      : "r"(addr)
      : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_ld_fence(float (&v)[N]) {
#pragma unroll
  for (int i = 0; i < N; ++i) asm volatile("" : "+f"(v[i]));
}

__device__ __forceinline__ void tmem_st16(uint32_t addr, const float (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(addr),
      "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
      "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
      "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
      "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15]))
      : "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float bf16_lo(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }

}  // namespace m3tc
