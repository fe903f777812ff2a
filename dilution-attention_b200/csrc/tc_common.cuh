// Blackwell (sm_100a) building blocks for the bf16 tensor-core path: mbarriers
// with bounded waits, TMA tile loads, TMEM allocation, tcgen05.mma issue/commit
// and tcgen05.ld, plus the shared-memory and instruction descriptors they take.
//
// Conventions used by every kernel built on these:
//  * operand tiles are [128 rows][64 bf16] = 16 KB, written by TMA with the
//    128-byte swizzle; row pitch 128 B, 8-row groups 1024 B apart, tile base
//    1024-byte aligned.  Read as a K-major operand the rows are the M/N index
//    and the 64 elements the contraction index; read as an MN-major operand the
//    64 elements are the M/N index and the rows the contraction index;
//  * accumulators live in TMEM with M = 128: row r of D is TMEM lane r, column
//    c of D is TMEM column base+c (fp32);
//  * every wait on an mbarrier gives up after kWaitCycles, records a code in the
//    device status word and raises the CTA's abort flag; later waits return at
//    once, the CTA drains, frees its TMEM and exits.  Loop bounds and addresses
//    never depend on data, so an aborted CTA stays in bounds.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace dil {
namespace tc {

constexpr int kTileRows = 128;
constexpr int kHeadDim = 64;
constexpr uint32_t kTileBytes = kTileRows * kHeadDim * 2;   // 16 KB
constexpr long long kWaitCycles = 4000000000LL;             // ~2 s: a live wait is microseconds

enum : int { kErrWaitTma = 101, kErrWaitMma = 102, kErrWaitDrain = 103, kErrAlign = 104, kErrWaitTile = 105, kErrSelfTest = 199 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Per-CTA control block in shared memory.
struct Ctl {
  volatile int abort;   // raised by the first wait that ran out
  uint32_t tmem;        // written by tcgen05.alloc
};

// Bounded wait.  Returns false (after one probe, if the CTA is already aborting) when
// the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, Ctl* ctl, int* status,
                                          int code, long long limit = kWaitCycles) {
  if (mbar_try(bar, parity)) return true;      // the common case costs one instruction
  if (ctl->abort) return false;
  const long long t0 = clock64();
  while (!mbar_try(bar, parity)) {
    if (clock64() - t0 > limit) {
      ctl->abort = 1;
      atomicCAS(status, 0, code);
      return false;
    }
  }
  return true;
}

// After a wait has given up, the CTA runs to its end without waiting for anything, so copies and
// MMAs it issued may still be in flight when it gets there.  Every kernel calls this in front of its
// last CTA-wide barrier: a CTA that gave up idles for a fixed grace period (about 0.2 ms, three
// orders of magnitude above a copy's or an MMA's latency) before it frees its TMEM and returns.
__device__ __forceinline__ void drain_if_aborted(const Ctl* ctl) {
  if (ctl->abort) {
    const long long t0 = clock64();
    while (clock64() - t0 < 400000LL) {
    }
  }
}

// ---- fences -------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA ----------------------------------------------------------------------
// One [box rows][64 bf16] tile of a (n, t, 64) tensor: coordinates (0, row, n).
__device__ __forceinline__ void tma_load_tile(uint32_t dst, const CUtensorMap* map, int row, int n,
                                              uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(0), "r"(row), "r"(n)
      : "memory");
}

// Element-wise add of a shared-memory tile into global memory (performed at L2), one
// instruction for the whole box; coordinates (col, row, n).  Rows/columns outside the
// tensor are dropped.  The issuing thread commits the group and, before the tile is
// overwritten, waits until the copy engine has read it.
__device__ __forceinline__ void tma_reduce_add_tile(const CUtensorMap* map, uint32_t src, int col, int row,
                                                    int n) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4}], [%1];"
      :
      : "l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(col), "r"(row), "r"(n)
      : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_wait_read_all() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// ---- TMEM -----------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {   // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t taddr, uint32_t cols) {         // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
               : "memory");
}

// 32 consecutive fp32 columns of this thread's lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
      " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31},"
      " [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// The same wait, tied to the 32 registers a load filled: the compiler cannot move
// a use of them above the wait.
__device__ __forceinline__ void tmem_ld_wait(float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]),
                 "+r"(r[14]), "+r"(r[15]), "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]),
                 "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]), "+r"(r[24]), "+r"(r[25]),
                 "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

// One fp32 column of this thread's lane.
__device__ __forceinline__ void tmem_ld1(uint32_t taddr, float* v) {
  uint32_t r;
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
  *v = __uint_as_float(r);
}

// 16 consecutive fp32 columns of this thread's lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait16(float* v) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]),
                 "+r"(r[7]), "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]),
                 "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}

// 16 consecutive 32-bit columns of this thread's lane, written from registers.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0],"
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ---- descriptors ------------------------------------------------------------------
// Shared-memory matrix descriptor, 128-byte swizzle, for the 16 KB tile layout above.
//   K-major view : 8-row groups 1024 B apart (SBO); LBO unused.
//   MN-major view: the 64 contiguous elements are one MN group (LBO = distance to the
//                  next group of 64, for tiles wider than 64); 8 contraction rows per
//                  1024 B (SBO).
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;   // descriptor version of this architecture
  d |= (uint64_t)2 << 61;   // 128-byte swizzle
  return d;
}

// Instruction descriptor: bf16 x bf16 -> fp32, M x N, operand majors (0 = K-major, 1 = MN-major).
__host__ __device__ constexpr uint32_t instr_desc(int m, int n, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// A descriptor is kept as two 32-bit halves.  The start address sits in the low half, so
// stepping through a tile is one 32-bit add of a constant to a value built once outside
// the loop: the issuing thread's own arithmetic, not the tensor pipe, limits the issue
// rate of small MMAs (about 45 cycles per instruction back to back, about 100 when each
// descriptor is rebuilt from an address).
struct Desc {
  uint32_t lo, hi;
};
__device__ __forceinline__ Desc make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  const uint64_t d = smem_desc(saddr, lbo_bytes, sbo_bytes);
  return Desc{(uint32_t)d, (uint32_t)(d >> 32)};
}
// D[tmem] (+)= A[smem] * B[smem]; one instruction covers 16 contraction elements.
// Offsets are added in descriptor units of 16 bytes.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, Desc a, uint32_t a_off16, Desc b, uint32_t b_off16,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\t"
      "mov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a.lo + a_off16), "r"(a.hi), "r"(b.lo + b_off16), "r"(b.hi), "r"(idesc),
        "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is an M x 16 bf16 operand held in TMEM, row m on
// lane m, two consecutive contraction elements per 32-bit column (8 columns).
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, Desc b, uint32_t b_off16,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b.lo + b_off16), "r"(b.hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

// S[128 x n_cols] = A[128 x 64] * B[n_cols x 64]^T, both K-major tiles: 4 instructions.
__device__ __forceinline__ void mma_scores(uint32_t d_tmem, uint32_t a_smem, uint32_t b_smem, int n_cols) {
  const uint32_t idesc = instr_desc(128, n_cols, 0, 0);
  const Desc a = make_desc(a_smem, 16, 1024), b = make_desc(b_smem, 16, 1024);
#pragma unroll
  for (int kk = 0; kk < 4; ++kk) mma_ss(d_tmem, a, 2 * kk, b, 2 * kk, idesc, kk > 0);
}

// Dynamic shared memory base rounded up to 1024 bytes.
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
  return p + ((1024u - (smem_u32(p) & 1023u)) & 1023u);
}

}  // namespace tc
}  // namespace dil
