// Blackwell (sm_100a) building blocks in inline PTX: mbarriers with bounded waits, TMA tile
// loads/stores through tensor maps, tensor-memory (TMEM) allocation, tcgen05.mma issue and
// completion, TMEM <-> register moves, and the shared-memory / instruction descriptors the
// tensor core consumes.  One CTA per tile, cta_group::1 everywhere, no cluster multicast.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fat {
namespace tc {

// ------------------------------------------------------------------------------- addresses
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One try: the hardware parks the thread until the phase completes or about `kWaitHintNs` pass, so a
// waiting warp does not compete for issue slots with the warps that are doing arithmetic.
#ifndef FAT_WAIT_HINT_NS
#define FAT_WAIT_HINT_NS 100000
#endif
constexpr uint32_t kWaitHintNs = FAT_WAIT_HINT_NS;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
#if FAT_WAIT_HINT_NS > 0
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs) : "memory");
#else
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
#endif
  return ok != 0;
}

// non-blocking test of a phase
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

// Every wait in these kernels is bounded.  When the bound is hit the kernel records a status
// word, raises a CTA-wide abort flag that makes all later waits fall through, and runs to
// its normal teardown (TMEM is released, the launch ends, the context stays usable).
#if defined(FAT_WAIT_SPINS)
constexpr uint32_t kWaitSpins = FAT_WAIT_SPINS;   // test builds: a wait gives up after FAT_WAIT_SPINS x kWaitHintNs
#elif FAT_WAIT_HINT_NS >= 100000
constexpr uint32_t kWaitSpins = 1u << 15;      // x kWaitHintNs: a few seconds at most
#elif FAT_WAIT_HINT_NS > 0
constexpr uint32_t kWaitSpins = (1u << 15) * (100000u / FAT_WAIT_HINT_NS);
#else
constexpr uint32_t kWaitSpins = 1u << 26;      // polls of a few dozen cycles each: a second or so
#endif

struct Guard {
  volatile int* abort_flag;   // shared memory, zeroed at kernel start
  int* status;                // global, may be null
  __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }
  __device__ __forceinline__ void fail(int where) const {
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, (1 << 24) | (where & 0xffffff));
  }
  // returns false when the wait was given up (or the CTA had already aborted)
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int where) const {
    for (uint32_t i = 0; i < kWaitSpins; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
      if (aborted()) return false;
    }
    fail(where);
    return false;
  }
  // The same for the single threads that sit on the critical path between two roles (the MMA issuers): they poll without
  // parking, which costs one warp's issue slots and wakes them some hundred cycles sooner.  Bounded like wait(): after
  // kPollSpins polls (about a second) it gives up.
  __device__ __forceinline__ bool wait_polling(uint64_t* bar, uint32_t parity, int where) const {
#ifdef FAT_WAIT_SPINS
    return wait(bar, parity, where);                      // test builds with short limits: one code path for the limit
#else
    constexpr uint32_t kPollSpins = 1u << 25;
    for (uint32_t i = 0; i < kPollSpins; ++i) {
      if (mbar_test_wait(bar, parity)) return true;
      if ((i & 63u) == 63u && aborted()) return false;
    }
    fail(where);
    return false;
#endif
  }
};

// ------------------------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 4-D tile load (coordinates: innermost first).  c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
        "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
// Element-wise add of a shared-memory tile into global memory (performed in L2).  Coordinates must not be negative.
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* m, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }   // all but the newest group
// generic-proxy writes to shared memory -> visible to the async proxy (TMA store, tcgen05.mma operands)
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ------------------------------------------------------------------------------- TMEM
// Allocation is a warp-wide instruction; `cols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// TMEM address: lane in bits 31..16, column in bits 15..0.
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 lanes x 32 columns of 32-bit: thread l of the warp receives lane (lane_base + l), columns col..col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

// ------------------------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for 128-byte-swizzled tiles (tile base 1024-byte aligned).
//   K-major  operand ([rows][64 elements] of 16-bit, 128 B per row): SBO = 1024 B between 8-row groups.
//   MN-major operand ([k rows][64 elements], chunks of 64 MN-elements `chunk_bytes` apart):
//            LBO = chunk_bytes, SBO = 1024 B between 8-k-row groups.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((saddr & 0x3ffff) >> 4);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fff) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fff) << 32;
  d |= uint64_t(1) << 46;       // descriptor version of this architecture
  d |= uint64_t(2) << 61;       // 128-byte swizzle
  return d;
}

// Instruction descriptor of tcgen05.mma kind::f16 with float32 accumulation.
//   a_fmt / b_fmt: 0 = f16, 1 = bf16 (the two operands may differ).
//   a_mn / b_mn: 1 when the operand is MN-major (transposed).
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, int a_fmt, int b_fmt, int a_mn, int b_mn) {
  return (1u << 4) | (uint32_t(a_fmt) << 7) | (uint32_t(b_fmt) << 10) | (uint32_t(a_mn) << 15) |
         (uint32_t(b_mn) << 16) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}
__host__ __device__ constexpr uint32_t idesc_f16(int M, int N, int ab_fmt, int a_mn, int b_mn) {
  return idesc_f16(M, N, ab_fmt, ab_fmt, a_mn, b_mn);
}

// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A holds two 16-bit elements per 32-bit column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(uint32_t(accumulate)) : "memory");
}
// The barrier receives one arrival when every tcgen05.mma issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Byte offset of element (row, 16-byte segment seg) inside a 128-byte-swizzled [rows][128 B] tile.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t seg) {
  return row * 128u + ((seg ^ (row & 7u)) << 4);
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

}  // namespace tc

// ------------------------------------------------------------------------------- host: tensor maps
// Encodes a 4-D tensor map over a [B,H,T,D] tensor of 16-bit elements with arbitrary (16-byte
// aligned) strides: dims {D, T, H, B}, box {box_d, box_t, 1, 1}, 128-byte swizzle, zero fill.
// Returns false (and sets the library error string) when the driver rejects the description.
bool make_tmap_bhtd(CUtensorMap* out, const void* base, int B, int H, int T, int D,
                    const int64_t* strides_bht, int box_d, int box_t);
// Same for a dense float32 [B,H,T,D] tensor, no swizzle (box rows are plain row-major in shared memory).
bool make_tmap_bhtd_f32(CUtensorMap* out, const void* base, int B, int H, int T, int D, int box_d, int box_t);

}  // namespace fat
