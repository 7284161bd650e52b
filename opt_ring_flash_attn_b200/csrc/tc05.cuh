// Thin inline-PTX layer for Blackwell (sm_100a): mbarrier, TMA tile loads,
// tcgen05 tensor-memory allocation, MMA issue, and TMEM <-> register moves.
//
// Conventions used by every kernel in this directory
//  * Shared-memory operand tiles use the 128-byte swizzle. A tile is a set of
//    "panels"; one panel is [rows][64 x 16-bit] = rows x 128 B, row r at byte
//    r*128, 16-byte chunk c stored at position c ^ (r & 7).  This is what a TMA
//    box of {64, rows} with CU_TENSOR_MAP_SWIZZLE_128B writes, and what the
//    UMMA shared-memory descriptor with layout type 2 reads.  Panels must start
//    on a 1024-byte boundary.
//  * "K-major" operand  : rows are the M/N index, the 64 columns of a panel are
//    the contraction index.  One MMA K-step (16 elements) = 32 bytes inside the
//    panel; the next panel holds the next 64 contraction elements.
//  * "MN-major" operand : rows are the contraction index, columns are the M/N
//    index.  One MMA K-step = 16 rows = 2048 bytes; the next panel holds the
//    next 64 M/N elements (leading byte offset = panel stride).
//  * Every wait on an mbarrier is bounded in wall-clock time.  When the bound
//    is hit the waiting thread raises a CTA-wide abort flag; all roles leave
//    their loops, meet at the final barrier, free TMEM and return.  The host
//    sees a non-zero status word; the context stays usable.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

namespace rfa {

// Status codes written to the device status word by kernels.
enum : int {
  kStatusOk = 0,
  kStatusWaitTimeout = 1,  // a bounded mbarrier wait ran out
};

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s per single wait

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
  // Makes barrier initialisation visible to the async proxy (TMA, tcgen05.commit).
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Non-blocking probe (try_wait may suspend the thread for a hardware-defined time before answering "not yet").
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait for the phase with the given parity to complete.  Returns false
// when the CTA is aborting (this thread timed out, or another one did).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (((++spins) & 0xffu) == 0) {
      if (*abort_flag) return false;
      if (global_timer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// Same, called by all 32 lanes of a warp; the result is made warp-uniform so
// that the warp-collective tcgen05 instructions that follow stay converged.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  bool ok = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, ok);
}

// ----------------------------------------------------------------------------
// Proxy / tcgen05 fences
// ----------------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
  // Orders generic-proxy shared-memory writes before async-proxy reads (MMA operand fetch).
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copy global -> shared, completion on an mbarrier)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tmap)) : "memory");
}

// 4-D tile load.  Coordinates are innermost first: (d, head, seq, batch).
// c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_4d(uint32_t smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(tmap)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2),
        "r"(c3)
      : "memory");
}

// 1-D bulk copy global -> shared (both 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gptr, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      :
      : "r"(smem_dst), "l"(reinterpret_cast<uint64_t>(gptr)), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

// ----------------------------------------------------------------------------
// Tensor memory allocation (whole warp executes these)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_holder, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_holder)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// Register re-balancing between warpgroups (all four warps of a warpgroup execute the same one).
// The counts used by a kernel must add up to at most the registers the launch allocated.
template <int N>
__device__ __forceinline__ void setmaxnreg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void setmaxnreg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ----------------------------------------------------------------------------
// MMA descriptors
// ----------------------------------------------------------------------------
// Instruction descriptor for kind::f16, fp32 accumulate.
//  bits [4,6) D format (1 = f32); [7,10) A format; [10,13) B format (0 = f16, 1 = bf16);
//  bit 15 A major (1 = MN); bit 16 B major (1 = MN); [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t make_idesc(int m, int n, bool is_bf16, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1.
//  bits [0,14) address >> 4; [16,30) leading byte offset >> 4; [32,46) stride byte
//  offset >> 4 (distance between groups of 8 rows = 1024 B); bits [46,48) = 1; [61,64) = 2.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes) {
  return static_cast<uint64_t>((saddr & 0x3ffffu) >> 4) | (static_cast<uint64_t>(lbo_bytes >> 4) << 16) |
         (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// K-major operand: the leading byte offset is not used by the hardware for swizzled layouts.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) { return smem_desc_sw128(saddr, 16); }
// MN-major operand: leading byte offset = distance between 64-element groups along M/N (panel stride).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t panel_stride_bytes) {
  return smem_desc_sw128(saddr, panel_stride_bytes);
}

// ----------------------------------------------------------------------------
// MMA issue (one thread) and completion tracking
// ----------------------------------------------------------------------------
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]   (A: 128 lanes x K, 16-bit elements packed two per column)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Cheap-to-issue variants: the MMA-issuing thread shares its scheduler with busy warps, so the
// per-instruction overhead matters.  A descriptor is split into a constant high word (stride byte
// offset 1024, version, 128-byte swizzle) and a low word (address >> 4 | leading byte offset << 16)
// that is advanced by adding (byte offset >> 4).
constexpr uint32_t kDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_kmajor(uint32_t saddr) { return ((saddr & 0x3ffffu) >> 4) | (1u << 16); }
__device__ __forceinline__ uint32_t desc_lo_mnmajor(uint32_t saddr, uint32_t panel_stride_bytes) {
  return ((saddr & 0x3ffffu) >> 4) | ((panel_stride_bytes >> 4) << 16);
}
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi)
      : "memory");
}
// Same with compile-time offsets (in 16-byte units) added to the base low words inside the asm block:
// only the bases stay live in registers of the issuing thread.
template <int A_OFF, int B_OFF>
__device__ __forceinline__ void mma_ss_off(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 da, {ra, %5};\n\t"
      "mov.b64 db, {rb, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "n"(A_OFF), "n"(B_OFF)
      : "memory");
}
template <int A_COL_OFF, int B_OFF>
__device__ __forceinline__ void mma_ts_off(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 db, {rb, %5};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "n"(A_COL_OFF), "n"(B_OFF)
      : "memory");
}
// Warp-converged issue.  All 32 lanes of the issuing warp run the surrounding loop (so the descriptor arithmetic is
// warp-uniform and cheap) and only the lane chosen once by elect_one() executes the instruction.  Measured on B200: an
// MMA issued from inside a single-lane branch costs the issuing thread 45-95 cycles depending on how busy the other
// warps of its scheduler are, the converged form 39-54 — the difference between starving and feeding a tensor pipe
// that retires one 128x128x16 MMA every 64 cycles.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t"
      "}"
      : "=r"(pred));
  return pred;
}
template <int A_OFF, int B_OFF>
__device__ __forceinline__ void mma_ss_off_e(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %8, 0;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 da, {ra, %5};\n\t"
      "mov.b64 db, {rb, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "n"(A_OFF), "n"(B_OFF),
        "r"(elected)
      : "memory");
}
template <int A_COL_OFF, int B_OFF>
__device__ __forceinline__ void mma_ts_off_e(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                             uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b32 ra, rb;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %8, 0;\n\t"
      "add.u32 ra, %1, %6;\n\t"
      "add.u32 rb, %2, %7;\n\t"
      "mov.b64 db, {rb, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "n"(A_COL_OFF), "n"(B_OFF),
        "r"(elected)
      : "memory");
}
__device__ __forceinline__ void mma_ss_lo_e(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc,
                                            uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b64 da, db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "mov.b64 da, {%1, %5};\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "r"(elected)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lo_e(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                            uint32_t accumulate, uint32_t elected) {
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      ".reg .b64 db;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "setp.ne.b32 q, %6, 0;\n\t"
      "mov.b64 db, {%2, %5};\n\t"
      "@q tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
      "}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(accumulate), "r"(kDescHi), "r"(elected)
      : "memory");
}
__device__ __forceinline__ void mma_commit_e(uint64_t* bar, uint32_t elected) {
  asm volatile(
      "{\n\t"
      ".reg .pred q;\n\t"
      "setp.ne.b32 q, %1, 0;\n\t"
      "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t"
      "}" ::"r"(smem_u32(bar)),
      "r"(elected)
      : "memory");
}
// Compile-time loop: f(std::integral_constant<int, I>) for I in [0, N).
template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F&& f) {
  if constexpr (I < N) {
    f(std::integral_constant<int, I>{});
    static_for<I + 1, N>(f);
  }
}
// The mbarrier receives one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// ----------------------------------------------------------------------------
// TMEM <-> registers.  Shape 32x32b: lane i of the warp accesses TMEM lane
// (32 * (warp_id % 4) + i); register j is column (base + j).
// ----------------------------------------------------------------------------
#define RFA_R8(r, o) "=r"(r[o + 0]), "=r"(r[o + 1]), "=r"(r[o + 2]), "=r"(r[o + 3]), "=r"(r[o + 4]), "=r"(r[o + 5]), "=r"(r[o + 6]), "=r"(r[o + 7])
#define RFA_RW8(r, o) "+r"(r[o + 0]), "+r"(r[o + 1]), "+r"(r[o + 2]), "+r"(r[o + 3]), "+r"(r[o + 4]), "+r"(r[o + 5]), "+r"(r[o + 6]), "+r"(r[o + 7])
#define RFA_I8(r, o) "r"(r[o + 0]), "r"(r[o + 1]), "r"(r[o + 2]), "r"(r[o + 3]), "r"(r[o + 4]), "r"(r[o + 5]), "r"(r[o + 6]), "r"(r[o + 7])

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : RFA_R8(r, 0), RFA_R8(r, 8), RFA_R8(r, 16), RFA_R8(r, 24)
      : "r"(taddr)
      : "memory");
}
// Completes all tcgen05.ld issued by this thread; the registers are listed as
// read-write operands so that the compiler cannot consume them earlier.
__device__ __forceinline__ void tmem_ld_wait32(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : RFA_RW8(r, 0), RFA_RW8(r, 8), RFA_RW8(r, 16), RFA_RW8(r, 24)
               :
               : "memory");
}
// Compiler-only fence for a second register block filled by an earlier tcgen05.ld: placed after
// tmem_ld_wait32 of the first block, it keeps uses of these registers behind the wait.
__device__ __forceinline__ void reg_fence32(uint32_t (&r)[32]) {
  asm volatile("" : RFA_RW8(r, 0), RFA_RW8(r, 8), RFA_RW8(r, 16), RFA_RW8(r, 24) : : "memory");
}
// 16-byte vector reduction (sm_90+): four consecutive floats, one L2 operation.
__device__ __forceinline__ void red_add_v4_f32(float* gptr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(gptr), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
// Cross-CTA counters in global memory: acquire load and release add at GPU scope.
__device__ __forceinline__ int ld_acquire_gpu(const int* gptr) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(gptr) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_gpu_add(int* gptr, int v) {
  asm volatile("red.release.gpu.global.add.s32 [%0], %1;" ::"l"(gptr), "r"(v) : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31};"
      :
      : RFA_I8(r, 0), RFA_I8(r, 8), RFA_I8(r, 16), RFA_I8(r, 24), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%16], "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15};"
      :
      : RFA_I8(r, 0), RFA_I8(r, 8), "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : RFA_R8(r, 0), RFA_R8(r, 8)
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;" : RFA_RW8(r, 0), RFA_RW8(r, 8) : : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ----------------------------------------------------------------------------
// Small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pairs of fp32 (Blackwell add/fma .f32x2: one issue slot for two lanes of arithmetic).
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack_u2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ void unpack_u2(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// 2^x for a pair, on the FMA pipe instead of the special-function unit: x = n + f with n = round(x) (magic-number
// rounding), 2^f by a cubic on [-0.5, 0.5] (relative error 7.5e-5, far below 16-bit rounding of the result), and n
// added to the exponent field.  x is clamped to >= -125 so that masked (-inf) entries come out as ~2^-125.
struct Exp2Poly {
  uint64_t magic, c0, c1, c2, c3, nc1, nc3;
  __device__ __forceinline__ Exp2Poly() {
    magic = pack_f2(12582912.f, 12582912.f);
    c0 = pack_f2(0.9999281168f, 0.9999281168f);
    c1 = pack_f2(0.6932609677f, 0.6932609677f);
    c2 = pack_f2(0.2426108569f, 0.2426108569f);
    c3 = pack_f2(0.0551714599f, 0.0551714599f);
    nc1 = pack_f2(-0.6932609677f, -0.6932609677f);
    nc3 = pack_f2(-0.0551714599f, -0.0551714599f);
  }
  __device__ __forceinline__ uint64_t operator()(uint64_t x2) const {
    float x0, x1;
    unpack_f2(x2, x0, x1);
    const uint64_t xc = pack_f2(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
    const uint64_t xr = add2(xc, magic);        // low mantissa bits = n (two's complement)
    const uint64_t n = sub2(xr, magic);         // round(x) as a float
    const uint64_t f = sub2(xc, n);
    uint64_t pl = fma2(c3, f, c2);
    pl = fma2(pl, f, c1);
    pl = fma2(pl, f, c0);
    uint32_t p0, p1, r0, r1;
    unpack_u2(pl, p0, p1);
    unpack_u2(xr, r0, r1);
    return pack_u2(p0 + (r0 << 23), p1 + (r1 << 23));
  }
  // 2^(-y) for a pair, for callers that hold the negated exponent.
  __device__ __forceinline__ uint64_t neg(uint64_t y2) const {
    float y0, y1;
    unpack_f2(y2, y0, y1);
    const uint64_t yc = pack_f2(fminf(y0, 125.f), fminf(y1, 125.f));
    const uint64_t xr = sub2(magic, yc);        // magic + x
    const uint64_t n = sub2(xr, magic);         // round(x)
    const uint64_t g = add2(yc, n);             // -(x - n)
    uint64_t pl = fma2(nc3, g, c2);
    pl = fma2(pl, g, nc1);
    pl = fma2(pl, g, c0);
    uint32_t p0, p1, r0, r1;
    unpack_u2(pl, p0, p1);
    unpack_u2(xr, r0, r1);
    return pack_u2(p0 + (r0 << 23), p1 + (r1 << 23));
  }
};

template <typename T>
struct Pack2;
template <>
struct Pack2<__nv_bfloat16> {
  static constexpr bool kIsBf16 = true;
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static float2 unpack(uint32_t u) {
    __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(v);
  }
};
template <>
struct Pack2<__half> {
  static constexpr bool kIsBf16 = false;
  __device__ __forceinline__ static uint32_t pack(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __device__ __forceinline__ static float2 unpack(uint32_t u) {
    __half2 v = *reinterpret_cast<__half2*>(&u);
    return __half22float2(v);
  }
};

// Optional per-role event trace (diagnostics): (tag << 48 | SM clock) records written by one
// designated thread per role into a caller-provided buffer laid out [cta][role][cap].
struct Tracer {
  unsigned long long* buf = nullptr;
  int cap = 0;
  int n = 0;
  __device__ __forceinline__ void init(unsigned long long* base, int n_ctas, int cap_, int n_roles, int role) {
    if (base != nullptr && static_cast<int>(blockIdx.x) < n_ctas) {
      buf = base + (static_cast<size_t>(blockIdx.x) * n_roles + role) * cap_;
      cap = cap_;
    }
  }
  __device__ __forceinline__ void mark(int tag) {
    if (buf != nullptr && n < cap) {
      buf[n++] = (static_cast<unsigned long long>(tag) << 48) | (static_cast<unsigned long long>(clock64()) & 0xffffffffffffull);
    }
  }
};

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a swizzled panel.
__device__ __forceinline__ uint32_t sw128_offset(int row, int chunk) {
  return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

}  // namespace rfa
