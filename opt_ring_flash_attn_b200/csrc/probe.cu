// Diagnostic kernel: one 128x128x128 product through each operand path used by
// the hop kernels (see rfa_debug_mma_probe in rfa_b200_debug.h).  It exists so
// that a wrong descriptor field or swizzle shows up as a wrong 128x128 matrix in
// a unit test instead of as a wrong attention result.
#include "common.h"
#include "tc05.cuh"

namespace rfa {

__global__ void __launch_bounds__(128, 1)
    mma_probe_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                     const __nv_bfloat16* __restrict__ a_gmem, float* __restrict__ c_out, int mode, int* status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t s_a = base;            // 2 panels x 16 KB
  const uint32_t s_b = base + 32768u;   // 2 panels x 16 KB
  constexpr uint32_t kPanel = 128 * 128;

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = tmem_holder;
  volatile int* abort_p = &abort_flag;
  const uint32_t lane_addr = static_cast<uint32_t>(warp * 32) << 16;
  const int row = warp * 32 + lane;
  constexpr uint32_t kTmC = 0, kTmA = 256;

  const bool a_by_tma = (mode == 0 || mode == 1 || mode == 3);
  if (tid == 0) {
    uint32_t bytes = 32768u + (a_by_tma ? 32768u : 0u);
    mbar_expect_tx(&bar_load, bytes);
    if (a_by_tma) {
      tma_load_4d(s_a, &tm_a, &bar_load, 0, 0, 0, 0);
      tma_load_4d(s_a + kPanel, &tm_a, &bar_load, 64, 0, 0, 0);
    }
    tma_load_4d(s_b, &tm_b, &bar_load, 0, 0, 0, 0);
    tma_load_4d(s_b + kPanel, &tm_b, &bar_load, 64, 0, 0, 0);
  }
  if (mode == 2) {
    // stage A in tensor memory: row = lane, 128 16-bit values packed two per column (64 columns)
    const uint4* arow = reinterpret_cast<const uint4*>(a_gmem + row * 128);
#pragma unroll 1
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint4 v = arow[c * 8 + k];
        r[4 * k + 0] = v.x; r[4 * k + 1] = v.y; r[4 * k + 2] = v.z; r[4 * k + 3] = v.w;
      }
      tmem_st32(tmem_base + lane_addr + kTmA + c * 32, r);
    }
    tmem_st_wait();
    tc_fence_before_sync();
  }
  if (mode == 4) {
    // write A into the swizzled K-major layout by hand: 16 chunks of 16 bytes per row
    const uint4* arow = reinterpret_cast<const uint4*>(a_gmem + row * 128);
#pragma unroll
    for (int ch = 0; ch < 16; ++ch) {
      const uint4 v = arow[ch];
      *reinterpret_cast<uint4*>(base_ptr + (ch >> 3) * kPanel + sw128_offset(row, ch & 7)) = v;
    }
    fence_proxy_async_smem();
  }
  __syncthreads();

  if (tid == 0) {
    bool ok = mbar_wait(&bar_load, 0, abort_p);
    if (ok) {
      tc_fence_after_sync();
      const uint32_t d = tmem_base + kTmC;
      if (mode == 0 || mode == 4) {
        const uint32_t idesc = make_idesc(128, 128, true, false, false);
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kPanel + (ks & 3) * 32;
          mma_ss(d, desc_kmajor(s_a + off), desc_kmajor(s_b + off), idesc, ks > 0);
        }
      } else if (mode == 1) {
        const uint32_t idesc = make_idesc(128, 128, true, false, true);
        for (int ks = 0; ks < 8; ++ks) {
          const uint32_t off = (ks >> 2) * kPanel + (ks & 3) * 32;
          mma_ss(d, desc_kmajor(s_a + off), desc_mnmajor(s_b + ks * 2048, kPanel), idesc, ks > 0);
        }
      } else if (mode == 2) {
        const uint32_t idesc = make_idesc(128, 128, true, false, true);
        for (int ks = 0; ks < 8; ++ks)
          mma_ts(d, tmem_base + kTmA + ks * 8, desc_mnmajor(s_b + ks * 2048, kPanel), idesc, ks > 0);
      } else {  // mode 3
        const uint32_t idesc = make_idesc(128, 128, true, true, true);
        for (int ks = 0; ks < 8; ++ks)
          mma_ss(d, desc_mnmajor(s_a + ks * 2048, kPanel), desc_mnmajor(s_b + ks * 2048, kPanel), idesc, ks > 0);
      }
      mma_commit(&bar_mma);
    }
  }
  __syncwarp();
  const bool done = mbar_wait_warp(&bar_mma, 0, abort_p);
  if (done) {
    tc_fence_after_sync();
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem_base + lane_addr + kTmC + c * 32, r);
      tmem_ld_wait32(r);
#pragma unroll
      for (int k = 0; k < 32; ++k) c_out[row * 128 + c * 32 + k] = __uint_as_float(r[k]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) atomicExch(status, kStatusWaitTimeout);
  }
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// A wait that nothing ever satisfies: one thread waits on an mbarrier with no arrival pending.  The bounded wait of
// tc05.cuh runs out (2 s), the CTA takes the same exit path as the hop kernels (abort flag, status word) and returns.
__global__ void __launch_bounds__(32, 1) wait_probe_kernel(int* status) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (*reinterpret_cast<volatile int*>(status) != 0) return;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(&bar, 0, &abort_flag);
  __syncthreads();
  if (abort_flag && threadIdx.x == 0) atomicExch(status, kStatusWaitTimeout);
}

}  // namespace rfa

extern "C" int rfa_debug_wait_timeout(int* status, void* stream) {
  if (!status) return RFA_ERR_INVALID_ARG;
  rfa::wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(status);
  return rfa::cuda_status(cudaGetLastError());
}

extern "C" int rfa_debug_mma_probe(int mode, const void* a, const void* b, float* c, int* status, void* stream) {
  using namespace rfa;
  if (!a || !b || !c || !status || mode < 0 || mode > 4) return RFA_ERR_INVALID_ARG;
  CUtensorMap ta, tb;
  int rc;
  if ((rc = make_tmap_bshd(&ta, a, RFA_DTYPE_BF16, 1, 128, 1, 128, 128)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tb, b, RFA_DTYPE_BF16, 1, 128, 1, 128, 128)) != RFA_OK) return rc;
  const int smem = 65536 + 1024 + 60 * 1024;  // above half an SM: one CTA per SM
  static bool attr_done[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return RFA_ERR_CUDA; }
  if (!attr_done[dev]) {
    if (cudaFuncSetAttribute(mma_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
      cudaGetLastError();
      return RFA_ERR_CUDA;
    }
    attr_done[dev] = true;
  }
  mma_probe_kernel<<<1, 128, smem, static_cast<cudaStream_t>(stream)>>>(ta, tb, static_cast<const __nv_bfloat16*>(a),
                                                                      c, mode, status);
  return cuda_status(cudaGetLastError());
}
