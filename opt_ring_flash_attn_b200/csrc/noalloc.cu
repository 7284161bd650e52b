// Backward hop for callers that cannot allocate device memory.
//
// rfa_bwd_hop needs a fp32 dQ accumulator next to its inputs and outputs, and its regular callers
// get that from their allocator (a torch tensor cached per shape).  Some callers have no allocator to
// ask: code that runs where cudaMalloc is forbidden or unavailable -- inside a region that must not
// synchronise the device or touch the driver's memory manager, in a process whose memory pool was
// handed out completely at start-up, or behind a plugin interface that only ever passes tensors in
// and out.  For them the accumulator lives in a fixed array inside this library.
//
// The array is a file-scope __device__ object: every GPU that loads the library carries
// RFA_NOALLOC_SCRATCH_BYTES of it until the process exits, which is why the limit is modest.
// In host code the array's name is only a handle; the device address is looked up once per device
// with cudaGetSymbolAddress (with that device current) and passed to the kernels as a pointer.
#include "bwd_common.cuh"
#include "common.h"

namespace {

constexpr size_t kScratchBytes = RFA_NOALLOC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

float* g_scratch_ptr[rfa::kMaxDevices] = {nullptr};

// Device address of the scratch array on the current device (looked up on first use).
int scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= rfa::kMaxDevices) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_scratch) != cudaSuccess || p == nullptr) {
      cudaGetLastError();
      return RFA_ERR_CUDA;
    }
    g_scratch_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_scratch_ptr[dev];
  return RFA_OK;
}

}  // namespace

extern "C" size_t rfa_noalloc_scratch_bytes(void) { return kScratchBytes; }

extern "C" int rfa_bwd_hop_noalloc(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                                   const float* delta, void* dq, const float* dkdv_prev, float* dkdv_out, int B,
                                   int Sq, int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale,
                                   int accumulate_prev, int causal_diag, int* status, void* stream) {
  if (!dq || (reinterpret_cast<uintptr_t>(dq) & 15u)) return RFA_ERR_INVALID_ARG;
  // every argument is checked before anything is enqueued on the stream
  {
    const int rc0 = rfa::bwd_check_args(q, k, v, dout, lse2, delta, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                                        softmax_scale, accumulate_prev, causal_diag, /*q_begin=*/0, /*kv_len=*/Skv,
                                        status);
    if (rc0 != RFA_OK) return rc0;
  }
  const size_t elems = rfa_dq_acc_elems(B, Sq, Hq, D);
  if (elems == 0) return RFA_ERR_UNSUPPORTED;
  if (elems * sizeof(float) > kScratchBytes) return RFA_ERR_TOO_LARGE;  // shape needs more than the fixed array
  float* acc = nullptr;
  int rc = scratch_for_current_device(&acc);
  if (rc != RFA_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // The array keeps whatever the previous call left in it; the accumulator must start at zero.
  if (cudaMemsetAsync(acc, 0, elems * sizeof(float), s) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  rc = rfa_bwd_hop(q, k, v, dout, lse2, delta, acc, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                   softmax_scale, accumulate_prev, causal_diag, status, stream);
  if (rc != RFA_OK) return rc;
  return rfa_bwd_dq_finalize(acc, dq, B, Sq, Hq, D, dtype, stream);
}
