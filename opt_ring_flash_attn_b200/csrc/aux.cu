// Host utilities (tensor-map factory) and the small bandwidth-bound kernels of
// the path: backward preprocessing, fp32 -> 16-bit casts, K/V packing.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math.h>

#include <type_traits>

#include "common.h"

namespace rfa {

TraceCfg g_trace = {nullptr, 0, 0};

// cuTensorMapEncodeTiled is reached through the runtime's driver entry point
// lookup so that the library carries no link-time dependency on libcuda.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* ptr = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr) {
    cudaGetLastError();
    return nullptr;
  }
  fn = reinterpret_cast<EncodeTiledFn>(ptr);
  return fn;
}

int make_tmap_bshd(CUtensorMap* out, const void* base, int dtype, int B, int S, int H, int D, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RFA_ERR_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0) return RFA_ERR_INVALID_ARG;
  const CUtensorMapDataType dt = (dtype == RFA_DTYPE_BF16) ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  cuuint64_t gdim[4] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(H), static_cast<cuuint64_t>(S),
                        static_cast<cuuint64_t>(B)};
  cuuint64_t gstride[3] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(H) * D * 2,
                           static_cast<cuuint64_t>(S) * H * D * 2};
  cuuint32_t box[4] = {64u, 1u, static_cast<cuuint32_t>(box_rows), 1u};
  cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RFA_OK : RFA_ERR_DRIVER;
}

// ----------------------------------------------------------------------------
// Backward preprocessing: one warp per (b, s, h) row.
//   delta = sum_d out*dout ; lse2 = lse*log2(e).
// Streams out, dout once (2*B*S*Hq*D*2 bytes): HBM-bound.  (The dQ accumulator is cleared by a memset the launcher
// enqueues in front of the kernel: a fill runs at the full write rate, a strided clear inside this kernel did not.)
// ----------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float dot8(const uint4& a, const uint4& b);
template <>
__device__ __forceinline__ float dot8<__nv_bfloat16>(const uint4& a, const uint4& b) {
  const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
  const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(pa[i]);
    const float2 y = __bfloat1622float2(pb[i]);
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
  return s;
}
template <>
__device__ __forceinline__ float dot8<__half>(const uint4& a, const uint4& b) {
  const __half2* pa = reinterpret_cast<const __half2*>(&a);
  const __half2* pb = reinterpret_cast<const __half2*>(&b);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __half22float2(pa[i]);
    const float2 y = __half22float2(pb[i]);
    s = fmaf(x.x, y.x, s);
    s = fmaf(x.y, y.y, s);
  }
  return s;
}

template <typename T>
__global__ void __launch_bounds__(256) bwd_prepare_kernel(const T* __restrict__ out, const T* __restrict__ dout,
                                                         const float* __restrict__ lse, float* __restrict__ delta,
                                                         float* __restrict__ lse2, int B, int Sq, int Spad, int Hq,
                                                         int D) {
  // A row of D 16-bit values is D/8 16-byte vectors; a group of gsz lanes (gsz = 4, 8, 16 or 32, the
  // power of two >= D/8) owns one row, so a warp streams 32/gsz rows at a time with every lane loading.
  const int vec_per_row = D / 8;
  int gsz = 4;
  while (gsz < vec_per_row) gsz <<= 1;
  const int lane = threadIdx.x & 31;
  const int sub = lane / gsz;            // row slot inside the warp
  const int gl = lane % gsz;             // lane inside the group
  const int rows_per_warp = 32 / gsz;
  const long long warp_global = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = (static_cast<long long>(gridDim.x) * blockDim.x) >> 5;
  const long long rows = static_cast<long long>(B) * Spad * Hq;
  for (long long r0 = warp_global * rows_per_warp; r0 < rows; r0 += nwarps * rows_per_warp) {
    // rows are enumerated (b, s, h) with h fastest so that consecutive groups stream consecutive memory
    const long long r = r0 + sub;
    const bool in_range = r < rows;
    const int h = in_range ? static_cast<int>(r % Hq) : 0;
    const long long bs = in_range ? r / Hq : 0;
    const int s = static_cast<int>(bs % Spad);
    const int b = static_cast<int>(bs / Spad);
    const size_t stat = (static_cast<size_t>(b) * Hq + h) * Spad + s;
    const bool real = in_range && s < Sq;
    float acc = 0.f;
    if (real && gl < vec_per_row) {
      const size_t row_off = ((static_cast<size_t>(b) * Sq + s) * Hq + h) * D;
      const uint4 a = *reinterpret_cast<const uint4*>(out + row_off + gl * 8);
      const uint4 g = *reinterpret_cast<const uint4*>(dout + row_off + gl * 8);
      acc = dot8<T>(a, g);
    }
    for (int o = gsz >> 1; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (in_range && gl == 0) {
      delta[stat] = real ? acc : 0.f;
      lse2[stat] = real ? lse[stat] * 1.4426950408889634f : INFINITY;
    }
  }
}

// dQ accumulator (fp32, tiled [b][h][tile of 128 rows][32 row groups][DP][4]) -> dq [B, Sq, Hq, D] in T.
// One block per (b, h, tile, 64-wide slice of the head dim); transposed through shared memory so that
// both the reads (16 B per thread, consecutive) and the writes (16 B per thread, row-contiguous) coalesce.
template <typename T>
__global__ void __launch_bounds__(256) dq_finalize_kernel(const float* __restrict__ acc, T* __restrict__ dq, int B,
                                                         int Sq, int Hq, int D, int DP, int nQt) {
  __shared__ __align__(16) T tile[128][64 + 8];
  const int nslice = DP / 64;
  int idx = blockIdx.x;
  const int slice = idx % nslice; idx /= nslice;
  const int qt = idx % nQt; idx /= nQt;
  const int h = idx % Hq;
  const int b = idx / Hq;
  const float* src = acc + ((static_cast<size_t>(b) * Hq + h) * nQt + qt) * (static_cast<size_t>(128) * DP);
  const int dl = threadIdx.x & 63;
  const int qsub = threadIdx.x >> 6;
#pragma unroll 2
  for (int qg = qsub; qg < 32; qg += 4) {
    const float4 v = *reinterpret_cast<const float4*>(src + (static_cast<size_t>(qg) * DP + slice * 64 + dl) * 4);
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      tile[4 * qg + 0][dl] = __float2bfloat16_rn(v.x); tile[4 * qg + 1][dl] = __float2bfloat16_rn(v.y);
      tile[4 * qg + 2][dl] = __float2bfloat16_rn(v.z); tile[4 * qg + 3][dl] = __float2bfloat16_rn(v.w);
    } else {
      tile[4 * qg + 0][dl] = __float2half_rn(v.x); tile[4 * qg + 1][dl] = __float2half_rn(v.y);
      tile[4 * qg + 2][dl] = __float2half_rn(v.z); tile[4 * qg + 3][dl] = __float2half_rn(v.w);
    }
  }
  __syncthreads();
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int id = it * 256 + threadIdx.x;
    const int q = id >> 3;
    const int part = id & 7;
    const int qg_ = qt * 128 + q;
    const int d = slice * 64 + part * 8;
    if (qg_ < Sq && d < D) {
      const uint4 w = *reinterpret_cast<const uint4*>(&tile[q][part * 8]);
      *reinterpret_cast<uint4*>(dq + ((static_cast<size_t>(b) * Sq + qg_) * Hq + h) * D + d) = w;
    }
  }
}

// out = a + b over n4 float4 elements (out may alias a or b): the ring accumulate of the partial dK/dV.
// Streams 3 * 16 bytes per element: HBM-bound.
__global__ void __launch_bounds__(256) add_f32_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                                     float4* out, size_t n4) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += stride) {
    const float4 x = a[i];
    const float4 y = b[i];
    out[i] = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
  }
}

// Two 16-bit values <-> two floats (round to nearest even on the way down).
template <typename T>
struct Cvt16;
template <>
struct Cvt16<__nv_bfloat16> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u));
  }
};
template <>
struct Cvt16<__half> {
  static __device__ __forceinline__ uint32_t pack(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  static __device__ __forceinline__ float2 unpack(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
  }
};

// out16 = round(float(prev16) + block32) over groups of 8 elements (prev may be null: out16 = round(block32)).
// Streams 32 + 16 + 16 bytes per group: HBM-bound.
template <typename T, bool kHasPrev>
__global__ void __launch_bounds__(256) accum_to16_kernel(const uint4* __restrict__ prev, const float4* __restrict__ block,
                                                        uint4* out, size_t n8) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = block[2 * i];
    const float4 b = block[2 * i + 1];
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    if (kHasPrev) {
      const uint4 pw = prev[i];
      const uint32_t w[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = Cvt16<T>::unpack(w[k]);
        v[2 * k] += f.x;
        v[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = Cvt16<T>::pack(v[0], v[1]);
    o.y = Cvt16<T>::pack(v[2], v[3]);
    o.z = Cvt16<T>::pack(v[4], v[5]);
    o.w = Cvt16<T>::pack(v[6], v[7]);
    out[i] = o;
  }
}

template <typename T>
__global__ void __launch_bounds__(256) cast_from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst,
                                                           size_t n8, size_t n) {
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += stride) {
    const float4 a = *reinterpret_cast<const float4*>(src + i * 8);
    const float4 b = *reinterpret_cast<const float4*>(src + i * 8 + 4);
    T tmp[8];
    if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
      tmp[0] = __float2bfloat16_rn(a.x); tmp[1] = __float2bfloat16_rn(a.y);
      tmp[2] = __float2bfloat16_rn(a.z); tmp[3] = __float2bfloat16_rn(a.w);
      tmp[4] = __float2bfloat16_rn(b.x); tmp[5] = __float2bfloat16_rn(b.y);
      tmp[6] = __float2bfloat16_rn(b.z); tmp[7] = __float2bfloat16_rn(b.w);
    } else {
      tmp[0] = __float2half_rn(a.x); tmp[1] = __float2half_rn(a.y);
      tmp[2] = __float2half_rn(a.z); tmp[3] = __float2half_rn(a.w);
      tmp[4] = __float2half_rn(b.x); tmp[5] = __float2half_rn(b.y);
      tmp[6] = __float2half_rn(b.z); tmp[7] = __float2half_rn(b.w);
    }
    *reinterpret_cast<uint4*>(dst + i * 8) = *reinterpret_cast<const uint4*>(tmp);
  }
  // tail (n not a multiple of 8)
  if (blockIdx.x == 0) {
    for (size_t i = n8 * 8 + threadIdx.x; i < n; i += blockDim.x) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) dst[i] = __float2bfloat16_rn(src[i]);
      else dst[i] = __float2half_rn(src[i]);
    }
  }
}

}  // namespace rfa

extern "C" int rfa_version(void) { return 100; }

extern "C" int rfa_debug_set_trace(unsigned long long* buf, int n_ctas, int cap) {
  if (buf != nullptr && (n_ctas <= 0 || cap <= 0)) return RFA_ERR_INVALID_ARG;
  rfa::g_trace.buf = buf;
  rfa::g_trace.ctas = buf ? n_ctas : 0;
  rfa::g_trace.cap = buf ? cap : 0;
  return RFA_OK;
}
extern "C" int rfa_seq_tile(void) { return 128; }

extern "C" int rfa_status_publish(const int* status, int* host_copy, void* stream) {
  if (!status || !host_copy) return RFA_ERR_INVALID_ARG;
  *host_copy = -1;  // "not landed yet"; the copy below overwrites it with the status word in stream order
  if (cudaMemcpyAsync(host_copy, status, sizeof(int), cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)) !=
      cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  return RFA_OK;
}

extern "C" int rfa_bwd_prepare(const void* out, const void* dout, const float* lse, float* delta, float* lse2,
                               float* dq_acc, int B, int Sq, int Hq, int D, int dtype, int* status, void* stream) {
  using namespace rfa;
  (void)status;
  if (!out || !dout || !lse || !delta || !lse2) return RFA_ERR_INVALID_ARG;
  if (B <= 0 || Sq <= 0 || Hq <= 0) return RFA_ERR_INVALID_ARG;
  if (padded_head_dim(D) == 0) return RFA_ERR_UNSUPPORTED;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  const int Spad = round_up(Sq, 128);
  const long long rows = static_cast<long long>(B) * Spad * Hq;
  const size_t dq_vec4 = static_cast<size_t>(B) * Hq * Spad * padded_head_dim(D) / 4;
  if (dq_acc && (reinterpret_cast<uintptr_t>(dq_acc) & 15u)) return RFA_ERR_INVALID_ARG;
  const int threads = 256;
  long long blocks = (rows + 15) / 16;  // 8 warps per block, at least two rows per warp pass
  if (blocks > 148ll * 16) blocks = 148ll * 16;
  if (blocks < 1) blocks = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dq_acc && cudaMemsetAsync(dq_acc, 0, dq_vec4 * sizeof(float4), s) != cudaSuccess) {
    cudaGetLastError();
    return RFA_ERR_CUDA;
  }
  if (dtype == RFA_DTYPE_BF16)
    bwd_prepare_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        static_cast<const __nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(dout), lse, delta, lse2, B, Sq, Spad,
        Hq, D);
  else
    bwd_prepare_kernel<__half><<<static_cast<unsigned>(blocks), threads, 0, s>>>(
        static_cast<const __half*>(out), static_cast<const __half*>(dout), lse, delta, lse2, B, Sq, Spad, Hq, D);
  return cuda_status(cudaGetLastError());
}

extern "C" size_t rfa_dq_acc_elems(int B, int Sq, int Hq, int D) {
  const int dp = rfa::padded_head_dim(D);
  if (dp == 0 || B <= 0 || Sq <= 0 || Hq <= 0) return 0;
  return static_cast<size_t>(B) * Hq * rfa::round_up(Sq, 128) * dp;
}

extern "C" int rfa_bwd_dq_finalize(const float* dq_acc, void* dq, int B, int Sq, int Hq, int D, int dtype,
                                   void* stream) {
  using namespace rfa;
  if (!dq_acc || !dq || B <= 0 || Sq <= 0 || Hq <= 0) return RFA_ERR_INVALID_ARG;
  const int dp = padded_head_dim(D);
  if (dp == 0) return RFA_ERR_UNSUPPORTED;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(dq_acc) & 15u) || (reinterpret_cast<uintptr_t>(dq) & 15u)) return RFA_ERR_INVALID_ARG;
  const int nQt = round_up(Sq, 128) / 128;
  const unsigned grid = static_cast<unsigned>(B) * Hq * nQt * (dp / 64);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == RFA_DTYPE_BF16)
    dq_finalize_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(dq_acc, static_cast<__nv_bfloat16*>(dq), B, Sq, Hq, D, dp, nQt);
  else
    dq_finalize_kernel<__half><<<grid, 256, 0, s>>>(dq_acc, static_cast<__half*>(dq), B, Sq, Hq, D, dp, nQt);
  return cuda_status(cudaGetLastError());
}

extern "C" int rfa_dkdv_accumulate(const float* prev, const float* block, float* out, size_t n, void* stream) {
  using namespace rfa;
  if (!prev || !block || !out) return RFA_ERR_INVALID_ARG;
  if ((n & 3u) != 0) return RFA_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(prev) & 15u) || (reinterpret_cast<uintptr_t>(block) & 15u) ||
      (reinterpret_cast<uintptr_t>(out) & 15u))
    return RFA_ERR_INVALID_ARG;
  if (n == 0) return RFA_OK;
  const size_t n4 = n / 4;
  size_t blocks = (n4 + 255) / 256;
  if (blocks > 148u * 16) blocks = 148u * 16;
  add_f32_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const float4*>(prev), reinterpret_cast<const float4*>(block), reinterpret_cast<float4*>(out), n4);
  return cuda_status(cudaGetLastError());
}

extern "C" int rfa_dkdv_accumulate_to16(const void* prev, const float* block, void* out, size_t n, int dtype,
                                        void* stream) {
  using namespace rfa;
  if (!block || !out) return RFA_ERR_INVALID_ARG;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  if (n == 0) return RFA_OK;
  if (n % 8) return RFA_ERR_INVALID_ARG;
  if ((reinterpret_cast<uintptr_t>(block) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u) ||
      (reinterpret_cast<uintptr_t>(prev) & 15u))
    return RFA_ERR_INVALID_ARG;
  const size_t n8 = n / 8;
  size_t blocks = (n8 + 255) / 256;
  if (blocks > 148u * 16) blocks = 148u * 16;
  const unsigned g = static_cast<unsigned>(blocks);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const uint4* p4 = static_cast<const uint4*>(prev);
  const float4* b4 = reinterpret_cast<const float4*>(block);
  uint4* o4 = static_cast<uint4*>(out);
  if (dtype == RFA_DTYPE_BF16) {
    if (prev) accum_to16_kernel<__nv_bfloat16, true><<<g, 256, 0, s>>>(p4, b4, o4, n8);
    else accum_to16_kernel<__nv_bfloat16, false><<<g, 256, 0, s>>>(p4, b4, o4, n8);
  } else {
    if (prev) accum_to16_kernel<__half, true><<<g, 256, 0, s>>>(p4, b4, o4, n8);
    else accum_to16_kernel<__half, false><<<g, 256, 0, s>>>(p4, b4, o4, n8);
  }
  return cuda_status(cudaGetLastError());
}

extern "C" int rfa_cast_from_f32(const float* src, void* dst, size_t n, int dtype, void* stream) {
  using namespace rfa;
  if (!src || !dst) return RFA_ERR_INVALID_ARG;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  if (n == 0) return RFA_OK;
  if ((reinterpret_cast<uintptr_t>(src) & 15u) || (reinterpret_cast<uintptr_t>(dst) & 15u)) return RFA_ERR_INVALID_ARG;
  const size_t n8 = n / 8;
  size_t blocks = (n8 + 255) / 256;
  if (blocks > 148u * 16) blocks = 148u * 16;
  if (blocks == 0) blocks = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == RFA_DTYPE_BF16)
    cast_from_f32_kernel<__nv_bfloat16><<<static_cast<unsigned>(blocks), 256, 0, s>>>(
        src, static_cast<__nv_bfloat16*>(dst), n8, n);
  else
    cast_from_f32_kernel<__half><<<static_cast<unsigned>(blocks), 256, 0, s>>>(src, static_cast<__half*>(dst), n8, n);
  return cuda_status(cudaGetLastError());
}

extern "C" int rfa_pack_kv(const void* k, const void* v, void* dst, size_t bytes_each, void* stream) {
  if (!k || !v || !dst) return RFA_ERR_INVALID_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(dst, k, bytes_each, cudaMemcpyDeviceToDevice, s);
  if (e == cudaSuccess)
    e = cudaMemcpyAsync(static_cast<char*>(dst) + bytes_each, v, bytes_each, cudaMemcpyDeviceToDevice, s);
  if (e != cudaSuccess) cudaGetLastError();
  return rfa::cuda_status(e);
}
