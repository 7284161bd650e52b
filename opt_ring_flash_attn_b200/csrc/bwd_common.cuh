// Launch parameters of the backward hop kernel and the GQA-group split that fills the last wave of CTAs.
#pragma once

#include <cuda_runtime.h>

#include "common.h"

namespace rfa {

struct BwdParams {
  const float* lse2;
  const float* delta;
  float* dq_acc;
  const float* dkdv_prev;
  float* dkdv_out;
  int B, Sq, Skv, Hq, Hkv, D;
  int Spad;
  float scale, scale_log2;
  int accumulate_prev, causal;
  int q_begin;  // window (zigzag layout): only query rows >= q_begin contribute
  int kv_len;   // only keys < kv_len are processed; dK/dV rows beyond keep the previous partial sums (or zero)
  int gsplit;      // CTAs per (kv tile, kv head): each takes G / gsplit query heads of the group
  int reduce_out;  // 1: the epilogue adds into dkdv_out with vector reductions (gsplit > 1); 0: plain stores
  int* dq_order;   // ordered (bit-reproducible) dQ reductions: per-tile counters, cleared by the launcher; null = unordered
  int* status;
  unsigned long long* trace;
  int trace_ctas, trace_cap;
};

int bwd_check_args(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                   const float* delta, const float* dkdv_prev, const float* dkdv_out, int B, int Sq, int Skv, int Hq,
                   int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev, int causal_diag, int q_begin,
                   int kv_len, const int* status);

// Work units are CTAs, one per SM at a time.  A grid that is not close to a multiple of 148 wastes the last
// wave, so a GQA group may be split over several CTAs whose partial dK/dV are added with vector reductions.
// Picks the smallest split that fills the waves to >= 90 % and prepares dkdv_out for the reducing epilogue (copy of
// the previous partial sums, or zeros).  Ordered mode never splits: three or more partial sums added by reductions
// would arrive in a varying order.
inline int choose_group_split(BwdParams& pr, long long base_units, cudaStream_t stream) {
  const int G = pr.Hq / pr.Hkv;
  int best = 1;
  double best_eff = 0.0;
  // Diagonal (causal) blocks: CTAs carry unequal work and are launched heaviest first, so the tail evens out by itself
  // once there are a few CTAs per SM; splitting only adds reductions and K/V reloads (measured 2 % slower at config 3).
  const bool balanced_by_order = pr.causal && base_units >= 2 * 148;
  for (int gsplit = 1; gsplit <= G && !balanced_by_order && pr.dq_order == nullptr; ++gsplit) {
    if (G % gsplit) continue;
    const long long units = base_units * gsplit;
    const double eff = static_cast<double>(units) / static_cast<double>((units + 147) / 148 * 148);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = gsplit; }
    if (eff >= 0.9) { best = gsplit; break; }
  }
  pr.gsplit = best;
  pr.reduce_out = best > 1 ? 1 : 0;
  // Rows of dkdv_out that the kernel does not write (keys beyond kv_len) must still hold prev (or zero): prepare the
  // whole buffer in that case too.
  const bool partial_rows = pr.kv_len < pr.Skv;
  if (pr.reduce_out || (partial_rows && (!pr.accumulate_prev || pr.dkdv_prev != pr.dkdv_out))) {
    const size_t bytes = static_cast<size_t>(2) * pr.B * pr.Skv * pr.Hkv * pr.D * sizeof(float);
    cudaError_t e = cudaSuccess;
    if (pr.accumulate_prev) {
      if (pr.dkdv_prev != pr.dkdv_out) e = cudaMemcpyAsync(pr.dkdv_out, pr.dkdv_prev, bytes, cudaMemcpyDeviceToDevice, stream);
    } else {
      e = cudaMemsetAsync(pr.dkdv_out, 0, bytes, stream);
    }
    if (e != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
  }
  return RFA_OK;
}

}  // namespace rfa
