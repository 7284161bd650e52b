// Host-side helpers shared by the launchers: error codes of the C ABI, the
// tensor-map factory for [B, S, H, D] operands, and small shape utilities.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rfa_b200.h"
#include "../../include/rfa_b200_debug.h"

namespace rfa {

// Per-device launcher state (function attributes, scratch addresses) is kept in arrays of this size.
constexpr int kMaxDevices = 64;

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
inline int ceil_div(int x, int m) { return (x + m - 1) / m; }

// Padded head dimension the kernels are instantiated for (64, 128 or 256), or 0.
inline int padded_head_dim(int d) {
  if (d <= 0 || d > 256 || (d % 8) != 0) return 0;
  if (d <= 64) return 64;
  if (d <= 128) return 128;
  return 256;
}

// Builds a 4-D tensor map over a contiguous [B, S, H, D] tensor of 16-bit
// elements.  The box is {64 elements of D, 1 head, box_rows rows of S, 1 batch}
// with the 128-byte swizzle; out-of-range elements read as zero, which is what
// pads ragged sequence tails and head dimensions below the padded size.
int make_tmap_bshd(CUtensorMap* out, const void* base, int dtype, int B, int S, int H, int D, int box_rows);

// Diagnostic event trace requested through rfa_debug_set_trace (null buffer = off).
struct TraceCfg {
  unsigned long long* buf;
  int ctas;
  int cap;
};
extern TraceCfg g_trace;
constexpr int kTraceRoles = 5;

// Translates a CUDA runtime error into an ABI error code (and clears it).
inline int cuda_status(cudaError_t e) { return e == cudaSuccess ? RFA_OK : RFA_ERR_CUDA; }

}  // namespace rfa
