// Forward ring hop: attention of the local query shard against one K/V block,
// folded into the running fp32 (m, l, acc) state that lives in device memory
// between hops.  Functionally this is one launch of the reference's
// `_native_fwd_step_kernel` (optimized_ring_flash_attn.py:519-615); the final
// hop also produces `out` and the log-sum-exp, so no separate merge pass
// (optimized_ring_flash_attn.py:328-417) exists.
//
// Structure of one CTA (sm_100a):
//   warp 0      TMA producer: Q tile(s) once, then K_j / V_j tiles through a ring
//               of shared-memory slots guarded by full/empty mbarriers.
//   warp 1      MMA issuer (loop run by the whole warp, one elected lane issues): S = Q K_j^T
//               (tcgen05.mma, operands in shared memory) and O += P_j V_j (P read from tensor memory).
//   warps 4..   one softmax warpgroup per Q tile: thread = query row = TMEM lane;
//               reads S from tensor memory, exp2-domain online softmax with lazy
//               rescaling of O, writes P (16-bit) back over S.
// Tensor memory: [0, NQ*DP) O accumulators, then NQ*NS score buffers of BN columns.
// Two variants: NQ=2 Q tiles with one score buffer each (D <= 128), and NQ=1 with
// two alternating score buffers and BN=64 (D = 256).
#include "common.h"
#include "tc05.cuh"

namespace rfa {

// Every n-th pair of exponentials of the softmax on the FMA pipe (a cubic) instead of the special-function unit,
// which needs as many cycles per K/V tile as the tensor pipe does; 0 = none.  Diagonal / full block at S = 8192,
// 32/8 heads, D = 128: every 2nd 0.486 / 0.905 ms, 3rd 0.467 / 0.867, 4th 0.465 / 0.862, 6th 0.469 / 0.866.
constexpr int kFwdPolyEvery = 4;

struct FwdParams {
  float* acc;
  float* m;
  float* l;
  void* out;
  float* lse;
  int B, Sq, Skv, Hq, Hkv, D;
  int Spad;  // Sq rounded up to 128
  int nQt;   // Spad / 128
  float scale_log2;
  int first, last, causal;
  // Window (zigzag layout): only query rows >= q_begin are processed, only keys < kv_len are visible, and
  // query rows < q_split take `last_lo` instead of `last` (their final hop can come earlier).
  int q_begin, kv_len, q_split, last_lo;
  int* status;
  unsigned long long* trace;
  int trace_ctas, trace_cap;
};

template <int DP, int BN, int NQ, int NS>
struct FwdCfg {
  static constexpr int kBM = 128;
  static constexpr int kPanels = DP / 64;
  static constexpr int kQBytes = kBM * DP * 2;
  static constexpr int kKVBytes = BN * DP * 2;
  static constexpr int kSlots = (DP == 64) ? 8 : 4;
  static constexpr int kSmemTiles = NQ * kQBytes + kSlots * kKVBytes;
  static constexpr int kSmemBytes = kSmemTiles + 1024;  // slack for 1024-byte alignment
  static constexpr int kThreads = 128 + NQ * 128;
  static constexpr int kTmO = 0;
  static constexpr int kTmS = NQ * DP;
  static_assert(kTmS + NQ * NS * BN <= 512, "tensor memory over budget");
  static_assert(kSmemBytes >= 120 * 1024, "one CTA per SM is assumed (whole TMEM is allocated)");
};

// S[128 x BN] = Q[128 x DP] * K[BN x DP]^T, both operands K-major.
template <int DP, int BN>
__device__ __forceinline__ void issue_qk(uint32_t s_tmem, uint32_t q_smem, uint32_t k_smem, uint32_t idesc,
                                         uint32_t el) {
  // q_smem / k_smem are descriptor low words of the tile bases; offsets are in 16-byte units
  static_for<0, DP / 16>([&](auto ks_) {
    constexpr int ks = decltype(ks_)::value;
    mma_ss_off_e<(((ks / 4) * (128 * 128) + (ks % 4) * 32) / 16), (((ks / 4) * (BN * 128) + (ks % 4) * 32) / 16)>(
        s_tmem, q_smem, k_smem, idesc, ks > 0 ? 1u : 0u, el);
  });
}

// O[128 x DP] (+)= P[128 x BN] * V[BN x DP] over the K-steps [KS0, KS1) of 16 keys each; P in tensor memory,
// V MN-major.  The product of one K/V tile is issued in kPvParts pieces so that the first keys of P are consumed
// while the softmax warps still exponentiate the rest of the row.
template <int DP, int BN, int KS0, int KS1>
__device__ __forceinline__ void issue_pv(uint32_t o_tmem, uint32_t p_tmem, uint32_t v_smem, uint32_t idesc,
                                         bool accumulate, uint32_t el) {
  static_for<KS0, KS1>([&](auto ks_) {
    constexpr int ks = decltype(ks_)::value;
    mma_ts_off_e<(ks * 8), (ks * 128)>(o_tmem, p_tmem, v_smem, idesc, (accumulate || ks > KS0) ? 1u : 0u, el);
  });
}

template <int DP, int BN, int NQ, int NS, typename T>
__global__ void __launch_bounds__(128 + NQ * 128, 1)
    fwd_hop_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using Cfg = FwdCfg<DP, BN, NQ, NS>;
  constexpr int kSlots = Cfg::kSlots;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;

  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full;
  __shared__ uint64_t bar_kv_full[kSlots];
  __shared__ uint64_t bar_kv_empty[kSlots];
  __shared__ uint64_t bar_s_full[NQ * NS];
  constexpr int kPvParts = BN / 32;  // one hand-off per 32 keys
  constexpr int kPolyEvery = kFwdPolyEvery;  // every n-th pair of exponentials on the FMA pipe (0 = none)
  __shared__ uint64_t bar_p_ready[NQ * NS * kPvParts];  // [score buffer][part of the keys]
  __shared__ uint64_t bar_pv_done[NQ];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;  // an earlier kernel gave up

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t s_q = smem_base;
  const uint32_t s_kv = smem_base + NQ * Cfg::kQBytes;

  // ---- tile coordinates: heaviest (latest rows) first, heads fastest ----
  const int tq0 = p.q_begin / 128;
  const int nQs = (p.nQt - tq0 + NQ - 1) / NQ;
  const int per_qs = p.Hq * p.B;
  const int qs = nQs - 1 - static_cast<int>(blockIdx.x) / per_qs;
  const int rem = static_cast<int>(blockIdx.x) % per_qs;
  const int b = rem / p.Hq;
  const int h = rem % p.Hq;
  const int hkv = h / (p.Hq / p.Hkv);

  const int nkv_total = (p.kv_len + BN - 1) / BN;
  int m0[NQ], ntile[NQ];
  int nmax = 0;
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    m0[q] = (tq0 + qs * NQ + q) * 128;
    int n = 0;
    if (m0[q] < p.Sq) {
      n = nkv_total;
      if (p.causal) n = min(n, (m0[q] + 127) / BN + 1);
    }
    ntile[q] = n;
    nmax = max(nmax, n);
  }

  // ---- setup ----
  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_q_full, 1);
    for (int i = 0; i < kSlots; ++i) {
      mbar_init(&bar_kv_full[i], 1);
      mbar_init(&bar_kv_empty[i], 1);
    }
    for (int i = 0; i < NQ * NS; ++i) {
      mbar_init(&bar_s_full[i], 1);
      for (int h = 0; h < kPvParts; ++h) mbar_init(&bar_p_ready[i * kPvParts + h], 128);
    }
    for (int i = 0; i < NQ; ++i) mbar_init(&bar_pv_done[i], 1);
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
  Tracer tr;
  {
    int role = -1;
    if (lane == 0) role = (warp == 0) ? 0 : (warp == 1) ? 1 : (warp == 4) ? 2 : (warp == 8) ? 3 : -1;
    if (role >= 0) tr.init(p.trace, p.trace_ctas, p.trace_cap, kTraceRoles, role);
  }

  if (warp == 0) {
    // =========================== TMA producer ===========================
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      int nvalid = 0;
#pragma unroll
      for (int q = 0; q < NQ; ++q) nvalid += (ntile[q] > 0) ? 1 : 0;
      mbar_expect_tx(&bar_q_full, static_cast<uint32_t>(nvalid) * Cfg::kQBytes);
#pragma unroll
      for (int q = 0; q < NQ; ++q) {
        if (ntile[q] > 0) {
#pragma unroll
          for (int pn = 0; pn < Cfg::kPanels; ++pn)
            tma_load_4d(s_q + q * Cfg::kQBytes + pn * (128 * 128), &tm_q, &bar_q_full, pn * 64, h, m0[q], b);
        }
      }
      bool ok = true;
      for (int j = 0; j < nmax && ok; ++j) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const int u = 2 * j + which;
          const int slot = u % kSlots;
          const int round = u / kSlots;
          if (!mbar_wait(&bar_kv_empty[slot], (round & 1) ^ 1, abort_p)) {
            ok = false;
            break;
          }
          tr.mark(40 + which);
          mbar_expect_tx(&bar_kv_full[slot], Cfg::kKVBytes);
#pragma unroll
          for (int pn = 0; pn < Cfg::kPanels; ++pn)
            tma_load_4d(s_kv + slot * Cfg::kKVBytes + pn * (BN * 128), which ? &tm_v : &tm_k, &bar_kv_full[slot],
                        pn * 64, hkv, j * BN, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // =========================== MMA issuer ===========================
    // The whole warp runs this loop converged; the elected lane issues.  A commit makes its mbarrier track every MMA
    // issued before it, so the arrival on bar_s_full for tile j+1 also tells the softmax warps that O += P_j V_j has
    // retired; bar_pv_done is only needed after the last tile.
    {
      const uint32_t el = elect_one();
      constexpr uint32_t idesc_qk = make_idesc(128, BN, kBf16, false, false);
      constexpr uint32_t idesc_pv = make_idesc(128, DP, kBf16, false, true);
      auto slot_of = [&](int u) { return u % kSlots; };
      auto par_of = [&](int u) { return static_cast<uint32_t>((u / kSlots) & 1); };
      // descriptor low words of the operand tiles (K: K-major, V: MN-major, Q: K-major)
      auto k_lo = [&](int u) { return desc_lo_kmajor(s_kv + slot_of(u) * Cfg::kKVBytes); };
      auto v_lo = [&](int u) { return desc_lo_mnmajor(s_kv + slot_of(u) * Cfg::kKVBytes, BN * 128); };
      uint32_t q_lo[NQ];
#pragma unroll
      for (int q = 0; q < NQ; ++q) q_lo[q] = desc_lo_kmajor(s_q + q * Cfg::kQBytes);
      auto s_tm = [&](int q, int sb) { return tmem_base + Cfg::kTmS + (q * NS + sb) * BN; };
      auto o_tm = [&](int q) { return tmem_base + Cfg::kTmO + q * DP; };
      bool ok = nmax > 0;
      if (ok) ok = mbar_wait_warp(&bar_q_full, 0, abort_p);
      if (ok) ok = mbar_wait_warp(&bar_kv_full[slot_of(0)], par_of(0), abort_p);
      if (ok) {
        tc_fence_after_sync();
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          if (ntile[q] > 0) {
            issue_qk<DP, BN>(s_tm(q, 0), q_lo[q], k_lo(0), idesc_qk, el);
            mma_commit_e(&bar_s_full[q * NS + 0], el);
          }
        }
        mma_commit_e(&bar_kv_empty[slot_of(0)], el);
      }
      for (int j = 0; j < nmax && ok; ++j) {
        if (NS == 2) {
          // Score buffer (j+1)&1 is free: P_{j-1} was consumed by the PV issued last iteration.
          if (j + 1 < ntile[0]) {
            const int uk = 2 * (j + 1);
            if (!mbar_wait_warp(&bar_kv_full[slot_of(uk)], par_of(uk), abort_p)) { ok = false; break; }
            tc_fence_after_sync();
            issue_qk<DP, BN>(s_tm(0, (j + 1) & 1), q_lo[0], k_lo(uk), idesc_qk, el);
            mma_commit_e(&bar_s_full[(j + 1) & 1], el);
            mma_commit_e(&bar_kv_empty[slot_of(uk)], el);
          }
        }
        const int uv = 2 * j + 1;
        tr.mark(9);
        if (!mbar_wait_warp(&bar_kv_full[slot_of(uv)], par_of(uv), abort_p)) { ok = false; break; }
        tr.mark(10);
#pragma unroll
        for (int q = 0; q < NQ; ++q) {
          if (j < ntile[q]) {
            const int sb = (NS == 2) ? (j & 1) : 0;
            const uint32_t par = (NS == 2) ? ((j >> 1) & 1) : (j & 1);
            static_for<0, kPvParts>([&](auto h_) {
              constexpr int h = decltype(h_)::value;
              if (ok) {
                if (!mbar_wait_warp(&bar_p_ready[(q * NS + sb) * kPvParts + h], par, abort_p)) {
                  ok = false;
                } else {
                  if (h == 0) tr.mark(11 + 2 * q);
                  tc_fence_after_sync();
                  issue_pv<DP, BN, 2 * h, 2 * h + 2>(o_tm(q), s_tm(q, sb), v_lo(uv), idesc_pv,
                                                     (h > 0) || (j > 0) || (p.first == 0), el);
                }
              }
            });
            if (!ok) break;
            if (NS == 2 || j + 1 == ntile[q]) mma_commit_e(&bar_pv_done[q], el);
            if (NS == 1 && j + 1 < ntile[q]) {
              const int uk = 2 * (j + 1);
              if (!mbar_wait_warp(&bar_kv_full[slot_of(uk)], par_of(uk), abort_p)) { ok = false; break; }
              tc_fence_after_sync();
              issue_qk<DP, BN>(s_tm(q, 0), q_lo[q], k_lo(uk), idesc_qk, el);
              mma_commit_e(&bar_s_full[q * NS + 0], el);
            }
            tr.mark(12 + 2 * q);
          }
        }
        if (!ok) break;
        mma_commit_e(&bar_kv_empty[slot_of(uv)], el);
        if (NS == 1 && j + 1 < nmax) mma_commit_e(&bar_kv_empty[slot_of(2 * (j + 1))], el);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // =========================== softmax warpgroups ===========================
    const int q = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int n = ntile[q];
    const int row_g = m0[q] + row;  // local query position
    const uint32_t o_addr = tmem_base + lane_addr + Cfg::kTmO + q * DP;
    const int qt = tq0 + qs * NQ + q;
    const bool last_here = (m0[q] < p.q_split) ? (p.last_lo != 0) : (p.last != 0);
    const size_t bh = static_cast<size_t>(b) * p.Hq + h;
    float* acc_tile = p.acc + ((bh * p.nQt + qt) * (DP / 4)) * 512;  // [DP/4][128][4]
    const size_t ml_idx = bh * p.Spad + row_g;

    bool ok = true;
    if (n > 0) {
      float m_used = -INFINITY;
      float l_sum = 0.f;
      if (!p.first) {
        m_used = p.m[ml_idx];
        l_sum = p.l[ml_idx];
#pragma unroll 1
        for (int c = 0; c < DP / 32; ++c) {
          uint32_t r[32];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float4 v = *reinterpret_cast<const float4*>(acc_tile + ((c * 8 + k) * 128 + row) * 4);
            r[4 * k + 0] = __float_as_uint(v.x);
            r[4 * k + 1] = __float_as_uint(v.y);
            r[4 * k + 2] = __float_as_uint(v.z);
            r[4 * k + 3] = __float_as_uint(v.w);
          }
          tmem_st32(o_addr + c * 32, r);
        }
        tmem_st_wait();
      }
      const Exp2Poly exp2_poly;
      // Highest visible local key index for this row.
      const int col_lim = p.causal ? min(row_g, p.kv_len - 1) : (p.kv_len - 1);

#pragma unroll 1
      for (int j = 0; j < n; ++j) {
        const int sb = (NS == 2) ? (j & 1) : 0;
        const uint32_t par = (NS == 2) ? ((j >> 1) & 1) : (j & 1);
        tr.mark(19);
        if (!mbar_wait_warp(&bar_s_full[q * NS + sb], par, abort_p)) { ok = false; break; }
        tr.mark(20);
        tc_fence_after_sync();
        const uint32_t s_addr = tmem_base + lane_addr + Cfg::kTmS + (q * NS + sb) * BN;
        const int n0 = j * BN;
        const bool masked = (p.causal && (n0 + BN - 1 > m0[q])) || (n0 + BN > p.kv_len);

        // The whole score row (BN fp32 values) goes to registers in one batch of loads.
        constexpr int NCH = BN / 32;
        uint32_t r[NCH][32];
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld32(s_addr + c * 32, r[c]);
        tmem_ld_wait32(r[0]);
#pragma unroll
        for (int c = 1; c < NCH; ++c) reg_fence32(r[c]);
        if (masked) {
          // keys beyond the causal limit of this row / beyond the end of the block count as -inf
#pragma unroll
          for (int c = 0; c < NCH; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (n0 + c * 32 + i > col_lim) r[c][i] = __float_as_uint(-INFINITY);
        }
        // row maximum of the raw scores (independent partial maxima keep the dependency chains short)
        float mxp[NCH][2];
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          mxp[c][0] = __uint_as_float(r[c][0]);
          mxp[c][1] = __uint_as_float(r[c][1]);
#pragma unroll
          for (int i = 2; i < 32; i += 2) {
            mxp[c][0] = fmaxf(mxp[c][0], __uint_as_float(r[c][i]));
            mxp[c][1] = fmaxf(mxp[c][1], __uint_as_float(r[c][i + 1]));
          }
        }
        float mx = fmaxf(mxp[0][0], mxp[0][1]);
#pragma unroll
        for (int c = 1; c < NCH; ++c) mx = fmaxf(mx, fmaxf(mxp[c][0], mxp[c][1]));
        const float m_new = fmaxf(m_used, mx * p.scale_log2);
        tr.mark(21);

        // lazy rescale: only when the maximum grew by more than 2^8
        bool need;
        if (j == 0 && p.first) {
          m_used = m_new;
          need = false;
        } else {
          need = (m_new - m_used) > 8.0f;
        }
        if (__any_sync(0xffffffffu, need)) {
          const float alpha = need ? fast_exp2(m_used - m_new) : 1.0f;
          if (need) m_used = m_new;
          l_sum *= alpha;
          // With one score buffer the arrival on bar_s_full that let this iteration start was committed after
          // O += P_{j-1} V_{j-1} was issued, so that product has retired; with two buffers it has its own barrier.
          if (NS == 2 && j > 0) {
            if (!mbar_wait_warp(&bar_pv_done[q], (j - 1) & 1, abort_p)) { ok = false; break; }
            tc_fence_after_sync();
          }
#pragma unroll 1
          for (int c = 0; c < DP / 16; ++c) {
            uint32_t o16[16];
            tmem_ld16(o_addr + c * 16, o16);
            tmem_ld_wait16(o16);
#pragma unroll
            for (int i = 0; i < 16; ++i) o16[i] = __float_as_uint(__uint_as_float(o16[i]) * alpha);
            tmem_st16(o_addr + c * 16, o16);
          }
          tmem_st_wait();
          tr.mark(23);
        }

        // P = exp2(s * scale_log2 - m_used), packed to 16 bit over the start of S.  Arithmetic runs on packed pairs;
        // one pair in kPolyEvery takes the polynomial route so that the special-function unit (16 exp2 per clock per
        // SM, as many cycles per tile as the tensor pipe needs for the two products) is not the only exp2 engine.
        const uint64_t scale2 = pack_f2(p.scale_log2, p.scale_log2);
        const uint64_t negm2 = pack_f2(-m_used, -m_used);
        uint64_t lp2[2] = {0ull, 0ull};
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t u[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const uint64_t x2 = fma2(pack_u2(r[c][2 * i], r[c][2 * i + 1]), scale2, negm2);
            uint64_t p2;
            float p0, p1;
            if (kPolyEvery > 0 && (i % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1) {
              p2 = exp2_poly(x2);
              unpack_f2(p2, p0, p1);
            } else {
              float x0, x1;
              unpack_f2(x2, x0, x1);
              p0 = fast_exp2(x0);
              p1 = fast_exp2(x1);
              p2 = pack_f2(p0, p1);
            }
            lp2[i & 1] = add2(lp2[i & 1], p2);
            u[i] = Pack2<T>::pack(p0, p1);
          }
          if (c > 0) {
            // the previous 32 keys of P have landed: the issuer may start O += P V on them
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(&bar_p_ready[(q * NS + sb) * kPvParts + c - 1]);
          }
          tmem_st16(s_addr + c * 16, u);
          if (c == NCH - 2) tr.mark(24);
        }
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(&bar_p_ready[(q * NS + sb) * kPvParts + NCH - 1]);
        {
          float a0, a1, b0, b1;
          unpack_f2(lp2[0], a0, a1);
          unpack_f2(lp2[1], b0, b1);
          l_sum += (a0 + a1) + (b0 + b1);
        }
        tr.mark(25);
      }

      // ---- epilogue: wait for the last PV, then spill state or write the result ----
      if (ok) ok = mbar_wait_warp(&bar_pv_done[q], (NS == 2) ? ((n - 1) & 1) : 0, abort_p);
      if (ok) {
        tc_fence_after_sync();
        if (last_here) {
          const float inv = 1.0f / l_sum;
          const bool row_ok = row_g < p.Sq;
          T* orow = reinterpret_cast<T*>(p.out) + ((static_cast<size_t>(b) * p.Sq + row_g) * p.Hq + h) * p.D;
#pragma unroll 1
          for (int c = 0; c < DP / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(o_addr + c * 32, r);
            tmem_ld_wait32(r);
            if (row_ok) {
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                if (c * 32 + k * 8 < p.D) {
                  uint4 w;
                  w.x = Pack2<T>::pack(__uint_as_float(r[8 * k + 0]) * inv, __uint_as_float(r[8 * k + 1]) * inv);
                  w.y = Pack2<T>::pack(__uint_as_float(r[8 * k + 2]) * inv, __uint_as_float(r[8 * k + 3]) * inv);
                  w.z = Pack2<T>::pack(__uint_as_float(r[8 * k + 4]) * inv, __uint_as_float(r[8 * k + 5]) * inv);
                  w.w = Pack2<T>::pack(__uint_as_float(r[8 * k + 6]) * inv, __uint_as_float(r[8 * k + 7]) * inv);
                  *reinterpret_cast<uint4*>(orow + c * 32 + k * 8) = w;
                }
              }
            }
          }
          if (row_ok) p.lse[ml_idx] = (m_used + log2f(l_sum)) * 0.6931471805599453f;
        } else {
#pragma unroll 1
          for (int c = 0; c < DP / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(o_addr + c * 32, r);
            tmem_ld_wait32(r);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float4 v;
              v.x = __uint_as_float(r[4 * k + 0]);
              v.y = __uint_as_float(r[4 * k + 1]);
              v.z = __uint_as_float(r[4 * k + 2]);
              v.w = __uint_as_float(r[4 * k + 3]);
              *reinterpret_cast<float4*>(acc_tile + ((c * 8 + k) * 128 + row) * 4) = v;
            }
          }
          p.m[ml_idx] = m_used;
          p.l[ml_idx] = l_sum;
        }
      }
    }
    __syncwarp();
  }

  // ---- teardown: every role arrives here, also after an abort ----
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    // Give copies that are still in flight time to land before the CTA's shared memory is released.
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) atomicExch(p.status, kStatusWaitTimeout);
  }
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

// ----------------------------------------------------------------------------
// Launcher
// ----------------------------------------------------------------------------
template <int DP, int BN, int NQ, int NS, typename T>
static int launch_fwd(const void* q, const void* k, const void* v, const FwdParams& prm, int dtype,
                      cudaStream_t stream) {
  using Cfg = FwdCfg<DP, BN, NQ, NS>;
  CUtensorMap tq, tk, tv;
  int rc;
  if ((rc = make_tmap_bshd(&tq, q, dtype, prm.B, prm.Sq, prm.Hq, prm.D, 128)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tk, k, dtype, prm.B, prm.Skv, prm.Hkv, prm.D, BN)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tv, v, dtype, prm.B, prm.Skv, prm.Hkv, prm.D, BN)) != RFA_OK) return rc;
  auto kern = fwd_hop_kernel<DP, BN, NQ, NS, T>;
  // Function attributes belong to a device: one flag per instantiation and device.
  static bool attr_done[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return RFA_ERR_CUDA; }
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
    attr_done[dev] = true;
  }
  const int nQs = (prm.nQt - prm.q_begin / 128 + NQ - 1) / NQ;
  const unsigned grid = static_cast<unsigned>(nQs) * prm.Hq * prm.B;
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, prm);
  return cuda_status(cudaGetLastError());
}

template <typename T>
static int dispatch_fwd(int dp, const void* q, const void* k, const void* v, const FwdParams& prm, int dtype,
                        cudaStream_t stream) {
  switch (dp) {
    case 64: return launch_fwd<64, 128, 2, 1, T>(q, k, v, prm, dtype, stream);
    case 128: return launch_fwd<128, 128, 2, 1, T>(q, k, v, prm, dtype, stream);
    case 256: return launch_fwd<256, 64, 1, 2, T>(q, k, v, prm, dtype, stream);
    default: return RFA_ERR_UNSUPPORTED;
  }
}

}  // namespace rfa

extern "C" size_t rfa_fwd_acc_elems(int B, int Sq, int Hq, int D) {
  const int dp = rfa::padded_head_dim(D);
  if (dp == 0 || B <= 0 || Sq <= 0 || Hq <= 0) return 0;
  return static_cast<size_t>(B) * Hq * rfa::round_up(Sq, 128) * dp;
}

extern "C" int rfa_fwd_hop_window(const void* q, const void* k, const void* v, float* acc, float* m, float* l,
                                  void* out, float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, int dtype,
                                  float softmax_scale, int first, int last, int causal_diag, int q_begin, int kv_len,
                                  int q_split, int last_lo, int* status, void* stream) {
  using namespace rfa;
  if (!q || !k || !v || !status) return RFA_ERR_INVALID_ARG;
  if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return RFA_ERR_INVALID_ARG;
  if (!(softmax_scale > 0.f)) return RFA_ERR_INVALID_ARG;
  if (q_begin < 0 || q_begin >= Sq || (q_begin % 128) != 0 || kv_len <= 0 || kv_len > Skv) return RFA_ERR_INVALID_ARG;
  if (q_split < 0 || (q_split % 128) != 0) return RFA_ERR_INVALID_ARG;
  const bool lo_exists = q_begin < q_split;
  const bool hi_exists = q_split < Sq;
  const bool all_final = first && (!hi_exists || last) && (!lo_exists || last_lo);
  if (!all_final && (!acc || !m || !l)) return RFA_ERR_INVALID_ARG;
  if (((hi_exists && last) || (lo_exists && last_lo)) && (!out || !lse)) return RFA_ERR_INVALID_ARG;
  if (causal_diag && Sq != Skv) return RFA_ERR_INVALID_ARG;
  const int dp = padded_head_dim(D);
  if (dp == 0) return RFA_ERR_UNSUPPORTED;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  FwdParams prm;
  prm.acc = acc;
  prm.m = m;
  prm.l = l;
  prm.out = out;
  prm.lse = lse;
  prm.B = B;
  prm.Sq = Sq;
  prm.Skv = Skv;
  prm.Hq = Hq;
  prm.Hkv = Hkv;
  prm.D = D;
  prm.Spad = round_up(Sq, 128);
  prm.nQt = prm.Spad / 128;
  prm.scale_log2 = softmax_scale * 1.4426950408889634f;
  prm.first = first ? 1 : 0;
  prm.last = last ? 1 : 0;
  prm.causal = causal_diag ? 1 : 0;
  prm.q_begin = q_begin;
  prm.kv_len = kv_len;
  prm.q_split = q_split;
  prm.last_lo = last_lo ? 1 : 0;
  prm.status = status;
  prm.trace = g_trace.buf;
  prm.trace_ctas = g_trace.ctas;
  prm.trace_cap = g_trace.cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == RFA_DTYPE_BF16) return dispatch_fwd<__nv_bfloat16>(dp, q, k, v, prm, dtype, s);
  return dispatch_fwd<__half>(dp, q, k, v, prm, dtype, s);
}

extern "C" int rfa_fwd_hop(const void* q, const void* k, const void* v, float* acc, float* m, float* l, void* out,
                           float* lse, int B, int Sq, int Skv, int Hq, int Hkv, int D, int dtype,
                           float softmax_scale, int first, int last, int causal_diag, int* status, void* stream) {
  return rfa_fwd_hop_window(q, k, v, acc, m, l, out, lse, B, Sq, Skv, Hq, Hkv, D, dtype, softmax_scale, first, last,
                            causal_diag, /*q_begin=*/0, /*kv_len=*/Skv, /*q_split=*/0, /*last_lo=*/0, status, stream);
}
