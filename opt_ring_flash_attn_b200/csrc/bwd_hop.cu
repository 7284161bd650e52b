// Backward ring hop against one K/V block.  One CTA owns a 128-row K/V tile of
// one kv head and walks over every query head of its GQA group and every query
// tile that can see it.  Five tensor-core products per (kv tile, q tile) pair,
// all computed in the transposed orientation so that the kv row is the TMEM
// lane and the accumulators dK, dV stay resident in tensor memory:
//   S^T  = K Q^T                (smem x smem)      -> P^T = exp2(scale*S^T - lse2[q])
//   dP^T = V dO^T               (smem x smem)      -> dS^T = P^T o (dP^T - delta[q])
//   dV  += P^T dO               (P^T from tensor memory, dO MN-major)
//   dK  += dS^T Q               (dS^T from shared memory, Q MN-major)
//   dQ^T = K^T dS^T             (both MN-major), reduced into the fp32 dQ
//                                accumulator in global memory with red.add.f32
// The epilogue adds the partial dK/dV that arrived from the previous rank and
// writes the packed fp32 buffer that travels on.  This one kernel covers the
// reference's `_bwd_dq_kernel` (optimized_ring_flash_attn.py:672-735),
// `_bwd_dkdv_kernel` (optimized_ring_flash_attn.py:738-805) and the accumulate
// kernels (optimized_ring_flash_attn.py:441-503); S and dP are computed once
// instead of once per kernel.
//
// Roles: warp 0 TMA producer, warp 1 MMA issuer, warps 4-11 two elementwise
// warpgroups (each owns half of the query columns of every tile: P^T, dS^T, then
// the dV / dK epilogues), warps 12-19 two dQ reduction warpgroups (half of the
// query columns each).
// Tensor memory: [0,BQ) S^T / P^T, [BQ,2BQ) dP^T then dQ^T, then dV (DH) and dK (DH).
// Head dim 256 runs as two CTAs per tile, each owning 128 columns of dK, dV, dQ.
#include <type_traits>

#include "bwd_common.cuh"
#include "common.h"
#include "tc05.cuh"

namespace rfa {

// Pause (ns) a reduction warp takes after each vector reduction.  An SM can push 32 B per clock towards the L2, so
// the 64 KB of dQ^T of a tile need >= 2048 cycles whatever issues them; unpaced, the eight reduction warps keep the
// load/store queue full of reductions and every shared-memory or tensor-memory access of the elementwise warps
// waits behind them.  The optimum is sharp (diagonal / full block at S = 8192, 32/8 heads: 0 ns 1.57 / 2.99 ms, 50 ns
// 1.54 / 2.97, 100 ns 1.35 / 2.52, 200 ns 2.13 / 4.20).
constexpr unsigned kRedSleepNs = 100;
// Every n-th group of four exponentials of the P^T phase on the FMA pipe (0 = all on the special-function unit, which
// measured best here: the phase is bound by shared-memory and load/store traffic, not by exp2).
constexpr int kBwdPolyEvery = 0;

}  // namespace rfa

namespace rfa {


template <int DP, int DH, int BQ, int NST>
struct BwdCfg {
  static constexpr int kPanels = DP / 64;
  static constexpr int kHalves = DP / DH;
  static constexpr int kKBytes = 128 * DP * 2;
  static constexpr int kQBytes = BQ * DP * 2;
  static constexpr int kDSBytes = 128 * BQ * 2;
  static constexpr int kStatBytes = 2 * BQ * 4;
  static constexpr int kOffK = 0;
  static constexpr int kOffV = kKBytes;
  static constexpr int kOffQ = 2 * kKBytes;
  static constexpr int kOffDO = kOffQ + NST * kQBytes;
  static constexpr int kOffDS = kOffDO + NST * kQBytes;
  static constexpr int kOffStat = kOffDS + kDSBytes;
  static constexpr int kSmemUsed = kOffStat + NST * kStatBytes;
  // Pad to more than half of the SM's shared memory so that two CTAs never share an SM
  // (each CTA allocates the whole tensor memory).
  static constexpr int kSmemBytes = kSmemUsed < 120 * 1024 ? 120 * 1024 : kSmemUsed;
  static constexpr int kThreads = 640;
  static constexpr int kTmS = 0;
  static constexpr int kTmDP = BQ;
  static constexpr int kTmDV = 2 * BQ;
  static constexpr int kTmDK = 2 * BQ + DH;
  static_assert(2 * BQ + 2 * DH <= 512, "tensor memory over budget");
  static_assert(kSmemBytes <= 232448 - 1024, "shared memory over budget");
};

template <int DP, int DH, int BQ, int NST, typename T>
__global__ void __launch_bounds__(640, 1)
    bwd_hop_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const BwdParams p) {
  using Cfg = BwdCfg<DP, DH, BQ, NST>;
  constexpr bool kBf16 = Pack2<T>::kIsBf16;
  constexpr int kPanelK = 128 * 128;  // bytes per panel of a 128-row tile
  constexpr int kPanelQ = BQ * 128;   // bytes per panel of a BQ-row tile

  extern __shared__ __align__(1024) uint8_t smem_raw[];
  __shared__ uint64_t bar_kv_full;
  __shared__ uint64_t bar_q_full[NST], bar_q_empty[NST], bar_do_full[NST], bar_do_empty[NST];
  __shared__ uint64_t bar_s_full, bar_p_ready, bar_dp_full, bar_ds_ready, bar_dq_full, bar_dq_drained, bar_final;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  if (*reinterpret_cast<volatile int*>(p.status) != 0) return;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const uint32_t smem_base = smem_u32(smem_raw);
  const uint32_t s_k = smem_base + Cfg::kOffK;
  const uint32_t s_v = smem_base + Cfg::kOffV;
  const uint32_t s_q = smem_base + Cfg::kOffQ;
  const uint32_t s_do = smem_base + Cfg::kOffDO;
  const uint32_t s_ds = smem_base + Cfg::kOffDS;
  const uint32_t s_stat = smem_base + Cfg::kOffStat;
  uint8_t* const stat_ptr = smem_raw + Cfg::kOffStat;
  uint8_t* const ds_ptr = smem_raw + Cfg::kOffDS;

  // ---- tile coordinates ----
  // Diagonal (causal) blocks: kv tile first, so that the CTAs with the most visible queries start first and the tail
  // of the grid evens out.  Full blocks (every CTA carries the same work): head group first, kv tile fastest, so that
  // the CTAs resident at one time work on the dQ accumulator and the Q/dO tiles of two or three head groups only --
  // some 20 MB instead of the whole 134 MB accumulator, which then stays in L2 between the reductions of
  // different kv tiles (kv-tile-first order re-fetched it from HBM: 4.3 GB of DRAM traffic per launch at
  // S = 8192, 32/8 heads, against 0.6 GB of algorithmic bytes).
  int kvt, hf, gs, hkv, b;
  {
    int rem = static_cast<int>(blockIdx.x);
    hf = rem % Cfg::kHalves;
    rem /= Cfg::kHalves;
    if (p.causal) {
      gs = rem % p.gsplit;  // CTAs that share a K/V tile are adjacent (the tile stays in L2)
      rem /= p.gsplit;
      hkv = rem % p.Hkv;
      rem /= p.Hkv;
      b = rem % p.B;
      kvt = rem / p.B;
    } else {
      const int nkvt = (p.kv_len + 127) / 128;
      kvt = rem % nkvt;
      rem /= nkvt;
      gs = rem % p.gsplit;
      rem /= p.gsplit;
      hkv = rem % p.Hkv;
      b = rem / p.Hkv;
    }
  }
  const int G = p.Hq / p.Hkv;
  const int Gc = G / p.gsplit;
  const int n0 = kvt * 128;
  const int nQtiles = (p.Sq + BQ - 1) / BQ;
  const int i_begin = max(p.causal ? (n0 / BQ) : 0, p.q_begin / BQ);
  const int nI = nQtiles - i_begin;
  const int T_total = Gc * nI;

  if (tid == 0) {
    abort_flag = ((smem_base & 1023u) != 0) ? 1 : 0;  // operand tiles need 1024-byte alignment
    mbar_init(&bar_kv_full, 1);
    for (int i = 0; i < NST; ++i) {
      mbar_init(&bar_q_full[i], 1);
      mbar_init(&bar_q_empty[i], 1);
      mbar_init(&bar_do_full[i], 1);
      mbar_init(&bar_do_empty[i], 1);
    }
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_p_ready, 256);
    mbar_init(&bar_dp_full, 1);
    mbar_init(&bar_ds_ready, 256);
    mbar_init(&bar_dq_full, 1);
    mbar_init(&bar_dq_drained, 256);
    mbar_init(&bar_final, 1);
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
  const bool run = (abort_flag == 0) && (T_total > 0);

  Tracer tr;
  {
    int role = -1;
    // traced roles: producer, issuer, one warp of each elementwise group, one reduction warp
    if (lane == 0) role = (warp == 0) ? 0 : (warp == 1) ? 1 : (warp == 4) ? 2 : (warp == 8) ? 3 : (warp == 12) ? 4 : -1;
    if (role >= 0) tr.init(p.trace, p.trace_ctas, p.trace_cap, kTraceRoles, role);
  }
  auto q_head = [&](int t) { return hkv * G + gs * Gc + t / nI; };
  auto q_tile = [&](int t) { return i_begin + t % nI; };

  // Register budget.  The launch gives every thread 96 registers (640 x 96 = 61440, the pool the warpgroups trade
  // inside); each role changes its own allowance on entry: 4 service warps x 64, 8 elementwise warps x 128,
  // 8 reduction warps x 80.  The raise waits until the other roles have lowered theirs, so the sum must fit the pool.
  static_assert(128 * 64 + 256 * 128 + 256 * 80 <= 640 * 96, "register allowances exceed what the launch allocated");
  if (warp < 4) {
    setmaxnreg_dec<64>();
    if (warp == 0) {
      // =========================== TMA producer ===========================
      if (lane == 0 && run) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
        tma_prefetch_desc(&tm_do);
        mbar_expect_tx(&bar_kv_full, 2 * Cfg::kKBytes);
#pragma unroll
        for (int pn = 0; pn < Cfg::kPanels; ++pn) {
          tma_load_4d(s_k + pn * kPanelK, &tm_k, &bar_kv_full, pn * 64, hkv, n0, b);
          tma_load_4d(s_v + pn * kPanelK, &tm_v, &bar_kv_full, pn * 64, hkv, n0, b);
        }
        for (int t = 0; t < T_total; ++t) {
          const int st = t % NST;
          const uint32_t par_empty = ((t / NST) & 1) ^ 1;
          const int hq = q_head(t);
          const int i = q_tile(t);
          // dO first: its slot frees earlier (after the dV product) than the Q slot (after dK).
          if (!mbar_wait(&bar_do_empty[st], par_empty, abort_p)) break;
          tr.mark(40);
          mbar_expect_tx(&bar_do_full[st], Cfg::kQBytes);
#pragma unroll
          for (int pn = 0; pn < Cfg::kPanels; ++pn)
            tma_load_4d(s_do + st * Cfg::kQBytes + pn * kPanelQ, &tm_do, &bar_do_full[st], pn * 64, hq, i * BQ, b);
          if (!mbar_wait(&bar_q_empty[st], par_empty, abort_p)) break;
          tr.mark(41);
          mbar_expect_tx(&bar_q_full[st], Cfg::kQBytes + Cfg::kStatBytes);
#pragma unroll
          for (int pn = 0; pn < Cfg::kPanels; ++pn)
            tma_load_4d(s_q + st * Cfg::kQBytes + pn * kPanelQ, &tm_q, &bar_q_full[st], pn * 64, hq, i * BQ, b);
          const size_t stat_off = (static_cast<size_t>(b) * p.Hq + hq) * p.Spad + static_cast<size_t>(i) * BQ;
          bulk_load_1d(s_stat + st * Cfg::kStatBytes, p.lse2 + stat_off, BQ * 4, &bar_q_full[st]);
          bulk_load_1d(s_stat + st * Cfg::kStatBytes + BQ * 4, p.delta + stat_off, BQ * 4, &bar_q_full[st]);
        }
      }
      __syncwarp();
    } else if (warp == 1) {
      // =========================== MMA issuer ===========================
      // The whole warp runs the loop converged (cheap, warp-uniform descriptor arithmetic); the elected lane issues.
      if (run) {
        const uint32_t el = elect_one();
        constexpr uint32_t idesc_s = make_idesc(128, BQ, kBf16, false, false);   // K-major x K-major
        constexpr uint32_t idesc_dv = make_idesc(128, DH, kBf16, false, true);   // A tmem / K-major smem, B MN-major
        constexpr uint32_t idesc_dq = make_idesc(128, BQ, kBf16, true, true);    // both MN-major
        const uint32_t tm_s = tmem_base + Cfg::kTmS;
        const uint32_t tm_dp = tmem_base + Cfg::kTmDP;
        const uint32_t tm_dv = tmem_base + Cfg::kTmDV;
        const uint32_t tm_dk = tmem_base + Cfg::kTmDK;

        // Descriptor low words of the resident tiles; offsets below are in 16-byte units.
        const uint32_t k_km = desc_lo_kmajor(s_k);                                   // K as K-major A (S^T)
        const uint32_t v_km = desc_lo_kmajor(s_v);                                   // V as K-major A (dP^T)
        const uint32_t k_mn = desc_lo_mnmajor(s_k + hf * (DH / 64) * kPanelK, kPanelK);  // K^T as MN-major A (dQ^T)
        const uint32_t ds_km = desc_lo_kmajor(s_ds);                                 // dS^T as K-major A (dK)
        const uint32_t ds_mn = desc_lo_mnmajor(s_ds, kPanelK);                       // dS^T as MN-major B (dQ^T)
        auto q_km = [&](int st) { return desc_lo_kmajor(s_q + st * Cfg::kQBytes); };
        auto do_km = [&](int st) { return desc_lo_kmajor(s_do + st * Cfg::kQBytes); };
        auto q_mn = [&](int st) {
          return desc_lo_mnmajor(s_q + st * Cfg::kQBytes + hf * (DH / 64) * kPanelQ, kPanelQ);
        };
        auto do_mn = [&](int st) {
          return desc_lo_mnmajor(s_do + st * Cfg::kQBytes + hf * (DH / 64) * kPanelQ, kPanelQ);
        };

        // S^T[128 x BQ] = K[128 x DP] * Q[BQ x DP]^T
        auto issue_s = [&](int st) {
          const uint32_t bq = q_km(st);
#pragma unroll
          for (int ks = 0; ks < DP / 16; ++ks)
            mma_ss_lo_e(tm_s, k_km + (((ks >> 2) * kPanelK + (ks & 3) * 32) >> 4),
                      bq + (((ks >> 2) * kPanelQ + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u, el);
        };
        // dP^T[128 x BQ] = V[128 x DP] * dO[BQ x DP]^T
        auto issue_dp = [&](int st) {
          const uint32_t bo = do_km(st);
#pragma unroll
          for (int ks = 0; ks < DP / 16; ++ks)
            mma_ss_lo_e(tm_dp, v_km + (((ks >> 2) * kPanelK + (ks & 3) * 32) >> 4),
                      bo + (((ks >> 2) * kPanelQ + (ks & 3) * 32) >> 4), idesc_s, ks > 0 ? 1u : 0u, el);
        };
        // dV[128 x DH] += P^T[128 x BQ] (tensor memory) * dO[BQ x DH]
        auto issue_dv = [&](int st, bool acc) {
          const uint32_t bo = do_mn(st);
#pragma unroll
          for (int ks = 0; ks < BQ / 16; ++ks) {
            // P^T of query columns [16ks, 16ks+16): each elementwise group packs its half over its own S^T columns
            const int grp = (ks * 16) / (BQ / 2);
            const uint32_t pa = tm_s + grp * (BQ / 2) + ((ks * 16) % (BQ / 2)) / 2;
            mma_ts_lo_e(tm_dv, pa, bo + ((ks * 2048) >> 4), idesc_dv, (acc || ks > 0) ? 1u : 0u, el);
          }
        };
        // dK[128 x DH] += dS^T[128 x BQ] (shared memory, K-major) * Q[BQ x DH]
        auto issue_dk = [&](int st, bool acc) {
          const uint32_t bq = q_mn(st);
#pragma unroll
          for (int ks = 0; ks < BQ / 16; ++ks)
            mma_ss_lo_e(tm_dk, ds_km + (((ks >> 2) * kPanelK + (ks & 3) * 32) >> 4), bq + ((ks * 2048) >> 4), idesc_dv,
                        (acc || ks > 0) ? 1u : 0u, el);
        };
        // dQ^T[128 (d) x BQ] = K^T[d x 128 (kv)] * dS^T[128 (kv) x BQ]; for head dim 64 the upper 64
        // rows of the A operand run into the V tile (results in those lanes are ignored).
        auto issue_dq = [&]() {
#pragma unroll
          for (int ks = 0; ks < 128 / 16; ++ks)
            mma_ss_lo_e(tm_dp, k_mn + ((ks * 2048) >> 4), ds_mn + ((ks * 2048) >> 4), idesc_dq, ks > 0 ? 1u : 0u, el);
        };

        bool ok = mbar_wait_warp(&bar_kv_full, 0, abort_p);
        if (ok) ok = mbar_wait_warp(&bar_q_full[0], 0, abort_p);
        if (ok) {
          tc_fence_after_sync();
          issue_s(0);
          mma_commit_e(&bar_s_full, el);
          ok = mbar_wait_warp(&bar_do_full[0], 0, abort_p);
        }
        if (ok) {
          tc_fence_after_sync();
          issue_dp(0);
          mma_commit_e(&bar_dp_full, el);
        }
        for (int t = 0; t < T_total && ok; ++t) {
          const int st = t % NST;
          const int st_n = (t + 1) % NST;
          const uint32_t par_n = ((t + 1) / NST) & 1;
          const bool more = (t + 1 < T_total);
          tr.mark(10);
          if (!mbar_wait_warp(&bar_p_ready, t & 1, abort_p)) break;
          tr.mark(11);
          tc_fence_after_sync();
          issue_dv(st, t > 0);
          mma_commit_e(&bar_do_empty[st], el);
          // S^T of the next tile goes out now if its Q tile has landed (a non-blocking probe); otherwise it is the
          // first thing issued once dS^T is ready.
          bool s_issued = !more;
          if (more && __all_sync(0xffffffffu, mbar_test_wait(&bar_q_full[st_n], par_n))) {
            tr.mark(12);
            tc_fence_after_sync();
            issue_s(st_n);
            mma_commit_e(&bar_s_full, el);
            s_issued = true;
          }
          tr.mark(13);
          if (!mbar_wait_warp(&bar_ds_ready, t & 1, abort_p)) break;
          tr.mark(14);
          tc_fence_after_sync();
          if (NST >= 2 && !s_issued) {
            // The elementwise warps have nothing to do until S^T of the next tile exists: it goes first.  (With a
            // single Q stage the next tile can only be loaded after dK below has released the slot.)
            if (!mbar_wait_warp(&bar_q_full[st_n], par_n, abort_p)) break;
            tc_fence_after_sync();
            issue_s(st_n);
            mma_commit_e(&bar_s_full, el);
            s_issued = true;
          }
          // dK before dQ^T: it releases the Q slot ~500 cycles earlier, which matters more than the reduction
          // starting earlier (a Q tile load takes 1500-3000 cycles under the L2 load of the reductions and only two
          // Q stages fit in shared memory).
          issue_dk(st, t > 0);
          mma_commit_e(&bar_q_empty[st], el);
          issue_dq();
          mma_commit_e(&bar_dq_full, el);
          tr.mark(15);
          if (!s_issued) {
            if (!mbar_wait_warp(&bar_q_full[st_n], par_n, abort_p)) break;
            tc_fence_after_sync();
            issue_s(st_n);
            mma_commit_e(&bar_s_full, el);
          }
          if (more) {
            if (!mbar_wait_warp(&bar_do_full[st_n], par_n, abort_p)) break;
            tr.mark(16);
            if (!mbar_wait_warp(&bar_dq_drained, t & 1, abort_p)) break;
            tr.mark(17);
            tc_fence_after_sync();
            issue_dp(st_n);
            mma_commit_e(&bar_dp_full, el);
            tr.mark(18);
          } else {
            mma_commit_e(&bar_final, el);
          }
        }
      }
      __syncwarp();
    }
  } else if (warp < 12) {
    // =========================== elementwise warpgroups ===========================
    // Two warpgroups share every tile: group cw owns query columns [cw*BQ/2, (cw+1)*BQ/2).
    setmaxnreg_inc<128>();
    constexpr int kHalfCols = BQ / 2;
    constexpr int NCH = kHalfCols / 32;  // 32-column chunks per thread
    const int cw = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // kv row inside the tile
    const int kvpos = n0 + row;
    // Queries before mask_lim get P = 0 for this key: the causal rule on a diagonal block (query before key), and every
    // query when the key lies at or beyond kv_len (a window that ends inside this tile: those keys are real rows of the
    // K/V tensors, so without the mask they would add to dQ).
    const int mask_lim = (kvpos >= p.kv_len) ? 0x7fffffff : (p.causal ? kvpos : static_cast<int>(0x80000000));
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int col0 = cw * kHalfCols;
    const uint32_t a_s = tmem_base + lane_addr + Cfg::kTmS + col0;
    const uint32_t a_dp = tmem_base + lane_addr + Cfg::kTmDP + col0;
    constexpr int kPolyEvery = kBwdPolyEvery;  // of the 8 groups of four exponentials per 32 columns
    const Exp2Poly exp2_poly;
    const uint64_t nscale2 = pack_f2(-p.scale_log2, -p.scale_log2);
    bool ok = run;
    for (int t = 0; t < T_total && ok; ++t) {
      const int st = t % NST;
      const int i = q_tile(t);
      const float* lse2_s = reinterpret_cast<const float*>(stat_ptr + st * Cfg::kStatBytes) + col0;
      const float* delta_s = lse2_s + BQ;
      if (!mbar_wait_warp(&bar_q_full[st], (t / NST) & 1, abort_p)) { ok = false; break; }
      tr.mark(19);
      if (!mbar_wait_warp(&bar_s_full, t & 1, abort_p)) { ok = false; break; }
      tr.mark(20);
      tc_fence_after_sync();
      const int q0 = i * BQ + col0;
      const bool masked = (p.causal && (i * BQ < n0 + 127)) || (n0 + 128 > p.kv_len);
      uint32_t pk[NCH * 16];
      {
        uint32_t r[NCH][32];
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld32(a_s + c * 32, r[c]);
        tmem_ld_wait32(r[0]);
#pragma unroll
        for (int c = 1; c < NCH; ++c) reg_fence32(r[c]);
        tr.mark(21);
        // P^T = exp2(scale*log2e * S^T - lse2[q]); masked only on diagonal tiles and on a tile that straddles kv_len.
        // Packed pairs: y = lse2 - c*s in one fma, then 2^(-y); every kPolyEvery-th pair on the FMA pipe.
        auto p_phase = [&](auto mask_tag) {
          constexpr bool kMask = decltype(mask_tag)::value;
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float4 l4 = *reinterpret_cast<const float4*>(lse2_s + c * 32 + k * 4);
              const uint64_t y01 = fma2(pack_u2(r[c][4 * k + 0], r[c][4 * k + 1]), nscale2, pack_f2(l4.x, l4.y));
              const uint64_t y23 = fma2(pack_u2(r[c][4 * k + 2], r[c][4 * k + 3]), nscale2, pack_f2(l4.z, l4.w));
              float e0, e1, e2, e3;
              if (kPolyEvery > 0 && (k % (kPolyEvery > 0 ? kPolyEvery : 1)) == kPolyEvery - 1) {
                unpack_f2(exp2_poly.neg(y01), e0, e1);
                unpack_f2(exp2_poly.neg(y23), e2, e3);
              } else {
                float y0, y1, y2, y3;
                unpack_f2(y01, y0, y1);
                unpack_f2(y23, y2, y3);
                e0 = fast_exp2(-y0);
                e1 = fast_exp2(-y1);
                e2 = fast_exp2(-y2);
                e3 = fast_exp2(-y3);
              }
              if (kMask) {
                const int qp = q0 + c * 32 + k * 4;
                if (qp + 0 < mask_lim) e0 = 0.f;
                if (qp + 1 < mask_lim) e1 = 0.f;
                if (qp + 2 < mask_lim) e2 = 0.f;
                if (qp + 3 < mask_lim) e3 = 0.f;
              }
              pk[c * 16 + 2 * k + 0] = Pack2<T>::pack(e0, e1);
              pk[c * 16 + 2 * k + 1] = Pack2<T>::pack(e2, e3);
            }
          }
        };
        if (masked) p_phase(std::true_type{});
        else p_phase(std::false_type{});
      }
      tr.mark(26);
      // P^T (16 bit, two per column) goes over the start of this group's own S^T columns.
#pragma unroll
      for (int c = 0; c < NCH; ++c) {
        uint32_t u[16];
#pragma unroll
        for (int k = 0; k < 16; ++k) u[k] = pk[c * 16 + k];
        tmem_st16(a_s + c * 16, u);
      }
      tmem_st_wait();
      tr.mark(27);
      tc_fence_before_sync();
      mbar_arrive(&bar_p_ready);
      tr.mark(22);

      if (!mbar_wait_warp(&bar_dp_full, t & 1, abort_p)) { ok = false; break; }
      tr.mark(23);
      tc_fence_after_sync();
      {
        uint32_t r[NCH][32];
#pragma unroll
        for (int c = 0; c < NCH; ++c) tmem_ld32(a_dp + c * 32, r[c]);
        tmem_ld_wait32(r[0]);
#pragma unroll
        for (int c = 1; c < NCH; ++c) reg_fence32(r[c]);
        tr.mark(24);
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          uint32_t w[16];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float4 d4 = *reinterpret_cast<const float4*>(delta_s + c * 32 + k * 4);
            const float2 p01 = Pack2<T>::unpack(pk[c * 16 + 2 * k + 0]);
            const float2 p23 = Pack2<T>::unpack(pk[c * 16 + 2 * k + 1]);
            float s0, s1, s2, s3;
            unpack_f2(mul2(pack_f2(p01.x, p01.y),
                           sub2(pack_u2(r[c][4 * k + 0], r[c][4 * k + 1]), pack_f2(d4.x, d4.y))), s0, s1);
            unpack_f2(mul2(pack_f2(p23.x, p23.y),
                           sub2(pack_u2(r[c][4 * k + 2], r[c][4 * k + 3]), pack_f2(d4.z, d4.w))), s2, s3);
            w[2 * k + 0] = Pack2<T>::pack(s0, s1);
            w[2 * k + 1] = Pack2<T>::pack(s2, s3);
          }
          // 32 columns = 64 bytes = four 16-byte chunks inside the panel that holds column col0 + c*32
          const int colg = col0 + c * 32;
          uint8_t* panel = ds_ptr + (colg / 64) * kPanelK;
          const int chunk0 = (colg % 64) / 8;
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            uint4 v4 = make_uint4(w[4 * k + 0], w[4 * k + 1], w[4 * k + 2], w[4 * k + 3]);
            *reinterpret_cast<uint4*>(panel + sw128_offset(row, chunk0 + k)) = v4;
          }
        }
      }
      tr.mark(28);
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bar_ds_ready);
      tr.mark(25);
    }
    // ---- epilogue: group 0 writes dV, group 1 writes dK (scaled) ----
    if (ok) ok = mbar_wait_warp(&bar_final, 0, abort_p);
    if (ok) {
      tc_fence_after_sync();
      const bool row_ok = kvpos < p.kv_len;
      const int which = (cw == 0) ? 1 : 0;  // packed buffer: [0] = dK, [1] = dV
      const float mul = (cw == 0) ? 1.0f : p.scale;
      const uint32_t a_acc = tmem_base + lane_addr + (cw == 0 ? Cfg::kTmDV : Cfg::kTmDK);
      const size_t base = (((static_cast<size_t>(which) * p.B + b) * p.Skv + kvpos) * p.Hkv + hkv) * p.D + hf * DH;
#pragma unroll 1
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(a_acc + c * 32, r);
        tmem_ld_wait32(r);
        if (row_ok) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int d = hf * DH + c * 32 + k * 4;
            if (d < p.D) {
              float4 v = make_float4(__uint_as_float(r[4 * k + 0]) * mul, __uint_as_float(r[4 * k + 1]) * mul,
                                     __uint_as_float(r[4 * k + 2]) * mul, __uint_as_float(r[4 * k + 3]) * mul);
              if (p.reduce_out) {
                // several CTAs (one per slice of the GQA group) add into the same rows; the host prepared dkdv_out
                red_add_v4_f32(p.dkdv_out + base + c * 32 + k * 4, v.x, v.y, v.z, v.w);
              } else {
                if (p.accumulate_prev) {
                  const float4 o = *reinterpret_cast<const float4*>(p.dkdv_prev + base + c * 32 + k * 4);
                  v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                }
                *reinterpret_cast<float4*>(p.dkdv_out + base + c * 32 + k * 4) = v;
              }
            }
          }
        }
      }
    }
    __syncwarp();
  } else {
    // =========================== dQ reduction warpgroups ===========================
    // Two warpgroups, each owning half of the query columns of dQ^T.  A thread pulls its whole share into registers
    // with one batch of loads and releases the tensor-memory columns at once (the next dP^T product is waiting for
    // them); the vector reductions into global memory, which drain at the rate the L2 can add, then overlap the next
    // tile's products instead of sitting in front of them.
    setmaxnreg_dec<80>();
    constexpr int kRedCols = BQ / 2;
    constexpr int NCR = kRedCols / 32;
    const int half = (warp - 12) >> 2;
    const int quarter = warp & 3;
    const int drow = quarter * 32 + lane;  // row of dQ^T = head-dim index inside this CTA's half
    const int d = hf * DH + drow;
    const bool d_ok = (drow < DH);
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t a_dq = tmem_base + lane_addr + Cfg::kTmDP + half * kRedCols;
    // dQ accumulator layout (fp32, private): [b][hq][Spad/128 tiles][32 groups of 4 rows][DP][4].
    // Lane = head-dim index, four consecutive registers = four consecutive query rows, so one
    // 16-byte vector reduction per (lane, row group) and 512 contiguous bytes per warp instruction.
    constexpr size_t kTileElems = static_cast<size_t>(128) * DP;
    const int nQt128 = p.Spad / 128;
    bool ok = run;
    for (int t = 0; t < T_total && ok; ++t) {
      const int hq = q_head(t);
      const int q0 = q_tile(t) * BQ;
      tr.mark(29);
      if (!mbar_wait_warp(&bar_dq_full, t & 1, abort_p)) { ok = false; break; }
      tr.mark(30);
      tc_fence_after_sync();
      float* base = p.dq_acc + ((static_cast<size_t>(b) * p.Hq + hq) * nQt128 + q0 / 128) * kTileElems +
                    (static_cast<size_t>((q0 % 128 + half * kRedCols) / 4) * DP + d) * 4;
      uint32_t r[NCR][32];
#pragma unroll
      for (int c = 0; c < NCR; ++c) tmem_ld32(a_dq + c * 32, r[c]);
      tmem_ld_wait32(r[0]);
#pragma unroll
      for (int c = 1; c < NCR; ++c) reg_fence32(r[c]);
      // every read of this half of dQ^T has completed: the columns may be overwritten by the next dP^T
      tc_fence_before_sync();
      mbar_arrive(&bar_dq_drained);
      tr.mark(31);
      // Ordered mode (bit-reproducible dQ): the contributions of the kv tiles to one accumulator tile are added in
      // kv-tile order.  One counter per (head, query tile, warp slice); the CTA of kv tile j adds after j earlier
      // tiles have.  The CTA of the previous kv tile (same heads) always has a lower block index, so it was
      // dispatched before this one: it is resident or finished, never pending behind the waiter.
      int* order_sem = nullptr;
      if (p.dq_order != nullptr) {
        order_sem = p.dq_order +
                    ((((static_cast<size_t>(b) * p.Hq + hq) * nQtiles + q_tile(t)) * Cfg::kHalves + hf) * 2 + half) * 4 +
                    quarter;
        bool got = true;
        if (lane == 0 && d_ok) {
          const unsigned long long t0 = global_timer_ns();
          uint32_t spins = 0;
          while (ld_acquire_gpu(order_sem) < kvt) {
            if (((++spins) & 0x3fu) == 0) {
              if (*abort_p) { got = false; break; }
              if (global_timer_ns() - t0 > kWaitLimitNs) { *abort_p = 1; got = false; break; }
            }
            __nanosleep(64);
          }
        }
        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
      }
      if (d_ok) {
        // rows beyond Sq and head-dim columns beyond D hold exact zeros (zero-filled operands, P = 0)
#pragma unroll
        for (int c = 0; c < NCR; ++c) {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            red_add_v4_f32(base + static_cast<size_t>(c * 8 + k) * DP * 4, __uint_as_float(r[c][4 * k + 0]) * p.scale,
                           __uint_as_float(r[c][4 * k + 1]) * p.scale, __uint_as_float(r[c][4 * k + 2]) * p.scale,
                           __uint_as_float(r[c][4 * k + 3]) * p.scale);
            if (kRedSleepNs > 0) __nanosleep(kRedSleepNs);
          }
        }
        if (order_sem != nullptr) {
          __threadfence();  // this lane's reductions are performed before the counter moves
          __syncwarp();
          if (lane == 0) red_release_gpu_add(order_sem, 1);
        }
      }
    }
    __syncwarp();
  }

  // ---- teardown ----
  tc_fence_before_sync();
  __syncthreads();
  if (abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    if (tid == 0) atomicExch(p.status, kStatusWaitTimeout);
  }
  if (warp == 0) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 512);
  }
}

template <int DP, int DH, int BQ, int NST, typename T>
static int launch_bwd(const void* q, const void* k, const void* v, const void* dout, const BwdParams& prm, int dtype,
                      cudaStream_t stream) {
  using Cfg = BwdCfg<DP, DH, BQ, NST>;
  CUtensorMap tq, tk, tv, tdo;
  int rc;
  if ((rc = make_tmap_bshd(&tq, q, dtype, prm.B, prm.Sq, prm.Hq, prm.D, BQ)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tdo, dout, dtype, prm.B, prm.Sq, prm.Hq, prm.D, BQ)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tk, k, dtype, prm.B, prm.Skv, prm.Hkv, prm.D, 128)) != RFA_OK) return rc;
  if ((rc = make_tmap_bshd(&tv, v, dtype, prm.B, prm.Skv, prm.Hkv, prm.D, 128)) != RFA_OK) return rc;
  auto kern = bwd_hop_kernel<DP, DH, BQ, NST, T>;
  // Function attributes belong to a device: the opt-in to large dynamic shared memory is made once per device.
  static bool attr_done[kMaxDevices] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) { cudaGetLastError(); return RFA_ERR_CUDA; }
  if (!attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
    // The kernel trades registers between its warpgroups inside the pool the launch allocates (threads x registers
    // per thread); a raise that the pool cannot satisfy would wait forever, so a build whose register count does not
    // cover the allowances is refused here instead of launched.
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, kern);
    if (e != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
    if (fa.numRegs * Cfg::kThreads < 128 * 64 + 256 * 128 + 256 * 80) return RFA_ERR_UNSUPPORTED;
    attr_done[dev] = true;
  }
  BwdParams pr = prm;
  const long long base_units = static_cast<long long>(ceil_div(prm.kv_len, 128)) * prm.Hkv * prm.B * Cfg::kHalves;
  {
    const int rc2 = choose_group_split(pr, base_units, stream);
    if (rc2 != RFA_OK) return rc2;
  }
  if (pr.dq_order != nullptr) {
    const size_t n = static_cast<size_t>(prm.B) * prm.Hq * ceil_div(prm.Sq, BQ) * Cfg::kHalves * 8;
    if (cudaMemsetAsync(pr.dq_order, 0, n * sizeof(int), stream) != cudaSuccess) { cudaGetLastError(); return RFA_ERR_CUDA; }
  }
  const unsigned grid = static_cast<unsigned>(base_units * pr.gsplit);
  kern<<<grid, Cfg::kThreads, Cfg::kSmemBytes, stream>>>(tq, tk, tv, tdo, pr);
  return cuda_status(cudaGetLastError());
}

template <typename T>
static int dispatch_bwd(int dp, const void* q, const void* k, const void* v, const void* dout, const BwdParams& prm,
                        int dtype, cudaStream_t stream) {
  switch (dp) {
    case 64: return launch_bwd<64, 64, 128, 2, T>(q, k, v, dout, prm, dtype, stream);
    case 128: return launch_bwd<128, 128, 128, 2, T>(q, k, v, dout, prm, dtype, stream);
    case 256: return launch_bwd<256, 128, 64, 1, T>(q, k, v, dout, prm, dtype, stream);
    default: return RFA_ERR_UNSUPPORTED;
  }
}

}  // namespace rfa

// Argument checks shared by every backward-hop entry point (nothing is enqueued before they pass).
int rfa::bwd_check_args(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                        const float* delta, const float* dkdv_prev, const float* dkdv_out, int B, int Sq, int Skv,
                        int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev, int causal_diag,
                        int q_begin, int kv_len, const int* status) {
  if (!q || !k || !v || !dout || !lse2 || !delta || !dkdv_out || !status) return RFA_ERR_INVALID_ARG;
  if (accumulate_prev && !dkdv_prev) return RFA_ERR_INVALID_ARG;
  if (B <= 0 || Sq <= 0 || Skv <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0) return RFA_ERR_INVALID_ARG;
  if (!(softmax_scale > 0.f)) return RFA_ERR_INVALID_ARG;
  if (causal_diag && Sq != Skv) return RFA_ERR_INVALID_ARG;
  if (q_begin < 0 || q_begin >= Sq || (q_begin % 128) != 0 || kv_len <= 0 || kv_len > Skv) return RFA_ERR_INVALID_ARG;
  if (padded_head_dim(D) == 0) return RFA_ERR_UNSUPPORTED;
  if (dtype != RFA_DTYPE_BF16 && dtype != RFA_DTYPE_FP16) return RFA_ERR_UNSUPPORTED;
  if ((reinterpret_cast<uintptr_t>(lse2) & 15u) || (reinterpret_cast<uintptr_t>(delta) & 15u) ||
      (reinterpret_cast<uintptr_t>(dkdv_out) & 15u) || (reinterpret_cast<uintptr_t>(dkdv_prev) & 15u))
    return RFA_ERR_INVALID_ARG;
  return RFA_OK;
}

// Query-tile width of the backward kernel for a padded head dim (the granularity of the ordering counters).
static int bwd_q_tile(int dp) { return dp == 256 ? 64 : 128; }

extern "C" size_t rfa_dq_order_elems(int B, int Sq, int Hq, int D) {
  const int dp = rfa::padded_head_dim(D);
  if (dp == 0 || B <= 0 || Sq <= 0 || Hq <= 0) return 0;
  return static_cast<size_t>(B) * Hq * rfa::ceil_div(Sq, bwd_q_tile(dp)) * (dp == 256 ? 2 : 1) * 8;
}

static int bwd_hop_impl(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                        const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B, int Sq,
                        int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev,
                        int causal_diag, int q_begin, int kv_len, int* dq_order, int* status, void* stream) {
  using namespace rfa;
  if (!dq_acc) return RFA_ERR_INVALID_ARG;
  {
    const int rc = bwd_check_args(q, k, v, dout, lse2, delta, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                                  softmax_scale, accumulate_prev, causal_diag, q_begin, kv_len, status);
    if (rc != RFA_OK) return rc;
  }
  if (reinterpret_cast<uintptr_t>(dq_order) & 3u) return RFA_ERR_INVALID_ARG;
  const int dp = padded_head_dim(D);
  BwdParams prm;
  prm.lse2 = lse2;
  prm.delta = delta;
  prm.dq_acc = dq_acc;
  prm.dkdv_prev = dkdv_prev;
  prm.dkdv_out = dkdv_out;
  prm.B = B;
  prm.Sq = Sq;
  prm.Skv = Skv;
  prm.Hq = Hq;
  prm.Hkv = Hkv;
  prm.D = D;
  prm.Spad = round_up(Sq, 128);
  prm.scale = softmax_scale;
  prm.scale_log2 = softmax_scale * 1.4426950408889634f;
  prm.accumulate_prev = accumulate_prev ? 1 : 0;
  prm.causal = causal_diag ? 1 : 0;
  prm.q_begin = q_begin;
  prm.kv_len = kv_len;
  prm.gsplit = 1;
  prm.reduce_out = 0;
  prm.dq_order = dq_order;
  prm.status = status;
  prm.trace = g_trace.buf;
  prm.trace_ctas = g_trace.ctas;
  prm.trace_cap = g_trace.cap;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == RFA_DTYPE_BF16) return dispatch_bwd<__nv_bfloat16>(dp, q, k, v, dout, prm, dtype, s);
  return dispatch_bwd<__half>(dp, q, k, v, dout, prm, dtype, s);
}

extern "C" int rfa_bwd_hop_window(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                                  const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B,
                                  int Sq, int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale,
                                  int accumulate_prev, int causal_diag, int q_begin, int kv_len, int* status,
                                  void* stream) {
  return bwd_hop_impl(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                      softmax_scale, accumulate_prev, causal_diag, q_begin, kv_len, /*dq_order=*/nullptr, status, stream);
}

extern "C" int rfa_bwd_hop_ordered(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                                   const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B,
                                   int Sq, int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale,
                                   int accumulate_prev, int causal_diag, int q_begin, int kv_len, int* dq_order,
                                   int* status, void* stream) {
  if (!dq_order) return RFA_ERR_INVALID_ARG;
  return bwd_hop_impl(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                      softmax_scale, accumulate_prev, causal_diag, q_begin, kv_len, dq_order, status, stream);
}

extern "C" int rfa_bwd_hop(const void* q, const void* k, const void* v, const void* dout, const float* lse2,
                           const float* delta, float* dq_acc, const float* dkdv_prev, float* dkdv_out, int B, int Sq,
                           int Skv, int Hq, int Hkv, int D, int dtype, float softmax_scale, int accumulate_prev,
                           int causal_diag, int* status, void* stream) {
  return bwd_hop_impl(q, k, v, dout, lse2, delta, dq_acc, dkdv_prev, dkdv_out, B, Sq, Skv, Hq, Hkv, D, dtype,
                      softmax_scale, accumulate_prev, causal_diag, /*q_begin=*/0, /*kv_len=*/Skv, /*dq_order=*/nullptr,
                      status, stream);
}
