// Forward attention kernel for sm_100a: O = softmax(scale * Q K^T [+ mask]) V, LSE.
//
// Replaces fused_mha_forward_kernel of the reference (kernel/fused_mha_kernel.cu:20-323):
// same mathematics (online softmax over KV tiles, running max / sum, O rescale), none of its
// structure.  The kernel is PERSISTENT: one CTA per SM walks a list of work items; a work item
// is 256 query rows (two 128-row tiles) of one (batch, head), processed against the KV sequence
// in 128-row tiles:
//
//   warp 16     TMA producer for K_0, V_0, K_1, V_1, ... through a ring of shared-memory slots
//               (full / empty mbarriers per slot); runs ahead into the next item as slots free
//   warp 18     TMA producer for the two Q tiles of an item, as soon as the previous item's
//               last S = Q K^T has released them
//   warp 17     MMA issuer: S_t = Q_t K_j^T (both operands in shared memory) and
//               O_t += P_t V_j (P_t read from tensor memory), accumulators in tensor memory.
//               The whole warp runs the loop so that descriptors stay in uniform registers;
//               one elected lane issues.
//   warps 0-7   softmax of query tile 0: two threads per row (64 score columns each), S_0 read
//               with tcgen05.ld, online exp2 softmax, P_0 written back over S_0 as fp16, lazy
//               O_0 rescale, epilogue
//   warps 8-15  the same for query tile 1
//
// While one softmax group works on its tile the tensor pipe runs the other tile's MMAs, and
// while the groups run an item's epilogue the producer and the MMA warp already start the next
// item (its Q / K loads and first S = Q K^T), so that the load latency at the head of an item
// and the store at its tail are hidden.
//
// Tensor memory (512 columns): S_0 [0,128) S_1 [128,256) O_0 [256,256+D) O_1 [256+D,256+2D);
// P_t aliases the first 64 columns of S_t (two fp16 per 32-bit column).
//
// Shared memory: rows of 64 fp16 (128 bytes) in the TMA / UMMA 128-byte swizzle.  A 128 x D
// tile is D/64 boxes of 128 x 64, box b at byte offset b * 16384.  Per softmax group one
// extra tile stages the output for the TMA store.
//
// Work items are paired (heaviest with lightest query block of a head) into super-items of
// equal cost, and super-items are dealt round-robin to the CTAs: balanced without a global
// work counter, and CTAs that run at the same time work on neighbouring heads (K/V stay in L2).
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace fmha {

struct FwdKernelParams {
  float* lse;
  int heads, seqlen_q, seqlen_k;
  int num_q_blocks;     // ceil(seqlen_q / 256)
  int num_heads_total;  // batch * heads
  float scale_log2;     // scale * log2(e)
  int causal, causal_shift;
  int* status;
  // debug builds (-DFMHA_TIMELINE) only: clock64 stamps of one CTA, see FMHA_TL
  long long* timeline;
  int timeline_block;
};

#ifndef FMHA_ABLATE
#define FMHA_ABLATE 0  // debug builds: bit 0 no exp2, bit 1 no row max, bit 2 no P store
#endif

template <int D>
struct FwdTraits {
  static constexpr int kBlockM = 128;  // rows per query tile
  static constexpr int kTilesM = 2;    // query tiles per work item
  static constexpr int kBlockN = 128;  // rows per KV tile
  static constexpr int kBoxes = D / 64;
  static constexpr int kBoxBytes = 128 * 128;  // 128 rows x 128 bytes
  static constexpr int kTileBytes = kBoxes * kBoxBytes;
  static constexpr int kStages = (D == 128) ? 3 : 6;
  static constexpr int kThreads = 640;  // 16 softmax warps (2 tiles x 2 column halves), 4 issue warps
  // Q tiles, K/V ring, one output staging tile per softmax group
  static constexpr int kSmemBytes = 1024 + (kTilesM + kStages + 2) * kTileBytes;
  static constexpr int kTmemCols = 512;
  static constexpr uint32_t kIdescQK = umma_idesc_f16(128, kBlockN, 0, 0);
  static constexpr uint32_t kIdescPV = umma_idesc_f16(128, D, 0, 1);
};

constexpr int kKvWarp = 16, kMmaWarp = 17, kQWarp = 18;
// 640 threads start at 96 registers each.  The issuing warpgroup (warps 16-19) gives up 32 per
// thread, which lets the four softmax warpgroups grow by 8.
// pairs out of every 4 whose exponential is a polynomial on the FMA pipe (the rest use MUFU)
#ifndef FMHA_FWD_POLY_PAIRS
#define FMHA_FWD_POLY_PAIRS 1
#endif
constexpr int kFwdPolyPairs = FMHA_FWD_POLY_PAIRS;
constexpr int kFwdRegsLaunch = 96, kFwdRegsIssue = 64, kFwdRegsSoftmax = 104;
static_assert(kFwdRegsIssue <= kFwdRegsLaunch && kFwdRegsSoftmax >= kFwdRegsLaunch,
              "setmaxnreg.dec must not raise and .inc must not lower the launch allocation");
// setmaxnreg.inc waits until the registers are there, and the pool it draws from is what the CTA
// was launched with (threads x launch registers), not the whole register file: asking for more
// than the other warpgroups give back blocks for ever.
static_assert(kFwdRegsSoftmax * 512 + kFwdRegsIssue * 128 <= kFwdRegsLaunch * 640,
              "setmaxnreg.inc would wait for registers that no warpgroup releases");

// lazy rescale threshold in the log2 domain: P may grow to 2^8 before O is rescaled
constexpr float kRescaleThreshold = 8.0f;

// The work list of one CTA.  Super-item s = (head zh, pair k): query blocks nqb-1-k (heavy,
// first) and k (light), one item only when they coincide.  Every role of the CTA walks the
// same list with its own copy of this iterator.
struct FwdWorkIter {
  int s, sub, n_super, pairs_per_head, nqb, stride;
  __device__ FwdWorkIter(int first, int stride_, int nqb_, int heads_total)
      : s(first), sub(0), pairs_per_head((nqb_ + 1) / 2), nqb(nqb_), stride(stride_) {
    n_super = pairs_per_head * heads_total;
  }
  __device__ bool next(int& zh, int& qb) {
    while (s < n_super) {
      const int k = s % pairs_per_head;
      const int hi = nqb - 1 - k;
      zh = s / pairs_per_head;
      if (sub == 0) {
        sub = 1;
        qb = hi;
        return true;
      }
      sub = 0;
      s += stride;
      if (k != hi) {
        qb = k;
        return true;
      }
    }
    return false;
  }
};

// KV tiles each of the two query tiles of an item has to visit (0 = none)
template <int D>
__device__ __forceinline__ void fwd_item_extent(const FwdKernelParams& p, int q0, int (&n_kv)[2]) {
  using T = FwdTraits<D>;
  const int nk_total = (p.seqlen_k + T::kBlockN - 1) / T::kBlockN;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * T::kBlockM;
    if (r0 >= p.seqlen_q) {
      n_kv[t] = 0;
    } else if (!p.causal) {
      n_kv[t] = nk_total;
    } else {
      const int r_last = min(r0 + T::kBlockM - 1, p.seqlen_q - 1);
      const long long lim = (long long)r_last + p.causal_shift;
      n_kv[t] = lim < 0 ? 0 : (int)min((long long)nk_total, lim / T::kBlockN + 1);
    }
  }
}

template <int D>
__global__ void __launch_bounds__(640, 1)
    fmha_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    const FwdKernelParams p) {
  using T = FwdTraits<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full[2];   // Q_t of the current item has landed
  __shared__ uint64_t bar_q_free[2];   // the last S_t = Q_t K^T of the item is done: Q_t reusable
  __shared__ uint64_t bar_kv_full[T::kStages];
  __shared__ uint64_t bar_kv_empty[T::kStages];
  __shared__ uint64_t bar_s_full[2];
  __shared__ uint64_t bar_p_full[2];
  __shared__ uint64_t bar_o_full[2];
  __shared__ uint64_t bar_o_read[2];   // the softmax group has O_t in registers: O_t reusable
  __shared__ float row_xch[2][128];    // per tile: row statistics passed between the two halves
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;
  __shared__ int skip_cta;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // a status word already set by an earlier launch / CTA means: drain the grid quickly
  if (threadIdx.x == 0) {
    skip_cta = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    abort_word = 0;
  }
  __syncthreads();
  if (skip_cta) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t q_smem = smem_base;                                    // 2 query tiles
  const uint32_t ring_smem = smem_base + T::kTilesM * T::kTileBytes;    // K/V ring
  const uint32_t ostage_smem = ring_smem + T::kStages * T::kTileBytes;  // 2 output tiles

  // ---- set-up: barriers (thread 0), tensor memory (warp 9)
  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(smem_u32(&bar_kv_full[s]), 1);
      mbar_init(smem_u32(&bar_kv_empty[s]), 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bar_q_full[t]), 1);
      mbar_init(smem_u32(&bar_q_free[t]), 1);
      mbar_init(smem_u32(&bar_s_full[t]), 1);
      mbar_init(smem_u32(&bar_p_full[t]), 256);
      mbar_init(smem_u32(&bar_o_full[t]), 1);
      mbar_init(smem_u32(&bar_o_read[t]), 256);
    }
    fence_barrier_init();
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(&tmem_base_slot), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  FwdWorkIter work(blockIdx.x, gridDim.x, p.num_q_blocks, p.num_heads_total);
  int zh, qb;

  if (warp >= 16) {
    reg_dealloc<kFwdRegsIssue>();
    if (warp == kKvWarp) {
      // =========================== TMA producer (converged warp, elected issue) ==========
      if (elect_one()) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
      }
      __syncwarp();
      uint32_t kv_it = 0;  // K/V tiles loaded so far (ring slot and phase)
      bool ok = true;
      while (ok && work.next(zh, qb)) {
        const int z = zh / p.heads, h = zh % p.heads;
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, q0, n_kv);
        const int n_loads = 2 * max(n_kv[0], n_kv[1]);  // K_0, V_0, K_1, V_1, ...
        for (int it = 0; it < n_loads; ++it, ++kv_it) {
          const uint32_t slot = kv_it % T::kStages;
          const uint32_t round = kv_it / T::kStages;
          if (round > 0 &&
              !mbar_wait_warp(smem_u32(&bar_kv_empty[slot]), (round - 1) & 1, &abort_word, 2)) {
            ok = false;
            break;
          }
          if (elect_one()) {
            const uint32_t fbar = smem_u32(&bar_kv_full[slot]);
            mbar_arrive_expect_tx(fbar, T::kTileBytes);
            const CUtensorMap* tm = (it & 1) ? &tm_v : &tm_k;
            const int row = (it >> 1) * T::kBlockN;
#pragma unroll
            for (int b = 0; b < T::kBoxes; ++b)
              tma_load_4d(ring_smem + slot * T::kTileBytes + b * T::kBoxBytes, tm, fbar, b * 64,
                          row, h, z);
          }
          __syncwarp();
        }
      }
    } else if (warp == kQWarp) {
      // =========================== Q producer ===========================
      // its own warp, so that waiting for the Q buffers of the running item never holds back
      // the K/V prefetch of the next one
      uint32_t items = 0;  // items with work seen so far (phase of the Q barriers)
      bool ok = true;
      while (ok && work.next(zh, qb)) {
        const int z = zh / p.heads, h = zh % p.heads;
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, q0, n_kv);
        if (max(n_kv[0], n_kv[1]) == 0) continue;
#pragma unroll
        for (int t = 0; t < T::kTilesM; ++t) {
          if (items > 0 &&
              !mbar_wait_warp(smem_u32(&bar_q_free[t]), (items - 1) & 1, &abort_word, 1)) {
            ok = false;
            break;
          }
          FMHA_TL(2, (int)items * 16 + 13, t);
          if (elect_one()) {
            const uint32_t qbar = smem_u32(&bar_q_full[t]);
            mbar_arrive_expect_tx(qbar, T::kTileBytes);
#pragma unroll
            for (int b = 0; b < T::kBoxes; ++b)
              tma_load_4d(q_smem + t * T::kTileBytes + b * T::kBoxBytes, &tm_q, qbar, b * 64,
                          q0 + t * T::kBlockM, h, z);
          }
          __syncwarp();
        }
        ++items;
        // the next item's Q tiles come cold from HBM (microseconds): start them towards L2 now,
        // a whole item ahead of the load that needs them
        {
          FwdWorkIter peek = work;
          int zh2, qb2;
          if (peek.next(zh2, qb2) && elect_one()) {
#pragma unroll
            for (int t = 0; t < T::kTilesM; ++t)
#pragma unroll
              for (int b = 0; b < T::kBoxes; ++b)
                tma_prefetch_l2_4d(&tm_q, b * 64, qb2 * (T::kBlockM * T::kTilesM) + t * T::kBlockM,
                                   zh2 % p.heads, zh2 / p.heads);
          }
          __syncwarp();
        }
      }
    } else if (warp == kMmaWarp) {
      // =========================== MMA issuer (converged warp, elected issue) ============
      // All 32 lanes run the loop so that addresses and descriptors live in uniform registers;
      // a loop run by one lane only makes every operand a per-thread value that has to be moved
      // to a uniform register before each tcgen05.mma, and the issue rate falls below the
      // tensor pipe's 64 cycles per 128x128x16 MMA.
      const uint32_t q_lo0 = umma_desc_lo(q_smem, kLboKMajor);
      auto issue_qk = [&](int t, uint32_t k_addr) {
        const uint32_t d = tmem_base + t * 128;
        const uint32_t a_lo = q_lo0 + ((t * T::kTileBytes) >> 4);
        const uint32_t b_lo = umma_desc_lo(k_addr, kLboKMajor);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * T::kBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss_elect(d, a_lo + off, b_lo + off, T::kIdescQK, ks > 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int t, uint32_t v_addr, bool accumulate) {
        const uint32_t d = tmem_base + 256 + t * D;
        const uint32_t a = tmem_base + t * 128;
        const uint32_t b_lo = umma_desc_lo(v_addr, kLboMnMajor);
#pragma unroll
        for (int ks = 0; ks < T::kBlockN / 16; ++ks)
          umma_ts_elect(d, a + ks * 8, b_lo + ((ks * 2048) >> 4), T::kIdescPV,
                        (accumulate || ks > 0) ? 1u : 0u);
      };
      uint32_t items = 0, kv_it = 0;
      int tl_base = 0;  // timeline slot offset of the current item (debug builds)
      uint32_t p_cnt[2] = {0, 0};  // P_t tiles consumed so far (phase of p_full[t])
      uint32_t o_cnt[2] = {0, 0};  // items in which tile t produced an O_t (phase of o_read[t])
      bool ok = true;
      // first S_t = Q_t K_0^T of an item (slot0 holds K_0), with the item's bookkeeping
      auto first_qk = [&](int t, int n_t, uint32_t slot0) {
        if (n_t > 0) {
          issue_qk(t, ring_smem + slot0 * T::kTileBytes);
          umma_commit_elect(smem_u32(&bar_s_full[t]));
        }
        // with at most one KV tile this was the item's last use of Q_t
        if (n_t <= 1) umma_commit_elect(smem_u32(&bar_q_free[t]));
      };
      while (ok && work.next(zh, qb)) {
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, q0, n_kv);
        const int n_max = max(n_kv[0], n_kv[1]);
        if (n_max == 0) continue;
        {
          const uint32_t slot0 = kv_it % T::kStages;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            ok = ok && mbar_wait_warp(smem_u32(&bar_q_full[t]), items & 1, &abort_word, 3) &&
                 mbar_wait_warp(smem_u32(&bar_kv_full[slot0]), (kv_it / T::kStages) & 1,
                                &abort_word, 4);
            if (!ok) break;
            tc_fence_after();
            first_qk(t, n_kv[t], slot0);
          }
          if (!ok) break;
          umma_commit_elect(smem_u32(&bar_kv_empty[slot0]));
        }
        for (int j = 0; ok && j < n_max; ++j) {
          const uint32_t it_v = kv_it + 2 * j + 1;
          const uint32_t slot_v = it_v % T::kStages;
          if (!mbar_wait_warp(smem_u32(&bar_kv_full[slot_v]), (it_v / T::kStages) & 1, &abort_word,
                              5)) {
            ok = false;
            break;
          }
          const bool have_next = (j + 1 < n_max);
          const uint32_t it_k = it_v + 1;
          const uint32_t slot_k = it_k % T::kStages;
          bool k_ready = false;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            if (j < n_kv[t]) {
              FMHA_TL(2, tl_base + j, t * 4 + 0);
              if (!mbar_wait_warp(smem_u32(&bar_p_full[t]), p_cnt[t] & 1, &abort_word, 6)) {
                ok = false;
                break;
              }
              ++p_cnt[t];
              // the first O_t += of an item overwrites O_t: the previous item's epilogue must
              // have read it out of tensor memory
              if (j == 0 && o_cnt[t] > 0 &&
                  !mbar_wait_warp(smem_u32(&bar_o_read[t]), (o_cnt[t] - 1) & 1, &abort_word, 7)) {
                ok = false;
                break;
              }
              tc_fence_after();
              FMHA_TL(2, tl_base + j, t * 4 + 1);
              issue_pv(t, ring_smem + slot_v * T::kTileBytes, j > 0);
              FMHA_TL(2, tl_base + j, t * 4 + 2);
              if (j + 1 < n_kv[t]) {
                if (!k_ready) {
                  if (!mbar_wait_warp(smem_u32(&bar_kv_full[slot_k]), (it_k / T::kStages) & 1,
                                      &abort_word, 8)) {
                    ok = false;
                    break;
                  }
                  tc_fence_after();
                  k_ready = true;
                }
                issue_qk(t, ring_smem + slot_k * T::kTileBytes);
                umma_commit_elect(smem_u32(&bar_s_full[t]));
                if (j + 2 == n_kv[t]) umma_commit_elect(smem_u32(&bar_q_free[t]));
              } else {
                umma_commit_elect(smem_u32(&bar_o_full[t]));
                ++o_cnt[t];
              }
              FMHA_TL(2, tl_base + j, t * 4 + 3);
            }
          }
          if (!ok) break;
          umma_commit_elect(smem_u32(&bar_kv_empty[slot_v]));
          if (have_next) umma_commit_elect(smem_u32(&bar_kv_empty[slot_k]));
        }
        kv_it += 2 * n_max;
        ++items;
        tl_base += 16;
      }
    }
  } else {
    // =========================== softmax / epilogue ===========================
    reg_alloc<kFwdRegsSoftmax>();
    // Two threads per query row (warps t*8 + hf*4 + quad: tile t, column half hf, TMEM lane
    // quadrant quad), each owning 64 of the 128 score columns.  One warp per scheduler issues at
    // most every other cycle; with two warps of the active tile on every scheduler the pass over
    // a tile is bound by the MUFU unit instead of by instruction issue.
    const int t = warp >> 3;         // query tile
    const int hf = (warp >> 2) & 1;  // column half of this thread
    const int quad = warp & 3;       // TMEM lane quadrant of this warp
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + t * 128 + hf * 64;          // my 64 score columns
    const uint32_t tP = tmem_base + lane_addr + t * 128 + hf * 32;          // my 32 packed P columns
    const uint32_t tO = tmem_base + lane_addr + 256 + t * D + hf * (D / 2); // my D/2 output columns
    const uint32_t o_stage = ostage_smem + t * T::kTileBytes;
    const uint32_t xch = smem_u32(&row_xch[t][row_in_tile]);  // fp32 view: row sums
    // 16-bit view of the same words: row references, one slot per thread of the row
    const uint32_t xch_mine = smem_u32(&row_xch[t][0]) + (hf * 128 + row_in_tile) * 2;
    const uint32_t xch_other = smem_u32(&row_xch[t][0]) + ((hf ^ 1) * 128 + row_in_tile) * 2;
    const uint32_t bar_id = 1 + t;               // named barrier of this tile's 256 threads
    const uint32_t pair_bar = 3 + t * 4 + quad;  // named barrier of the two warps sharing my rows
    bool stored = false;  // a TMA store of this tile may still be reading the staging tile
    const float c = p.scale_log2;
    // a masked score must give exp2(s * c - m * c) = 0 whatever the sign of c
    const float mask_val = (c >= 0.f) ? -CUDART_INF_F : CUDART_INF_F;
    const bool tl = (lane == 0 && quad == 0 && hf == 0);
    uint32_t s_cnt = 0;  // S_t tiles consumed so far (phase of s_full[t])
    uint32_t o_cnt = 0;  // O_t tiles read so far (phase of o_full[t])
    int tl_base = 0;     // timeline slot offset of the current item (debug builds)

    while (work.next(zh, qb)) {
      const int z = zh / p.heads, h = zh % p.heads;
      const int q0 = qb * (T::kBlockM * T::kTilesM);
      int n_kv[2];
      fwd_item_extent<D>(p, q0, n_kv);
      const int n = n_kv[t];
      const bool tile_valid = (q0 + t * T::kBlockM) < p.seqlen_q;
      const int row = q0 + t * T::kBlockM + row_in_tile;
      long long lim_ll = p.causal ? (long long)row + p.causal_shift : (long long)p.seqlen_k - 1;
      lim_ll = min(lim_ll, (long long)p.seqlen_k - 1);
      lim_ll = max(lim_ll, -1ll);
      const int row_limit = (int)lim_ll;  // last visible key of this row (-1 = none)

      float m_ref = mask_val;  // reference score of the running softmax (raw, unscaled)
      float l = 0.f;           // this thread's share of the running sum of exp2((s - m_ref) * c)

      for (int j = 0; j < n; ++j, ++s_cnt) {
        if (tl) FMHA_TL(t, tl_base + j, 0);
        // on a time-out keep going: every later wait returns at once, and all threads of the
        // tile still meet at the named barriers
        mbar_wait(smem_u32(&bar_s_full[t]), s_cnt & 1, &abort_word, 9);
        tc_fence_after();
        if (tl) FMHA_TL(t, tl_base + j, 1);
        uint32_t s[2][32];
        tmem_ld32(tS + 0, s[0]);
        tmem_ld32(tS + 32, s[1]);
        tmem_wait_ld();
        if (tl) FMHA_TL(t, tl_base + j, 2);

        // columns > lim of this tile are masked (lim counted within my 64 columns)
        const int lim = row_limit - j * T::kBlockN - hf * 64;
        if (lim < 63) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cc * 32 + i > lim) s[cc][i] = __float_as_uint(mask_val);
        }

        // extreme of my 64 scores: max when c >= 0, min when c < 0, so that m * c = max(s * c)
        float mx0 = __uint_as_float(s[0][0]), mx1 = __uint_as_float(s[1][0]);
        if (c >= 0.f) {
          mx0 = fmaxf(mx0, __uint_as_float(s[0][1]));
          mx1 = fmaxf(mx1, __uint_as_float(s[1][1]));
#pragma unroll
          for (int i = 2; i < 32; i += 2) {
            mx0 = max3(mx0, __uint_as_float(s[0][i]), __uint_as_float(s[0][i + 1]));
            mx1 = max3(mx1, __uint_as_float(s[1][i]), __uint_as_float(s[1][i + 1]));
          }
        } else {
          mx0 = fminf(mx0, __uint_as_float(s[0][1]));
          mx1 = fminf(mx1, __uint_as_float(s[1][1]));
#pragma unroll
          for (int i = 2; i < 32; i += 2) {
            mx0 = min3(mx0, __uint_as_float(s[0][i]), __uint_as_float(s[0][i + 1]));
            mx1 = min3(mx1, __uint_as_float(s[1][i]), __uint_as_float(s[1][i + 1]));
          }
        }
        float mx = (c >= 0.f) ? fmaxf(mx0, mx1) : fminf(mx0, mx1);
        // The row reference has to be the same number in both threads of the row, but not the
        // exact extreme: anything between the extreme and a little beyond it will do.  Each
        // thread rounds its value away from the scores to 16 bits, the two swap them through
        // shared memory, and both take the extreme of the same two numbers.
        // The barrier of the pair also orders half 0's tcgen05.ld of S columns 32..63 before
        // half 1 overwrites them with its packed P.  The slot is reused every tile: the partner
        // has read it before it arrives on p_full, which the next S tile is ordered after.
        {
          uint32_t b = __float_as_uint(mx);
          const bool grow = ((b >> 31) == 0u) == (c >= 0.f);  // larger magnitude = away
          b = (grow ? b + 0xffffu : b) & 0xffff0000u;
          asm volatile("st.shared.u16 [%0], %1;" ::"r"(xch_mine), "h"((uint16_t)(b >> 16))
                       : "memory");
          named_bar_sync(pair_bar, 64);
          uint16_t o16;
          asm volatile("ld.shared.u16 %0, [%1];" : "=h"(o16) : "r"(xch_other) : "memory");
          const float other = __uint_as_float((uint32_t)o16 << 16);
          mx = __uint_as_float(b);
          mx = (c >= 0.f) ? fmaxf(mx, other) : fminf(mx, other);
        }

        if (j == 0) {
          m_ref = mx;
        } else {
          const float m_new = (c >= 0.f) ? fmaxf(m_ref, mx) : fminf(m_ref, mx);
          // growth of the scaled maximum; NaN (inf - inf) compares false.  Both threads of a
          // row see the same numbers, and both half-warps hold the same rows: same decision.
          const bool need = (m_new - m_ref) * c > kRescaleThreshold;
          if (__any_sync(0xffffffffu, need)) {
            // O_t is idle here: S_t(j) is committed after O_t += P_t V_(j-1) was issued
            const float alpha = isinf(m_new) ? 1.f : fast_exp2((m_ref - m_new) * c);
            l *= alpha;
            m_ref = m_new;
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {  // my half of the output columns
              uint32_t o[16];
              tmem_ld16(tO + cc * 16, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st16(tO + cc * 16, o);
            }
          }
        }

        if (tl) FMHA_TL(t, tl_base + j, 3);
        const float neg_mc = isinf(m_ref) ? 0.f : -m_ref * c;
        const uint64_t c2 = pack2f(c, c), nm2 = pack2f(neg_mc, neg_mc);
        uint64_t la = pack2f(0.f, 0.f), lb = pack2f(0.f, 0.f);
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {  // 32 scores -> 16 packed columns of P at a time
          uint32_t pk[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x2 = fma2(pack2(s[cc][i], s[cc][i + 1]), c2, nm2);
            uint64_t p2;
            // kFwdPolyPairs of every 4 pairs go through the FMA pipe instead of the MUFU unit
            if (((i >> 1) & 3) < kFwdPolyPairs) {
              p2 = poly_exp2_pair(x2);
            } else {
              uint32_t x0, x1;
              unpack2(x2, x0, x1);
              p2 = pack2f(fast_exp2(__uint_as_float(x0)), fast_exp2(__uint_as_float(x1)));
            }
            if (i & 2) lb = add2(lb, p2); else la = add2(la, p2);
            uint32_t p0, p1;
            unpack2(p2, p0, p1);
            pk[i >> 1] = pack_half2(__uint_as_float(p0), __uint_as_float(p1));
          }
          tmem_st16(tP + cc * 16, pk);
        }
        {
          uint32_t a0, a1;
          unpack2(add2(la, lb), a0, a1);
          l += __uint_as_float(a0) + __uint_as_float(a1);
        }
        if (tl) FMHA_TL(t, tl_base + j, 4);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_p_full[t]));
        if (tl) FMHA_TL(t, tl_base + j, 5);
      }
      if (tl) FMHA_TL(t, tl_base + 15, 6);

      // ---- epilogue: my half of O_t / l -> fp16 registers (tensor memory released) ->
      //      staging tile -> TMA store; LSE
      if (tile_valid) {
        if (n > 0) {
          // O_t complete.  It also tells that every thread of the tile is through its last
          // exchange of row references, whose 16-bit slots the row sums below reuse.
          mbar_wait(smem_u32(&bar_o_full[t]), o_cnt & 1, &abort_word, 10);
          ++o_cnt;
          tc_fence_after();
          if (tl) FMHA_TL(t, tl_base + 15, 8);
        }
        // the row sum: half 1 hands its share to half 0, which hands the total back
        if (hf == 1) asm volatile("st.shared.f32 [%0], %1;" ::"r"(xch), "f"(l) : "memory");
        named_bar_sync(bar_id, 256);
        if (hf == 0) {
          float other;
          asm volatile("ld.shared.f32 %0, [%1];" : "=f"(other) : "r"(xch) : "memory");
          l += other;
          asm volatile("st.shared.f32 [%0], %1;" ::"r"(xch), "f"(l) : "memory");
        }
        named_bar_sync(bar_id, 256);
        if (hf == 1) asm volatile("ld.shared.f32 %0, [%1];" : "=f"(l) : "r"(xch) : "memory");

        uint32_t oh[D / 4];  // my half of the output row, fp16 pairs
        if (n > 0) {
          const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
#pragma unroll
          for (int cc = 0; cc < D / 64; ++cc) {  // 32 columns at a time keeps the registers low
            uint32_t o[32];
            tmem_ld32(tO + cc * 32, o);
            tmem_wait_ld();
            if (cc == D / 64 - 1) {  // O_t is in registers: the next item may overwrite it
              tc_fence_before();
              mbar_arrive(smem_u32(&bar_o_read[t]));
              if (tl) FMHA_TL(t, tl_base + 15, 9);
            }
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              oh[cc * 16 + (i >> 1)] = pack_half2(__uint_as_float(o[i]) * inv_l,
                                                  __uint_as_float(o[i + 1]) * inv_l);
          }
        } else {
#pragma unroll
          for (int i = 0; i < D / 4; ++i) oh[i] = 0u;
        }
        if (hf == 0 && row < p.seqlen_q) {
          const float lse =
              (l > 0.f) ? (m_ref * c + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
          p.lse[((size_t)z * p.heads + h) * p.seqlen_q + row] = lse;
        }
        // through the staging tile and TMA stores (per-thread stores of whole rows are
        // uncoalesced and clog the load/store pipe for everybody)
        if (row_in_tile == 0 && hf == 0 && stored) tma_wait_group_read<0>();  // previous item
        named_bar_sync(bar_id, 256);
#pragma unroll
        for (int ch = 0; ch < D / 16; ++ch) {  // my 16-byte chunks (8 fp16 each)
          const int gch = hf * (D / 16) + ch;  // chunk index within the whole row
          sts128(o_stage + (gch >> 3) * T::kBoxBytes + row_in_tile * 128 +
                     (((gch & 7) ^ (row_in_tile & 7)) << 4),
                 oh[ch * 4 + 0], oh[ch * 4 + 1], oh[ch * 4 + 2], oh[ch * 4 + 3]);
        }
        fence_proxy_async_smem();
        named_bar_sync(bar_id, 256);
        if (row_in_tile == 0 && hf == 0) {
#pragma unroll
          for (int b = 0; b < T::kBoxes; ++b)
            tma_store_4d(&tm_o, o_stage + b * T::kBoxBytes, b * 64, q0 + t * T::kBlockM, h, z);
          tma_commit_group();
        }
        stored = true;
      }
      if (tl) FMHA_TL(t, tl_base + 15, 7);
      tl_base += 16;
    }
    if (row_in_tile == 0 && hf == 0) tma_wait_group<0>();
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (abort_word != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, abort_word);
    // let copies that may still be in flight land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace fmha
