// Forward attention kernel for sm_100a: O = softmax(scale * Q K^T [+ mask]) V, LSE.
//
// Replaces fused_mha_forward_kernel of the reference (kernel/fused_mha_kernel.cu:20-323):
// same mathematics (online softmax over KV tiles, running max / sum, O rescale), none of its
// structure.  The kernel is PERSISTENT: one CTA per SM walks a list of work items; a work item
// is 256 query rows (two 128-row tiles) of one (batch, head), processed against the KV sequence
// in 128-row tiles, each consumed in two 64-row halves ("steps"):
//
//   warp 8      TMA producer for K and V, in half tiles of 64 rows, through a ring of
//               shared-memory slots (full / empty mbarriers per slot); a slot holds what one
//               step consumes, V(h) and K(h+2); runs ahead into the next item as slots free
//   warp 10     TMA producer for the two Q tiles of an item, as soon as the previous item's
//               last S = Q K^T has released them
//   warps 9, 11 MMA issuers, one per query tile t: S_t(h) = Q_t K(h)^T (128 x 64, both operands
//               in shared memory) and O_t += P_t(h) V(h) (P_t read from tensor memory),
//               accumulators in tensor memory.  The whole warp runs the loop so that
//               descriptors stay in uniform registers; one elected lane issues.  Two issuers
//               because the tensor pipe queues very little: with one, every barrier wait
//               between two blocks of MMAs let the pipe run dry.
//   warps 0-3   softmax of query tile 0: one thread per row, S_0(h) read with tcgen05.ld,
//               online exp2 softmax, P_0(h) written back over S_0(h) as fp16, lazy O_0
//               rescale, epilogue
//   warps 4-7   the same for query tile 1
//
// S_t is double buffered in tensor memory: while the softmax group works on S_t(h), the tensor
// pipe already holds or computes S_t(h+1), so the group never waits for the latency of an MMA
// round trip, and the MMA warps only ever wait for P.  The price is N = 64 per S MMA, which the
// tensor pipe runs at 3/4 of the rate of N = 128.
//
// While the groups run an item's epilogue the producer and the MMA warp already start the next
// item (its Q / K loads and first S = Q K^T), so that the load latency at the head of an item
// and the store at its tail are hidden.
//
// Element type: fp16 (the reference's only type, kernel/fused_mha_api.cpp:25-29) or bf16
// (kBf16): the tensor cores take either by two bits of the instruction descriptor; P and O are
// then rounded to bf16 instead of fp16, everything in between stays fp32.
//
// Tensor memory (512 columns): S_t buffer b at [t * 128 + b * 64, + 64); O_0 [256, 256 + D),
// O_1 [256 + D, 256 + 2 D); P_t(h) aliases the first 32 columns of the S_t buffer it came from
// (two fp16 per 32-bit column).
//
// Shared memory: rows of 64 fp16 (128 bytes) in the TMA / UMMA 128-byte swizzle.  A 128 x D
// tile is D/64 boxes of 128 x 64, box b at byte offset b * 16384 (a 64-row half tile of K or V:
// boxes of 64 x 64, 8192 bytes apart).  Per softmax group one extra tile stages the output for
// the TMA store.
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
  // optional per-batch lengths (right-padded batches): rows >= seqused_q[z] and keys >=
  // seqused_k[z] are padding, skipped tile-wise and masked inside partial tiles
  const int* seqused_q;
  const int* seqused_k;
  // debug builds (-DFMHA_TIMELINE) only: clock64 stamps of one CTA, see FMHA_TL
  long long* timeline;
  int timeline_block;
};

#ifndef FMHA_ABLATE
#define FMHA_ABLATE 0  // debug builds: bit 0 no exp2, bit 1 no row max, bit 2 no P store
#endif

// pairs out of every 4 whose exponential is a polynomial on the FMA pipe (the rest use MUFU),
// for head_dim 128 and for head_dim 64
#ifndef FMHA_FWD_POLY_PAIRS
#define FMHA_FWD_POLY_PAIRS 0
#endif
#ifndef FMHA_FWD_POLY_PAIRS_D64
#define FMHA_FWD_POLY_PAIRS_D64 0
#endif

template <int D, bool kBf16 = false>
struct FwdTraits {
  static constexpr int kBlockM = 128;  // rows per query tile
  static constexpr int kTilesM = 2;    // query tiles per work item
  static constexpr int kBlockN = 128;  // rows per KV tile (one TMA load)
  static constexpr int kStepN = 64;    // KV rows per S = Q K^T / softmax / O += P V step
  static constexpr int kBoxes = D / 64;
  static constexpr int kBoxBytes = 128 * 128;  // 128 rows x 128 bytes
  static constexpr int kTileBytes = kBoxes * kBoxBytes;
  // K and V travel in half tiles of kStepN rows: the same shared memory holds twice as many
  // ring slots, each released as soon as its step is done, so loads run several steps ahead
  static constexpr int kHalfBoxBytes = kStepN * 128;  // 64 rows x 128 bytes
  static constexpr int kHalfTileBytes = kBoxes * kHalfBoxBytes;
  // a ring slot holds the two half tiles one step consumes: V(h) and K(h+2) (one barrier pair
  // and one release per step); the slot of an item's head holds K(0) and K(1)
  static constexpr int kSlotBytes = 2 * kHalfTileBytes;
  static constexpr int kStages = (D == 128) ? 3 : 6;
  static constexpr int kThreads = 384;  // softmax 0, softmax 1, {TMA, MMA, 2 idle} warpgroups
  // Q tiles, K/V ring, one output staging tile per softmax group
  static constexpr int kSmemBytes = 1024 + (kTilesM + 2) * kTileBytes + kStages * kSlotBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kPolyPairs = (D == 64) ? FMHA_FWD_POLY_PAIRS_D64 : FMHA_FWD_POLY_PAIRS;
  static constexpr uint32_t kIdescQK = umma_idesc_f16(128, kStepN, 0, 0, kBf16);
  static constexpr uint32_t kIdescPV = umma_idesc_f16(128, D, 0, 1, kBf16);
};

constexpr int kFwdRegsIssue = 88;                                 // warps 8-11
constexpr int kFwdRegsSoftmax = 168 + (168 - kFwdRegsIssue) / 2;  // warps 0-7: 208
static_assert(kFwdRegsIssue <= 168 && kFwdRegsSoftmax >= 168 && kFwdRegsSoftmax % 8 == 0,
              "setmaxnreg.dec must not raise and .inc must not lower the 168 registers of the launch");

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

// the lengths that count for batch entry z: the tensors' own, or the caller's per-batch ones
__device__ __forceinline__ void fwd_lengths(const FwdKernelParams& p, int z, int& sq, int& sk) {
  sq = p.seqused_q == nullptr ? p.seqlen_q : max(0, min(p.seqlen_q, __ldg(p.seqused_q + z)));
  sk = p.seqused_k == nullptr ? p.seqlen_k : max(0, min(p.seqlen_k, __ldg(p.seqused_k + z)));
}

// KV tiles each of the two query tiles of an item has to visit (0 = none)
template <int D>
__device__ __forceinline__ void fwd_item_extent(const FwdKernelParams& p, int z, int q0,
                                                int (&n_kv)[2]) {
  using T = FwdTraits<D>;
  int sq, sk;
  fwd_lengths(p, z, sq, sk);
  const int nk_total = (sk + T::kBlockN - 1) / T::kBlockN;
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int r0 = q0 + t * T::kBlockM;
    if (r0 >= sq) {
      n_kv[t] = 0;
    } else if (!p.causal) {
      n_kv[t] = nk_total;
    } else {
      const int r_last = min(r0 + T::kBlockM - 1, sq - 1);
      const long long lim = (long long)r_last + p.causal_shift;
      n_kv[t] = lim < 0 ? 0 : (int)min((long long)nk_total, lim / T::kBlockN + 1);
    }
  }
}

template <int D, bool kBf16 = false>
__global__ void __launch_bounds__(384, 1)
    fmha_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                    const FwdKernelParams p) {
  using T = FwdTraits<D, kBf16>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_q_full[2];   // Q_t of the current item has landed
  __shared__ uint64_t bar_q_free[2];   // the last S_t = Q_t K^T of the item is done: Q_t reusable
  __shared__ uint64_t bar_kv_full[T::kStages];
  __shared__ uint64_t bar_kv_empty[T::kStages];
  __shared__ uint64_t bar_s_full[2][2];  // [tile][buffer]
  __shared__ uint64_t bar_pv_done[2];    // one of the last two O_t += of an item has completed
  // One barrier per S/P buffer: a softmax warp may be a step ahead of its neighbours, and its
  // arrival for step h+1 must not be counted towards step h.  Per buffer that cannot happen:
  // the buffer's next S only exists after everybody's P of this step has been consumed.
  __shared__ uint64_t bar_p_full[2][2];  // [tile][buffer]
  __shared__ uint64_t bar_o_full[2];
  __shared__ uint64_t bar_o_read[2];   // the softmax group has O_t in registers: O_t reusable
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
  const uint32_t ostage_smem = ring_smem + T::kStages * T::kSlotBytes;  // 2 output tiles

  // ---- set-up: barriers (thread 0), tensor memory (warp 9)
  if (threadIdx.x == 0) {
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(smem_u32(&bar_kv_full[s]), 1);
      mbar_init(smem_u32(&bar_kv_empty[s]), 2);  // one release by each MMA warp
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(smem_u32(&bar_q_full[t]), 1);
      mbar_init(smem_u32(&bar_q_free[t]), 1);
      mbar_init(smem_u32(&bar_s_full[t][0]), 1);
      mbar_init(smem_u32(&bar_s_full[t][1]), 1);
      mbar_init(smem_u32(&bar_pv_done[t]), 1);
      // one arrival per softmax warp: 128 arrivals on one word are 128 serialised atomics
      mbar_init(smem_u32(&bar_p_full[t][0]), 4);
      mbar_init(smem_u32(&bar_p_full[t][1]), 4);
      mbar_init(smem_u32(&bar_o_full[t]), 1);
      mbar_init(smem_u32(&bar_o_read[t]), 4);
    }
    fence_barrier_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(&tmem_base_slot), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  FwdWorkIter work(blockIdx.x, gridDim.x, p.num_q_blocks, p.num_heads_total);
  int zh, qb;

  // Register budget: 384 threads leave 168 per thread.  The producer / MMA warpgroup hands part
  // of its share to the softmax warpgroups, whose threads hold a 128-column row of S.  Each
  // setmaxnreg sits at the top of its warpgroup's own branch.
  if (warp >= 8) {
    reg_dealloc<kFwdRegsIssue>();
    if (warp == 8) {
      // =========================== TMA producer (converged warp, elected issue) ==========
      if (elect_one()) {
        tma_prefetch_desc(&tm_q);
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
      }
      __syncwarp();
      uint32_t kv_it = 0;  // ring slots loaded so far (slot index and phase)
      bool ok = true;
      while (ok && work.next(zh, qb)) {
        const int z = zh / p.heads, h = zh % p.heads;
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, z, q0, n_kv);
        // slot loads in the order the MMA warps consume them:
        //   [K(0) K(1)]  [V(0) K(2)]  [V(1) K(3)]  ...  [V(nh-3) K(nh-1)]  [V(nh-2)]  [V(nh-1)]
        const int nh = 2 * max(n_kv[0], n_kv[1]);
        const int n_loads = nh > 0 ? nh + 1 : 0;
        for (int it = 0; it < n_loads; ++it, ++kv_it) {
          const uint32_t slot = kv_it % T::kStages;
          const uint32_t round = kv_it / T::kStages;
          if (round > 0 &&
              !mbar_wait_warp(smem_u32(&bar_kv_empty[slot]), (round - 1) & 1, &abort_word, 2)) {
            ok = false;
            break;
          }
          // first and second half tile of the slot (-1 = none)
          const int k_first = (it == 0) ? 0 : -1;               // K half in the first place
          const int v_first = (it == 0) ? -1 : it - 1;          // V(h), h = it - 1
          const int k_second = (it == 0) ? 1 : (it + 1 < nh ? it + 1 : -1);  // K(h+2)
          if (elect_one()) {
            const uint32_t fbar = smem_u32(&bar_kv_full[slot]);
            const uint32_t base = ring_smem + slot * T::kSlotBytes;
            mbar_arrive_expect_tx(fbar, (k_second >= 0 ? 2 : 1) * T::kHalfTileBytes);
#pragma unroll
            for (int b = 0; b < T::kBoxes; ++b) {
              if (k_first >= 0)
                tma_load_4d(base + b * T::kHalfBoxBytes, &tm_k, fbar, b * 64, k_first * T::kStepN, h, z);
              else
                tma_load_4d(base + b * T::kHalfBoxBytes, &tm_v, fbar, b * 64, v_first * T::kStepN, h, z);
              if (k_second >= 0)
                tma_load_4d(base + T::kHalfTileBytes + b * T::kHalfBoxBytes, &tm_k, fbar, b * 64,
                            k_second * T::kStepN, h, z);
            }
          }
          __syncwarp();
        }
      }
    } else if (warp == 10) {
      // =========================== Q producer ===========================
      // its own warp, so that waiting for the Q buffers of the running item never holds back
      // the K/V prefetch of the next one
      uint32_t items = 0;  // items with work seen so far (phase of the Q barriers)
      bool ok = true;
      while (ok && work.next(zh, qb)) {
        const int z = zh / p.heads, h = zh % p.heads;
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, z, q0, n_kv);
        if (max(n_kv[0], n_kv[1]) == 0) continue;
#pragma unroll
        for (int t = 0; t < T::kTilesM; ++t) {
          if (items > 0 &&
              !mbar_wait_warp(smem_u32(&bar_q_free[t]), (items - 1) & 1, &abort_word, 1)) {
            ok = false;
            break;
          }
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
    } else if (warp == 9 || warp == 11) {
      // =========================== MMA issuers, one warp per query tile ===================
      // Two issuers, because the tensor pipe queues very little: whenever a single issuer sat in
      // a barrier wait between two blocks of MMAs the pipe ran dry.  With one warp per tile the
      // other warp's MMAs fill those gaps.
      // (converged warp, elected issue)
      // All 32 lanes run the loop so that addresses and descriptors live in uniform registers;
      // a loop run by one lane only makes every operand a per-thread value that has to be moved
      // to a uniform register before each tcgen05.mma, and the issue rate falls below the
      // tensor pipe's 64 cycles per 128x128x16 MMA.
      const uint32_t q_lo0 = umma_desc_lo(q_smem, kLboKMajor);
      // S_t buffer `buf` = Q_t K(h)^T, K(h) = the half tile at k_addr
      auto issue_qk = [&](int t, int buf, uint32_t k_addr) {
        const uint32_t d = tmem_base + t * 128 + buf * T::kStepN;
        const uint32_t a_lo = q_lo0 + ((t * T::kTileBytes) >> 4);
        const uint32_t b_lo = umma_desc_lo(k_addr, kLboKMajor);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t a_off = ((ks >> 2) * T::kBoxBytes + (ks & 3) * 32) >> 4;
          const uint32_t b_off = ((ks >> 2) * T::kHalfBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss_elect(d, a_lo + a_off, b_lo + b_off, T::kIdescQK, ks > 0 ? 1u : 0u);
        }
      };
      // O_t (+)= P_t (in S_t buffer `buf`) V(h), V(h) = the half tile at v_addr; its 64-column
      // boxes are kHalfBoxBytes apart
      auto issue_pv = [&](int t, int buf, uint32_t v_addr, bool accumulate) {
        const uint32_t d = tmem_base + 256 + t * D;
        const uint32_t a = tmem_base + t * 128 + buf * T::kStepN;
        const uint32_t b_lo = umma_desc_lo(v_addr, T::kHalfBoxBytes);
#pragma unroll
        for (int ks = 0; ks < T::kStepN / 16; ++ks)
          umma_ts_elect(d, a + ks * 8, b_lo + ((ks * 2048) >> 4), T::kIdescPV,
                        (accumulate || ks > 0) ? 1u : 0u);
      };
      auto kv_addr = [&](uint32_t it) { return ring_smem + (it % T::kStages) * T::kSlotBytes; };
      auto kv_wait = [&](uint32_t it, int who) {
        return mbar_wait_warp(smem_u32(&bar_kv_full[it % T::kStages]), (it / T::kStages) & 1,
                              &abort_word, who);
      };
      auto kv_release = [&](uint32_t it) {
        umma_commit_elect(smem_u32(&bar_kv_empty[it % T::kStages]));
      };
      const int t = (warp == 9) ? 0 : 1;  // the query tile this warp issues for
      uint32_t items = 0, kv_it = 0;  // kv_it: ring slots consumed before this item
      int tl_base = 0;     // timeline slot offset of the current item (debug builds)
      uint32_t p_cnt = 0;  // P_t steps consumed so far (even at item boundaries)
      uint32_t o_cnt = 0;  // items in which tile t produced an O_t (phase of o_read[t])
      bool ok = true;
      while (ok && work.next(zh, qb)) {
        const int q0 = qb * (T::kBlockM * T::kTilesM);
        int n_kv[2];
        fwd_item_extent<D>(p, zh / p.heads, q0, n_kv);
        const int n_max = max(n_kv[0], n_kv[1]);
        if (n_max == 0) continue;
        const int nh = 2 * n_kv[t];  // steps of this tile
        const int nhm = 2 * n_max;   // steps of the item (the K/V ring serves both tiles)
        {
          // the first two S_t of the item, one per buffer, from K(0) and K(1) in the head slot
          ok = ok && mbar_wait_warp(smem_u32(&bar_q_full[t]), items & 1, &abort_word, 3) &&
               kv_wait(kv_it, 4);
          if (!ok) break;
          tc_fence_after();
          if (nh > 0) {
#pragma unroll
            for (int b = 0; b < 2; ++b) {
              issue_qk(t, b, kv_addr(kv_it) + b * T::kHalfTileBytes);
              umma_commit_elect(smem_u32(&bar_s_full[t][b]));
            }
          }
          // with at most one KV tile these were the item's last uses of Q_t
          if (nh <= 2) umma_commit_elect(smem_u32(&bar_q_free[t]));
          kv_release(kv_it);
        }
        for (int h = 0; ok && h < nhm; ++h) {
          const int buf = h & 1;
          const uint32_t it_s = kv_it + 1 + h;  // the slot with V(h) and K(h+2)
          // The step's two waits (its slot, P_t(h)) with both probes in flight together; when
          // both are ready, as they normally are, the bounded waits below are skipped.  A slot
          // is only released after it was seen full, used or not: otherwise this warp could
          // release the same slot twice within one round of the ring.
          const uint32_t bs = smem_u32(&bar_kv_full[it_s % T::kStages]);
          const uint32_t ps = (it_s / T::kStages) & 1;
          const bool use_p = h < nh;
          const uint32_t bp = use_p ? smem_u32(&bar_p_full[t][buf]) : bs;
          const uint32_t pp = use_p ? ((p_cnt >> 1) & 1) : ps;
          const bool all_ready = __all_sync(0xffffffffu, mbar_try_wait3(bs, ps, bp, pp, bs, ps));
          if (!all_ready && !kv_wait(it_s, 5)) {
            ok = false;
            break;
          }
          if (h < nh) {
            FMHA_TL(2, tl_base + h, t * 4 + 0);
            if (!all_ready &&
                !mbar_wait_warp(smem_u32(&bar_p_full[t][buf]), (p_cnt >> 1) & 1, &abort_word, 6)) {
              ok = false;
              break;
            }
            ++p_cnt;
            // the first O_t += of an item overwrites O_t: the previous item's epilogue must
            // have read it out of tensor memory
            if (h == 0 && o_cnt > 0 &&
                !mbar_wait_warp(smem_u32(&bar_o_read[t]), (o_cnt - 1) & 1, &abort_word, 7)) {
              ok = false;
              break;
            }
            tc_fence_after();
            FMHA_TL(2, tl_base + h, t * 4 + 1);
            issue_pv(t, buf, kv_addr(it_s), h > 0);
            FMHA_TL(2, tl_base + h, t * 4 + 2);
            if (h + 2 < nh) {
              // S_t(h+2) goes where P_t(h) was; the tensor pipe runs one warp's MMAs in order.
              // Its commit also tells the softmax group that O_t += P_t(h) V(h) is complete.
              issue_qk(t, buf, kv_addr(it_s) + T::kHalfTileBytes);
              umma_commit_elect(smem_u32(&bar_s_full[t][buf]));
              if (h + 3 == nh) umma_commit_elect(smem_u32(&bar_q_free[t]));
            } else {
              // no S follows: the completion of this O_t += gets a barrier of its own
              umma_commit_elect(smem_u32(&bar_pv_done[t]));
              if (h + 1 == nh) {
                umma_commit_elect(smem_u32(&bar_o_full[t]));
                ++o_cnt;
              }
            }
            FMHA_TL(2, tl_base + h, t * 4 + 3);
          }
          kv_release(it_s);
        }
        kv_it += nhm + 1;
        ++items;
        tl_base += 64;
      }
    }
  } else {
    // =========================== softmax / epilogue ===========================
    reg_alloc<kFwdRegsSoftmax>();
    const int t = warp >> 2;    // query tile of this warpgroup
    const int quad = warp & 3;  // TMEM lane quadrant of this warp
    const int row_in_tile = quad * 32 + lane;
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const uint32_t tS = tmem_base + lane_addr + t * 128;
    const uint32_t tO = tmem_base + lane_addr + 256 + t * D;
    const uint32_t o_stage = ostage_smem + t * T::kTileBytes;
    bool stored = false;  // a TMA store of this group may still be reading the staging box
    const float c = p.scale_log2;
    // a masked score must give exp2(s * c - m * c) = 0 whatever the sign of c
    const float mask_val = (c >= 0.f) ? -CUDART_INF_F : CUDART_INF_F;
    const bool tl = (lane == 0 && quad == 0);
    uint32_t step = 0;    // steps of this tile so far, over all items (even at item boundaries)
    uint32_t o_cnt = 0;   // O_t tiles read so far (phase of o_full[t])
    int tl_base = 0;      // timeline slot offset of the current item (debug builds)

    while (work.next(zh, qb)) {
      const int z = zh / p.heads, h = zh % p.heads;
      const int q0 = qb * (T::kBlockM * T::kTilesM);
      int n_kv[2];
      fwd_item_extent<D>(p, z, q0, n_kv);
      int sq, sk;
      fwd_lengths(p, z, sq, sk);
      const int n = n_kv[t];
      const bool tile_valid = (q0 + t * T::kBlockM) < p.seqlen_q;
      const int row = q0 + t * T::kBlockM + row_in_tile;
      long long lim_ll = p.causal ? (long long)row + p.causal_shift : (long long)sk - 1;
      lim_ll = min(lim_ll, (long long)sk - 1);
      if (row >= sq) lim_ll = -1;  // a padding row sees nothing: O = 0, LSE = -inf
      lim_ll = max(lim_ll, -1ll);
      const int row_limit = (int)lim_ll;  // last visible key of this row (-1 = none)

      float m_ref = mask_val;  // reference score of the running softmax (raw, unscaled)
      float l = 0.f;           // running sum of exp2((s - m_ref) * c)

      for (int hs = 0; hs < 2 * n; ++hs, ++step) {
        const uint32_t buf = step & 1;  // == hs & 1
        const uint32_t tSb = tS + buf * T::kStepN;
        if (tl) FMHA_TL(t, tl_base + hs, 0);
        // on a time-out keep going: every later wait returns at once, and all 128 threads of
        // the group still meet at the named barriers of the epilogue
        mbar_wait(smem_u32(&bar_s_full[t][buf]), (step >> 1) & 1, &abort_word, 9);
        tc_fence_after();
        if (tl) FMHA_TL(t, tl_base + hs, 1);
        uint32_t s[2][32];
        tmem_ld32(tSb + 0, s[0]);
        tmem_ld32(tSb + 32, s[1]);
        tmem_wait_ld();
        if (tl) FMHA_TL(t, tl_base + hs, 2);

        const int lim = row_limit - hs * T::kStepN;  // columns > lim of this step are masked
        if (lim < T::kStepN - 1) {
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (cc * 32 + i > lim) s[cc][i] = __float_as_uint(mask_val);
        }

        // row extreme: max of s when c >= 0, min when c < 0, so that m * c = max(s * c)
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
        if (FMHA_ABLATE & 2) mx = __uint_as_float(s[0][0]);

        if (hs == 0) {
          m_ref = mx;
        } else {
          const float m_new = (c >= 0.f) ? fmaxf(m_ref, mx) : fminf(m_ref, mx);
          // growth of the scaled maximum; NaN (inf - inf) compares false
          const bool need = (m_new - m_ref) * c > kRescaleThreshold;
          const bool any_need = __any_sync(0xffffffffu, need);
#ifdef FMHA_COUNT_RESCALE
          // debug builds: how often a warp takes the rescale path (word 0), per warp-step (word 1)
          if (lane == 0 && p.timeline != nullptr) {
            atomicAdd(reinterpret_cast<unsigned long long*>(p.timeline) + 1, 1ull);
            if (any_need) atomicAdd(reinterpret_cast<unsigned long long*>(p.timeline), 1ull);
          }
#endif
          if (any_need) {
            // O_t may still be accumulating the previous step: wait for that MMA.  The next
            // one is not issued before this thread has arrived on p_full.
            // That is known from the commit of S_t(hs+1), issued right behind it, or, for
            // the last step of an item (no S follows the last two O_t +=, which complete
            // bar_pv_done twice per item), from the first of those two completions.
            if (hs + 1 < 2 * n)
              mbar_wait(smem_u32(&bar_s_full[t][buf ^ 1]), ((step + 1) >> 1) & 1, &abort_word, 11);
            else
              mbar_wait(smem_u32(&bar_pv_done[t]), 0, &abort_word, 11);
            tc_fence_after();
            const float alpha = isinf(m_new) ? 1.f : fast_exp2((m_ref - m_new) * c);
            l *= alpha;
            m_ref = m_new;
#pragma unroll
            for (int cc = 0; cc < D / 32; ++cc) {
              uint32_t o[32];
              tmem_ld32(tO + cc * 32, o);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(tO + cc * 32, o);
            }
          }
        }

        if (tl) FMHA_TL(t, tl_base + hs, 3);
        const float neg_mc = isinf(m_ref) ? 0.f : -m_ref * c;
        const uint64_t c2 = pack2f(c, c), nm2 = pack2f(neg_mc, neg_mc);
        uint64_t la = pack2f(0.f, 0.f), lb = pack2f(0.f, 0.f);
        uint32_t pk[32];  // 64 scores -> 32 packed columns of P
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x2 = fma2(pack2(s[cc][i], s[cc][i + 1]), c2, nm2);
            uint64_t p2;
            // kPolyPairs of every 4 pairs go through the FMA pipe instead of the MUFU unit
            if (((i >> 1) & 3) < T::kPolyPairs) {
              p2 = poly_exp2_pair(x2);
            } else {
              uint32_t x0, x1;
              unpack2(x2, x0, x1);
              p2 = pack2f(fast_exp2(__uint_as_float(x0)), fast_exp2(__uint_as_float(x1)));
            }
            if (i & 2) lb = add2(lb, p2); else la = add2(la, p2);
            uint32_t p0, p1;
            unpack2(p2, p0, p1);
            pk[cc * 16 + (i >> 1)] = pack16x2<kBf16>(__uint_as_float(p0), __uint_as_float(p1));
          }
        }
        if (!(FMHA_ABLATE & 4)) tmem_st32(tSb, pk);
        {
          uint32_t a0, a1;
          unpack2(add2(la, lb), a0, a1);
          l += __uint_as_float(a0) + __uint_as_float(a1);
        }
        if (tl) FMHA_TL(t, tl_base + hs, 4);
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&bar_p_full[t][buf]));
        if (tl) FMHA_TL(t, tl_base + hs, 5);
      }
      if (tl) FMHA_TL(t, tl_base + 31, 6);

      // ---- epilogue: O_t / l -> fp16 registers (tensor memory released) -> staging box -> TMA
      //      store; LSE
      if (tile_valid) {
        uint32_t oh[D / 2];  // the output row, fp16 pairs
        if (n > 0) {
          mbar_wait(smem_u32(&bar_o_full[t]), o_cnt & 1, &abort_word, 10);
          ++o_cnt;
          tc_fence_after();
          if (tl) FMHA_TL(t, tl_base + 31, 8);
          const float inv_l = (l > 0.f) ? 1.f / l : 0.f;
          uint32_t o[D / 32][32];
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(tO + cc * 32, o[cc]);
          tmem_wait_ld();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&bar_o_read[t]));
          if (tl) FMHA_TL(t, tl_base + 31, 9);
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc)
#pragma unroll
            for (int i = 0; i < 32; i += 2)
              oh[cc * 16 + (i >> 1)] = pack16x2<kBf16>(__uint_as_float(o[cc][i]) * inv_l,
                                                       __uint_as_float(o[cc][i + 1]) * inv_l);
        } else {
#pragma unroll
          for (int i = 0; i < D / 2; ++i) oh[i] = 0u;
        }
        if (row < p.seqlen_q) {
          const float lse =
              (l > 0.f) ? (m_ref * c + log2f(l)) * 0.6931471805599453f : -CUDART_INF_F;
          p.lse[((size_t)z * p.heads + h) * p.seqlen_q + row] = lse;
        }
        // through this group's staging tile and TMA stores (per-thread stores of whole rows are
        // uncoalesced and clog the load/store pipe for everybody)
        if (row_in_tile == 0 && stored) tma_wait_group_read<0>();  // previous item's store
        named_bar_sync(1 + t, 128);
#pragma unroll
        for (int ch = 0; ch < D / 8; ++ch)  // 16-byte chunk (8 fp16) of this row
          sts128(o_stage + (ch >> 3) * T::kBoxBytes + row_in_tile * 128 +
                     (((ch & 7) ^ (row_in_tile & 7)) << 4),
                 oh[ch * 4 + 0], oh[ch * 4 + 1], oh[ch * 4 + 2], oh[ch * 4 + 3]);
        fence_proxy_async_smem();
        named_bar_sync(1 + t, 128);
        if (row_in_tile == 0) {
#pragma unroll
          for (int b = 0; b < T::kBoxes; ++b)
            tma_store_4d(&tm_o, o_stage + b * T::kBoxBytes, b * 64, q0 + t * T::kBlockM, h, z);
          tma_commit_group();
        }
        stored = true;
      }
      if (tl) FMHA_TL(t, tl_base + 31, 7);
      tl_base += 64;
    }
    if (row_in_tile == 0) tma_wait_group<0>();
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (abort_word != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, abort_word);
    // let copies that may still be in flight land before the shared memory is released
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace fmha
