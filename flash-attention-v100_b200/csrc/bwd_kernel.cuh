// Backward attention kernel for sm_100a: fused dK / dV / dQ.
//
// Replaces fused_mha_backward_kernel of the reference (kernel/fused_mha_kernel.cu:325-735):
// the same identities  P = exp(scale*S - lse),  dV = P^T dO,  dP = dO V^T,
// dS = P o (dP - D) * scale,  dQ = dS K,  dK = dS^T Q  (kernel/fused_mha_kernel.cu:453-458,
// 503-506), with dQ accumulated in fp32 instead of the reference's fp16 atomics (:543,693).
//
// One CTA owns one 128-row KV tile of one (batch, head) and walks the query tiles (128 rows)
// that can see it.  Everything is computed TRANSPOSED so that the KV rows sit on the 128
// tensor-memory lanes, which lets P^T feed the dV MMA straight from tensor memory:
//
//   S^T  = K  Q_i^T    (A = K  smem K-major,  B = Q_i  smem K-major)      -> TMEM [0,128)
//   dP^T = V  dO_i^T   (A = V  smem K-major,  B = dO_i smem K-major)      -> TMEM [128,256)
//   dV  += P^T dO_i    (A = P^T TMEM fp16 over S^T, B = dO_i smem MN-major)-> TMEM [256+D, ..)
//                      (P^T columns [0,32) and [64,96): one 32-column block per compute group)
//   dK  += dS^T Q_i    (A = dS^T smem K-major, B = Q_i smem MN-major)      -> TMEM [256, 256+D)
//   dQ_i = dS  K       (A = dS^T smem read MN-major, B = K smem MN-major)  -> TMEM [128,128+D)
//                      (aliases dP^T, which is dead once dS^T is in shared memory)
//
//   warps 0-3, 4-7  two compute groups: one thread per KV row, group g owns query columns
//                   [64g, 64g+64) of the tile: P^T = exp2(S^T*c - lse2) (two exp2 per MUFU op,
//                   fp16) and dS^T = P^T o (dP^T - D)
//   warps 8-11      dQ group: one thread per query row; tensor memory -> registers ->
//                   shared-memory staging -> TMA reduce-add into the fp32 dQ accumulator
//                   (bulk async adds: no per-thread atomics in the load/store pipeline)
//   warp 12         TMA producer (K, V once; Q_i through a 2-stage ring, dO_i single stage)
//   warp 13         MMA issuer: the whole warp runs the loop, one elected lane issues
//
// The per-row statistics come from the workspace the preprocess kernel fills:
// lse2 = lse * log2(e) (+inf on padding rows) and delta = rowsum(dO o O) (0 on padding rows),
// both padded to a multiple of 128 rows per (batch, head); a tile's 2 x 128 values are staged
// through shared memory once instead of being re-read by every thread.
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace fmha {

struct BwdKernelParams {
  const float* lse2;    // fp32 (Z*H, seqlen_q_pad)
  const float* delta;   // fp32 (Z*H, seqlen_q_pad)
  float* dk_accum;      // optional fp32 (Z, seqlen_k, H, D) contiguous
  float* dv_accum;      // optional
  long long accum_batch_stride;  // elements between batch entries of dk_accum / dv_accum
  int accum_overwrite;  // 1: dK / dV REPLACE what dk_accum / dv_accum hold (FMHA_BWD_ACCUM_OVERWRITE)
  int heads, seqlen_q, seqlen_k, seqlen_q_pad;
  int num_kv_blocks;    // ceil(seqlen_k / 128)
  int num_heads_total;  // batch * heads
  int head_group;       // heads whose CTAs are interleaved in the grid (>= 1)
  int q_tile_begin;     // query tiles before this one take no part (FmhaBwdParams.q_row_begin / 128)
  float scale, scale_log2;
  int causal, causal_shift;
  int* status;
  // Deterministic dQ (not NULL): one word per (batch*head, query tile), zero at launch.  The
  // CTAs that add into a query tile's dQ do so in the order of their KV tiles: CTA kb waits
  // for the word to reach kb, adds, waits for its adds to complete and sets kb + 1.  The fp32
  // additions then happen in one fixed order and dQ is the same bits on every run; the price
  // is that the CTAs of a head run staggered by one query tile each.
  int* dq_order;
  // optional per-batch lengths (right-padded batches), see FmhaBwdParams
  const int* seqused_q;
  const int* seqused_k;
  long long* timeline;  // debug builds (-DFMHA_TIMELINE) only
  int timeline_block;
};

constexpr int kBwdRegsIssue = 80;     // warps 12-15
constexpr int kBwdRegsCompute = 120;  // warps 0-7
constexpr int kBwdRegsDq = 128 + (128 - kBwdRegsIssue) + 2 * (128 - kBwdRegsCompute);  // warps 8-11
static_assert(kBwdRegsIssue <= 128 && kBwdRegsCompute <= 128 && kBwdRegsDq >= 128,
              "setmaxnreg.dec must not raise and .inc must not lower the 128 registers of the launch");

template <int D, bool kBf16 = false>
struct BwdTraits {
  static constexpr int kBlock = 128;
  static constexpr int kBoxes = D / 64;
  static constexpr int kBoxBytes = 128 * 128;
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a 128 x D fp16 tile
  static constexpr int kDsBytes = 2 * kBoxBytes;         // dS^T: 128 x 128 fp16
  static constexpr int kQStages = 2;
  static constexpr int kStageBytes = 2 * 16384;          // dQ staging: 2 x (128 rows x 32 fp32)
  static constexpr int kStatBytes = 256 * 4;             // lse2[128] + delta[128] of one tile
  static constexpr int kThreads = 512;  // 4 warpgroups; warps 14, 15 only take part in barriers
  // K, V, Q x2, dO, dS^T, dQ staging, statistics
  static constexpr int kSmemBytes =
      1024 + (3 + kQStages) * kTileBytes + kDsBytes + kStageBytes + kStatBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDP = 128, kColDQ = 128, kColDK = 256, kColDV = 256 + D;
  static constexpr uint32_t kIdescST = umma_idesc_f16(128, 128, 0, 0, kBf16);  // S^T, dP^T
  static constexpr uint32_t kIdescDV = umma_idesc_f16(128, D, 0, 1, kBf16);    // dV, dK
  static constexpr uint32_t kIdescDQ = umma_idesc_f16(128, D, 1, 1, kBf16);    // dQ
};

// DR <= D: elements per row of the tensors.  96 runs at D = 128: the tile loads fill columns
// 96-127 with zeros, so those columns of dQ, dK and dV are zeros that are never written out, and
// the fp32 buffers have DR elements per row.
template <int D, bool kBf16 = false, int DR = D>
__global__ void __launch_bounds__(512, 1)
    fmha_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                    const __grid_constant__ CUtensorMap tm_dqacc, const BwdKernelParams p) {
  using T = BwdTraits<D, kBf16>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_kv_full;
  __shared__ uint64_t bar_q_full[T::kQStages], bar_q_empty[T::kQStages];
  __shared__ uint64_t bar_do_full, bar_do_empty;
  __shared__ uint64_t bar_s_full, bar_dp_full, bar_p_ready, bar_ds_ready, bar_dq_full,
      bar_dq_empty, bar_ds_free, bar_done;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_word;
  __shared__ int skip_cta;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    skip_cta = (p.status != nullptr && *reinterpret_cast<volatile int*>(p.status) != 0) ? 1 : 0;
    abort_word = 0;
  }
  __syncthreads();
  if (skip_cta) return;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t k_smem = smem_base;
  const uint32_t v_smem = k_smem + T::kTileBytes;
  const uint32_t q_smem = v_smem + T::kTileBytes;                   // kQStages tiles
  const uint32_t do_smem = q_smem + T::kQStages * T::kTileBytes;    // one tile
  const uint32_t ds_smem = do_smem + T::kTileBytes;                 // dS^T
  const uint32_t stg_smem = ds_smem + T::kDsBytes;                  // dQ staging, 2 x 16 KB
  const uint32_t stat_smem = stg_smem + T::kStageBytes;             // statistics

  // ---- coordinates.  Heads are taken in groups of head_group; within a group the CTAs are
  // ordered by KV tile first (early KV tiles see the most query tiles under a causal mask and
  // live longest), head second: the CTAs running at any time still belong to a handful of heads
  // (their Q / dO tiles and dQ accumulators stay in L2), and what is dispatched last, at the end
  // of a group and of the grid, are the short CTAs.  head_group = 1: all CTAs of a head in a row.
  const int nkb = p.num_kv_blocks;
  const int per_group = p.head_group * nkb;
  const int group = blockIdx.x / per_group;
  const int within = blockIdx.x % per_group;
  const int heads_here = min(p.head_group, p.num_heads_total - group * p.head_group);
  const int zh = group * p.head_group + within % heads_here;
  const int kb = within / heads_here;
  const int z = zh / p.heads;
  const int h = zh % p.heads;
  const int kv0 = kb * T::kBlock;

  // the lengths that count for this batch entry: query tiles and keys beyond them are padding
  const int sq = p.seqused_q == nullptr ? p.seqlen_q : max(0, min(p.seqlen_q, __ldg(p.seqused_q + z)));
  const int sk = p.seqused_k == nullptr ? p.seqlen_k : max(0, min(p.seqlen_k, __ldg(p.seqused_k + z)));
  const int nq_tiles = (sq + T::kBlock - 1) / T::kBlock;
  int i_begin = 0;
  if (p.causal) {
    // query row r sees key kv0 iff r + shift >= kv0
    const long long first_row = (long long)kv0 - p.causal_shift;
    i_begin = first_row <= 0 ? 0 : (int)min((long long)nq_tiles, first_row / T::kBlock);
  }
  i_begin = max(i_begin, p.q_tile_begin);
  // query tiles this CTA walks (may be 0; a KV tile that is all padding walks none)
  const int cnt = kv0 < sk ? max(0, nq_tiles - i_begin) : 0;
  // the n-th query tile this CTA visits
  auto tile_of = [&](int n) { return i_begin + n; };

  // The producer warp sets the barriers up itself and sends the loads of K, V and of the first
  // Q / dO tile off at once, before the CTA-wide barrier below that waits for the tensor-memory
  // allocation: the load latency at the head of a CTA runs beside the rest of the set-up.
  if (warp == 12) {
    if (lane == 0) {
      mbar_init(smem_u32(&bar_kv_full), 1);
      for (int s = 0; s < T::kQStages; ++s) {
        mbar_init(smem_u32(&bar_q_full[s]), 1);
        mbar_init(smem_u32(&bar_q_empty[s]), 1);
      }
      mbar_init(smem_u32(&bar_do_full), 1);
      mbar_init(smem_u32(&bar_do_empty), 1);
      mbar_init(smem_u32(&bar_s_full), 1);
      mbar_init(smem_u32(&bar_dp_full), 1);
      mbar_init(smem_u32(&bar_p_ready), 256);
      mbar_init(smem_u32(&bar_ds_ready), 256);
      mbar_init(smem_u32(&bar_dq_full), 1);
      mbar_init(smem_u32(&bar_dq_empty), 128);
      mbar_init(smem_u32(&bar_ds_free), 1);
      mbar_init(smem_u32(&bar_done), 1);
      fence_barrier_init();
    }
    __syncwarp();
    if (cnt > 0 && elect_one()) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      const uint32_t kvbar = smem_u32(&bar_kv_full);
      mbar_arrive_expect_tx(kvbar, 2 * T::kTileBytes);
      const uint32_t qbar = smem_u32(&bar_q_full[0]);
      mbar_arrive_expect_tx(qbar, T::kTileBytes);
      const uint32_t dbar = smem_u32(&bar_do_full);
      mbar_arrive_expect_tx(dbar, T::kTileBytes);
      const int row0 = tile_of(0) * T::kBlock;
#pragma unroll
      for (int b = 0; b < T::kBoxes; ++b) {
        tma_load_4d(k_smem + b * T::kBoxBytes, &tm_k, kvbar, b * 64, kv0, h, z);
        tma_load_4d(q_smem + b * T::kBoxBytes, &tm_q, qbar, b * 64, row0, h, z);
      }
#pragma unroll
      for (int b = 0; b < T::kBoxes; ++b) {
        tma_load_4d(v_smem + b * T::kBoxBytes, &tm_v, kvbar, b * 64, kv0, h, z);
        tma_load_4d(do_smem + b * T::kBoxBytes, &tm_do, dbar, b * 64, row0, h, z);
      }
    }
    __syncwarp();
  }
  if (warp == 13) {
    tmem_alloc(smem_u32(&tmem_base_slot), T::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  // Register budget: 512 threads leave 128 per thread.  The producer / MMA warpgroup and the
  // compute warpgroups hand part of their share to the dQ warpgroup, which must hold a whole
  // 128-column dQ row per thread to drain tensor memory in one go (the next dP^T waits for
  // those columns).  Each setmaxnreg sits at the top of its warpgroup's own branch: the
  // compiler budgets registers per region only when the instruction dominates the region.
  if (warp >= 12) {
    reg_dealloc<kBwdRegsIssue>();
  if (warp == 12) {
    // =========================== TMA producer ===========================
    if (cnt > 0) {
      // K, V and the first Q / dO tile were sent off during the set-up
      for (int n = 1; n < cnt; ++n) {
        const int st = n % T::kQStages;
        const int round = n / T::kQStages;
        const int row = tile_of(n) * T::kBlock;
        if (round > 0 &&
            !mbar_wait_warp(smem_u32(&bar_q_empty[st]), (round - 1) & 1, &abort_word, 1))
          break;
        if (elect_one()) {
          const uint32_t qbar = smem_u32(&bar_q_full[st]);
          mbar_arrive_expect_tx(qbar, T::kTileBytes);
#pragma unroll
          for (int b = 0; b < T::kBoxes; ++b)
            tma_load_4d(q_smem + st * T::kTileBytes + b * T::kBoxBytes, &tm_q, qbar, b * 64, row, h,
                        z);
        }
        __syncwarp();
        if (!mbar_wait_warp(smem_u32(&bar_do_empty), (n - 1) & 1, &abort_word, 2)) break;
        if (elect_one()) {
          const uint32_t dbar = smem_u32(&bar_do_full);
          mbar_arrive_expect_tx(dbar, T::kTileBytes);
#pragma unroll
          for (int b = 0; b < T::kBoxes; ++b)
            tma_load_4d(do_smem + b * T::kBoxBytes, &tm_do, dbar, b * 64, row, h, z);
        }
        __syncwarp();
      }
    }
  } else if (warp == 13) {
    // =========================== MMA issuer (converged warp) ===========================
    if (cnt > 0) {
      // C[128 x 128] = A[128 x D] B[128 x D]^T, both K-major in shared memory
      auto issue_kmajor = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
        const uint32_t a_lo = umma_desc_lo(a_addr, kLboKMajor);
        const uint32_t b_lo = umma_desc_lo(b_addr, kLboKMajor);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * T::kBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss_elect(tmem_base + d_col, a_lo + off, b_lo + off, T::kIdescST, ks > 0 ? 1u : 0u);
        }
      };
      const uint32_t ds_lo_k = umma_desc_lo(ds_smem, kLboKMajor);    // dS^T as K-major A (dK)
      const uint32_t ds_lo_mn = umma_desc_lo(ds_smem, kLboMnMajor);  // dS^T read as MN-major A (dQ)
      const uint32_t k_lo_mn = umma_desc_lo(k_smem, kLboMnMajor);    // K as MN-major B (dQ)
      const uint32_t do_lo_mn = umma_desc_lo(do_smem, kLboMnMajor);  // dO as MN-major B (dV)

      bool ok = mbar_wait_warp(smem_u32(&bar_kv_full), 0, &abort_word, 3);
      ok = ok && mbar_wait_warp(smem_u32(&bar_q_full[0]), 0, &abort_word, 4);
      if (ok) {
        tc_fence_after();
        issue_kmajor(T::kColS, k_smem, q_smem);
        umma_commit_elect(smem_u32(&bar_s_full));
      }
      ok = ok && mbar_wait_warp(smem_u32(&bar_do_full), 0, &abort_word, 5);
      if (ok) {
        tc_fence_after();
        issue_kmajor(T::kColDP, v_smem, do_smem);
        umma_commit_elect(smem_u32(&bar_dp_full));
      }
      for (int n = 0; ok && n < cnt; ++n) {
        const int st = n % T::kQStages;
        const uint32_t q_addr = q_smem + st * T::kTileBytes;
        // ---- dV += P^T dO_i
        FMHA_TL(2, n, 0);
        if (!mbar_wait_warp(smem_u32(&bar_p_ready), n & 1, &abort_word, 6)) break;
        tc_fence_after();
        FMHA_TL(2, n, 1);
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks)
          umma_ts_elect(tmem_base + T::kColDV,
                        tmem_base + T::kColS + (ks >> 2) * 64 + (ks & 3) * 8, do_lo_mn + ks * 128,
                        T::kIdescDV, (n > 0 || ks > 0) ? 1u : 0u);
        umma_commit_elect(smem_u32(&bar_do_empty));
        // ---- S^T of the next query tile (the S region is free once dV has read P^T)
        if (n + 1 < cnt) {
          const int st1 = (n + 1) % T::kQStages;
          if (!mbar_wait_warp(smem_u32(&bar_q_full[st1]), ((n + 1) / T::kQStages) & 1, &abort_word,
                              7))
            break;
          tc_fence_after();
          issue_kmajor(T::kColS, k_smem, q_smem + st1 * T::kTileBytes);
          umma_commit_elect(smem_u32(&bar_s_full));
        }
        // ---- dQ_i = dS K first (its read-out is on the critical path), then dK += dS^T Q_i
        FMHA_TL(2, n, 2);
        if (!mbar_wait_warp(smem_u32(&bar_ds_ready), n & 1, &abort_word, 8)) break;
        tc_fence_after();
        FMHA_TL(2, n, 3);
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks)
          umma_ss_elect(tmem_base + T::kColDQ, ds_lo_mn + ks * 128, k_lo_mn + ks * 128, T::kIdescDQ,
                        ks > 0 ? 1u : 0u);
        umma_commit_elect(smem_u32(&bar_dq_full));
        const uint32_t q_lo_mn = umma_desc_lo(q_addr, kLboMnMajor);
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * T::kBoxBytes + (ks & 3) * 32) >> 4;
          umma_ss_elect(tmem_base + T::kColDK, ds_lo_k + off, q_lo_mn + ks * 128, T::kIdescDV,
                        (n > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit_elect(smem_u32(&bar_q_empty[st]));
        umma_commit_elect(smem_u32(&bar_ds_free));
        FMHA_TL(2, n, 4);
        // ---- dP^T of the next query tile (its columns hold dQ_i until the dQ group read it)
        if (n + 1 < cnt) {
          if (!mbar_wait_warp(smem_u32(&bar_do_full), (n + 1) & 1, &abort_word, 9)) break;
          if (!mbar_wait_warp(smem_u32(&bar_dq_empty), n & 1, &abort_word, 10)) break;
          tc_fence_after();
          FMHA_TL(2, n, 5);
          issue_kmajor(T::kColDP, v_smem, do_smem);
          umma_commit_elect(smem_u32(&bar_dp_full));
          FMHA_TL(2, n, 6);
        }
      }
      umma_commit_elect(smem_u32(&bar_done));
    }
  }
  } else {
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // TMEM lane of this thread
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const size_t stat_base = (size_t)zh * p.seqlen_q_pad;

    if (warp < 8) {
      // =========================== compute groups: P^T, dS^T ===========================
      reg_dealloc<kBwdRegsCompute>();
      const int cg = warp >> 2;           // query-column half of this group
      const int ct = threadIdx.x;         // 0..255 among the compute threads
      const int kvi = kv0 + r;            // key of this thread
      const float c = p.scale_log2;
      const uint32_t tS = tmem_base + lane_addr + T::kColS + cg * 64;
      // P^T (32 packed columns) goes over the start of this group's own S^T half, which only
      // this group reads: no ordering between the two groups is needed
      const uint32_t tP = tS;
      const uint32_t tDP = tmem_base + lane_addr + T::kColDP + cg * 64;
      // statistics: thread ct < 128 carries lse2[q0 + ct], the others delta[q0 + ct - 128]
      const float* stat_src = (ct < 128 ? p.lse2 : p.delta) + stat_base + (ct & 127);
      float stat_next = (cnt > 0) ? __ldg(stat_src + (size_t)tile_of(0) * T::kBlock) : 0.f;
      const bool tl = (threadIdx.x == 0);

      for (int n = 0; n < cnt; ++n) {
        const int qbase = tile_of(n) * T::kBlock;
        const uint32_t sb = stat_smem;  // lse2 at [0, 512), delta at [512, 1024)
        named_bar_sync(3, 256);  // every thread is done reading the previous tile's values
        asm volatile("st.shared.f32 [%0], %1;" ::"r"(sb + ct * 4), "f"(stat_next) : "memory");
        if (n + 1 < cnt) stat_next = __ldg(stat_src + (size_t)tile_of(n + 1) * T::kBlock);
        named_bar_sync(4, 256);  // this tile's values are visible

        // first visible query column of this thread's half (>= 64: none)
        int first_visible = 0;
        if (kvi >= sk) {
          first_visible = T::kBlock;
        } else if (p.causal) {
          const long long fv = (long long)kvi - p.causal_shift - qbase;
          first_visible = fv <= 0 ? 0 : (int)min(fv, (long long)T::kBlock);
        }
        const int fvh = first_visible - cg * 64;

        uint32_t pp[32];  // P^T of this row and half, 16-bit pairs
        // fp16 only: -(P^T o delta) as fp16 pairs, so that dS^T = P^T o dP^T - P^T o delta is one
        // half2 FMA per pair; with bf16 (8 mantissa bits) dS^T is formed in fp32 instead
        uint32_t npd[kBf16 ? 1 : 32];
        if (tl) FMHA_TL(0, n, 0);
        mbar_wait(smem_u32(&bar_s_full), n & 1, &abort_word, 11);  // on a time-out: keep going,
        // every later wait returns at once and all 256 threads still meet at the named barrier
        tc_fence_after();
        if (tl) FMHA_TL(0, n, 1);
        {
          uint32_t s[2][32];
          tmem_ld32(tS, s[0]);
          tmem_ld32(tS + 32, s[1]);
          tmem_wait_ld();
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              const float4 L = lds128(sb + (cg * 64 + cc * 32 + i) * 4);
              const float x0 = fmaf(__uint_as_float(s[cc][i + 0]), c, -L.x);
              const float x1 = fmaf(__uint_as_float(s[cc][i + 1]), c, -L.y);
              const float x2 = fmaf(__uint_as_float(s[cc][i + 2]), c, -L.z);
              const float x3 = fmaf(__uint_as_float(s[cc][i + 3]), c, -L.w);
              if constexpr (kBf16) {
                // a bf16 argument would cost P two to three digits: exponentials in fp32
                pp[cc * 16 + (i >> 1) + 0] = pack_bf16x2(fast_exp2(x0), fast_exp2(x1));
                pp[cc * 16 + (i >> 1) + 1] = pack_bf16x2(fast_exp2(x2), fast_exp2(x3));
              } else {
                pp[cc * 16 + (i >> 1) + 0] = exp2_half2(pack_half2(x0, x1));
                pp[cc * 16 + (i >> 1) + 1] = exp2_half2(pack_half2(x2, x3));
              }
            }
          if (fvh > 0) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {  // pair j = columns 2j, 2j+1 of this half
              if (2 * j + 1 < fvh) pp[j] = 0u;
              else if (2 * j < fvh) pp[j] &= 0xffff0000u;
            }
          }
        }
        tmem_st32(tP, pp);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_p_ready));
        if (tl) FMHA_TL(0, n, 2);
        // off the critical path (dP^T is not there yet): -(P o delta)
        if constexpr (!kBf16) {
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float4 Dl = lds128(sb + 512 + (cg * 64 + 2 * j) * 4);
            npd[j + 0] = mul_half2(pp[j + 0], pack_half2(-Dl.x, -Dl.y));
            npd[j + 1] = mul_half2(pp[j + 1], pack_half2(-Dl.z, -Dl.w));
          }
        }

        mbar_wait(smem_u32(&bar_dp_full), n & 1, &abort_word, 12);
        if (tl) FMHA_TL(0, n, 3);
        // dS^T of the previous tile must have been consumed by its dK / dQ MMAs
        if (n > 0) mbar_wait(smem_u32(&bar_ds_free), (n - 1) & 1, &abort_word, 13);
        tc_fence_after();
        if (tl) FMHA_TL(0, n, 4);
        {
          uint32_t dp[2][32];
          tmem_ld32(tDP, dp[0]);
          tmem_ld32(tDP + 32, dp[1]);
          tmem_wait_ld();
          const uint32_t row_addr = ds_smem + cg * T::kBoxBytes + r * 128;
#pragma unroll
          for (int cc = 0; cc < 2; ++cc)
#pragma unroll
            for (int k8 = 0; k8 < 4; ++k8) {  // 8 columns = one 16-byte chunk
              uint32_t w[4];
              float dl[8];  // bf16 only: delta of this chunk's 8 query columns
              if constexpr (kBf16) {
                const float4 Da = lds128(sb + 512 + (cg * 64 + cc * 32 + k8 * 8) * 4);
                const float4 Db = lds128(sb + 512 + (cg * 64 + cc * 32 + k8 * 8 + 4) * 4);
                dl[0] = Da.x, dl[1] = Da.y, dl[2] = Da.z, dl[3] = Da.w;
                dl[4] = Db.x, dl[5] = Db.y, dl[6] = Db.z, dl[7] = Db.w;
              }
#pragma unroll
              for (int q2 = 0; q2 < 4; ++q2) {
                const int i = k8 * 8 + q2 * 2;     // column within this 32-column block
                const int j = cc * 16 + (i >> 1);  // its fp16 pair
                if constexpr (kBf16) {
                  w[q2] = pack_bf16x2(bf16_lo(pp[j]) * (__uint_as_float(dp[cc][i]) - dl[q2 * 2]),
                                      bf16_hi(pp[j]) * (__uint_as_float(dp[cc][i + 1]) - dl[q2 * 2 + 1]));
                } else {
                  w[q2] = fma_half2(pp[j],
                                    pack_half2(__uint_as_float(dp[cc][i]), __uint_as_float(dp[cc][i + 1])),
                                    npd[j]);
                }
              }
              const int ch = cc * 4 + k8;  // chunk of this thread's 128-byte row
              sts128(row_addr + ((ch ^ (r & 7)) << 4), w[0], w[1], w[2], w[3]);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_ds_ready));
        if (tl) FMHA_TL(0, n, 5);
      }
    } else {
      // =========================== dQ group ===========================
      reg_alloc<kBwdRegsDq>();
      const uint32_t tDQ = tmem_base + lane_addr + T::kColDQ;
      const bool tl = (r == 0);
      constexpr int kChunks = (DR + 31) / 32;  // 32-column chunks of a dQ row
      // an odd number of chunks per tile breaks the alternation of the two staging buffers by
      // chunk index: count the chunks staged so far instead
      [[maybe_unused]] uint32_t chunk_no = 0;
      for (int n = 0; n < cnt; ++n) {
        if (tl) FMHA_TL(1, n, 0);
        // on a time-out keep going (like the compute groups): every later wait returns at once,
        // and all 128 threads still meet at the named barriers
        mbar_wait(smem_u32(&bar_dq_full), n & 1, &abort_word, 14);
        tc_fence_after();
        if (tl) FMHA_TL(1, n, 1);
        // The whole dQ row goes to registers first so that the dQ columns are released to the
        // next dP^T as early as possible; then 32-column chunks go out through shared memory.
        uint32_t acc[D / 32][32];
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(tDQ + cc * 32, acc[cc]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_dq_empty));
        if (tl) FMHA_TL(1, n, 2);
#pragma unroll
        for (int cc = 0; cc < kChunks; ++cc) {
          // One reduce-add per 32-column chunk for the whole 128-row tile (16 KB): few large
          // bulk operations instead of many small ones.  The buffer was last used two
          // reduce-adds ago: at most one group may still be reading.
          uint32_t stg_buf;
          if constexpr (kChunks % 2 == 0) {
            stg_buf = stg_smem + (cc & 1) * 16384;
          } else {
            stg_buf = stg_smem + (chunk_no & 1u) * 16384;
            ++chunk_no;
          }
          if (r == 0) tma_wait_group_read<1>();
          named_bar_sync(2, 128);
          const uint32_t buf_row = stg_buf + r * 128;
#pragma unroll
          for (int k4 = 0; k4 < 8; ++k4)
            sts128(buf_row + ((k4 ^ (r & 7)) << 4), acc[cc][k4 * 4 + 0], acc[cc][k4 * 4 + 1],
                   acc[cc][k4 * 4 + 2], acc[cc][k4 * 4 + 3]);
          fence_proxy_async_smem();
          named_bar_sync(2, 128);
          if (r == 0) {
            int* order_word = p.dq_order == nullptr
                                  ? nullptr
                                  : p.dq_order + (size_t)zh * (p.seqlen_q_pad / T::kBlock) + tile_of(n);
            if (order_word != nullptr && cc == 0) {
              // the KV tiles before this one have added their share of this query tile
              global_flag_wait(order_word, kb, &abort_word, p.status, 17);
              fence_proxy_async_all();
            }
            tma_reduce_add_4d(&tm_dqacc, stg_buf, cc * 32,
                              tile_of(n) * T::kBlock, h, z);
            tma_commit_group();
            if (order_word != nullptr && cc == kChunks - 1) {
              tma_wait_group<0>();  // the adds have been performed, not just read from shared memory
              fence_proxy_async_all();
              __threadfence();
              global_flag_release(order_word, kb + 1);
            }
          }
        }
        if (tl) FMHA_TL(1, n, 3);
      }
      if (r == 0) tma_wait_group<0>();
      named_bar_sync(2, 128);  // the group leaves its loop together
    }

    // ============ epilogue: dK (warps 0-3), dV (warps 4-7) ============
    // The two compute groups, which are done with the last query tile before the dQ group is:
    // dK and dV leave while the last dQ tile is still being staged and reduce-added.
    if (warp < 8) {
      const bool is_dk = warp < 4;
      if (cnt > 0) mbar_wait(smem_u32(&bar_done), 0, &abort_word, 15);
      tc_fence_after();
      const uint32_t tAcc = tmem_base + lane_addr + (is_dk ? T::kColDK : T::kColDV);
      const float mul = is_dk ? p.scale : 1.f;
      float* accum = is_dk ? p.dk_accum : p.dv_accum;
      const int kvi = kv0 + r;
      if (accum != nullptr) {
        // ring attention: this block's contribution goes into an fp32 buffer, added to what is
        // there or (accum_overwrite) in its place; then also rows nobody contributes to are
        // written, as zeros, so that the buffer needs no clearing beforehand
        const bool have = cnt > 0 && kvi < sk;                  // this thread's row has a result
        const bool touch = kvi < p.seqlen_k && (have || p.accum_overwrite != 0);
        float* dst =
            accum + (size_t)z * p.accum_batch_stride + ((size_t)kvi * p.heads + h) * DR;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t a[32];
          if (cnt > 0) {  // uniform over the CTA: the tensor-memory load is a warp-wide instruction
            tmem_ld32(tAcc + cc * 32, a);
            tmem_wait_ld();
          }
          if (touch && cc * 32 < DR) {
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 cur = make_float4(0.f, 0.f, 0.f, 0.f);
              if (p.accum_overwrite == 0) cur = *reinterpret_cast<float4*>(dst + cc * 32 + i);
              if (have) {
                cur.x += __uint_as_float(a[i + 0]) * mul;
                cur.y += __uint_as_float(a[i + 1]) * mul;
                cur.z += __uint_as_float(a[i + 2]) * mul;
                cur.w += __uint_as_float(a[i + 3]) * mul;
              }
              *reinterpret_cast<float4*>(dst + cc * 32 + i) = cur;
            }
          }
        }
      } else {
        // fp16 tile -> shared memory (over Q stage 0 / dO) -> TMA store
        const uint32_t out_smem = is_dk ? q_smem : do_smem;
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) {
          uint32_t a[32];
          if (cnt > 0) {
            tmem_ld32(tAcc + cc * 32, a);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = 0u;
          }
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int ch = cc * 4 + k4;
            const uint32_t addr =
                out_smem + (ch >> 3) * T::kBoxBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            sts128(addr,
                   pack16x2<kBf16>(__uint_as_float(a[k4 * 8 + 0]) * mul, __uint_as_float(a[k4 * 8 + 1]) * mul),
                   pack16x2<kBf16>(__uint_as_float(a[k4 * 8 + 2]) * mul, __uint_as_float(a[k4 * 8 + 3]) * mul),
                   pack16x2<kBf16>(__uint_as_float(a[k4 * 8 + 4]) * mul, __uint_as_float(a[k4 * 8 + 5]) * mul),
                   pack16x2<kBf16>(__uint_as_float(a[k4 * 8 + 6]) * mul, __uint_as_float(a[k4 * 8 + 7]) * mul));
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(is_dk ? 1 : 5, 128);
        if (r == 0) {
          const CUtensorMap* tm = is_dk ? &tm_dk : &tm_dv;
#pragma unroll
          for (int b = 0; b < T::kBoxes; ++b)
            tma_store_4d(tm, out_smem + b * T::kBoxBytes, b * 64, kv0, h, z);
          tma_commit_group();
          tma_wait_group<0>();
        }
      }
    }
  }

  // ---- teardown
  tc_fence_before();
  __syncthreads();
  if (abort_word != 0) {
    if (threadIdx.x == 0 && p.status != nullptr) atomicCAS(p.status, 0, abort_word);
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
  }
  if (warp == 13) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace fmha
