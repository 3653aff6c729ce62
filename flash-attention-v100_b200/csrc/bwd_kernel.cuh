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
//   dK  += dS^T Q_i    (A = dS^T smem K-major, B = Q_i smem MN-major)      -> TMEM [256, 256+D)
//   dQ_i = dS  K       (A = dS^T smem read MN-major, B = K smem MN-major)  -> TMEM [128,128+D)
//                      (aliases dP^T, which is dead once dS^T is in shared memory)
//
//   warps 0-3  compute group: one thread per KV row; P^T and dS^T
//   warps 4-7  dQ group: one thread per query row; moves dQ_i from tensor memory into the fp32
//              accumulator in global memory with vector reductions
//   warp 8     TMA producer (K, V once; Q_i, dO_i through 2-stage rings)
//   warp 9     MMA issuer (one thread)
//
// The per-row statistics come from the workspace the preprocess kernel fills:
// lse2 = lse * log2(e) (+inf on padding rows) and delta = rowsum(dO o O) (0 on padding rows),
// both padded to a multiple of 128 rows per (batch, head).
#pragma once
#include <cuda.h>
#include <math_constants.h>

#include "ptx.cuh"

namespace fmha {

struct BwdKernelParams {
  float* dq_accum;      // fp32 (Z, seqlen_q, H, D) contiguous
  const float* lse2;    // fp32 (Z*H, seqlen_q_pad)
  const float* delta;   // fp32 (Z*H, seqlen_q_pad)
  float* dk_accum;      // optional fp32 (Z, seqlen_k, H, D) contiguous
  float* dv_accum;      // optional
  int heads, seqlen_q, seqlen_k, seqlen_q_pad;
  int num_kv_blocks;    // ceil(seqlen_k / 128)
  float scale, scale_log2;
  int causal, causal_shift;
  int* status;
};

template <int D>
struct BwdTraits {
  static constexpr int kBlock = 128;
  static constexpr int kBoxes = D / 64;
  static constexpr int kBoxBytes = 128 * 128;
  static constexpr int kTileBytes = kBoxes * kBoxBytes;  // a 128 x D fp16 tile
  static constexpr int kDsBytes = 2 * kBoxBytes;         // dS^T: 128 x 128 fp16
  static constexpr int kStages = 2;
  static constexpr int kThreads = 320;
  // K, V, Q x2, dO x2, dS^T
  static constexpr int kSmemBytes = 1024 + (2 + 2 * kStages) * kTileBytes + kDsBytes;
  static constexpr int kTmemCols = 512;
  static constexpr int kColS = 0, kColDP = 128, kColDQ = 128, kColDK = 256, kColDV = 256 + D;
  static constexpr uint32_t kIdescST = umma_idesc_f16(128, 128, 0, 0);  // S^T, dP^T
  static constexpr uint32_t kIdescDV = umma_idesc_f16(128, D, 0, 1);    // dV, dK
  static constexpr uint32_t kIdescDQ = umma_idesc_f16(128, D, 1, 1);    // dQ
};

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c),
               "f"(d)
               : "memory");
}

template <int D>
__global__ void __launch_bounds__(320, 1)
    fmha_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                    const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                    const __grid_constant__ CUtensorMap tm_dk, const __grid_constant__ CUtensorMap tm_dv,
                    const BwdKernelParams p) {
  using T = BwdTraits<D>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar_kv_full;
  __shared__ uint64_t bar_q_full[T::kStages], bar_q_empty[T::kStages];
  __shared__ uint64_t bar_do_full[T::kStages], bar_do_empty[T::kStages];
  __shared__ uint64_t bar_s_full, bar_dp_full, bar_p_ready, bar_ds_ready, bar_dq_full,
      bar_dq_empty, bar_done;
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
  const uint32_t q_smem = v_smem + T::kTileBytes;                  // kStages tiles
  const uint32_t do_smem = q_smem + T::kStages * T::kTileBytes;    // kStages tiles
  const uint32_t ds_smem = do_smem + T::kStages * T::kTileBytes;   // dS^T

  // ---- coordinates: consecutive CTAs = same head; early KV tiles (most query tiles) first
  const int nkb = p.num_kv_blocks;
  const int zh = blockIdx.x / nkb;
  const int kb = blockIdx.x % nkb;
  const int z = zh / p.heads;
  const int h = zh % p.heads;
  const int kv0 = kb * T::kBlock;

  const int nq_tiles = (p.seqlen_q + T::kBlock - 1) / T::kBlock;
  int i_begin = 0;
  if (p.causal) {
    // query row r sees key kv0 iff r + shift >= kv0
    const long long first_row = (long long)kv0 - p.causal_shift;
    i_begin = first_row <= 0 ? 0 : (int)min((long long)nq_tiles, first_row / T::kBlock);
  }
  const int cnt = nq_tiles - i_begin;  // query tiles this CTA walks (may be 0)

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar_kv_full), 1);
    for (int s = 0; s < T::kStages; ++s) {
      mbar_init(smem_u32(&bar_q_full[s]), 1);
      mbar_init(smem_u32(&bar_q_empty[s]), 1);
      mbar_init(smem_u32(&bar_do_full[s]), 1);
      mbar_init(smem_u32(&bar_do_empty[s]), 1);
    }
    mbar_init(smem_u32(&bar_s_full), 1);
    mbar_init(smem_u32(&bar_dp_full), 1);
    mbar_init(smem_u32(&bar_p_ready), 128);
    mbar_init(smem_u32(&bar_ds_ready), 128);
    mbar_init(smem_u32(&bar_dq_full), 1);
    mbar_init(smem_u32(&bar_dq_empty), 128);
    mbar_init(smem_u32(&bar_done), 1);
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

  if (warp == 8) {
    // =========================== TMA producer ===========================
    if (lane == 0 && cnt > 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      tma_prefetch_desc(&tm_v);
      tma_prefetch_desc(&tm_do);
      const uint32_t kvbar = smem_u32(&bar_kv_full);
      mbar_arrive_expect_tx(kvbar, 2 * T::kTileBytes);
#pragma unroll
      for (int b = 0; b < T::kBoxes; ++b) {
        tma_load_4d(k_smem + b * T::kBoxBytes, &tm_k, kvbar, b * 64, kv0, h, z);
        tma_load_4d(v_smem + b * T::kBoxBytes, &tm_v, kvbar, b * 64, kv0, h, z);
      }
      for (int n = 0; n < cnt; ++n) {
        const int st = n % T::kStages;
        const int round = n / T::kStages;
        const int row = (i_begin + n) * T::kBlock;
        if (round > 0 && !mbar_wait(smem_u32(&bar_q_empty[st]), (round - 1) & 1, &abort_word, 1))
          break;
        const uint32_t qbar = smem_u32(&bar_q_full[st]);
        mbar_arrive_expect_tx(qbar, T::kTileBytes);
#pragma unroll
        for (int b = 0; b < T::kBoxes; ++b)
          tma_load_4d(q_smem + st * T::kTileBytes + b * T::kBoxBytes, &tm_q, qbar, b * 64, row, h,
                      z);
        if (round > 0 && !mbar_wait(smem_u32(&bar_do_empty[st]), (round - 1) & 1, &abort_word, 2))
          break;
        const uint32_t dbar = smem_u32(&bar_do_full[st]);
        mbar_arrive_expect_tx(dbar, T::kTileBytes);
#pragma unroll
        for (int b = 0; b < T::kBoxes; ++b)
          tma_load_4d(do_smem + st * T::kTileBytes + b * T::kBoxBytes, &tm_do, dbar, b * 64, row,
                      h, z);
      }
    }
    __syncwarp();
  } else if (warp == 9) {
    // =========================== MMA issuer ===========================
    if (lane == 0 && cnt > 0) {
      // C[128 x 128] = A[128 x D] B[128 x D]^T, both K-major in shared memory
      auto issue_kmajor = [&](uint32_t d_col, uint32_t a_addr, uint32_t b_addr) {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * T::kBoxBytes + (ks & 3) * 32;
          umma_ss(tmem_base + d_col, umma_smem_desc(a_addr + off, 16, 1024),
                  umma_smem_desc(b_addr + off, 16, 1024), T::kIdescST, ks > 0 ? 1u : 0u);
        }
      };
      bool ok = mbar_wait(smem_u32(&bar_kv_full), 0, &abort_word, 3);
      ok = ok && mbar_wait(smem_u32(&bar_q_full[0]), 0, &abort_word, 4);
      if (ok) {
        tc_fence_after();
        issue_kmajor(T::kColS, k_smem, q_smem);
        umma_commit(smem_u32(&bar_s_full));
      }
      ok = ok && mbar_wait(smem_u32(&bar_do_full[0]), 0, &abort_word, 5);
      if (ok) {
        tc_fence_after();
        issue_kmajor(T::kColDP, v_smem, do_smem);
        umma_commit(smem_u32(&bar_dp_full));
      }
      for (int n = 0; ok && n < cnt; ++n) {
        const int st = n % T::kStages;
        const uint32_t q_addr = q_smem + st * T::kTileBytes;
        const uint32_t do_addr = do_smem + st * T::kTileBytes;
        // ---- dV += P^T dO_i
        if (!mbar_wait(smem_u32(&bar_p_ready), n & 1, &abort_word, 6)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks)
          umma_ts(tmem_base + T::kColDV, tmem_base + T::kColS + ks * 8,
                  umma_smem_desc(do_addr + ks * 2048, T::kBoxBytes, 1024), T::kIdescDV,
                  (n > 0 || ks > 0) ? 1u : 0u);
        umma_commit(smem_u32(&bar_do_empty[st]));
        // ---- S^T of the next query tile (the S region is free once dV has read P^T)
        if (n + 1 < cnt) {
          const int st1 = (n + 1) % T::kStages;
          if (!mbar_wait(smem_u32(&bar_q_full[st1]), ((n + 1) / T::kStages) & 1, &abort_word, 7))
            break;
          tc_fence_after();
          issue_kmajor(T::kColS, k_smem, q_smem + st1 * T::kTileBytes);
          umma_commit(smem_u32(&bar_s_full));
        }
        // ---- dK += dS^T Q_i ; dQ_i = dS K
        if (!mbar_wait(smem_u32(&bar_ds_ready), n & 1, &abort_word, 8)) break;
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks) {
          const uint32_t off = (ks >> 2) * T::kBoxBytes + (ks & 3) * 32;
          umma_ss(tmem_base + T::kColDK, umma_smem_desc(ds_smem + off, 16, 1024),
                  umma_smem_desc(q_addr + ks * 2048, T::kBoxBytes, 1024), T::kIdescDV,
                  (n > 0 || ks > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int ks = 0; ks < T::kBlock / 16; ++ks)
          umma_ss(tmem_base + T::kColDQ, umma_smem_desc(ds_smem + ks * 2048, T::kBoxBytes, 1024),
                  umma_smem_desc(k_smem + ks * 2048, T::kBoxBytes, 1024), T::kIdescDQ,
                  ks > 0 ? 1u : 0u);
        umma_commit(smem_u32(&bar_dq_full));
        umma_commit(smem_u32(&bar_q_empty[st]));
        // ---- dP^T of the next query tile (its columns hold dQ_i until the dQ group read it)
        if (n + 1 < cnt) {
          const int st1 = (n + 1) % T::kStages;
          if (!mbar_wait(smem_u32(&bar_do_full[st1]), ((n + 1) / T::kStages) & 1, &abort_word, 9))
            break;
          if (!mbar_wait(smem_u32(&bar_dq_empty), n & 1, &abort_word, 10)) break;
          tc_fence_after();
          issue_kmajor(T::kColDP, v_smem, do_smem + st1 * T::kTileBytes);
          umma_commit(smem_u32(&bar_dp_full));
        }
      }
      umma_commit(smem_u32(&bar_done));
    }
    __syncwarp();
  } else {
    const int group = warp >> 2;  // 0 = compute, 1 = dQ
    const int quad = warp & 3;
    const int r = quad * 32 + lane;  // TMEM lane of this thread
    const uint32_t lane_addr = uint32_t(quad * 32) << 16;
    const size_t stat_base = (size_t)zh * p.seqlen_q_pad;

    if (group == 0) {
      // =========================== compute group: P^T, dS^T ===========================
      const int kvi = kv0 + r;  // key of this thread
      const float c = p.scale_log2;
      const uint32_t tS = tmem_base + lane_addr + T::kColS;
      const uint32_t tDP = tmem_base + lane_addr + T::kColDP;
      for (int n = 0; n < cnt; ++n) {
        const int qbase = (i_begin + n) * T::kBlock;
        const float* lse2_p = p.lse2 + stat_base + qbase;
        const float* dl_p = p.delta + stat_base + qbase;
        // first visible query column of this tile for this key (>= 128: none)
        int first_visible = 0;
        if (kvi >= p.seqlen_k) {
          first_visible = T::kBlock;
        } else if (p.causal) {
          const long long fv = (long long)kvi - p.causal_shift - qbase;
          first_visible = fv <= 0 ? 0 : (int)min(fv, (long long)T::kBlock);
        }
        uint32_t pp[2][32];  // P^T of this row, fp16 pairs
        if (!mbar_wait(smem_u32(&bar_s_full), n & 1, &abort_word, 11)) break;
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t s[32];
          tmem_ld32(tS + cc * 32, s);
          tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 L = __ldg(reinterpret_cast<const float4*>(lse2_p + cc * 32 + i));
            float p0 = fast_exp2(fmaf(__uint_as_float(s[i + 0]), c, -L.x));
            float p1 = fast_exp2(fmaf(__uint_as_float(s[i + 1]), c, -L.y));
            float p2 = fast_exp2(fmaf(__uint_as_float(s[i + 2]), c, -L.z));
            float p3 = fast_exp2(fmaf(__uint_as_float(s[i + 3]), c, -L.w));
            if (first_visible > 0) {
              const int col = cc * 32 + i;
              if (col + 0 < first_visible) p0 = 0.f;
              if (col + 1 < first_visible) p1 = 0.f;
              if (col + 2 < first_visible) p2 = 0.f;
              if (col + 3 < first_visible) p3 = 0.f;
            }
            pp[cc >> 1][(cc & 1) * 16 + (i >> 1) + 0] = pack_half2(p0, p1);
            pp[cc >> 1][(cc & 1) * 16 + (i >> 1) + 1] = pack_half2(p2, p3);
          }
        }
        tmem_st32(tS + 0, pp[0]);
        tmem_st32(tS + 32, pp[1]);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_p_ready));

        if (!mbar_wait(smem_u32(&bar_dp_full), n & 1, &abort_word, 12)) break;
        // dS^T of the previous tile must have been consumed by its dK / dQ MMAs
        if (n > 0 && !mbar_wait(smem_u32(&bar_dq_full), (n - 1) & 1, &abort_word, 13)) break;
        tc_fence_after();
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint32_t dp[32];
          tmem_ld32(tDP + cc * 32, dp);
          tmem_wait_ld();
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float4 Dl = __ldg(reinterpret_cast<const float4*>(dl_p + cc * 32 + i));
            const uint32_t pk0 = pp[cc >> 1][(cc & 1) * 16 + (i >> 1) + 0];
            const uint32_t pk1 = pp[cc >> 1][(cc & 1) * 16 + (i >> 1) + 1];
            const float2 pa = __half22float2(*reinterpret_cast<const __half2*>(&pk0));
            const float2 pb = __half22float2(*reinterpret_cast<const __half2*>(&pk1));
            const float d0 = pa.x * (__uint_as_float(dp[i + 0]) - Dl.x);
            const float d1 = pa.y * (__uint_as_float(dp[i + 1]) - Dl.y);
            const float d2 = pb.x * (__uint_as_float(dp[i + 2]) - Dl.z);
            const float d3 = pb.y * (__uint_as_float(dp[i + 3]) - Dl.w);
            w[(i >> 1) + 0] = pack_half2(d0, d1);
            w[(i >> 1) + 1] = pack_half2(d2, d3);
          }
#pragma unroll
          for (int k4 = 0; k4 < 4; ++k4) {
            const int ch = cc * 4 + k4;  // 16-byte chunk (8 query columns) of this row
            const uint32_t addr =
                ds_smem + (ch >> 3) * T::kBoxBytes + r * 128 + (((ch & 7) ^ (r & 7)) << 4);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w[k4 * 4 + 0]),
                         "r"(w[k4 * 4 + 1]), "r"(w[k4 * 4 + 2]), "r"(w[k4 * 4 + 3])
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_ds_ready));
      }
    } else {
      // =========================== dQ group ===========================
      const uint32_t tDQ = tmem_base + lane_addr + T::kColDQ;
      for (int n = 0; n < cnt; ++n) {
        const int qrow = (i_begin + n) * T::kBlock + r;
        if (!mbar_wait(smem_u32(&bar_dq_full), n & 1, &abort_word, 14)) break;
        tc_fence_after();
        uint32_t acc[D / 32][32];
#pragma unroll
        for (int cc = 0; cc < D / 32; ++cc) tmem_ld32(tDQ + cc * 32, acc[cc]);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(smem_u32(&bar_dq_empty));
        if (qrow < p.seqlen_q) {
          float* dst = p.dq_accum + (((size_t)z * p.seqlen_q + qrow) * p.heads + h) * D;
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc)
#pragma unroll
            for (int i = 0; i < 32; i += 4)
              red_add_v4(dst + cc * 32 + i, __uint_as_float(acc[cc][i + 0]),
                         __uint_as_float(acc[cc][i + 1]), __uint_as_float(acc[cc][i + 2]),
                         __uint_as_float(acc[cc][i + 3]));
        }
      }
    }

    // =========================== epilogue: dK (group 0), dV (group 1) ===========================
    {
      if (cnt > 0) mbar_wait(smem_u32(&bar_done), 0, &abort_word, 15);
      tc_fence_after();
      const uint32_t tAcc = tmem_base + lane_addr + (group == 0 ? T::kColDK : T::kColDV);
      const float mul = (group == 0) ? p.scale : 1.f;
      float* accum = (group == 0) ? p.dk_accum : p.dv_accum;
      const int kvi = kv0 + r;
      if (accum != nullptr) {
        // ring attention: add this block's contribution into the travelling fp32 buffer
        if (cnt > 0 && kvi < p.seqlen_k) {
          float* dst = accum + (((size_t)z * p.seqlen_k + kvi) * p.heads + h) * D;
#pragma unroll
          for (int cc = 0; cc < D / 32; ++cc) {
            uint32_t a[32];
            tmem_ld32(tAcc + cc * 32, a);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              float4 cur = *reinterpret_cast<float4*>(dst + cc * 32 + i);
              cur.x += __uint_as_float(a[i + 0]) * mul;
              cur.y += __uint_as_float(a[i + 1]) * mul;
              cur.z += __uint_as_float(a[i + 2]) * mul;
              cur.w += __uint_as_float(a[i + 3]) * mul;
              *reinterpret_cast<float4*>(dst + cc * 32 + i) = cur;
            }
          }
        }
      } else {
        // fp16 tile -> shared memory (over Q stage 0 / dO stage 0) -> TMA store
        const uint32_t out_smem = (group == 0) ? q_smem : do_smem;
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
            const uint32_t w0 = pack_half2(__uint_as_float(a[k4 * 8 + 0]) * mul,
                                           __uint_as_float(a[k4 * 8 + 1]) * mul);
            const uint32_t w1 = pack_half2(__uint_as_float(a[k4 * 8 + 2]) * mul,
                                           __uint_as_float(a[k4 * 8 + 3]) * mul);
            const uint32_t w2 = pack_half2(__uint_as_float(a[k4 * 8 + 4]) * mul,
                                           __uint_as_float(a[k4 * 8 + 5]) * mul);
            const uint32_t w3 = pack_half2(__uint_as_float(a[k4 * 8 + 6]) * mul,
                                           __uint_as_float(a[k4 * 8 + 7]) * mul);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w0), "r"(w1),
                         "r"(w2), "r"(w3)
                         : "memory");
          }
        }
        fence_proxy_async_smem();
        named_bar_sync(1 + group, 128);
        if (r == 0) {
          const CUtensorMap* tm = (group == 0) ? &tm_dk : &tm_dv;
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
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, T::kTmemCols);
  }
}

}  // namespace fmha
