// HBM-bound helper kernels around the two tensor-core kernels:
//   - backward preprocess: D = rowsum(dO o O) in fp32, lse * log2(e), zero the fp32 dQ
//     accumulator.  Replaces the two eager PyTorch ops of the reference
//     (flash_attn_v100/flash_attn_interface.py:43-44, fp16 there) and its zero-fill (:84).
//   - dQ convert: fp16(scale * dq_accum).  Replaces the reference's fp16 atomicAdd
//     accumulation (kernel/fused_mha_kernel.cu:543,693) together with the fp32 accumulator.
//   - merge: LSE-weighted merge of a partial attention result into running fp32
//     accumulators (ring attention; no counterpart in the reference).
// Each thread owns 8 consecutive head_dim elements (one 16-byte load of fp16 or bf16) of one row.
// D is the head dimension the tensor-core kernels run at (64 or 128); DR <= D is the one the
// tensors have (96 runs at D = 128: the threads of a row beyond DR have nothing to do, and the
// fp32 accumulators are laid out with DR elements per row).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <math_constants.h>
#include <stdint.h>

#include <type_traits>

namespace fmha {

struct Strides3 {
  long long batch, row, head;
};

// E = __half or __nv_bfloat16: the 16-bit element type of the tensors
template <typename E>
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  if constexpr (sizeof(E) == 2 && std::is_same<E, __nv_bfloat16>::value) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 t = __half22float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
}
template <typename E>
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  if constexpr (std::is_same<E, __nv_bfloat16>::value) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  } else {
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
  return u;
}

// rows are indexed (zh, q) over the PADDED query length so that lse2 / delta are complete
template <int D, typename E, int DR = D>
__global__ void __launch_bounds__(256)
    fmha_bwd_preprocess_kernel(const E* __restrict__ o, Strides3 so,
                               const E* __restrict__ dout, Strides3 sdo,
                               const float* __restrict__ lse, float* __restrict__ dq_accum,
                               float* __restrict__ lse2, float* __restrict__ delta, int heads,
                               int seqlen_q, int seqlen_q_pad, long long total_rows,
                               const int* __restrict__ seqused_q) {
  constexpr int kGroup = D / 8;  // threads per row
  constexpr int kRowsPerBlock = 256 / kGroup;
  const int part = threadIdx.x % kGroup;
  const long long row_id = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / kGroup;
  if (row_id >= total_rows) return;  // whole groups leave together (256 % kGroup == 0)
  const long long zh = row_id / seqlen_q_pad;
  const int q = (int)(row_id % seqlen_q_pad);
  const int z = (int)(zh / heads);
  const int h = (int)(zh % heads);
  if (q >= seqlen_q) {
    if (part == 0) {
      lse2[row_id] = CUDART_INF_F;
      delta[row_id] = 0.f;
    }
    return;
  }
  // a padding row of a right-padded batch: P = exp2(s - inf) = 0 for it, it adds nothing to any
  // gradient, and its own dQ stays zero
  const bool padding = seqused_q != nullptr && q >= __ldg(seqused_q + z);
  const bool mine = (DR == D) || part * 8 < DR;  // this thread's 8 elements exist
  float acc = 0.f;
  if (mine) {
    const uint4 uo =
        *reinterpret_cast<const uint4*>(o + z * so.batch + q * so.row + h * so.head + part * 8);
    const uint4 ud =
        *reinterpret_cast<const uint4*>(dout + z * sdo.batch + q * sdo.row + h * sdo.head + part * 8);
    float fo[8], fd[8];
    unpack8<E>(uo, fo);
    unpack8<E>(ud, fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc = fmaf(fo[i], fd[i], acc);
  }
#pragma unroll
  for (int off = kGroup / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (part == 0) {
    delta[row_id] = padding ? 0.f : acc;
    lse2[row_id] = padding ? CUDART_INF_F : lse[zh * seqlen_q + q] * 1.4426950408889634f;
  }
  if (dq_accum != nullptr && mine) {
    float4* dst = reinterpret_cast<float4*>(
        dq_accum + ((((long long)z * seqlen_q + q) * heads + h) * DR + part * 8));
    dst[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    dst[1] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

template <int D, typename E, int DR = D>
__global__ void __launch_bounds__(256)
    fmha_bwd_convert_dq_kernel(const float* __restrict__ dq_accum, E* __restrict__ dq,
                               Strides3 sdq, int heads, int seqlen_q, float scale,
                               long long total_rows) {
  constexpr int kGroup = D / 8;
  constexpr int kRowsPerBlock = 256 / kGroup;
  const int part = threadIdx.x % kGroup;
  const long long row_id = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / kGroup;
  if (row_id >= total_rows || (DR != D && part * 8 >= DR)) return;
  // row_id enumerates (z, q, h): the accumulator's own order
  const int h = (int)(row_id % heads);
  const long long zq = row_id / heads;
  const int q = (int)(zq % seqlen_q);
  const int z = (int)(zq / seqlen_q);
  const float4* src = reinterpret_cast<const float4*>(dq_accum + row_id * DR + part * 8);
  const float4 a = src[0], b = src[1];
  float f[8] = {a.x * scale, a.y * scale, a.z * scale, a.w * scale,
                b.x * scale, b.y * scale, b.z * scale, b.w * scale};
  *reinterpret_cast<uint4*>(dq + z * sdq.batch + q * sdq.row + h * sdq.head + part * 8) = pack8<E>(f);
}

template <int D, typename E, int DR = D>
__global__ void __launch_bounds__(256)
    fmha_merge_kernel(float* __restrict__ o_acc, float* __restrict__ lse_acc,
                      const E* __restrict__ o_part, Strides3 sp,
                      const float* __restrict__ lse_part, E* __restrict__ o_out, int heads,
                      int rows, int acc_rows, int row_offset, long long total_rows) {
  constexpr int kGroup = D / 8;
  constexpr int kRowsPerBlock = 256 / kGroup;
  const int part = threadIdx.x % kGroup;
  const long long row_id = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / kGroup;
  const bool active = row_id < total_rows && (DR == D || part * 8 < DR);
  float la = 0.f, lb = 0.f, ln = 0.f;
  long long stat_idx = 0;
  if (active) {
    // row_id enumerates (z, q, h) of the partial result; it covers rows [row_offset,
    // row_offset + rows) of the accumulators, which have acc_rows rows
    const int h = (int)(row_id % heads);
    const long long zq = row_id / heads;
    const int q = (int)(zq % rows);
    const int z = (int)(zq / rows);
    const long long acc_row = ((long long)z * acc_rows + row_offset + q) * heads + h;
    stat_idx = ((long long)z * heads + h) * acc_rows + row_offset + q;
    la = lse_acc[stat_idx];
    lb = lse_part[((long long)z * heads + h) * rows + q];
    const float mx = fmaxf(la, lb);
    float wa = 0.f, wb = 0.f;
    ln = -CUDART_INF_F;
    if (mx > -CUDART_INF_F) {
      const float ea = __expf(la - mx), eb = __expf(lb - mx);
      const float inv = 1.f / (ea + eb);
      wa = ea * inv;
      wb = eb * inv;
      ln = mx + __logf(ea + eb);
    }
    float4* acc = reinterpret_cast<float4*>(o_acc + acc_row * DR + part * 8);
    // a row whose accumulated LSE is -inf holds nothing yet: its o_acc is not read (it may be
    // uninitialised memory), so the first merge of a row initialises it
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    if (la > -CUDART_INF_F) a0 = acc[0], a1 = acc[1];
    const uint4 up =
        *reinterpret_cast<const uint4*>(o_part + z * sp.batch + q * sp.row + h * sp.head + part * 8);
    float fp[8];
    unpack8<E>(up, fp);
    float f[8] = {wa * a0.x + wb * fp[0], wa * a0.y + wb * fp[1], wa * a0.z + wb * fp[2],
                  wa * a0.w + wb * fp[3], wa * a1.x + wb * fp[4], wa * a1.y + wb * fp[5],
                  wa * a1.z + wb * fp[6], wa * a1.w + wb * fp[7]};
    acc[0] = make_float4(f[0], f[1], f[2], f[3]);
    acc[1] = make_float4(f[4], f[5], f[6], f[7]);
    if (o_out != nullptr)
      *reinterpret_cast<uint4*>(o_out + acc_row * DR + part * 8) = pack8<E>(f);
  }
  // every thread of a row has read lse_acc before its first thread overwrites it
  __syncwarp();
  if (active && part == 0) lse_acc[stat_idx] = ln;
}

}  // namespace fmha
