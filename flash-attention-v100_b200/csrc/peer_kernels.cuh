// Small kernels behind the multi-GPU plumbing of ring attention (no counterpart in the
// reference, which is single-GPU): flags that one GPU sets in another GPU's memory and waits
// for in its own, a device-side iteration counter so that a captured sequence of launches can
// be replayed, and the final sum of the per-source dK / dV partial results.
//
// Every wait is bounded by wall-clock time; a wait that runs out writes a code to the status
// word, after which the attention kernels launched behind it return at once.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "aux_kernels.cuh"

namespace fmha {

constexpr int kMaxPeers = 16;
constexpr int kErrPeerTimeout = 0x200;  // status word: a flag from another GPU did not arrive

struct PeerFlagList {
  int* ptr[kMaxPeers];
  int n;
};

// word[0] += 1, word[1] = the old value (one thread): the iteration number the flags of this
// call carry, and the previous one
__global__ void counter_bump_kernel(int* word) {
  const int old = word[0];
  word[1] = old;
  word[0] = old + 1;
}

// flags[i] <- *value for every peer, after everything this GPU wrote before
__global__ void peer_signal_kernel(PeerFlagList list, const int* value) {
  const int i = threadIdx.x;
  if (i >= list.n) return;
  const int v = *value;
  __threadfence_system();
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(list.ptr[i]), "r"(v) : "memory");
}

// thread i waits until *flags[i] >= *value (set by another GPU); gives up after timeout_ns
__global__ void peer_wait_kernel(PeerFlagList list, const int* value, int* status,
                                 unsigned long long timeout_ns) {
  const int i = threadIdx.x;
  if (i >= list.n) return;
  if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return;
  const int want = *value;
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (;;) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(list.ptr[i]) : "memory");
    if (v >= want) return;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > timeout_ns) break;
    __nanosleep(200);
  }
  if (status != nullptr) atomicCAS(status, 0, kErrPeerTimeout | (i & 0xff));
}

struct PartList {
  const float* ptr[kMaxPeers];
  int rows[kMaxPeers];  // part s covers rows [0, rows[s]) of every batch entry
  int n;
};

// out (16-bit, strided) = sum over parts of fp32 (Z, rows, H, D) buffers, each dense with
// `rows` rows per batch entry although only its first rows[s] rows count.  D = 64 or 128 sets the
// threads per row; the tensors have DR <= D elements per row (96 runs at D = 128).
template <int D, typename E, int DR = D>
__global__ void __launch_bounds__(256)
    sum_partials_kernel(PartList parts, E* __restrict__ out, Strides3 so, int heads, int rows,
                        long long total_rows) {
  constexpr int kGroup = D / 8;
  constexpr int kRowsPerBlock = 256 / kGroup;
  const int part = threadIdx.x % kGroup;
  const long long row_id = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / kGroup;
  if (row_id >= total_rows || (DR != D && part * 8 >= DR)) return;
  // row_id enumerates (z, n, h)
  const int h = (int)(row_id % heads);
  const long long zn = row_id / heads;
  const int n = (int)(zn % rows);
  const int z = (int)(zn / rows);
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
  for (int s = 0; s < parts.n; ++s) {
    if (n < parts.rows[s]) {
      const float4* src = reinterpret_cast<const float4*>(parts.ptr[s] + row_id * DR + part * 8);
      const float4 a = src[0], b = src[1];
      f[0] += a.x, f[1] += a.y, f[2] += a.z, f[3] += a.w;
      f[4] += b.x, f[5] += b.y, f[6] += b.z, f[7] += b.w;
    }
  }
  *reinterpret_cast<uint4*>(out + z * so.batch + n * so.row + h * so.head + part * 8) = pack8<E>(f);
}

struct MergeList {
  const void* o[kMaxPeers];     // 16-bit (Z, rows[s], H, DR) contiguous
  const float* lse[kMaxPeers];  // fp32 (Z, H, rows[s]) contiguous
  int row0[kMaxPeers];          // part s covers output rows [row0[s], row0[s] + rows[s])
  int rows[kMaxPeers];
  int n;
};

// All partial attention results of a ring forward merged in ONE pass (instead of one
// read-modify-write pass over fp32 accumulators per step): for every output row
//   lse = log sum_s e^lse_s,   o = sum_s e^(lse_s - lse) o_s      over the parts that cover the row.
// out 16-bit (Z, rows, H, DR) contiguous, lse_out fp32 (Z, H, rows).
template <int D, typename E, int DR = D>
__global__ void __launch_bounds__(256)
    merge_parts_kernel(MergeList parts, E* __restrict__ out, float* __restrict__ lse_out, int heads,
                       int rows, long long total_rows) {
  constexpr int kGroup = D / 8;
  constexpr int kRowsPerBlock = 256 / kGroup;
  const int part = threadIdx.x % kGroup;
  const long long row_id = (long long)blockIdx.x * kRowsPerBlock + threadIdx.x / kGroup;
  if (row_id >= total_rows || (DR != D && part * 8 >= DR)) return;
  // row_id enumerates (z, n, h) of the output
  const int h = (int)(row_id % heads);
  const long long zn = row_id / heads;
  const int n = (int)(zn % rows);
  const int z = (int)(zn / rows);
  float mx = -CUDART_INF_F;
  for (int s = 0; s < parts.n; ++s) {
    const int r = n - parts.row0[s];
    if (r >= 0 && r < parts.rows[s])
      mx = fmaxf(mx, parts.lse[s][((long long)z * heads + h) * parts.rows[s] + r]);
  }
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float sum = 0.f;
  if (mx > -CUDART_INF_F) {
    for (int s = 0; s < parts.n; ++s) {
      const int r = n - parts.row0[s];
      if (r < 0 || r >= parts.rows[s]) continue;
      const float w = __expf(parts.lse[s][((long long)z * heads + h) * parts.rows[s] + r] - mx);
      if (w == 0.f) continue;
      sum += w;
      const uint4 u = *reinterpret_cast<const uint4*>(
          static_cast<const E*>(parts.o[s]) + (((long long)z * parts.rows[s] + r) * heads + h) * DR + part * 8);
      float fp[8];
      unpack8<E>(u, fp);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = fmaf(w, fp[i], f[i]);
    }
    const float inv = 1.f / sum;
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] *= inv;
  }
  *reinterpret_cast<uint4*>(out + row_id * DR + part * 8) = pack8<E>(f);
  if (part == 0)
    lse_out[((long long)z * heads + h) * rows + n] = mx > -CUDART_INF_F ? mx + __logf(sum) : -CUDART_INF_F;
}

}  // namespace fmha
