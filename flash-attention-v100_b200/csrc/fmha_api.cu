// C-ABI launch layer of the B200 attention library (declared in include/fmha_b200.h).
//
// Replaces the host launchers of the reference (kernel/fused_mha_kernel.cu:891-916): validate
// plain-pointer parameters, build the TMA tensor maps, raise the dynamic shared-memory limit,
// launch, and return a status.  Nothing here allocates device memory or synchronises.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "../../include/fmha_b200.h"
#include "aux_kernels.cuh"
#include "bwd_kernel.cuh"
#include "fwd_kernel.cuh"
#include "peer_kernels.cuh"

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  // resolved once; the pointer is process-wide and immutable afterwards
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) !=
            cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// 16-bit (Z, N, H, D) tensor with element strides -> 4-D map (D, N, H, Z), box 64 x box_rows x 1
// x 1, 128-byte swizzle, zero fill outside the tensor
int make_tensor_map(CUtensorMap* map, const void* base, int Z, int N, int H, int D,
                    const FmhaStrides& s, bool bf16, unsigned box_rows = 128) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return FMHA_ERR_NO_DEVICE;
  // a stride of a size-1 dimension is never used for addressing; make it well-formed
  const int64_t row = (N > 1) ? s.row : (int64_t)H * D;
  const int64_t head = (H > 1) ? s.head : (int64_t)D;
  const int64_t batch = (Z > 1) ? s.batch : row * N;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)Z};
  const cuuint64_t strides[3] = {(cuuint64_t)row * 2, (cuuint64_t)head * 2, (cuuint64_t)batch * 2};
  const cuuint32_t box[4] = {64, box_rows, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = encode(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                            4, const_cast<void*>(base), dims,
                            strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMHA_OK : FMHA_ERR_TENSOR_MAP;
}

// fp32 dQ accumulator (Z, N, H, D) contiguous -> 4-D map, box 32 x 128 x 1 x 1 (a tile's 128 query
// rows x 32 columns = 128-byte rows), 128-byte swizzle; used by TMA reduce-add
int make_accum_map(CUtensorMap* map, float* base, int Z, int N, int H, int D) {
  EncodeTiledFn encode = get_encode_fn();
  if (encode == nullptr) return FMHA_ERR_NO_DEVICE;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)N, (cuuint64_t)H, (cuuint64_t)Z};
  const cuuint64_t strides[3] = {(cuuint64_t)H * D * 4, (cuuint64_t)D * 4, (cuuint64_t)N * H * D * 4};
  const cuuint32_t box[4] = {32, 128, 1, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, base, dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FMHA_OK : FMHA_ERR_TENSOR_MAP;
}

// debug builds (-DFMHA_TIMELINE) set these through fmha_debug_set_timeline; otherwise unused
long long* g_timeline = nullptr;
int g_timeline_block = 0;

int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
    return 148;
  return n;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_strides(const FmhaStrides& s, int N, int H, int Z) {
  if ((N > 1 && (s.row % 8 != 0 || s.row <= 0)) || (H > 1 && (s.head % 8 != 0 || s.head <= 0)) ||
      (Z > 1 && (s.batch % 8 != 0 || s.batch <= 0)))
    return FMHA_ERR_BAD_STRIDE;
  return FMHA_OK;
}

int check_common(int batch, int heads, int seqlen_q, int seqlen_k, int head_dim, float scale,
                 int dtype = FMHA_DTYPE_FP16) {
  if (dtype != FMHA_DTYPE_FP16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_BAD_DTYPE;
  if (head_dim != 64 && head_dim != 96 && head_dim != 128) return FMHA_ERR_BAD_HEAD_DIM;
  if (batch <= 0 || heads <= 0 || seqlen_q <= 0 || seqlen_k <= 0) return FMHA_ERR_BAD_SHAPE;
  if (!std::isfinite(scale) || scale == 0.f) return FMHA_ERR_BAD_SHAPE;
  if ((long long)batch * heads * ((seqlen_q + 127) / 128 + 1) >= (1ll << 31) ||
      (long long)batch * heads * ((seqlen_k + 127) / 128 + 1) >= (1ll << 31))
    return FMHA_ERR_TOO_LARGE;
  return FMHA_OK;
}

// head_dim -> (D, DR) = (width the kernels run at, elements per row of the tensors):
// 64 -> (64, 64), 96 -> (128, 96), 128 -> (128, 128)
#define FMHA_DISPATCH_DIMS(head_dim, ...)       \
  if ((head_dim) == 128) {                      \
    constexpr int D = 128, DR = 128;            \
    __VA_ARGS__                                 \
  } else if ((head_dim) == 96) {                \
    constexpr int D = 128, DR = 96;             \
    __VA_ARGS__                                 \
  } else {                                      \
    constexpr int D = 64, DR = 64;              \
    __VA_ARGS__                                 \
  }

fmha::Strides3 to3(const FmhaStrides& s) { return fmha::Strides3{s.batch, s.row, s.head}; }

int round_up_128(int x) { return (x + 127) / 128 * 128; }

// Heads whose CTAs are interleaved in the backward grid (see the coordinates in bwd_kernel.cuh),
// for up to 32 KV tiles per head.  Measured on the fused kernel at Z=8, H=32, N=2048, D=128,
// alternating runs: causal 0.809 ms with one head at a time, 0.794 with groups of 4, 0.778 with 8,
// 0.771 with 16, 0.770 with 24, 0.769 with 32, 0.773 with 37 (the last CTAs of a group and of the
// grid being the short ones); without a mask, where all CTAs are equally long and only the L2
// matters, 1.351 ms with 8 against 1.37-1.40 with 16 to 37.  Longer sequences keep one head at a
// time: their grids are long, and many heads' query tiles would not share the L2.
// FMHA_BWD_HEAD_GROUP overrides (tuning experiments).
int bwd_head_group(int num_kv_blocks, bool causal) {
  static const int forced = []() {
    const char* e = std::getenv("FMHA_BWD_HEAD_GROUP");
    return e != nullptr ? std::atoi(e) : 0;
  }();
  if (forced >= 1) return forced;
  if (num_kv_blocks > 32) return 1;
  return causal ? 16 : 8;
}

struct BwdWorkspace {
  float* dq_accum;
  float* lse2;
  float* delta;
  int* dq_order;       // one word per (batch*head, query tile): FMHA_BWD_DETERMINISTIC
  size_t order_bytes;
  size_t bytes;
};

BwdWorkspace carve_workspace(void* ws, int Z, int H, int Nq, int D) {
  BwdWorkspace w;
  const size_t dq_bytes = (size_t)Z * Nq * H * D * sizeof(float);  // multiple of 256
  const size_t stat_bytes = (size_t)Z * H * round_up_128(Nq) * sizeof(float);
  char* base = static_cast<char*>(ws);
  w.dq_accum = reinterpret_cast<float*>(base);
  w.lse2 = reinterpret_cast<float*>(base + dq_bytes);
  w.delta = reinterpret_cast<float*>(base + dq_bytes + stat_bytes);
  w.dq_order = reinterpret_cast<int*>(base + dq_bytes + 2 * stat_bytes);
  w.order_bytes = (size_t)Z * H * (round_up_128(Nq) / 128) * sizeof(int);
  w.bytes = dq_bytes + 2 * stat_bytes + (w.order_bytes + 255) / 256 * 256;
  return w;
}

// D is the head dimension the kernel runs at; the tensors have p->head_dim <= D elements per row
// (96 runs at D = 128: the tensor maps describe 96 columns, the loads fill the rest of a
// 128-wide tile with zeros and the stores clip it)
template <int D, bool kBf16>
int launch_fwd(const FmhaFwdParams* p, cudaStream_t stream) {
  using T = fmha::FwdTraits<D, kBf16>;
  CUtensorMap tq, tk, tv, to;
  int rc;
  const int Dr = p->head_dim;
  if ((rc = make_tensor_map(&tq, p->q, p->batch, p->seqlen_q, p->heads, Dr, p->q_strides, kBf16)))
    return rc;
  // K and V are loaded in half tiles of kStepN rows
  if ((rc = make_tensor_map(&tk, p->k, p->batch, p->seqlen_k, p->heads, Dr, p->k_strides, kBf16,
                            T::kStepN)))
    return rc;
  if ((rc = make_tensor_map(&tv, p->v, p->batch, p->seqlen_k, p->heads, Dr, p->v_strides, kBf16,
                            T::kStepN)))
    return rc;
  if ((rc = make_tensor_map(&to, p->o, p->batch, p->seqlen_q, p->heads, Dr, p->o_strides, kBf16)))
    return rc;
  fmha::FwdKernelParams kp;
  kp.lse = p->lse;
  kp.heads = p->heads;
  kp.seqlen_q = p->seqlen_q;
  kp.seqlen_k = p->seqlen_k;
  kp.num_q_blocks = (p->seqlen_q + 255) / 256;
  kp.num_heads_total = p->batch * p->heads;
  kp.scale_log2 = p->scale * 1.4426950408889634f;
  kp.causal = p->causal ? 1 : 0;
  kp.causal_shift = p->causal_shift;
  kp.status = p->status;
  kp.seqused_q = p->seqused_q;
  kp.seqused_k = p->seqused_k;
  kp.timeline = g_timeline;
  kp.timeline_block = g_timeline_block;
  auto kernel = fmha::fmha_fwd_kernel<D, kBf16>;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes) !=
      cudaSuccess)
    return FMHA_ERR_LAUNCH;
  // persistent grid: one CTA per SM (or per super-item = pair of query blocks, if fewer)
  const long long n_super = (long long)((kp.num_q_blocks + 1) / 2) * kp.num_heads_total;
  const int sms = std::max(1, sm_count() - std::max(0, (int)p->sm_margin));
  const unsigned grid = (unsigned)std::min<long long>(n_super, sms);
  kernel<<<grid, T::kThreads, T::kSmemBytes, stream>>>(tq, tk, tv, to, kp);
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

// D: the head dimension the kernels run at; DR <= D: what the tensors have (p->head_dim)
template <int D, bool kBf16, int DR = D>
int launch_bwd(const FmhaBwdParams* p, const BwdWorkspace& w, cudaStream_t stream) {
  using T = fmha::BwdTraits<D, kBf16>;
  using E = typename std::conditional<kBf16, __nv_bfloat16, __half>::type;
  const int Z = p->batch, H = p->heads, Nq = p->seqlen_q, Nk = p->seqlen_k;
  const int Nq_pad = round_up_128(Nq);
  constexpr int Dr = DR;

  if (!(p->flags & FMHA_BWD_KEEP_WORKSPACE)) {
    const long long rows = (long long)Z * H * Nq_pad;
    constexpr int rows_per_block = 256 / (D / 8);
    const unsigned grid = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    fmha::fmha_bwd_preprocess_kernel<D, E, DR><<<grid, 256, 0, stream>>>(
        static_cast<const E*>(p->o), to3(p->o_strides), static_cast<const E*>(p->dout),
        to3(p->dout_strides), p->lse, w.dq_accum, w.lse2, w.delta, H, Nq, Nq_pad, rows, p->seqused_q);
    if (cudaGetLastError() != cudaSuccess) return FMHA_ERR_LAUNCH;
  }
  if (p->flags & FMHA_BWD_PREPROCESS_ONLY) return FMHA_OK;

  {
    CUtensorMap tq, tk, tv, tdo, tdk, tdv, tacc;
    int rc;
    if ((rc = make_accum_map(&tacc, w.dq_accum, Z, Nq, H, Dr))) return rc;
    if ((rc = make_tensor_map(&tq, p->q, Z, Nq, H, Dr, p->q_strides, kBf16))) return rc;
    if ((rc = make_tensor_map(&tk, p->k, Z, Nk, H, Dr, p->k_strides, kBf16))) return rc;
    if ((rc = make_tensor_map(&tv, p->v, Z, Nk, H, Dr, p->v_strides, kBf16))) return rc;
    if ((rc = make_tensor_map(&tdo, p->dout, Z, Nq, H, Dr, p->dout_strides, kBf16))) return rc;
    // with fp32 accumulation the fp16 outputs are not touched: any valid map will do
    const bool acc_k = p->dk_accum != nullptr, acc_v = p->dv_accum != nullptr;
    if ((rc = make_tensor_map(&tdk, acc_k ? p->k : p->dk, Z, Nk, H, Dr,
                              acc_k ? p->k_strides : p->dk_strides, kBf16)))
      return rc;
    if ((rc = make_tensor_map(&tdv, acc_v ? p->v : p->dv, Z, Nk, H, Dr,
                              acc_v ? p->v_strides : p->dv_strides, kBf16)))
      return rc;
    fmha::BwdKernelParams kp;
    kp.lse2 = w.lse2;
    kp.delta = w.delta;
    kp.dk_accum = p->dk_accum;
    kp.dv_accum = p->dv_accum;
    kp.accum_batch_stride =
        p->accum_batch_stride > 0 ? p->accum_batch_stride : (long long)Nk * H * Dr;
    kp.accum_overwrite = (p->flags & FMHA_BWD_ACCUM_OVERWRITE) ? 1 : 0;
    kp.heads = H;
    kp.seqlen_q = Nq;
    kp.seqlen_k = Nk;
    kp.seqlen_q_pad = Nq_pad;
    kp.num_kv_blocks = (Nk + 127) / 128;
    kp.num_heads_total = Z * H;
    kp.head_group = bwd_head_group(kp.num_kv_blocks, p->causal != 0);
    kp.q_tile_begin = p->q_row_begin / 128;
    kp.scale = p->scale;
    kp.scale_log2 = p->scale * 1.4426950408889634f;
    kp.causal = p->causal ? 1 : 0;
    kp.causal_shift = p->causal_shift;
    kp.status = p->status;
    kp.seqused_q = p->seqused_q;
    kp.seqused_k = p->seqused_k;
    kp.dq_order = nullptr;
    if (p->flags & FMHA_BWD_DETERMINISTIC) {
      // a memset node, not an allocation; every call starts its own count at zero
      if (cudaMemsetAsync(w.dq_order, 0, w.order_bytes, stream) != cudaSuccess) return FMHA_ERR_LAUNCH;
      kp.dq_order = w.dq_order;
    }
    kp.timeline = g_timeline;
    kp.timeline_block = g_timeline_block;
    auto kernel = fmha::fmha_bwd_kernel<D, kBf16, DR>;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T::kSmemBytes) !=
        cudaSuccess)
      return FMHA_ERR_LAUNCH;
    const unsigned grid = (unsigned)((long long)kp.num_kv_blocks * H * Z);
    kernel<<<grid, T::kThreads, T::kSmemBytes, stream>>>(tq, tk, tv, tdo, tdk, tdv, tacc, kp);
    if (cudaGetLastError() != cudaSuccess) return FMHA_ERR_LAUNCH;
  }

  if (!(p->flags & FMHA_BWD_SKIP_DQ_CONVERT)) {
    const long long rows = (long long)Z * Nq * H;
    constexpr int rows_per_block = 256 / (D / 8);
    const unsigned grid = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
    fmha::fmha_bwd_convert_dq_kernel<D, E, DR><<<grid, 256, 0, stream>>>(
        w.dq_accum, static_cast<E*>(p->dq), to3(p->dq_strides), H, Nq, p->scale, rows);
    if (cudaGetLastError() != cudaSuccess) return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

FmhaStrides dense_strides(int n, int head, int k) {
  FmhaStrides s;
  s.head = k;
  s.row = (int64_t)head * k;
  s.batch = (int64_t)n * head * k;
  return s;
}

// ---------------------------------------------------------------------------------------
// Built-in scratch for fmha_bwd_static_scratch: part of the device image, so it exists on every
// GPU that loads the library and costs no allocation call at run time.
// In HOST code the name below is only a handle for cudaGetSymbolAddress: it is not a device
// address and must never be handed to a kernel.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_fmha_static_scratch[FMHA_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
std::atomic<void*> g_static_scratch_addr[kMaxDevices];  // per device, filled on first use

// Device address of the scratch area on the CURRENT device, or nullptr (rc set) on failure.
void* static_scratch_for_current_device(int* rc) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *rc = FMHA_ERR_NO_DEVICE;
    return nullptr;
  }
  void* ptr = g_static_scratch_addr[dev].load(std::memory_order_acquire);
  if (ptr == nullptr) {
    // once per device, with that device current; the address differs from device to device
    if (cudaGetSymbolAddress(&ptr, g_fmha_static_scratch) != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      *rc = FMHA_ERR_NO_DEVICE;
      return nullptr;
    }
    g_static_scratch_addr[dev].store(ptr, std::memory_order_release);
  }
  *rc = FMHA_OK;
  return ptr;
}

}  // namespace

extern "C" {

int fmha_fwd(const FmhaFwdParams* p, void* stream) {
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->o == nullptr ||
      p->lse == nullptr)
    return FMHA_ERR_NULL_POINTER;
  int rc = check_common(p->batch, p->heads, p->seqlen_q, p->seqlen_k, p->head_dim, p->scale, p->dtype);
  if (rc) return rc;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->o))
    return FMHA_ERR_BAD_ALIGNMENT;
  if ((rc = check_strides(p->q_strides, p->seqlen_q, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->k_strides, p->seqlen_k, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->v_strides, p->seqlen_k, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->o_strides, p->seqlen_q, p->heads, p->batch))) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->dtype == FMHA_DTYPE_BF16)
    return p->head_dim > 64 ? launch_fwd<128, true>(p, s) : launch_fwd<64, true>(p, s);
  return p->head_dim > 64 ? launch_fwd<128, false>(p, s) : launch_fwd<64, false>(p, s);
}

size_t fmha_bwd_workspace_bytes(const FmhaBwdParams* p) {
  if (p == nullptr || p->batch <= 0 || p->heads <= 0 || p->seqlen_q <= 0 || p->head_dim <= 0)
    return 0;
  return carve_workspace(nullptr, p->batch, p->heads, p->seqlen_q, p->head_dim).bytes;
}

int fmha_bwd(const FmhaBwdParams* p, void* workspace, size_t workspace_bytes, void* stream) {
  if (p == nullptr || p->q == nullptr || p->k == nullptr || p->v == nullptr || p->dout == nullptr ||
      p->lse == nullptr)
    return FMHA_ERR_NULL_POINTER;
  const bool keep = (p->flags & FMHA_BWD_KEEP_WORKSPACE) != 0;
  const bool pre_only = (p->flags & FMHA_BWD_PREPROCESS_ONLY) != 0;
  const bool skip_convert = pre_only || (p->flags & FMHA_BWD_SKIP_DQ_CONVERT) != 0;
  if (keep && pre_only) return FMHA_ERR_WORKSPACE;
  if (!keep && p->o == nullptr) return FMHA_ERR_NULL_POINTER;
  if (!skip_convert && p->dq == nullptr) return FMHA_ERR_NULL_POINTER;
  if (p->dk_accum == nullptr && p->dk == nullptr) return FMHA_ERR_NULL_POINTER;
  if (p->dv_accum == nullptr && p->dv == nullptr) return FMHA_ERR_NULL_POINTER;
  int rc = check_common(p->batch, p->heads, p->seqlen_q, p->seqlen_k, p->head_dim, p->scale, p->dtype);
  if (rc) return rc;
  if (!aligned16(p->q) || !aligned16(p->k) || !aligned16(p->v) || !aligned16(p->dout) ||
      (!keep && !aligned16(p->o)) || (!skip_convert && !aligned16(p->dq)) ||
      (p->dk_accum == nullptr && !aligned16(p->dk)) || (p->dv_accum == nullptr && !aligned16(p->dv)) ||
      !aligned16(p->dk_accum) || !aligned16(p->dv_accum))
    return FMHA_ERR_BAD_ALIGNMENT;
  if ((rc = check_strides(p->q_strides, p->seqlen_q, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->k_strides, p->seqlen_k, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->v_strides, p->seqlen_k, p->heads, p->batch))) return rc;
  if ((rc = check_strides(p->dout_strides, p->seqlen_q, p->heads, p->batch))) return rc;
  if (!keep && (rc = check_strides(p->o_strides, p->seqlen_q, p->heads, p->batch))) return rc;
  if (!skip_convert && (rc = check_strides(p->dq_strides, p->seqlen_q, p->heads, p->batch)))
    return rc;
  if (p->dk_accum == nullptr && (rc = check_strides(p->dk_strides, p->seqlen_k, p->heads, p->batch)))
    return rc;
  if (p->dv_accum == nullptr && (rc = check_strides(p->dv_strides, p->seqlen_k, p->heads, p->batch)))
    return rc;
  if (p->q_row_begin < 0 || p->q_row_begin % 128 != 0 ||
      (p->q_row_begin != 0 && p->q_row_begin >= p->seqlen_q))
    return FMHA_ERR_BAD_SHAPE;
  if (p->dk_accum != nullptr || p->dv_accum != nullptr) {
    // the epilogue adds with 16-byte accesses at accum + z * stride: the stride must keep them
    // aligned, and batch entries must not overlap
    const int64_t st = p->accum_batch_stride;
    if (st < 0 || (st != 0 && (st % 4 != 0 || st < (int64_t)p->seqlen_k * p->heads * p->head_dim)))
      return FMHA_ERR_BAD_STRIDE;
  }
  const BwdWorkspace w = carve_workspace(workspace, p->batch, p->heads, p->seqlen_q, p->head_dim);
  if (workspace == nullptr || workspace_bytes < w.bytes) return FMHA_ERR_WORKSPACE;
  if (!aligned16(workspace)) return FMHA_ERR_BAD_ALIGNMENT;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (p->dtype == FMHA_DTYPE_BF16)
    return p->head_dim == 128 ? launch_bwd<128, true>(p, w, s)
           : p->head_dim == 96 ? launch_bwd<128, true, 96>(p, w, s)
                               : launch_bwd<64, true>(p, w, s);
  return p->head_dim == 128 ? launch_bwd<128, false>(p, w, s)
         : p->head_dim == 96 ? launch_bwd<128, false, 96>(p, w, s)
                             : launch_bwd<64, false>(p, w, s);
}

int fmha_bwd_static_scratch(const FmhaBwdParams* p, void* stream) {
  if (p == nullptr) return FMHA_ERR_NULL_POINTER;
  // the shared area cannot carry an accumulator over from an earlier call, nor hand an
  // unconverted fp32 dQ to a later one (the caller has no address for it)
  if (p->flags & (FMHA_BWD_KEEP_WORKSPACE | FMHA_BWD_PREPROCESS_ONLY | FMHA_BWD_SKIP_DQ_CONVERT))
    return FMHA_ERR_WORKSPACE;
  if (p->batch <= 0 || p->heads <= 0 || p->seqlen_q <= 0 || p->head_dim <= 0)
    return FMHA_ERR_BAD_SHAPE;
  const size_t need = fmha_bwd_workspace_bytes(p);
  if (need == 0 || need > (size_t)FMHA_STATIC_SCRATCH_BYTES) return FMHA_ERR_TOO_LARGE;
  int rc = FMHA_OK;
  void* scratch = static_scratch_for_current_device(&rc);
  if (scratch == nullptr) return rc;
  // same validation, kernels and launch order as the caller-workspace entry point
  return fmha_bwd(p, scratch, (size_t)FMHA_STATIC_SCRATCH_BYTES, stream);
}

int fmha_bwd_convert_dq(const void* workspace, void* dq, FmhaStrides dq_strides, int32_t batch,
                        int32_t heads, int32_t seqlen_q, int32_t head_dim, float scale,
                        int32_t dtype, void* stream) {
  if (workspace == nullptr || dq == nullptr) return FMHA_ERR_NULL_POINTER;
  if (dtype != FMHA_DTYPE_FP16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_BAD_DTYPE;
  if (head_dim != 64 && head_dim != 96 && head_dim != 128) return FMHA_ERR_BAD_HEAD_DIM;
  if (batch <= 0 || heads <= 0 || seqlen_q <= 0) return FMHA_ERR_BAD_SHAPE;
  if (!aligned16(workspace) || !aligned16(dq)) return FMHA_ERR_BAD_ALIGNMENT;
  int rc = check_strides(dq_strides, seqlen_q, heads, batch);
  if (rc) return rc;
  const long long rows = (long long)batch * seqlen_q * heads;
  const int rows_per_block = 256 / ((head_dim > 64 ? 128 : 64) / 8);  // 16 or 8 threads per row
  const unsigned grid = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const float* acc = static_cast<const float*>(workspace);
  const fmha::Strides3 sd = to3(dq_strides);
  if (dtype == FMHA_DTYPE_BF16) {
    auto* out = static_cast<__nv_bfloat16*>(dq);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::fmha_bwd_convert_dq_kernel<D, __nv_bfloat16, DR><<<grid, 256, 0, s>>>(
                           acc, out, sd, heads, seqlen_q, scale, rows);)
  } else {
    auto* out = static_cast<__half*>(dq);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::fmha_bwd_convert_dq_kernel<D, __half, DR><<<grid, 256, 0, s>>>(
                           acc, out, sd, heads, seqlen_q, scale, rows);)
  }
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_merge_rows(float* o_acc, float* lse_acc, const void* o_part, FmhaStrides o_part_strides,
                    const float* lse_part, void* o_out, int32_t batch, int32_t heads, int32_t rows,
                    int32_t acc_rows, int32_t row_offset, int32_t head_dim, int32_t dtype,
                    void* stream) {
  if (o_acc == nullptr || lse_acc == nullptr || o_part == nullptr || lse_part == nullptr)
    return FMHA_ERR_NULL_POINTER;
  if (dtype != FMHA_DTYPE_FP16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_BAD_DTYPE;
  if (head_dim != 64 && head_dim != 96 && head_dim != 128) return FMHA_ERR_BAD_HEAD_DIM;
  if (batch <= 0 || heads <= 0 || rows <= 0 || row_offset < 0 ||
      (long long)row_offset + rows > (long long)acc_rows)
    return FMHA_ERR_BAD_SHAPE;
  if (!aligned16(o_acc) || !aligned16(o_part) || !aligned16(o_out)) return FMHA_ERR_BAD_ALIGNMENT;
  int rc = check_strides(o_part_strides, rows, heads, batch);
  if (rc) return rc;
  const long long total = (long long)batch * rows * heads;
  const int rows_per_block = 256 / ((head_dim > 64 ? 128 : 64) / 8);  // 16 or 8 threads per row
  const unsigned grid = (unsigned)((total + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fmha::Strides3 sp = to3(o_part_strides);
  if (dtype == FMHA_DTYPE_BF16) {
    auto* part = static_cast<const __nv_bfloat16*>(o_part);
    auto* out = static_cast<__nv_bfloat16*>(o_out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::fmha_merge_kernel<D, __nv_bfloat16, DR><<<grid, 256, 0, s>>>(
                           o_acc, lse_acc, part, sp, lse_part, out, heads, rows, acc_rows, row_offset, total);)
  } else {
    auto* part = static_cast<const __half*>(o_part);
    auto* out = static_cast<__half*>(o_out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::fmha_merge_kernel<D, __half, DR><<<grid, 256, 0, s>>>(
                           o_acc, lse_acc, part, sp, lse_part, out, heads, rows, acc_rows, row_offset, total);)
  }
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_merge(float* o_acc, float* lse_acc, const void* o_part, FmhaStrides o_part_strides,
               const float* lse_part, void* o_out, int32_t batch, int32_t heads, int32_t rows,
               int32_t head_dim, int32_t dtype, void* stream) {
  return fmha_merge_rows(o_acc, lse_acc, o_part, o_part_strides, lse_part, o_out, batch, heads,
                         rows, rows, 0, head_dim, dtype, stream);
}

// ---------------------------------------------------------------------------------------
// multi-GPU plumbing
// ---------------------------------------------------------------------------------------
int fmha_ipc_export(const void* ptr, void* handle64, int64_t* offset) {
  if (ptr == nullptr || handle64 == nullptr || offset == nullptr) return FMHA_ERR_NULL_POINTER;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the header promises 64 bytes");
  using RangeFn = CUresult (*)(CUdeviceptr*, size_t*, CUdeviceptr);
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return FMHA_ERR_NO_DEVICE;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (reinterpret_cast<RangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS)
    return FMHA_ERR_BAD_ALIGNMENT;
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)) != cudaSuccess) {
    (void)cudaGetLastError();
    return FMHA_ERR_LAUNCH;
  }
  std::memcpy(handle64, &h, sizeof(h));
  *offset = (int64_t)(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return FMHA_OK;
}

int fmha_ipc_open(const void* handle64, int64_t offset, void** ptr) {
  if (handle64 == nullptr || ptr == nullptr) return FMHA_ERR_NULL_POINTER;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
    (void)cudaGetLastError();
    return FMHA_ERR_LAUNCH;
  }
  *ptr = static_cast<char*>(base) + offset;
  return FMHA_OK;
}

int fmha_ipc_close(void* ptr, int64_t offset) {
  if (ptr == nullptr) return FMHA_ERR_NULL_POINTER;
  if (cudaIpcCloseMemHandle(static_cast<char*>(ptr) - offset) != cudaSuccess) {
    (void)cudaGetLastError();
    return FMHA_ERR_LAUNCH;
  }
  return FMHA_OK;
}

int fmha_peer_copy(void* dst, const void* src, size_t bytes, void* stream) {
  if (dst == nullptr || src == nullptr) return FMHA_ERR_NULL_POINTER;
  if (bytes == 0) return FMHA_OK;
  return cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? FMHA_OK
             : FMHA_ERR_LAUNCH;
}

int fmha_peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t row_bytes, size_t rows, void* stream) {
  if (dst == nullptr || src == nullptr) return FMHA_ERR_NULL_POINTER;
  if (row_bytes == 0 || rows == 0) return FMHA_OK;
  if (row_bytes > dst_pitch || row_bytes > src_pitch) return FMHA_ERR_BAD_STRIDE;
  return cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, row_bytes, rows, cudaMemcpyDefault,
                           static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? FMHA_OK
             : FMHA_ERR_LAUNCH;
}

int fmha_counter_bump(int32_t* word, void* stream) {
  if (word == nullptr) return FMHA_ERR_NULL_POINTER;
  fmha::counter_bump_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(word);
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_peer_signal(int32_t* const* flags, int32_t n, const int32_t* value, void* stream) {
  if (flags == nullptr || value == nullptr) return FMHA_ERR_NULL_POINTER;
  if (n <= 0) return FMHA_OK;
  if (n > fmha::kMaxPeers) return FMHA_ERR_TOO_LARGE;
  fmha::PeerFlagList list;
  list.n = n;
  for (int i = 0; i < n; ++i) {
    if (flags[i] == nullptr) return FMHA_ERR_NULL_POINTER;
    list.ptr[i] = flags[i];
  }
  fmha::peer_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(list, value);
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_peer_wait(const int32_t* const* flags, int32_t n, const int32_t* value, int32_t* status,
                   int32_t timeout_ms, void* stream) {
  if (flags == nullptr || value == nullptr) return FMHA_ERR_NULL_POINTER;
  if (n <= 0) return FMHA_OK;
  if (n > fmha::kMaxPeers) return FMHA_ERR_TOO_LARGE;
  if (timeout_ms <= 0 || timeout_ms > 60000) return FMHA_ERR_BAD_SHAPE;
  fmha::PeerFlagList list;
  list.n = n;
  for (int i = 0; i < n; ++i) {
    if (flags[i] == nullptr) return FMHA_ERR_NULL_POINTER;
    list.ptr[i] = const_cast<int*>(flags[i]);
  }
  fmha::peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      list, value, status, (unsigned long long)timeout_ms * 1000000ull);
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_sum_partials(const float* const* parts, const int32_t* rows_per_part, int32_t n_parts,
                      void* out, FmhaStrides out_strides, int32_t batch, int32_t heads, int32_t rows,
                      int32_t head_dim, int32_t dtype, void* stream) {
  if (parts == nullptr || rows_per_part == nullptr || out == nullptr) return FMHA_ERR_NULL_POINTER;
  if (dtype != FMHA_DTYPE_FP16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_BAD_DTYPE;
  if (head_dim != 64 && head_dim != 96 && head_dim != 128) return FMHA_ERR_BAD_HEAD_DIM;
  if (batch <= 0 || heads <= 0 || rows <= 0 || n_parts <= 0) return FMHA_ERR_BAD_SHAPE;
  if (n_parts > fmha::kMaxPeers) return FMHA_ERR_TOO_LARGE;
  if (!aligned16(out)) return FMHA_ERR_BAD_ALIGNMENT;
  int rc = check_strides(out_strides, rows, heads, batch);
  if (rc) return rc;
  fmha::PartList list;
  list.n = n_parts;
  for (int i = 0; i < n_parts; ++i) {
    if (parts[i] == nullptr) return FMHA_ERR_NULL_POINTER;
    if (!aligned16(parts[i])) return FMHA_ERR_BAD_ALIGNMENT;
    if (rows_per_part[i] < 0 || rows_per_part[i] > rows) return FMHA_ERR_BAD_SHAPE;
    list.ptr[i] = parts[i];
    list.rows[i] = rows_per_part[i];
  }
  const long long total = (long long)batch * rows * heads;
  const int rows_per_block = 256 / ((head_dim > 64 ? 128 : 64) / 8);  // 16 or 8 threads per row
  const unsigned grid = (unsigned)((total + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const fmha::Strides3 so = to3(out_strides);
  if (dtype == FMHA_DTYPE_BF16) {
    auto* o = static_cast<__nv_bfloat16*>(out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::sum_partials_kernel<D, __nv_bfloat16, DR><<<grid, 256, 0, s>>>(
                           list, o, so, heads, rows, total);)
  } else {
    auto* o = static_cast<__half*>(out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::sum_partials_kernel<D, __half, DR><<<grid, 256, 0, s>>>(
                           list, o, so, heads, rows, total);)
  }
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_merge_parts(const void* const* o_parts, const float* const* lse_parts,
                     const int32_t* row_offset, const int32_t* rows_per_part, int32_t n_parts,
                     void* o_out, float* lse_out, int32_t batch, int32_t heads, int32_t rows,
                     int32_t head_dim, int32_t dtype, void* stream) {
  if (o_parts == nullptr || lse_parts == nullptr || row_offset == nullptr || rows_per_part == nullptr ||
      o_out == nullptr || lse_out == nullptr)
    return FMHA_ERR_NULL_POINTER;
  if (dtype != FMHA_DTYPE_FP16 && dtype != FMHA_DTYPE_BF16) return FMHA_ERR_BAD_DTYPE;
  if (head_dim != 64 && head_dim != 96 && head_dim != 128) return FMHA_ERR_BAD_HEAD_DIM;
  if (batch <= 0 || heads <= 0 || rows <= 0 || n_parts <= 0) return FMHA_ERR_BAD_SHAPE;
  if (n_parts > fmha::kMaxPeers) return FMHA_ERR_TOO_LARGE;
  if (!aligned16(o_out)) return FMHA_ERR_BAD_ALIGNMENT;
  fmha::MergeList list;
  list.n = n_parts;
  for (int i = 0; i < n_parts; ++i) {
    if (o_parts[i] == nullptr || lse_parts[i] == nullptr) return FMHA_ERR_NULL_POINTER;
    if (!aligned16(o_parts[i])) return FMHA_ERR_BAD_ALIGNMENT;
    if (rows_per_part[i] <= 0 || row_offset[i] < 0 ||
        (long long)row_offset[i] + rows_per_part[i] > (long long)rows)
      return FMHA_ERR_BAD_SHAPE;
    list.o[i] = o_parts[i];
    list.lse[i] = lse_parts[i];
    list.row0[i] = row_offset[i];
    list.rows[i] = rows_per_part[i];
  }
  const long long total = (long long)batch * rows * heads;
  const int rows_per_block = 256 / ((head_dim > 64 ? 128 : 64) / 8);  // 16 or 8 threads per row
  const unsigned grid = (unsigned)((total + rows_per_block - 1) / rows_per_block);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == FMHA_DTYPE_BF16) {
    auto* o = static_cast<__nv_bfloat16*>(o_out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::merge_parts_kernel<D, __nv_bfloat16, DR><<<grid, 256, 0, s>>>(
                           list, o, lse_out, heads, rows, total);)
  } else {
    auto* o = static_cast<__half*>(o_out);
    FMHA_DISPATCH_DIMS(head_dim,
                       fmha::merge_parts_kernel<D, __half, DR><<<grid, 256, 0, s>>>(
                           list, o, lse_out, heads, rows, total);)
  }
  return cudaGetLastError() == cudaSuccess ? FMHA_OK : FMHA_ERR_LAUNCH;
}

int fmha_b200_forward(const void* query_ptr, const void* key_ptr, const void* value_ptr,
                      void* output_ptr, void* lse_ptr, int batch, int head, int m, int n, int k,
                      float scale, int causal, void* stream) {
  FmhaFwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = query_ptr;
  p.k = key_ptr;
  p.v = value_ptr;
  p.o = output_ptr;
  p.lse = static_cast<float*>(lse_ptr);
  p.q_strides = p.o_strides = dense_strides(m, head, k);
  p.k_strides = p.v_strides = dense_strides(n, head, k);
  p.batch = batch;
  p.heads = head;
  p.seqlen_q = m;
  p.seqlen_k = n;
  p.head_dim = k;
  p.scale = scale;
  p.causal = causal;
  return fmha_fwd(&p, stream);
}

int fmha_b200_backward(const void* query_ptr, const void* key_ptr, const void* value_ptr,
                       const void* output_ptr, const void* d_output_ptr, const void* lse_ptr,
                       void* d_query_ptr, void* d_key_ptr, void* d_value_ptr, void* workspace,
                       size_t workspace_bytes, int batch, int head, int m, int n, int k,
                       float scale, int causal, void* stream) {
  FmhaBwdParams p;
  std::memset(&p, 0, sizeof(p));
  p.q = query_ptr;
  p.k = key_ptr;
  p.v = value_ptr;
  p.o = output_ptr;
  p.dout = d_output_ptr;
  p.lse = static_cast<const float*>(lse_ptr);
  p.dq = d_query_ptr;
  p.dk = d_key_ptr;
  p.dv = d_value_ptr;
  p.q_strides = p.o_strides = p.dout_strides = p.dq_strides = dense_strides(m, head, k);
  p.k_strides = p.v_strides = p.dk_strides = p.dv_strides = dense_strides(n, head, k);
  p.batch = batch;
  p.heads = head;
  p.seqlen_q = m;
  p.seqlen_k = n;
  p.head_dim = k;
  p.scale = scale;
  p.causal = causal;
  return fmha_bwd(&p, workspace, workspace_bytes, stream);
}

const char* fmha_status_string(int status) {
  switch (status) {
    case FMHA_OK: return "ok";
    case FMHA_ERR_NULL_POINTER: return "a required pointer is NULL";
    case FMHA_ERR_BAD_HEAD_DIM: return "head_dim must be 64, 96 or 128";
    case FMHA_ERR_BAD_SHAPE: return "sizes must be positive and scale finite and non-zero";
    case FMHA_ERR_BAD_STRIDE: return "strides must be positive multiples of 8 elements";
    case FMHA_ERR_BAD_ALIGNMENT: return "pointers must be 16-byte aligned";
    case FMHA_ERR_WORKSPACE: return "backward workspace missing or too small";
    case FMHA_ERR_TENSOR_MAP: return "cuTensorMapEncodeTiled rejected a tensor";
    case FMHA_ERR_NO_DEVICE: return "CUDA driver entry point unavailable";
    case FMHA_ERR_LAUNCH: return "kernel launch failed";
    case FMHA_ERR_TOO_LARGE: return "a size exceeds the supported maximum";
    case FMHA_ERR_BAD_DTYPE: return "dtype must be FMHA_DTYPE_FP16 or FMHA_DTYPE_BF16";
    default: return "unknown status";
  }
}

const char* fmha_version(void) { return "0.2.0"; }

#ifdef FMHA_TIMELINE
// debug builds only: device buffer (>= 3 * 512 int64) and the CTA whose events are recorded
void fmha_debug_set_timeline(long long* buf, int block) {
  g_timeline = buf;
  g_timeline_block = block;
}
#endif

}  // extern "C"
