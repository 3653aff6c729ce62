// Thin inline-PTX wrappers for the sm_100a primitives the attention kernels use:
// mbarrier, TMA tensor copies (load / store / reduce-add, each issued by one CTA for itself),
// tcgen05 (TMEM allocation, MMA issue, commit, TMEM load/store) and the UMMA
// shared-memory / instruction descriptors.
//
// Every wait in here is bounded: a wait that runs out records an error code in a
// shared abort word (and the caller copies it to a global status word), after which
// every later wait in the CTA returns at once so that the CTA can drain and exit.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Timeline instrumentation, compiled in only with -DFMHA_TIMELINE: the chosen CTA's elected
// threads store clock64() at pipeline events so that stalls can be located without a profiler.
#ifndef FMHA_ABLATE
#define FMHA_ABLATE 0  // debug builds: bit 0 no exp2, bit 1 no row max, bit 2 no P store
#endif
#ifdef FMHA_TIMELINE
#define FMHA_TL(role, j, k)                                                        \
  do {                                                                              \
    if (p.timeline != nullptr && (int)blockIdx.x == p.timeline_block && (j) < 32)  \
      p.timeline[(role)*512 + (j)*16 + (k)] = clock64();                           \
  } while (0)
#else
#define FMHA_TL(role, j, k) \
  do {                      \
  } while (0)
#endif

namespace fmha {

// ---------------------------------------------------------------------------------
// error codes written to the status word (0 = ok)
// ---------------------------------------------------------------------------------
enum : int {
  kErrNone = 0,
  kErrWaitTimeout = 0x100,  // low byte = id of the barrier class that timed out
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31u; }

// ---------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// orders accesses of the generic proxy (ordinary loads / stores, flags) with those of the async
// proxy (TMA copies and reductions), all state spaces
__device__ __forceinline__ void fence_proxy_async_all() {
  asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait. `abort_word` is a word in shared memory shared by the whole CTA:
// non-zero means some wait already ran out, and every wait then returns false at once.
// The limit (about 2^22 polls, each a try_wait with the hardware's own short suspend)
// is seconds of wall time, far above any legitimate wait in these kernels.
constexpr uint32_t kWaitPollLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_word,
                                          int who) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_word != 0) return false;  // some wait already gave up: drain without polling
  for (uint32_t i = 0; i < kWaitPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_word != 0) return false;
  }
  atomicCAS(const_cast<int*>(abort_word), 0, kErrWaitTimeout | (who & 0xff));
  return false;
}

// Bounded wait for a word in global memory to reach `want`; another CTA of the same grid with a
// LOWER block index sets it (blocks are dispatched in index order, so that CTA is running or
// done).  Gives up at once when this CTA, or the grid (status word), is already aborting.
constexpr uint32_t kFlagPollLimit = 1u << 21;
__device__ __forceinline__ bool global_flag_wait(const int* flag, int want, volatile int* abort_word,
                                                 const int* status, int who) {
  for (uint32_t i = 0; i < kFlagPollLimit; ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= want) return true;
    if (*abort_word != 0) return false;
    if (status != nullptr && (i & 31u) == 31u && *reinterpret_cast<const volatile int*>(status) != 0)
      break;
    __nanosleep(64);
  }
  atomicCAS(const_cast<int*>(abort_word), 0, kErrWaitTimeout | (who & 0xff));
  return false;
}
__device__ __forceinline__ void global_flag_release(int* flag, int value) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(flag), "r"(value) : "memory");
}

// ---------------------------------------------------------------------------------
// named barriers (sub-CTA sync among `count` threads)
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---------------------------------------------------------------------------------
// TMA: 4-D tiled tensor copies.  Coordinates are (c0 innermost .. c3 outermost);
// c0 * sizeof(element) must be a multiple of 16 bytes.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst_smem, const void* tmap, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];"
      :
      : "r"(dst_smem), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_4d(const void* tmap, uint32_t src_smem, int c0, int c1,
                                             int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
      :
      : "l"(tmap), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_reduce_add_4d(const void* tmap, uint32_t src_smem, int c0,
                                                  int c1, int c2, int c3) {
  asm volatile(
      "cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.bulk_group [%0, {%2, %3, %4, %5}], "
      "[%1];"
      :
      : "l"(tmap), "r"(src_smem), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// wait until at most N groups still read their shared-memory source
template <int N>
__device__ __forceinline__ void tma_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// wait until at most N groups are incomplete (writes visible)
template <int N>
__device__ __forceinline__ void tma_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
// bring a tile into L2 only (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_l2_4d(const void* tmap, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(tmap),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------------------------
// tcgen05: tensor memory
// A TMEM address is (lane << 16) | column.  Warp w of the CTA may touch only lanes
// 32*(w%4) .. 32*(w%4)+31 with tcgen05.ld/st.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// the mbarrier gets one arrival when every tcgen05.mma issued so far by this thread is done
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}

// 32 lanes x 32 columns of 32-bit: thread i of the warp gets lane (base_lane + i),
// register j holds column (col + j).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}


// ---------------------------------------------------------------------------------
// UMMA descriptors (16-bit operands, fp32 accumulate, dense, cta_group::1, M = 128)
// ---------------------------------------------------------------------------------
// Instruction descriptor bits: [4,6) D format (1 = f32); [7,10) A format (0 = f16, 1 = bf16);
// [10,13) B format; 15 A major (0 = K, 1 = MN); 16 B major; [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n, int a_mn_major,
                                                      int b_mn_major, bool bf16 = false) {
  return (1u << 4) | (uint32_t(bf16) << 7) | (uint32_t(bf16) << 10) | (uint32_t(a_mn_major) << 15) |
         (uint32_t(b_mn_major) << 16) | (uint32_t(n >> 3) << 17) | (uint32_t(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.  Bits: [0,14) address >> 4;
// [16,30) leading byte offset >> 4; [32,46) stride byte offset >> 4; [46,48) version = 1;
// [61,64) layout type (2 = 128-byte swizzle).
//
// Tiles here are stored as rows of 128 bytes (64 fp16), 8 rows per 1024-byte swizzle atom,
// exactly what a TMA box of 64 x rows with CU_TENSOR_MAP_SWIZZLE_128B writes:
//   K-major operand  (the 128-byte row runs along K):   SBO = 1024 (next 8 rows of M/N),
//     LBO unused; advancing K by 16 elements moves the start address by 32 bytes.
//   MN-major operand (the 128-byte row runs along M/N): SBO = 1024 (next 8 rows of K),
//     LBO = byte distance between successive 64-element blocks along M/N; advancing K by
//     16 moves the start address by 16 rows = 2048 bytes.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= uint64_t((saddr >> 4) & 0x3fffu);
  d |= uint64_t((lbo_bytes >> 4) & 0x3fffu) << 16;
  d |= uint64_t((sbo_bytes >> 4) & 0x3fffu) << 32;
  d |= uint64_t(1) << 46;
  d |= uint64_t(2) << 61;
  return d;
}

// The descriptor split in two 32-bit words, so that an MMA issue loop only adds a constant
// to the low word (address field) instead of rebuilding 64-bit values:
//   low  word = address >> 4 | (LBO >> 4) << 16
//   high word = SBO >> 4 | version 1 << 14 | layout 2 << 29      (the same for every tile here)
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo_bytes) {
  return ((sbo_bytes >> 4) & 0x3fffu) | (1u << 14) | (2u << 29);
}
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t saddr, uint32_t lbo_bytes) {
  return ((saddr >> 4) & 0x3fffu) | (((lbo_bytes >> 4) & 0x3fffu) << 16);
}
constexpr uint32_t kDescHi = umma_desc_hi(1024);
constexpr uint32_t kLboKMajor = 16;      // unused by the hardware for swizzled K-major tiles
constexpr uint32_t kLboMnMajor = 16384;  // next 64-element block along M/N = next TMA box

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %3};\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, {%6, %6, %6, %6}, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]   (A: 128 lanes x K fp16, two per 32-bit column)
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\t"
      "mov.b64 db, {%2, %3};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, {%6, %6, %6, %6}, p;\n\t}"
      :
      : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kDescHi), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

// ---- converged-warp variants.  The MMA / TMA issue loops are run by all 32 lanes of a warp so
// that addresses and descriptors stay in uniform registers; only the instruction itself is
// issued by one elected lane.  Call these from a converged warp only.
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred;
}
__device__ __forceinline__ void umma_ss_elect(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                              uint32_t idesc, uint32_t accumulate) {
  if (elect_one()) umma_ss(d_tmem, a_lo, b_lo, idesc, accumulate);
}
__device__ __forceinline__ void umma_ts_elect(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                              uint32_t idesc, uint32_t accumulate) {
  if (elect_one()) umma_ts(d_tmem, a_tmem, b_lo, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
  if (elect_one()) umma_commit(bar);
}
// Three barriers tested with the three probes in flight together: a probe that finds its phase
// complete still costs a round trip through the shared-memory pipe, and three in a row cost
// three.  Returns true when all three phases are complete.
__device__ __forceinline__ bool mbar_try_wait3(uint32_t bar0, uint32_t par0, uint32_t bar1,
                                               uint32_t par1, uint32_t bar2, uint32_t par2) {
  uint32_t r0, r1, r2;
  asm volatile(
      "{\n\t.reg .pred p0, p1, p2;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p0, [%3], %4;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p1, [%5], %6;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p2, [%7], %8;\n\t"
      "selp.u32 %0, 1, 0, p0;\n\t"
      "selp.u32 %1, 1, 0, p1;\n\t"
      "selp.u32 %2, 1, 0, p2;\n\t}"
      : "=r"(r0), "=r"(r1), "=r"(r2)
      : "r"(bar0), "r"(par0), "r"(bar1), "r"(par1), "r"(bar2), "r"(par2)
      : "memory");
  return (r0 & r1 & r2) != 0;
}
// bounded wait by a whole converged warp, with a warp-uniform result
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity,
                                               volatile int* abort_word, int who) {
  const bool ok = mbar_wait(bar, parity, abort_word, who);
  return __all_sync(0xffffffffu, ok);
}

// warpgroup-wide register re-budgeting: every warp of an aligned group of 4 warps executes it
template <int N>
__device__ __forceinline__ void reg_alloc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// ---------------------------------------------------------------------------------
// small math helpers
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float fast_exp2(float x) {
#if defined(FMHA_ABLATE) && (FMHA_ABLATE & 1)
  return x;  // timing experiments only
#else
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
#endif
}
// ---- packed pairs of fp32 (one instruction works on two values; sm_100 f32x2 forms) ----
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ uint64_t pack2f(float lo, float hi) {
  return pack2(__float_as_uint(lo), __float_as_uint(hi));
}
__device__ __forceinline__ void unpack2(uint64_t v, uint32_t& lo, uint32_t& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t add2_rm(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rm.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// three-input maximum / minimum
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// exp2 on the FMA / ALU pipes (no MUFU): x = n + f with n = floor(x) from a round-down add of
// 1.5 * 2^23, 2^f by a cubic (relative error 7.5e-5, far below the fp16 rounding P gets anyway),
// 2^n by adding n into the exponent field.  An option of the forward kernel (FMHA_FWD_POLY_PAIRS) for a
// fraction of the softmax exponentials, off by default.  x is clamped to >= -126
// (masked -inf scores give 2^-126, which rounds to 0 in fp16).
// Works on a packed pair; the result is the packed pair of 2^x.
__device__ __forceinline__ uint64_t poly_exp2_pair(uint64_t x2) {
  uint32_t x0, x1;
  unpack2(x2, x0, x1);
  x2 = pack2f(fmaxf(__uint_as_float(x0), -126.f), fmaxf(__uint_as_float(x1), -126.f));
  const uint64_t magic = pack2f(12582912.f, 12582912.f);
  const uint64_t t2 = add2_rm(x2, magic);
  const uint64_t f2 = sub2(x2, sub2(t2, magic));
  uint64_t p2 = fma2(f2, pack2f(0.0780244917f, 0.0780244917f), pack2f(0.2260672003f, 0.2260672003f));
  p2 = fma2(p2, f2, pack2f(0.6958335042f, 0.6958335042f));
  p2 = fma2(p2, f2, pack2f(0.9999251962f, 0.9999251962f));
  uint32_t p0, p1, t0, t1;
  unpack2(p2, p0, p1);
  unpack2(t2, t0, t1);
  // 2^n: n sits in the low mantissa bits of t; n * 2^23 added into the exponent field
  p0 += t0 << 23;
  p1 += t1 << 23;
  return pack2(p0, p1);
}
// two exp2 per MUFU operation, fp16 in and out (inputs here are <= ~0, results in [0, 1])
__device__ __forceinline__ uint32_t exp2_half2(uint32_t x) {
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}
__device__ __forceinline__ uint32_t mul_half2(uint32_t a, uint32_t b) {
  uint32_t y;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(y) : "r"(a), "r"(b));
  return y;
}
__device__ __forceinline__ uint32_t fma_half2(uint32_t a, uint32_t b, uint32_t c) {
  uint32_t y;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(y) : "r"(a), "r"(b), "r"(c));
  return y;
}
__device__ __forceinline__ float4 lds128(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t a, uint32_t b, uint32_t c,
                                       uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// two fp32 values -> one 32-bit word of the kernel's 16-bit element type (low half = first)
template <bool kBf16>
__device__ __forceinline__ uint32_t pack16x2(float lo, float hi) {
  if constexpr (kBf16) return pack_bf16x2(lo, hi);
  else return pack_half2(lo, hi);
}
// the two bf16 values of a word as fp32 (a bf16 is the upper half of an fp32)
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

}  // namespace fmha
