/*
 * fmha_b200.h - C ABI of the B200 (sm_100a) fused multi-head attention library.
 *
 * This header is the drop-in boundary for the attention hot path of
 * flash-attention-v100.  It replaces the two C++-linkage launchers of the reference
 * (include/fused_mha.h:1-2 `fused_mha_forward`, include/fused_mha.h:4-6
 * `fused_mha_backward`, defined in kernel/fused_mha_kernel.cu:891-916) with `extern "C"`
 * entry points that take plain pointers and sizes, return a status code instead of
 * `void`, and never abort the process.
 *
 * Conventions
 *  - All tensors are 16-bit floating point unless stated: fp16, the reference's only type
 *    (kernel/fused_mha_api.cpp:25-29), or bf16, chosen by the `dtype` field / argument
 *    (FMHA_DTYPE_*; 0 = fp16, so zero-initialised parameters mean what they always meant).
 *    Every tensor of a call has the same type.  Logical layout (Z, N, H, D) = (batch, sequence,
 *    heads, head_dim) as in the reference (kernel/fused_mha_api.cpp:37-47).  Strides are in
 *    ELEMENTS and the head_dim stride must be 1.  Row/head/batch strides must be multiples
 *    of 8 elements and base pointers 16-byte aligned (TMA requirement).
 *  - head_dim is 64, 96 or 128 (the reference: 128 only, kernel/fused_mha_api.cpp:44).  96 runs on
 *    the 128-wide kernels: the tensor maps describe 96 columns, tile loads fill columns 96-127
 *    with zeros and stores clip them, so the result is exact and the cost is that of 128.  The
 *    fp32 buffers (workspace, dk_accum / dv_accum, o_acc, partial sums) have head_dim elements
 *    per row like the 16-bit tensors.
 *  - `lse` is fp32 (Z, H, seqlen_q) contiguous: lse = max + ln(sum) of the scaled scores,
 *    i.e. the reference's `softmax_max` and `softmax_sum` (kernel/fused_mha_api.cpp:65-66)
 *    folded into one number per row.
 *  - Causal masking: key j is visible to query i iff j <= i + causal_shift.  The reference
 *    (square, kernel/fused_mha_kernel.cu:232-235) is causal_shift = 0.
 *  - The library allocates no device memory: the caller owns every buffer, including the
 *    backward workspace whose size `fmha_bwd_workspace_bytes` reports.
 *  - `stream` is a cudaStream_t passed as void*.  All launches are asynchronous on it.
 *  - `status` (optional, may be NULL) points to one int32 in DEVICE memory that the caller
 *    zeroes once; a kernel that gives up on a bounded wait writes a non-zero code there.
 *  - Sequence lengths: the C ABI accepts any positive seqlen_q / seqlen_k; tails of the
 *    128-row tiles are masked inside the kernels.  The reference's "multiple of 32" contract
 *    (README.md:3) is enforced one level up, by the torch extension's `fwd` / `bwd`.
 *  - Thread safety: entry points may be called from any thread with the target device
 *    current.  The only process-wide state is read-mostly: the resolved driver entry point
 *    for tensor-map encoding, and, for fmha_bwd_static_scratch, the per-device address of the
 *    built-in scratch area (looked up once per device ordinal in the primary context; it
 *    goes stale if that context is destroyed with cudaDeviceReset) and the area itself,
 *    which every call of that entry point on a device shares (see there).
 */
#ifndef FMHA_B200_H_
#define FMHA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes returned by every entry point */
enum {
  FMHA_OK = 0,
  FMHA_ERR_NULL_POINTER = 1,
  FMHA_ERR_BAD_HEAD_DIM = 2,   /* head_dim not in {64, 96, 128} */
  FMHA_ERR_BAD_SHAPE = 3,      /* non-positive sizes */
  FMHA_ERR_BAD_STRIDE = 4,     /* stride not a multiple of 8 elements, or too small */
  FMHA_ERR_BAD_ALIGNMENT = 5,  /* pointer not 16-byte aligned */
  FMHA_ERR_WORKSPACE = 6,      /* workspace missing or too small */
  FMHA_ERR_TENSOR_MAP = 7,     /* cuTensorMapEncodeTiled failed */
  FMHA_ERR_NO_DEVICE = 8,      /* no sm_100 device / driver entry point unavailable */
  FMHA_ERR_LAUNCH = 9,         /* cudaLaunchKernel failed (see cudaGetLastError) */
  FMHA_ERR_TOO_LARGE = 10,     /* a size exceeds a stated limit */
  FMHA_ERR_BAD_DTYPE = 11      /* dtype is not one of FMHA_DTYPE_* */
};

/* element type of q, k, v, o, dout, dq, dk, dv (accumulation is fp32 either way) */
#define FMHA_DTYPE_FP16 0
#define FMHA_DTYPE_BF16 1

/* element strides of one (Z, N, H, D) tensor; the D stride is 1 */
typedef struct {
  int64_t batch;
  int64_t row;
  int64_t head;
} FmhaStrides;

typedef struct {
  const void* q; /* (Z, seqlen_q, H, D) fp16 */
  const void* k; /* (Z, seqlen_k, H, D) fp16 */
  const void* v; /* (Z, seqlen_k, H, D) fp16 */
  void* o;       /* (Z, seqlen_q, H, D) fp16, written */
  float* lse;    /* (Z, H, seqlen_q) fp32, written */
  FmhaStrides q_strides, k_strides, v_strides, o_strides;
  int32_t batch, heads, seqlen_q, seqlen_k, head_dim;
  float scale;          /* softmax scale applied to q.k^T */
  int32_t causal;       /* 0 / 1 */
  int32_t causal_shift; /* see above; 0 for the reference's square causal mask */
  int32_t* status;      /* optional device status word */
  /* SMs to leave free (0 = none).  The forward kernel is persistent, one CTA per SM for its whole
   * run; a caller that has a copy or collective kernel in flight on another stream (ring
   * attention posts the next K/V exchange before it launches the step) gives those kernels room
   * to run beside it instead of after it. */
  int32_t sm_margin;
  int32_t dtype; /* FMHA_DTYPE_FP16 (0) or FMHA_DTYPE_BF16 */
  /* Right-padded batches (optional, NULL = every row counts): int32 device arrays of `batch`
   * entries.  Batch entry z has seqused_q[z] real query rows and seqused_k[z] real keys; the
   * rest of its seqlen_q / seqlen_k rows is padding.  Tiles that are all padding are skipped,
   * not computed and thrown away; padding keys are masked; padding rows of o are written as
   * zeros and their lse as -inf.  The padding must hold finite values.  The reference only has
   * the contract "the caller pads" (README.md:3) and computes the padding like real rows. */
  const int32_t* seqused_q;
  const int32_t* seqused_k;
} FmhaFwdParams;

typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* o;    /* forward output */
  const void* dout; /* (Z, seqlen_q, H, D) fp16 upstream gradient */
  const float* lse; /* (Z, H, seqlen_q) fp32 from the forward */
  void* dq;         /* (Z, seqlen_q, H, D) fp16, written */
  void* dk;         /* (Z, seqlen_k, H, D) fp16, written (may be NULL if dk_accum is set) */
  void* dv;         /* (Z, seqlen_k, H, D) fp16, written (may be NULL if dv_accum is set) */
  float* dk_accum;  /* optional fp32 (Z, seqlen_k, H, D): dK is ADDED into it */
  float* dv_accum;  /* optional fp32 (Z, seqlen_k, H, D): dV is ADDED into it */
  /* element stride between batch entries of dk_accum / dv_accum; 0 = dense
   * (seqlen_k * H * D).  Rows and heads are dense.  Lets a row range of a larger buffer be
   * the target (ring attention adds into the first half of a travelling block).  Must be 0, or
   * a multiple of 4 elements (the adds are 16-byte accesses) that is at least
   * seqlen_k * H * D (batch entries must not overlap); anything else, negative values
   * included, is rejected with FMHA_ERR_BAD_STRIDE. */
  int64_t accum_batch_stride;
  FmhaStrides q_strides, k_strides, v_strides, o_strides, dout_strides;
  FmhaStrides dq_strides, dk_strides, dv_strides;
  int32_t batch, heads, seqlen_q, seqlen_k, head_dim;
  float scale;
  int32_t causal;
  int32_t causal_shift;
  /* ring attention: 0 = normal (compute D, zero the fp32 dQ accumulator, convert dQ to fp16);
   * bit 0 set = do not zero the dQ accumulator nor recompute D (workspace carries both over
   * from an earlier call); bit 1 set = do not convert dQ (a later call will); bit 2 set = run
   * the preprocess step only; bit 3 set = deterministic dQ (see FMHA_BWD_DETERMINISTIC); bit 4 set =
   * dk_accum / dv_accum are overwritten, not added into (FMHA_BWD_ACCUM_OVERWRITE). */
  int32_t flags;
  int32_t* status;
  int32_t dtype; /* FMHA_DTYPE_FP16 (0) or FMHA_DTYPE_BF16 */
  /* Right-padded batches, as in FmhaFwdParams: padding rows contribute nothing to dk / dv, and
   * the padding rows of dq, dk and dv are written as zeros. */
  const int32_t* seqused_q;
  const int32_t* seqused_k;
  /* Query rows before this index take no part in the call: nothing is added to their dQ, and
   * they contribute nothing to dK / dV.  0 = all rows; otherwise a multiple of 128 below
   * seqlen_q (FMHA_ERR_BAD_SHAPE if not).  q, o, dout, lse and the workspace stay those of ALL
   * seqlen_q rows, so calls over different row ranges share one workspace (ring attention: a
   * step in which only the second half of the local queries sees the visiting block).  The
   * causal mask keeps counting rows from 0. */
  int32_t q_row_begin;
} FmhaBwdParams;

#define FMHA_BWD_KEEP_WORKSPACE 1
#define FMHA_BWD_SKIP_DQ_CONVERT 2
/* Only prepare the workspace (D, the rescaled LSE, zeroed dQ accumulator) and return; the
 * gradients come from a later call with FMHA_BWD_KEEP_WORKSPACE.  For callers that have O and dO
 * before the first K/V block arrives, and for timing the three kernels of a backward pass one by
 * one.  Not combinable with FMHA_BWD_KEEP_WORKSPACE (FMHA_ERR_WORKSPACE). */
#define FMHA_BWD_PREPROCESS_ONLY 4
/* Deterministic dQ: the fp32 partial sums of dQ from different key/value tiles are added in the
 * order of the tiles instead of the order in which they happen to finish, so dQ is bit-for-bit
 * the same on every run (dK, dV, O and LSE always are).  The CTAs of a (batch, head) then run
 * staggered, one query tile apart, which costs up to a factor of two in the fused kernel.  The
 * reference's dQ is a 64-way fp16 atomicAdd (kernel/fused_mha_kernel.cu:543,693) and has no
 * such mode.  The order words live in the workspace (fmha_bwd_workspace_bytes accounts for
 * them) and are cleared by every call that carries the flag. */
#define FMHA_BWD_DETERMINISTIC 8
/* dk_accum / dv_accum are WRITTEN instead of added into: the fp32 dK / dV of this call replace
 * what the buffers hold, every row of the seqlen_k rows included (zeros where no query row
 * sees a key), so the caller need not clear them first (ring attention: the partial result of
 * one step, sent to the block's owner). */
#define FMHA_BWD_ACCUM_OVERWRITE 16

/* Forward: O = softmax(scale * Q K^T [+ causal mask]) V and LSE.
 * Replaces fused_mha_forward (include/fused_mha.h:1-2, kernel/fused_mha_kernel.cu:891-902). */
int fmha_fwd(const FmhaFwdParams* p, void* stream);

/* Bytes of device workspace the backward needs for these sizes: an fp32 dQ accumulator
 * (Z, seqlen_q, H, D) followed by fp32 lse * log2(e) and D = rowsum(dO * O), each (Z, H, seqlen_q
 * padded to 128), and one int32 per (batch, head, 128-row query tile) for FMHA_BWD_DETERMINISTIC.  The reference
 * has no counterpart: it accumulates dQ with fp16 atomics in place
 * (kernel/fused_mha_kernel.cu:543,693) and computes D in PyTorch
 * (flash_attn_v100/flash_attn_interface.py:43-44). */
size_t fmha_bwd_workspace_bytes(const FmhaBwdParams* p);

/* Backward: dQ, dK, dV.  Runs the D/zero preprocess kernel, the fused dK/dV/dQ kernel and the
 * dQ convert kernel on `stream`.
 * Replaces fused_mha_backward (include/fused_mha.h:4-6, kernel/fused_mha_kernel.cu:904-916)
 * together with the D computation of flash_attn_v100/flash_attn_interface.py:43-44 and the
 * zero-fill of :84. */
int fmha_bwd(const FmhaBwdParams* p, void* workspace, size_t workspace_bytes, void* stream);

/* Capacity in bytes of the scratch area built into the library for fmha_bwd_static_scratch. */
#define FMHA_STATIC_SCRATCH_BYTES (32u << 20)

/* Backward without a caller workspace and without any allocation: the same computation and the
 * same results as fmha_bwd, with the workspace taken from a fixed FMHA_STATIC_SCRATCH_BYTES
 * (32 MiB) area that is part of the library's device image.  It has no counterpart in the
 * reference (which keeps no scratch: fp16 atomics in place, kernel/fused_mha_kernel.cu:543,693).
 *
 * It is meant for hosts that cannot obtain device memory at the moment they need a backward
 * pass: a serving or training process that handed all free HBM to its own pool at start-up, so
 * that a cudaMalloc for our workspace would fail or force the pool to shrink; a plugin called
 * from a latency-critical section where the device-wide synchronisation hidden in
 * cudaMalloc/cudaFree is not acceptable; an embedding runtime whose policy forbids a library
 * to allocate on its own.  Such a caller still passes every input and output buffer; only the
 * workspace comes from the library.
 *
 *  - Limit: fmha_bwd_workspace_bytes(p) must not exceed FMHA_STATIC_SCRATCH_BYTES, otherwise
 *    FMHA_ERR_TOO_LARGE is returned and nothing is launched (e.g. Z*N*H*D <= ~8.3M elements).
 *  - Cost: every GPU on which the library's device code is loaded holds the 32 MiB until the
 *    process exits, whether or not this entry point is ever called.  The CUDA runtime
 *    reserves it when it loads the library's module on a device, which with lazy module
 *    loading happens at the first fmha_* launch (or the first call of this entry point) on
 *    that device, not at dlopen.  A host that hands all free HBM to its own pool must
 *    therefore make one warm-up fmha_* call per device BEFORE it does so, outside stream
 *    capture and outside any latency-critical section (module loading allocates and
 *    synchronises inside the driver); after that warm-up this entry point never allocates.
 *  - The first call on each device looks up the device address of the area and caches it
 *    per device ordinal.  Make that first call outside any stream capture.
 *  - All calls on a device share the one area and it keeps whatever the last call left; each
 *    call re-initialises the parts it needs (dQ accumulator zeroed, statistics rewritten), so
 *    stale contents are harmless, but two calls that overlap on the GPU (different streams,
 *    or different host threads without ordering) race on it.  Serialise them on one stream.
 *  - FMHA_BWD_KEEP_WORKSPACE, FMHA_BWD_PREPROCESS_ONLY and FMHA_BWD_SKIP_DQ_CONVERT are rejected
 *    with FMHA_ERR_WORKSPACE: a shared area cannot carry state from one call to the next, and
 *    an unconverted dQ left in it would be out of the caller's reach.
 */
int fmha_bwd_static_scratch(const FmhaBwdParams* p, void* stream);

/* dQ = fp16(scale * accumulator) from a backward workspace, for callers that ran fmha_bwd with
 * FMHA_BWD_SKIP_DQ_CONVERT (several calls accumulating into one workspace).  The sizes must be
 * those the workspace was used with.  Replaces the reference's in-place fp16 atomics
 * (kernel/fused_mha_kernel.cu:543,693). */
int fmha_bwd_convert_dq(const void* workspace, void* dq, FmhaStrides dq_strides, int32_t batch,
                        int32_t heads, int32_t seqlen_q, int32_t head_dim, float scale,
                        int32_t dtype, void* stream);

/* Ring-attention merge of a partial result into running fp32 accumulators, in place:
 *   lse' = logaddexp(lse_acc, lse_part);  o_acc = e^(lse_acc-lse') o_acc + e^(lse_part-lse') o_part
 * o_acc fp32 (Z, N, H, D) contiguous, lse_acc fp32 (Z, H, N) contiguous; o_part 16-bit (`dtype`)
 * with strides, lse_part fp32 (Z, H, N).  rows = N.  When `o_out` is not NULL the merged result
 * is also written in `dtype` as (Z, N, H, D) contiguous (used on the last ring step).
 * A row with lse_acc = -inf holds nothing yet: its o_acc is not read, so accumulators start as
 * lse_acc = -inf and o_acc uninitialised.
 * No counterpart in the reference (it has no multi-GPU path). */
int fmha_merge(float* o_acc, float* lse_acc, const void* o_part, FmhaStrides o_part_strides,
               const float* lse_part, void* o_out, int32_t batch, int32_t heads, int32_t rows,
               int32_t head_dim, int32_t dtype, void* stream);

/* The same merge for a partial result that covers only rows [row_offset, row_offset + rows) of
 * accumulators with acc_rows rows (zig-zag ring attention: some steps compute the second half of
 * the local query rows only).  o_part (Z, rows, H, D) with strides, lse_part (Z, H, rows);
 * o_acc / o_out (Z, acc_rows, H, D), lse_acc (Z, H, acc_rows), all contiguous.
 * No counterpart in the reference. */
int fmha_merge_rows(float* o_acc, float* lse_acc, const void* o_part, FmhaStrides o_part_strides,
                    const float* lse_part, void* o_out, int32_t batch, int32_t heads, int32_t rows,
                    int32_t acc_rows, int32_t row_offset, int32_t head_dim, int32_t dtype,
                    void* stream);

/* ------------------------------------------------------------------------------------------
 * Multi-GPU plumbing for ring attention between the processes of one node, one process per GPU.
 * None of it has a counterpart in the reference (single GPU).  The attention kernels never
 * read another GPU's memory: a K/V block is first copied into this GPU's own memory by a copy
 * engine (fmha_peer_copy from an address obtained with fmha_ipc_open), flags tell the two sides
 * when a buffer may be read or overwritten.  Everything is asynchronous on the stream given.
 * ------------------------------------------------------------------------------------------ */

/* CUDA IPC handle (64 bytes) of the allocation that holds `ptr`, and the offset of `ptr` in it;
 * another process of the node turns the pair back into an address it can use as the source or
 * the destination of fmha_peer_copy, or as a flag for fmha_peer_signal. */
int fmha_ipc_export(const void* ptr, void* handle64, int64_t* offset);
int fmha_ipc_open(const void* handle64, int64_t offset, void** ptr);
/* Unmap an address obtained from fmha_ipc_open (pass the same offset). */
int fmha_ipc_close(void* ptr, int64_t offset);

/* bytes from src to dst, either of which may be another GPU's memory (copy engine, no SM). */
int fmha_peer_copy(void* dst, const void* src, size_t bytes, void* stream);
/* `rows` rows of `row_bytes` each, the rows `dst_pitch` / `src_pitch` bytes apart. */
int fmha_peer_copy_2d(void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                      size_t row_bytes, size_t rows, void* stream);

/* word[0] += 1 and word[1] = the old word[0], on the stream: the iteration number the flags of
 * one call carry, and the previous one.  Kept on the device so that a recorded sequence of
 * these calls can be replayed. */
int fmha_counter_bump(int32_t* word, void* stream);
/* flags[i] <- *value for i < n (n <= 16), ordered after everything the stream did before; the
 * flags may live in other GPUs' memory (fmha_ipc_open). */
int fmha_peer_signal(int32_t* const* flags, int32_t n, const int32_t* value, void* stream);
/* The stream waits until *flags[i] >= *value for every i < n (n <= 16; peers' fmha_peer_signal),
 * at most timeout_ms (1..60000); a wait that runs out writes a non-zero code to *status (device
 * memory, optional), which makes the attention kernels launched afterwards with that status
 * word return at once. */
int fmha_peer_wait(const int32_t* const* flags, int32_t n, const int32_t* value, int32_t* status,
                   int32_t timeout_ms, void* stream);

/* out (fp16 / bf16 with strides, (Z, rows, H, D)) = sum of n_parts (<= 16) fp32 buffers, each
 * (Z, rows, H, D) contiguous, of which only the first rows_per_part[s] rows of every batch entry
 * count (zig-zag ring attention: some ranks contribute to the first half of a block only). */
int fmha_sum_partials(const float* const* parts, const int32_t* rows_per_part, int32_t n_parts,
                      void* out, FmhaStrides out_strides, int32_t batch, int32_t heads, int32_t rows,
                      int32_t head_dim, int32_t dtype, void* stream);

/* All partial results of a ring-attention forward merged in one pass: for every output row
 *   lse = log sum_s e^(lse_s),  o = sum_s e^(lse_s - lse) o_s     over the parts that cover it.
 * Part s (s < n_parts <= 16): o_parts[s] 16-bit (Z, rows_per_part[s], H, D) contiguous,
 * lse_parts[s] fp32 (Z, H, rows_per_part[s]) contiguous, covering the output rows
 * [row_offset[s], row_offset[s] + rows_per_part[s]).  o_out 16-bit (Z, rows, H, D) contiguous,
 * lse_out fp32 (Z, H, rows); a row no part covers (or whose parts are all empty, LSE = -inf)
 * gets o = 0, lse = -inf.  Replaces n_parts calls of fmha_merge_rows on fp32 accumulators and
 * the final conversion.  No counterpart in the reference. */
int fmha_merge_parts(const void* const* o_parts, const float* const* lse_parts,
                     const int32_t* row_offset, const int32_t* rows_per_part, int32_t n_parts,
                     void* o_out, float* lse_out, int32_t batch, int32_t heads, int32_t rows,
                     int32_t head_dim, int32_t dtype, void* stream);

/* Reference-shaped launchers: same argument meaning as include/fused_mha.h:1-6, dense fp16
 * (batch, m|n, head, k) tensors, except that the `max`/`sum` pair becomes one `lse` buffer,
 * the backward's `d_ptr` (fp16 D) is dropped in favour of a caller workspace, and a status
 * is returned.  m = seqlen_q, n = seqlen_k, k = head_dim. */
int fmha_b200_forward(const void* query_ptr, const void* key_ptr, const void* value_ptr,
                      void* output_ptr, void* lse_ptr, int batch, int head, int m, int n, int k,
                      float scale, int causal, void* stream);
int fmha_b200_backward(const void* query_ptr, const void* key_ptr, const void* value_ptr,
                       const void* output_ptr, const void* d_output_ptr, const void* lse_ptr,
                       void* d_query_ptr, void* d_key_ptr, void* d_value_ptr, void* workspace,
                       size_t workspace_bytes, int batch, int head, int m, int n, int k,
                       float scale, int causal, void* stream);

/* Human-readable text for a status code (static storage). */
const char* fmha_status_string(int status);

/* Library version, "major.minor.patch". */
const char* fmha_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FMHA_B200_H_ */
