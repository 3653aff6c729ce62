// Torch extension `flash_attn_v100_cuda`: the module the Python package imports, with the
// entry points `fwd` and `bwd` of the reference's extension (kernel/fused_mha_api.cpp:13-72,
// :74-162, exported at :164-168).  All it does is check tensors, allocate outputs and the
// backward workspace with torch, and call the C ABI of libfmha_b200 on torch's current
// stream under a device guard (as kernel/fused_mha_api.cpp:61,67).  No kernel lives here and
// there is no fallback: without a CUDA device the checks raise.
//
// Differences from the reference extension, all widenings:
//   - any sm_100 device instead of the sm_70 gate (kernel/fused_mha_api.cpp:21-23);
//   - bf16 beside fp16 (reference: fp16 only, :25-29); head_dim 64, 96 or 128 (reference: 128 only, :44); sequence length a multiple of 32 is
//     CHECKED (the reference only documents it, README.md:3);
//   - q and k/v may differ in sequence length; row/head/batch strides are honoured;
//   - `fwd` returns {out, softmax_max, softmax_sum} like the reference (:71), where
//     softmax_max carries lse = max + ln(sum) and softmax_sum is all ones, so that the
//     reference's relation P = exp(scale*S - max) / sum (kernel/fused_mha_kernel.cu:457,602)
//     still holds for a caller that uses the pair;
//   - `bwd` ignores the fp16 `D` argument (flash_attn_interface.py:43-44) and computes
//     D = rowsum(dO o O) itself in fp32.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <optional>
#include <vector>

#include "../../include/fmha_b200.h"

namespace {

FmhaStrides strides_of(const at::Tensor& t) {
  FmhaStrides s;
  s.batch = t.stride(0);
  s.row = t.stride(1);
  s.head = t.stride(2);
  return s;
}

void check_input(const at::Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be on CUDA");
  TORCH_CHECK(t.scalar_type() == at::kHalf || t.scalar_type() == at::kBFloat16,
              "This repo only supports fp16 and bf16 data types (", name, ")");
  TORCH_CHECK(t.dim() == 4, name, " must have shape (batch, seqlen, heads, head_size)");
  TORCH_CHECK(t.stride(-1) == 1, name, " must have contiguous last dimension");
}

void check_status(int rc, const char* what) {
  TORCH_CHECK(rc == FMHA_OK, what, " failed: ", fmha_status_string(rc), " (status ", rc, ")");
}

void check_shapes(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v) {
  const auto B = q.size(0), Nq = q.size(1), H = q.size(2), D = q.size(3);
  const auto Nk = k.size(1);
  TORCH_CHECK(B > 0, "batch size must be positive");
  TORCH_CHECK(D == 64 || D == 96 || D == 128, "head dimension must be 64, 96 or 128, got ", D);
  TORCH_CHECK(k.size(0) == B && k.size(2) == H && k.size(3) == D,
              "k must have shape (batch_size, seqlen_k, num_heads, head_size)");
  TORCH_CHECK(v.sizes() == k.sizes(), "v must have the shape of k");
  TORCH_CHECK(k.scalar_type() == q.scalar_type() && v.scalar_type() == q.scalar_type(),
              "q, k and v must have the same data type");
  TORCH_CHECK(Nq % 32 == 0 && Nk % 32 == 0,
              "sequence lengths must be multiples of 32 (pad the inputs), got ", Nq, " and ", Nk);
}

// per-batch lengths of a right-padded batch -> device pointer (or NULL)
const int32_t* seqused_ptr(const std::optional<at::Tensor>& t, const at::Tensor& q, const char* name) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->dim() == 1 &&
                  t->size(0) == q.size(0) && t->is_contiguous(),
              name, " must be a contiguous int32 CUDA tensor with one entry per batch");
  return t->data_ptr<int32_t>();
}

std::vector<at::Tensor> fwd_impl(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                 std::optional<at::Tensor> out_, double softmax_scale,
                                 bool is_causal, bool want_sum,
                                 std::optional<at::Tensor> seqused_q = std::nullopt,
                                 std::optional<at::Tensor> seqused_k = std::nullopt) {
  check_input(q, "q");
  check_input(k, "k");
  check_input(v, "v");
  check_shapes(q, k, v);
  const int B = q.size(0), Nq = q.size(1), H = q.size(2), D = q.size(3), Nk = k.size(1);

  at::Tensor out;
  if (out_.has_value()) {
    out = out_.value();
    check_input(out, "out");
    TORCH_CHECK(out.sizes() == q.sizes() && out.scalar_type() == q.scalar_type(),
                "out must have the shape and type of q");
  } else {
    out = at::empty_like(q);
  }
  c10::cuda::CUDAGuard guard(q.device());
  auto fopts = q.options().dtype(at::kFloat);
  at::Tensor lse = at::empty({B, H, Nq}, fopts);

  FmhaFwdParams p = {};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.o = out.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.q_strides = strides_of(q);
  p.k_strides = strides_of(k);
  p.v_strides = strides_of(v);
  p.o_strides = strides_of(out);
  p.batch = B;
  p.heads = H;
  p.seqlen_q = Nq;
  p.seqlen_k = Nk;
  p.head_dim = D;
  p.scale = static_cast<float>(softmax_scale);
  p.causal = is_causal ? 1 : 0;
  p.causal_shift = 0;
  p.dtype = q.scalar_type() == at::kBFloat16 ? FMHA_DTYPE_BF16 : FMHA_DTYPE_FP16;
  p.seqused_q = seqused_ptr(seqused_q, q, "seqused_q");
  p.seqused_k = seqused_ptr(seqused_k, q, "seqused_k");
  check_status(fmha_fwd(&p, at::cuda::getCurrentCUDAStream().stream()), "fmha_fwd");
  if (!want_sum) return {out, lse};
  return {out, lse, at::ones({B, H, Nq}, fopts)};
}

// the reference's entry point: {out, softmax_max := lse, softmax_sum := 1}
std::vector<at::Tensor> mha_fwd(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                std::optional<at::Tensor> out_, double softmax_scale,
                                bool is_causal) {
  return fwd_impl(q, k, v, out_, softmax_scale, is_causal, true);
}

// {out, lse} only: what this package's own autograd glue uses (no tensor of ones to fill)
std::vector<at::Tensor> mha_fwd_lse(const at::Tensor& q, const at::Tensor& k, const at::Tensor& v,
                                    std::optional<at::Tensor> out_, double softmax_scale,
                                    bool is_causal, std::optional<at::Tensor> seqused_q,
                                    std::optional<at::Tensor> seqused_k) {
  return fwd_impl(q, k, v, out_, softmax_scale, is_causal, false, seqused_q, seqused_k);
}

std::vector<at::Tensor> bwd_impl(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                 const at::Tensor& v, const at::Tensor& out,
                                 std::optional<at::Tensor> softmax_sum, const at::Tensor& softmax_max,
                                 std::optional<at::Tensor> dq_, std::optional<at::Tensor> dk_,
                                 std::optional<at::Tensor> dv_, double softmax_scale, bool is_causal,
                                 std::optional<at::Tensor> seqused_q, std::optional<at::Tensor> seqused_k,
                                 bool deterministic) {
  check_input(q, "q");
  check_input(k, "k");
  check_input(v, "v");
  check_input(out, "out");
  check_input(dout, "dout");
  check_shapes(q, k, v);
  TORCH_CHECK(out.sizes() == q.sizes() && out.scalar_type() == q.scalar_type(),
              "out must have the shape and type of q");
  TORCH_CHECK(dout.sizes() == q.sizes() && dout.scalar_type() == q.scalar_type(),
              "dout must have the shape and type of q");
  const int B = q.size(0), Nq = q.size(1), H = q.size(2), D = q.size(3), Nk = k.size(1);
  TORCH_CHECK(softmax_max.is_cuda() && softmax_max.scalar_type() == at::kFloat &&
                  softmax_max.sizes() == at::IntArrayRef({B, H, Nq}),
              "softmax_max must be a CUDA fp32 tensor of shape (batch_size, num_heads, seqlen_q)");

  c10::cuda::CUDAGuard guard(q.device());
  at::Tensor lse = softmax_max;
  if (softmax_sum.has_value()) {
    TORCH_CHECK(softmax_sum->sizes() == softmax_max.sizes(), "softmax_sum must have the shape of softmax_max");
    lse = softmax_max + softmax_sum->log();
  }
  lse = lse.contiguous();

  auto take = [&](std::optional<at::Tensor>& t, const at::Tensor& like, const char* name) {
    if (t.has_value()) {
      check_input(t.value(), name);
      TORCH_CHECK(t->sizes() == like.sizes() && t->scalar_type() == like.scalar_type(), name,
                  " must have the shape and type of its input");
      return t.value();
    }
    return at::empty_like(like);
  };
  at::Tensor dq = take(dq_, q, "dq");
  at::Tensor dk = take(dk_, k, "dk");
  at::Tensor dv = take(dv_, v, "dv");

  FmhaBwdParams p = {};
  p.q = q.data_ptr();
  p.k = k.data_ptr();
  p.v = v.data_ptr();
  p.o = out.data_ptr();
  p.dout = dout.data_ptr();
  p.lse = lse.data_ptr<float>();
  p.dq = dq.data_ptr();
  p.dk = dk.data_ptr();
  p.dv = dv.data_ptr();
  p.q_strides = strides_of(q);
  p.k_strides = strides_of(k);
  p.v_strides = strides_of(v);
  p.o_strides = strides_of(out);
  p.dout_strides = strides_of(dout);
  p.dq_strides = strides_of(dq);
  p.dk_strides = strides_of(dk);
  p.dv_strides = strides_of(dv);
  p.batch = B;
  p.heads = H;
  p.seqlen_q = Nq;
  p.seqlen_k = Nk;
  p.head_dim = D;
  p.scale = static_cast<float>(softmax_scale);
  p.causal = is_causal ? 1 : 0;
  p.dtype = q.scalar_type() == at::kBFloat16 ? FMHA_DTYPE_BF16 : FMHA_DTYPE_FP16;
  p.seqused_q = seqused_ptr(seqused_q, q, "seqused_q");
  p.seqused_k = seqused_ptr(seqused_k, q, "seqused_k");
  p.flags = deterministic ? FMHA_BWD_DETERMINISTIC : 0;
  const size_t ws_bytes = fmha_bwd_workspace_bytes(&p);
  at::Tensor ws = at::empty({static_cast<int64_t>(ws_bytes)}, q.options().dtype(at::kByte));
  check_status(fmha_bwd(&p, ws.data_ptr(), ws_bytes, at::cuda::getCurrentCUDAStream().stream()),
               "fmha_bwd");
  return {dq, dk, dv};
}

// the reference's entry point (kernel/fused_mha_api.cpp:74-87); its fp16 D argument is ignored
std::vector<at::Tensor> mha_bwd(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                const at::Tensor& v, const at::Tensor& out,
                                std::optional<at::Tensor> D_unused,
                                std::optional<at::Tensor> softmax_sum, const at::Tensor& softmax_max,
                                std::optional<at::Tensor> dq_, std::optional<at::Tensor> dk_,
                                std::optional<at::Tensor> dv_, double softmax_scale,
                                bool is_causal) {
  (void)D_unused;
  return bwd_impl(dout, q, k, v, out, softmax_sum, softmax_max, dq_, dk_, dv_, softmax_scale,
                  is_causal, std::nullopt, std::nullopt, false);
}

// this package's own glue: lse instead of (max, sum), per-batch lengths, deterministic dQ
std::vector<at::Tensor> mha_bwd_lse(const at::Tensor& dout, const at::Tensor& q, const at::Tensor& k,
                                    const at::Tensor& v, const at::Tensor& out, const at::Tensor& lse,
                                    double softmax_scale, bool is_causal,
                                    std::optional<at::Tensor> seqused_q,
                                    std::optional<at::Tensor> seqused_k, bool deterministic) {
  return bwd_impl(dout, q, k, v, out, std::nullopt, lse, std::nullopt, std::nullopt, std::nullopt,
                  softmax_scale, is_causal, seqused_q, seqused_k, deterministic);
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "B200 (sm_100a) fused multi-head attention";
  // positional calls only, like the reference's pybind exports (kernel/fused_mha_api.cpp:166-167)
  m.def("fwd", &mha_fwd, "Forward pass: fwd(q, k, v, out|None, softmax_scale, is_causal)");
  m.def("fwd_lse", &mha_fwd_lse,
        "Forward pass returning [out, lse]: fwd_lse(q, k, v, out|None, softmax_scale, is_causal, "
        "seqused_q|None, seqused_k|None)");
  m.def("bwd_lse", &mha_bwd_lse,
        "Backward pass: bwd_lse(dout, q, k, v, out, lse, softmax_scale, is_causal, seqused_q|None, "
        "seqused_k|None, deterministic)");
  m.def("bwd", &mha_bwd,
        "Backward pass: bwd(dout, q, k, v, out, D|None, softmax_sum|None, softmax_max, dq|None, "
        "dk|None, dv|None, softmax_scale, is_causal)");
  m.def("version", []() { return std::string(fmha_version()); });
}
