"""Python surface and autograd glue of the B200 attention library.

Mirrors ``flash_attn_v100/flash_attn_interface.py`` of the reference: the same public
``flash_attn_func(q, k, v, softmax_scale=None, causal=False)`` (reference :101-110), the same
``FlashAttnFunc`` autograd Function with five inputs and ``(dq, dk, dv, None, None)`` gradients
(:62-99), the same helper names ``_flash_attn_forward`` / ``_flash_attn_backward`` (:11-60), on
fp16 CUDA tensors of shape (Z, N_CTX, H, D_HEAD).

What changed underneath:
  * the extension ``flash_attn_v100_cuda`` runs hand-written sm_100a kernels and returns one
    log-sum-exp per row instead of the (max, sum) pair (the pair is still returned for
    compatibility: max carries the LSE and sum is all ones);
  * D = rowsum(dO * O) is computed in fp32 inside the extension, not here in fp16 (:43-44);
  * dq/dk/dv need no zero-fill (:84): the kernels overwrite them;
  * the contract "N_CTX is a multiple of 32, right-padded by the caller" (README.md:3) is
    checked, and tail tiles are masked inside the kernels.

  * the two extension calls are registered as ``torch.library`` custom ops
    (``flash_attn_v100::fwd`` / ``flash_attn_v100::bwd``, each with a fake implementation that
    only describes output shapes), so that ``flash_attn_func`` can sit inside a
    ``torch.compile(fullgraph=True)`` region: the compiler sees two opaque ops instead of a
    pybind call it cannot trace.  The reference's glue (:62-99) calls the extension directly
    and breaks the graph.

There is no CPU path: importing this module needs the compiled extension, and calling it needs
a CUDA device.
"""
from typing import Optional, Tuple

import torch

# the CUDA kernels must be imported after torch (same order as the reference, :8-9)
import flash_attn_v100_cuda as flash_attn_cuda


def _maybe_contiguous(x):
    return x.contiguous() if x.stride(-1) != 1 else x


@torch.library.custom_op("flash_attn_v100::fwd", mutates_args=(), device_types="cuda")
def _fwd_op(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, softmax_scale: float, causal: bool,
            seqused_q: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None
            ) -> Tuple[torch.Tensor, torch.Tensor]:
    out, softmax_lse = flash_attn_cuda.fwd_lse(q, k, v, None, softmax_scale, causal, seqused_q, seqused_k)
    return out, softmax_lse


@_fwd_op.register_fake
def _fwd_fake(q, k, v, softmax_scale, causal, seqused_q=None, seqused_k=None):
    Z, N, H, _ = q.shape
    return torch.empty_like(q), q.new_empty((Z, H, N), dtype=torch.float32)


@torch.library.custom_op("flash_attn_v100::bwd", mutates_args=(), device_types="cuda")
def _bwd_op(dout: torch.Tensor, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: torch.Tensor,
            softmax_lse: torch.Tensor, softmax_scale: float, causal: bool,
            seqused_q: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None,
            deterministic: bool = False) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    # D = rowsum(dO * O) is computed by the extension in fp32; softmax_lse already is max + ln(sum)
    dq, dk, dv = flash_attn_cuda.bwd_lse(dout, q, k, v, out, softmax_lse, softmax_scale, causal,
                                         seqused_q, seqused_k, deterministic)
    return dq, dk, dv


@_bwd_op.register_fake
def _bwd_fake(dout, q, k, v, out, softmax_lse, softmax_scale, causal, seqused_q=None, seqused_k=None,
              deterministic=False):
    return torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)


def _flash_attn_forward(q, k, v, softmax_scale, causal):
    q, k, v = [_maybe_contiguous(x) for x in (q, k, v)]
    out, softmax_lse = _fwd_op(q, k, v, float(softmax_scale), bool(causal))
    return out, q, k, v, softmax_lse, None


def _flash_attn_backward(dout, q, k, v, out, softmax_lse, softmax_sum, dq, dk, dv,
                         softmax_scale, causal):
    """Same arguments as the reference's (:26-60).  With preallocated ``dq, dk, dv`` or a
    ``softmax_sum`` (the reference's calling convention) the extension is called directly;
    otherwise through the registered op, which allocates the gradients itself."""
    dout, q, k, v, out = [_maybe_contiguous(x) for x in (dout, q, k, v, out)]
    if dq is None and dk is None and dv is None and softmax_sum is None:
        return _bwd_op(dout, q, k, v, out, softmax_lse, float(softmax_scale), bool(causal))
    dq, dk, dv = flash_attn_cuda.bwd(
        dout, q, k, v, out,
        None,          # D: computed by the extension in fp32
        softmax_sum,
        softmax_lse,
        dq, dk, dv, softmax_scale, causal,
    )
    return dq, dk, dv


class FlashAttnFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, q, k, v, softmax_lse, _ = _flash_attn_forward(q, k, v, softmax_scale, causal=causal)
        ctx.save_for_backward(q, k, v, out, softmax_lse)
        ctx.softmax_scale = softmax_scale
        ctx.causal = causal
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, softmax_lse = ctx.saved_tensors
        # no zero-filled gradients as in the reference (:84): the kernels overwrite them
        dq, dk, dv = _flash_attn_backward(dout, q, k, v, out, softmax_lse, None, None, None, None,
                                          ctx.softmax_scale, ctx.causal)
        return dq, dk, dv, None, None


class FlashAttnPaddedFunc(torch.autograd.Function):
    """``FlashAttnFunc`` with per-batch real lengths and the deterministic-dQ switch; no
    counterpart in the reference, whose callers pad and pay for the padding (README.md:3)."""

    @staticmethod
    def forward(ctx, q, k, v, seqused_q, seqused_k, softmax_scale, causal, deterministic):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        q, k, v = [_maybe_contiguous(x) for x in (q, k, v)]
        out, softmax_lse = _fwd_op(q, k, v, float(softmax_scale), bool(causal), seqused_q, seqused_k)
        ctx.save_for_backward(q, k, v, out, softmax_lse, seqused_q, seqused_k)
        ctx.softmax_scale, ctx.causal, ctx.deterministic = float(softmax_scale), bool(causal), bool(deterministic)
        return out

    @staticmethod
    def backward(ctx, dout, *args):
        q, k, v, out, softmax_lse, seqused_q, seqused_k = ctx.saved_tensors
        dq, dk, dv = _bwd_op(_maybe_contiguous(dout), q, k, v, out, softmax_lse, ctx.softmax_scale,
                             ctx.causal, seqused_q, seqused_k, ctx.deterministic)
        return dq, dk, dv, None, None, None, None, None


def flash_attn_padded_func(q, k, v, seqused_q=None, seqused_k=None, softmax_scale: Optional[float] = None,
                           causal: bool = False, deterministic: bool = False):
    """``flash_attn_func`` for right-padded batches: ``seqused_q`` / ``seqused_k`` (int32 CUDA
    tensors, one entry per batch, or None) give the real number of query rows / keys of every
    batch entry.  Padding keys are masked, padding tiles are skipped instead of computed, the
    padding rows of the output and of every gradient are zero.  ``deterministic=True`` adds the
    partial sums of dQ in a fixed order (bit-for-bit reproducible, slower)."""
    return FlashAttnPaddedFunc.apply(q, k, v, seqused_q, seqused_k, softmax_scale, causal, deterministic)


def flash_attn_func(q, k, v, softmax_scale: Optional[float] = None, causal: bool = False):
    """softmax(q k^T * softmax_scale [+ causal mask]) v with autograd.

    q, k, v: fp16 (or bf16) CUDA tensors (batch, seqlen, heads, head_dim), head_dim 64, 96 or 128,
    seqlen a multiple of 32.  softmax_scale defaults to head_dim ** -0.5.  Returns (batch,
    seqlen, heads, head_dim) in the inputs' type.
    """
    return FlashAttnFunc.apply(q, k, v, softmax_scale, causal)
