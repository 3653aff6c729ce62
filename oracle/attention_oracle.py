"""CPU oracle for the attention hot path.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of
``bench.py`` may import this module; the product (the CUDA library and the
``flash_attn_v100`` package) never does and has no CPU fallback.

It restates the reference's own math path, the code the reference's test compares its kernel
against (``test.py:13-26``):

    p = (q @ k^T) * sm_scale                      test.py:17
    p[:, :, tril == 0] = -inf   (if causal)       test.py:16,18-19
    p = softmax(p.float(), dim=-1)                test.py:20
    out = p @ v                                   test.py:21-22
    out.backward(dout)  ->  dq, dk, dv            test.py:23-26

with ALL arithmetic in fp32 (or fp64) on the up-cast fp16 inputs, i.e. without the fp16
matmuls and the ``.half()`` of ``p`` that ``test.py`` itself uses; that fp32 form is the
correctness reference the build's tolerances (O <= 2e-3 max-abs, gradients <= 1e-2 relative
L2) are stated against.  Gradients are the closed form the reference kernel uses
(``kernel/fused_mha_kernel.cu:453-458,503-506`` and
``flash_attn_v100/flash_attn_interface.py:43-44``):

    P  = exp(scale * S - lse)          D  = rowsum(dO o O)
    dV = P^T dO                        dP = dO V^T
    dS = P o (dP - D) * scale          dQ = dS K        dK = dS^T Q

``lse = max + ln(sum)`` folds the reference's per-row ``softmax_max`` / ``softmax_sum``
(``kernel/fused_mha_kernel.cu:62-67,298-303``) into one number.

Parity pin: the reference ships no golden vectors (its only check is the relational
``allclose(atol=1e-2)`` of ``test.py:42-45``), so the oracle is pinned against OUTPUTS OF THE
REFERENCE'S MATH PATH ITSELF: ``tests/golden/make_golden.py`` executes the statements of
``test.py:13-26`` (read from the reference file, device changed to CPU) on seeded inputs and
stores them under ``tests/golden/``; ``tests/test_oracle.py`` checks this module against
those fixtures and against ``torch.autograd``.

Layout everywhere: (Z, N, H, D) = (batch, sequence, heads, head_dim), as the reference.
Masking: key j is visible to query i iff j <= i + causal_shift (the reference's square
``tril`` mask is causal_shift = 0).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch


def default_scale(head_dim: int) -> float:
    """flash_attn_v100/flash_attn_interface.py:67-68."""
    return head_dim ** (-0.5)


def make_inputs(Z: int, N: int, H: int, D: int, seed: int = 0, n_k: Optional[int] = None,
                dtype=torch.float16):
    """Seeded N(0,1) fp16 q, k, v, dout of shape (Z, N, H, D), drawn on the CPU in fp32 from one
    generator in the order q, k, v, dout and then rounded to fp16 (the reference draws N(0,1)
    fp16 tensors, test.py:5-10).  ``dtype=torch.bfloat16`` rounds the same draws to bf16."""
    g = torch.Generator().manual_seed(seed)
    n_k = N if n_k is None else n_k
    q = torch.randn((Z, N, H, D), generator=g, dtype=torch.float32).to(dtype)
    k = torch.randn((Z, n_k, H, D), generator=g, dtype=torch.float32).to(dtype)
    v = torch.randn((Z, n_k, H, D), generator=g, dtype=torch.float32).to(dtype)
    dout = torch.randn((Z, N, H, D), generator=g, dtype=torch.float32).to(dtype)
    return q, k, v, dout


def _visible(n_q: int, n_k: int, causal: bool, causal_shift: int, device=None) -> Optional[torch.Tensor]:
    if not causal:
        return None
    i = torch.arange(n_q, device=device).unsqueeze(1)
    j = torch.arange(n_k, device=device).unsqueeze(0)
    return j <= i + causal_shift


def attention_forward(q, k, v, scale: Optional[float] = None, causal: bool = False,
                      causal_shift: int = 0, dtype=torch.float32) -> Tuple[torch.Tensor, torch.Tensor]:
    """O (Z, N, H, D) and LSE (Z, H, N), both in ``dtype``, one (batch) slice at a time so that the
    (H, N, N) score block bounds memory.  Rows that see no key give O = 0, LSE = -inf."""
    Z, Nq, H, D = q.shape
    Nk = k.shape[1]
    scale = default_scale(D) if scale is None else scale
    out = torch.empty((Z, Nq, H, D), dtype=dtype, device=q.device)
    lse = torch.empty((Z, H, Nq), dtype=dtype, device=q.device)
    vis = _visible(Nq, Nk, causal, causal_shift, q.device)
    for z in range(Z):
        qz = q[z].to(dtype).transpose(0, 1)  # (H, N, D)
        kz = k[z].to(dtype).transpose(0, 1)
        vz = v[z].to(dtype).transpose(0, 1)
        s = torch.matmul(qz, kz.transpose(1, 2)) * scale  # test.py:17
        if vis is not None:
            s = s.masked_fill(~vis, float("-inf"))  # test.py:18-19
        m = s.max(dim=-1, keepdim=True).values
        m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
        e = torch.exp(s - m)
        l = e.sum(dim=-1, keepdim=True)
        p = torch.where(l > 0, e / l, torch.zeros_like(e))  # test.py:20
        out[z] = torch.matmul(p, vz).transpose(0, 1)  # test.py:21-22
        lse[z] = (m + torch.log(l)).squeeze(-1)
    return out, lse


def attention_backward(q, k, v, out, lse, dout, scale: Optional[float] = None, causal: bool = False,
                       causal_shift: int = 0, dtype=torch.float32):
    """dQ, dK, dV in ``dtype`` from the closed form above.  ``out`` / ``lse`` are the forward's
    results (any dtype); D = rowsum(dO o O) is taken in ``dtype``."""
    Z, Nq, H, D = q.shape
    Nk = k.shape[1]
    scale = default_scale(D) if scale is None else scale
    dq = torch.empty((Z, Nq, H, D), dtype=dtype, device=q.device)
    dk = torch.empty((Z, Nk, H, D), dtype=dtype, device=q.device)
    dv = torch.empty((Z, Nk, H, D), dtype=dtype, device=q.device)
    vis = _visible(Nq, Nk, causal, causal_shift, q.device)
    for z in range(Z):
        qz = q[z].to(dtype).transpose(0, 1)
        kz = k[z].to(dtype).transpose(0, 1)
        vz = v[z].to(dtype).transpose(0, 1)
        oz = out[z].to(dtype).transpose(0, 1)
        doz = dout[z].to(dtype).transpose(0, 1)
        lz = lse[z].to(dtype).unsqueeze(-1)  # (H, N, 1)
        s = torch.matmul(qz, kz.transpose(1, 2)) * scale
        p = torch.exp(s - torch.where(torch.isinf(lz), torch.zeros_like(lz), lz))
        p = torch.where(torch.isinf(lz), torch.zeros_like(p), p)
        if vis is not None:
            p = p.masked_fill(~vis, 0.0)
        delta = (doz * oz).sum(dim=-1, keepdim=True)  # flash_attn_interface.py:43-44
        dv[z] = torch.matmul(p.transpose(1, 2), doz).transpose(0, 1)
        dp = torch.matmul(doz, vz.transpose(1, 2))
        ds = p * (dp - delta) * scale
        dq[z] = torch.matmul(ds, kz).transpose(0, 1)
        dk[z] = torch.matmul(ds.transpose(1, 2), qz).transpose(0, 1)
    return dq, dk, dv


def attention_fwd_bwd(q, k, v, dout, scale=None, causal=False, causal_shift=0, dtype=torch.float32):
    """Forward + backward of the math path; returns (out, lse, dq, dk, dv) in ``dtype``."""
    out, lse = attention_forward(q, k, v, scale, causal, causal_shift, dtype)
    dq, dk, dv = attention_backward(q, k, v, out, lse, dout, scale, causal, causal_shift, dtype)
    return out, lse, dq, dk, dv


def attention_autograd(q, k, v, dout, scale=None, causal=False, dtype=torch.float32):
    """The same math path written exactly like test.py:13-26 (transpose, matmul, tril mask,
    softmax, matmul, ``backward``) but in ``dtype`` throughout; gradients by torch.autograd.
    Used to cross-check the closed-form gradients."""
    D = q.shape[-1]
    scale = default_scale(D) if scale is None else scale
    qf = q.detach().to(dtype).requires_grad_()
    kf = k.detach().to(dtype).requires_grad_()
    vf = v.detach().to(dtype).requires_grad_()
    qt, kt, vt = qf.transpose(1, 2), kf.transpose(1, 2), vf.transpose(1, 2)
    n_q, n_k = q.shape[1], k.shape[1]
    p = torch.matmul(qt, kt.transpose(2, 3)) * scale
    if causal:
        M = torch.tril(torch.ones((n_q, n_k)))
        p = p.masked_fill(M == 0, float("-inf"))
    p = torch.softmax(p, dim=-1)
    ref_out = torch.matmul(p, vt).transpose(1, 2)
    ref_out.backward(dout.to(dtype))
    return ref_out.detach(), qf.grad, kf.grad, vf.grad


def merge_partials(o_a, lse_a, o_b, lse_b):
    """LSE merge of two partial attention results over disjoint key sets (ring attention):
    o (Z, N, H, D), lse (Z, H, N); float tensors."""
    lse = torch.logaddexp(lse_a, lse_b)
    wa = torch.exp(lse_a - lse).transpose(1, 2).unsqueeze(-1)
    wb = torch.exp(lse_b - lse).transpose(1, 2).unsqueeze(-1)
    wa = torch.nan_to_num(wa, nan=0.0)
    wb = torch.nan_to_num(wb, nan=0.0)
    return wa * o_a + wb * o_b, lse


def numpy_forward_f64(q, k, v, scale=None, causal=False, causal_shift=0):
    """Independent float64 numpy forward for small cases (loops over batch and head)."""
    qn, kn, vn = (t.detach().cpu().numpy().astype(np.float64) for t in (q, k, v))
    Z, Nq, H, D = qn.shape
    Nk = kn.shape[1]
    scale = default_scale(D) if scale is None else scale
    out = np.zeros((Z, Nq, H, D))
    lse = np.full((Z, H, Nq), -np.inf)
    ii = np.arange(Nq)[:, None]
    jj = np.arange(Nk)[None, :]
    for z in range(Z):
        for h in range(H):
            s = qn[z, :, h, :] @ kn[z, :, h, :].T * scale
            if causal:
                s = np.where(jj <= ii + causal_shift, s, -np.inf)
            m = s.max(axis=1, keepdims=True)
            m = np.where(np.isinf(m), 0.0, m)
            e = np.exp(s - m)
            l = e.sum(axis=1, keepdims=True)
            with np.errstate(divide="ignore", invalid="ignore"):
                p = np.where(l > 0, e / l, 0.0)
                lse[z, h] = (m + np.log(l))[:, 0]
            out[z, :, h, :] = p @ vn[z, :, h, :]
    return out, lse


def max_abs(a, b) -> float:
    return (a.double() - b.double()).abs().max().item()


def rel_l2(a, b) -> float:
    """||a - b||_2 / ||b||_2 with b the reference."""
    a, b = a.double(), b.double()
    den = b.norm().item()
    return (a - b).norm().item() / (den if den > 0 else 1.0)


def attention_flops(Z: int, H: int, n_q: int, n_k: int, D: int, causal: bool, backward: bool = False) -> float:
    """Algorithmic FLOPs: forward 4*Z*H*N^2*D (halved when causal), backward 2.5x forward."""
    f = 4.0 * Z * H * n_q * n_k * D
    if causal:
        f *= 0.5
    return f * (2.5 if backward else 1.0)
