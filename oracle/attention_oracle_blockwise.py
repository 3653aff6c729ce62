"""Blockwise form of the oracle for sizes the plain one cannot hold.  TEST INFRASTRUCTURE ONLY.

Only ``tests/``, ``__graft_entry__.smoke()`` and the checking legs of ``bench.py`` (parity
figures printed beside a timing, never inside a timed region) may import this module; the
product never does.

The same math path as ``oracle/attention_oracle.py`` (the reference's ``test.py:13-26`` in fp32
with the closed-form gradients of ``kernel/fused_mha_kernel.cu:453-458,503-506``), evaluated one
batch entry, one group of heads and one chunk of query rows at a time, so that the score block
is (heads, rows, N_k) instead of (H, N, N): the full score matrix of a 32768-token sequence
would be 137 GB.  It runs on whatever device its inputs live on.  On a GPU every matmul is
plain fp32 (TF32 is switched off for the duration of the call), so the result differs from the
CPU oracle only by the summation order of fp32 dot products; ``tests/test_oracle.py`` checks the
two against each other.

A row subset can be asked for (``q_rows``): the forward and dQ are then produced for those
query rows only (dK/dV are sums over ALL query rows and always need the whole of q and dout).
"""
from __future__ import annotations

import contextlib
from typing import Optional, Tuple

import torch

from oracle.attention_oracle import default_scale


@contextlib.contextmanager
def _plain_fp32_matmul():
    old_mm = torch.backends.cuda.matmul.allow_tf32
    old_cudnn = torch.backends.cudnn.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    try:
        yield
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old_mm
        torch.backends.cudnn.allow_tf32 = old_cudnn


def _masked_scores(qc, kz, scale, causal, causal_shift, row0):
    """scale * qc kz^T with -inf where key j > query (row0 + i) + causal_shift."""
    s = torch.matmul(qc, kz.transpose(1, 2)) * scale  # test.py:17
    if causal:
        i = torch.arange(row0, row0 + qc.shape[1], device=qc.device).unsqueeze(1)
        j = torch.arange(kz.shape[1], device=qc.device).unsqueeze(0)
        s = s.masked_fill(~(j <= i + causal_shift), float("-inf"))  # test.py:18-19
    return s


def _softmax_lse(s):
    m = s.max(dim=-1, keepdim=True).values
    m = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    e = torch.exp(s - m)
    l = e.sum(dim=-1, keepdim=True)
    p = torch.where(l > 0, e / l, torch.zeros_like(e))  # test.py:20
    return p, (m + torch.log(l)).squeeze(-1)


def attention_fwd_bwd_blockwise(q, k, v, dout, scale: Optional[float] = None, causal: bool = False,
                                causal_shift: int = 0, row_chunk: int = 2048, head_chunk: int = 8,
                                want_grads: bool = True
                                ) -> Tuple[torch.Tensor, torch.Tensor, Optional[torch.Tensor],
                                           Optional[torch.Tensor], Optional[torch.Tensor]]:
    """(out, lse, dq, dk, dv) in fp32 on the inputs' device; q, dout (Z, N_q, H, D), k, v
    (Z, N_k, H, D) of any float dtype (up-cast to fp32 first, as the oracle does)."""
    Z, Nq, H, D = q.shape
    Nk = k.shape[1]
    scale = default_scale(D) if scale is None else scale
    dev = q.device
    out = torch.empty((Z, Nq, H, D), dtype=torch.float32, device=dev)
    lse = torch.empty((Z, H, Nq), dtype=torch.float32, device=dev)
    dq = torch.empty_like(out) if want_grads else None
    dk = torch.zeros((Z, Nk, H, D), dtype=torch.float32, device=dev) if want_grads else None
    dv = torch.zeros_like(dk) if want_grads else None
    with _plain_fp32_matmul():
        for z in range(Z):
            for h0 in range(0, H, head_chunk):
                hs = slice(h0, min(H, h0 + head_chunk))
                kz = k[z, :, hs].float().transpose(0, 1)  # (h, N_k, D)
                vz = v[z, :, hs].float().transpose(0, 1)
                for r0 in range(0, Nq, row_chunk):
                    rs = slice(r0, min(Nq, r0 + row_chunk))
                    qc = q[z, rs, hs].float().transpose(0, 1)  # (h, rows, D)
                    p, l = _softmax_lse(_masked_scores(qc, kz, scale, causal, causal_shift, r0))
                    oc = torch.matmul(p, vz)  # test.py:21-22
                    out[z, rs, hs] = oc.transpose(0, 1)
                    lse[z, hs, rs] = l
                    if not want_grads:
                        continue
                    doc = dout[z, rs, hs].float().transpose(0, 1)
                    delta = (doc * oc).sum(dim=-1, keepdim=True)  # flash_attn_interface.py:43-44
                    dv[z, :, hs] += torch.matmul(p.transpose(1, 2), doc).transpose(0, 1)
                    dp = torch.matmul(doc, vz.transpose(1, 2))
                    ds = p * (dp - delta) * scale
                    dq[z, rs, hs] = torch.matmul(ds, kz).transpose(0, 1)
                    dk[z, :, hs] += torch.matmul(ds.transpose(1, 2), qc).transpose(0, 1)
    return out, lse, dq, dk, dv


def attention_rows_blockwise(q, k, v, dout, q_rows: slice, scale: Optional[float] = None,
                             causal: bool = False, causal_shift: int = 0, row_chunk: int = 2048,
                             head_chunk: int = 8):
    """Forward and dQ for the query rows ``q_rows`` only (row indices keep their meaning for the
    causal mask): returns (out, lse, dq) of those rows in fp32."""
    start = q_rows.start or 0
    out, lse, dq, _, _ = _rows(q[:, q_rows], k, v, dout[:, q_rows], scale, causal,
                               causal_shift + start, row_chunk, head_chunk)
    return out, lse, dq


def _rows(q, k, v, dout, scale, causal, shift, row_chunk, head_chunk):
    # a row subset starting at row `start` is the same problem with causal_shift + start
    return attention_fwd_bwd_blockwise(q, k, v, dout, scale, causal, shift, row_chunk, head_chunk)
