"""ctypes binding of the C ABI in ``include/fmha_b200.h`` for torch tensors.

This is the same boundary a non-Python host would bind (the reference's launchers,
``include/fused_mha.h:1-6``): plain pointers, sizes and a stream.  It exposes what the public
``flash_attn_func`` does not need but the multi-GPU layer and the tests do: different query /
key lengths, ``causal_shift``, fp32 dK/dV accumulation, the LSE merge, and the status word.

Loading fails loudly if ``lib/libfmha_b200.so`` has not been built; nothing here computes on
the CPU.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_LIB_PATH = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "lib",
                         "libfmha_b200.so")

FMHA_OK = 0
FMHA_BWD_KEEP_WORKSPACE = 1
FMHA_BWD_SKIP_DQ_CONVERT = 2
FMHA_BWD_PREPROCESS_ONLY = 4
FMHA_BWD_DETERMINISTIC = 8
FMHA_BWD_ACCUM_OVERWRITE = 16
FMHA_DTYPE_FP16 = 0
FMHA_DTYPE_BF16 = 1

EXPORTED_SYMBOLS = (
    "fmha_fwd", "fmha_bwd_workspace_bytes", "fmha_bwd", "fmha_bwd_static_scratch", "fmha_bwd_convert_dq", "fmha_merge", "fmha_merge_rows", "fmha_b200_forward",
    "fmha_b200_backward", "fmha_status_string", "fmha_version",
    "fmha_ipc_export", "fmha_ipc_open", "fmha_ipc_close", "fmha_peer_copy", "fmha_peer_copy_2d",
    "fmha_counter_bump", "fmha_peer_signal", "fmha_peer_wait", "fmha_sum_partials", "fmha_merge_parts",
)


class FmhaStrides(ctypes.Structure):
    _fields_ = [("batch", ctypes.c_int64), ("row", ctypes.c_int64), ("head", ctypes.c_int64)]


class FmhaFwdParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("q_strides", FmhaStrides), ("k_strides", FmhaStrides), ("v_strides", FmhaStrides),
        ("o_strides", FmhaStrides),
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seqlen_q", ctypes.c_int32),
        ("seqlen_k", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("scale", ctypes.c_float), ("causal", ctypes.c_int32), ("causal_shift", ctypes.c_int32),
        ("status", ctypes.c_void_p), ("sm_margin", ctypes.c_int32), ("dtype", ctypes.c_int32),
        ("seqused_q", ctypes.c_void_p), ("seqused_k", ctypes.c_void_p),
    ]


class FmhaBwdParams(ctypes.Structure):
    _fields_ = [
        ("q", ctypes.c_void_p), ("k", ctypes.c_void_p), ("v", ctypes.c_void_p),
        ("o", ctypes.c_void_p), ("dout", ctypes.c_void_p), ("lse", ctypes.c_void_p),
        ("dq", ctypes.c_void_p), ("dk", ctypes.c_void_p), ("dv", ctypes.c_void_p),
        ("dk_accum", ctypes.c_void_p), ("dv_accum", ctypes.c_void_p),
        ("accum_batch_stride", ctypes.c_int64),
        ("q_strides", FmhaStrides), ("k_strides", FmhaStrides), ("v_strides", FmhaStrides),
        ("o_strides", FmhaStrides), ("dout_strides", FmhaStrides),
        ("dq_strides", FmhaStrides), ("dk_strides", FmhaStrides), ("dv_strides", FmhaStrides),
        ("batch", ctypes.c_int32), ("heads", ctypes.c_int32), ("seqlen_q", ctypes.c_int32),
        ("seqlen_k", ctypes.c_int32), ("head_dim", ctypes.c_int32),
        ("scale", ctypes.c_float), ("causal", ctypes.c_int32), ("causal_shift", ctypes.c_int32),
        ("flags", ctypes.c_int32), ("status", ctypes.c_void_p), ("dtype", ctypes.c_int32),
        ("seqused_q", ctypes.c_void_p), ("seqused_k", ctypes.c_void_p),
        ("q_row_begin", ctypes.c_int32),
    ]


_lib = None


def load_library() -> ctypes.CDLL:
    """dlopen ``lib/libfmha_b200.so`` (once) and declare the prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(_LIB_PATH):
        raise RuntimeError(
            f"{_LIB_PATH} is missing: build it with `python flash-attention-v100_b200/build.py` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(_LIB_PATH)
    lib.fmha_fwd.restype = ctypes.c_int
    lib.fmha_fwd.argtypes = [ctypes.POINTER(FmhaFwdParams), ctypes.c_void_p]
    lib.fmha_bwd_workspace_bytes.restype = ctypes.c_size_t
    lib.fmha_bwd_workspace_bytes.argtypes = [ctypes.POINTER(FmhaBwdParams)]
    lib.fmha_bwd.restype = ctypes.c_int
    lib.fmha_bwd.argtypes = [ctypes.POINTER(FmhaBwdParams), ctypes.c_void_p, ctypes.c_size_t,
                             ctypes.c_void_p]
    lib.fmha_bwd_static_scratch.restype = ctypes.c_int
    lib.fmha_bwd_static_scratch.argtypes = [ctypes.POINTER(FmhaBwdParams), ctypes.c_void_p]
    lib.fmha_bwd_convert_dq.restype = ctypes.c_int
    lib.fmha_bwd_convert_dq.argtypes = [ctypes.c_void_p, ctypes.c_void_p, FmhaStrides, ctypes.c_int32,
                                        ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_float,
                                        ctypes.c_int32, ctypes.c_void_p]
    lib.fmha_merge.restype = ctypes.c_int
    lib.fmha_merge.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, FmhaStrides,
                               ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int32, ctypes.c_int32,
                               ctypes.c_int32, ctypes.c_int32, ctypes.c_int32, ctypes.c_void_p]
    lib.fmha_merge_rows.restype = ctypes.c_int
    lib.fmha_merge_rows.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, FmhaStrides,
                                    ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int32] * 7 + [
                                        ctypes.c_void_p]
    lib.fmha_b200_forward.restype = ctypes.c_int
    lib.fmha_b200_forward.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 5 + [
        ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    lib.fmha_b200_backward.restype = ctypes.c_int
    lib.fmha_b200_backward.argtypes = [ctypes.c_void_p] * 10 + [ctypes.c_size_t] + [
        ctypes.c_int] * 5 + [ctypes.c_float, ctypes.c_int, ctypes.c_void_p]
    vp, i32, i64, sz = ctypes.c_void_p, ctypes.c_int32, ctypes.c_int64, ctypes.c_size_t
    for name, args in (
            ("fmha_ipc_export", [vp, vp, ctypes.POINTER(i64)]),
            ("fmha_ipc_open", [vp, i64, ctypes.POINTER(vp)]),
            ("fmha_ipc_close", [vp, i64]),
            ("fmha_peer_copy", [vp, vp, sz, vp]),
            ("fmha_peer_copy_2d", [vp, sz, vp, sz, sz, sz, vp]),
            ("fmha_counter_bump", [vp, vp]),
            ("fmha_peer_signal", [ctypes.POINTER(vp), i32, vp, vp]),
            ("fmha_peer_wait", [ctypes.POINTER(vp), i32, vp, vp, i32, vp]),
            ("fmha_sum_partials", [ctypes.POINTER(vp), ctypes.POINTER(i32), i32, vp, FmhaStrides, i32, i32,
                                   i32, i32, i32, vp]),
            ("fmha_merge_parts", [ctypes.POINTER(vp), ctypes.POINTER(vp), ctypes.POINTER(i32),
                                  ctypes.POINTER(i32), i32, vp, vp, i32, i32, i32, i32, i32, vp])):
        getattr(lib, name).restype = ctypes.c_int
        getattr(lib, name).argtypes = args
    lib.fmha_status_string.restype = ctypes.c_char_p
    lib.fmha_status_string.argtypes = [ctypes.c_int]
    lib.fmha_version.restype = ctypes.c_char_p
    lib.fmha_version.argtypes = []
    _lib = lib
    return lib


def status_string(rc: int) -> str:
    return load_library().fmha_status_string(rc).decode()


def _check(rc: int, what: str):
    if rc != FMHA_OK:
        raise RuntimeError(f"{what} failed: {status_string(rc)} (status {rc})")


def _strides(t: torch.Tensor) -> FmhaStrides:
    return FmhaStrides(t.stride(0), t.stride(1), t.stride(2))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream(stream) -> ctypes.c_void_p:
    if stream is None:
        stream = torch.cuda.current_stream()
    return ctypes.c_void_p(stream.cuda_stream)


def _dtype_code(t: torch.Tensor) -> int:
    return FMHA_DTYPE_BF16 if t.dtype == torch.bfloat16 else FMHA_DTYPE_FP16


def _require_cuda_half(*tensors):
    """fp16 or bf16 (all the same) CUDA tensors of rank 4 with a contiguous last dimension."""
    first = None
    for t in tensors:
        if t is None:
            continue
        first = t if first is None else first
        if not t.is_cuda or t.dtype not in (torch.float16, torch.bfloat16) or t.dtype != first.dtype \
                or t.dim() != 4 or t.stride(-1) != 1:
            raise RuntimeError("expected fp16 or bf16 CUDA tensors of one type (batch, seqlen, heads, "
                               "head_dim) with a contiguous last dimension")


def _seqused_ptr(t: Optional[torch.Tensor], batch: int):
    if t is None:
        return None
    if not t.is_cuda or t.dtype != torch.int32 or t.dim() != 1 or t.numel() != batch or not t.is_contiguous():
        raise RuntimeError("seqused_q / seqused_k must be contiguous int32 CUDA tensors with one entry per batch")
    return t.data_ptr()


def fwd_params(q, k, v, o, lse, scale, causal, causal_shift=0, status=None, sm_margin=0,
               seqused_q=None, seqused_k=None) -> FmhaFwdParams:
    p = FmhaFwdParams()
    p.q, p.k, p.v, p.o, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr()
    p.q_strides, p.k_strides, p.v_strides, p.o_strides = _strides(q), _strides(k), _strides(v), _strides(o)
    p.batch, p.seqlen_q, p.heads, p.head_dim = q.shape
    p.seqlen_k = k.shape[1]
    p.scale = float(scale)
    p.causal = int(bool(causal))
    p.causal_shift = int(causal_shift)
    p.status = None if status is None else status.data_ptr()
    p.sm_margin = int(sm_margin)
    p.dtype = _dtype_code(q)
    p.seqused_q = _seqused_ptr(seqused_q, q.shape[0])
    p.seqused_k = _seqused_ptr(seqused_k, q.shape[0])
    return p


def fwd(q, k, v, scale: float, causal: bool = False, causal_shift: int = 0,
        out: Optional[torch.Tensor] = None, lse: Optional[torch.Tensor] = None,
        status: Optional[torch.Tensor] = None, stream=None, sm_margin: int = 0,
        seqused_q: Optional[torch.Tensor] = None, seqused_k: Optional[torch.Tensor] = None):
    """O, LSE through ``fmha_fwd`` on the current (or given) stream; outputs allocated with torch
    unless passed in.  ``sm_margin``: SMs the persistent kernel leaves to other streams' kernels.
    ``seqused_q`` / ``seqused_k``: per-batch real lengths of right-padded batches (int32)."""
    _require_cuda_half(q, k, v, out)
    Z, Nq, H, D = q.shape
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((Z, H, Nq), dtype=torch.float32, device=q.device)
    p = fwd_params(q, k, v, out, lse, scale, causal, causal_shift, status, sm_margin, seqused_q, seqused_k)
    with torch.cuda.device(q.device):
        _check(load_library().fmha_fwd(ctypes.byref(p), _stream(stream)), "fmha_fwd")
    return out, lse


def bwd_params(q, k, v, o, dout, lse, dq, dk, dv, scale, causal, causal_shift=0, dk_accum=None,
               dv_accum=None, flags=0, status=None, seqused_q=None, seqused_k=None,
               q_row_begin=0) -> FmhaBwdParams:
    p = FmhaBwdParams()
    p.q, p.k, p.v, p.dout, p.lse = q.data_ptr(), k.data_ptr(), v.data_ptr(), dout.data_ptr(), lse.data_ptr()
    p.o = None if o is None else o.data_ptr()
    p.dq = None if dq is None else dq.data_ptr()
    p.dk = None if dk is None else dk.data_ptr()
    p.dv = None if dv is None else dv.data_ptr()
    p.dk_accum = None if dk_accum is None else dk_accum.data_ptr()
    p.dv_accum = None if dv_accum is None else dv_accum.data_ptr()
    for acc in (dk_accum, dv_accum):
        if acc is not None:
            # (Z, N, H, D) fp32 with dense rows and heads; the batch stride is free
            if acc.dtype != torch.float32 or acc.stride(3) != 1 or acc.stride(2) != acc.shape[3] or \
                    acc.stride(1) != acc.shape[2] * acc.shape[3]:
                raise RuntimeError("dk_accum / dv_accum must be fp32 (Z, N, H, D) with dense rows and heads")
            p.accum_batch_stride = acc.stride(0)
    p.q_strides, p.k_strides, p.v_strides = _strides(q), _strides(k), _strides(v)
    p.dout_strides = _strides(dout)
    if o is not None:
        p.o_strides = _strides(o)
    if dq is not None:
        p.dq_strides = _strides(dq)
    if dk is not None:
        p.dk_strides = _strides(dk)
    if dv is not None:
        p.dv_strides = _strides(dv)
    p.batch, p.seqlen_q, p.heads, p.head_dim = q.shape
    p.seqlen_k = k.shape[1]
    p.scale = float(scale)
    p.causal = int(bool(causal))
    p.causal_shift = int(causal_shift)
    p.flags = int(flags)
    p.status = None if status is None else status.data_ptr()
    p.dtype = _dtype_code(q)
    p.seqused_q = _seqused_ptr(seqused_q, q.shape[0])
    p.seqused_k = _seqused_ptr(seqused_k, q.shape[0])
    p.q_row_begin = int(q_row_begin)
    return p


def bwd_workspace_bytes(Z: int, Nq: int, H: int, D: int) -> int:
    p = FmhaBwdParams()
    p.batch, p.seqlen_q, p.heads, p.head_dim = Z, Nq, H, D
    return int(load_library().fmha_bwd_workspace_bytes(ctypes.byref(p)))


def bwd(q, k, v, o, dout, lse, scale: float, causal: bool = False, causal_shift: int = 0,
        dq=None, dk=None, dv=None, dk_accum=None, dv_accum=None, workspace=None, flags: int = 0,
        status=None, stream=None, seqused_q=None, seqused_k=None, q_row_begin: int = 0):
    """dQ, dK, dV through ``fmha_bwd``.  Outputs and workspace are allocated with torch unless
    passed in; with ``dk_accum`` / ``dv_accum`` (fp32) the fp16 dK / dV are not produced.
    ``q_row_begin`` (a multiple of 128): query rows before it take no part in the call."""
    _require_cuda_half(q, k, v, o, dout, dq, dk, dv)
    Z, Nq, H, D = q.shape
    if dq is None and not (flags & (FMHA_BWD_SKIP_DQ_CONVERT | FMHA_BWD_PREPROCESS_ONLY)):
        dq = torch.empty_like(q)
    if dk is None and dk_accum is None:
        dk = torch.empty_like(k)
    if dv is None and dv_accum is None:
        dv = torch.empty_like(v)
    if workspace is None:
        workspace = torch.empty(bwd_workspace_bytes(Z, Nq, H, D), dtype=torch.uint8, device=q.device)
    p = bwd_params(q, k, v, o, dout, lse, dq, dk, dv, scale, causal, causal_shift, dk_accum,
                   dv_accum, flags, status, seqused_q, seqused_k, q_row_begin)
    with torch.cuda.device(q.device):
        _check(load_library().fmha_bwd(ctypes.byref(p), ctypes.c_void_p(workspace.data_ptr()),
                                       workspace.numel() * workspace.element_size(),
                                       _stream(stream)), "fmha_bwd")
    return dq, dk, dv


STATIC_SCRATCH_BYTES = 32 << 20


def bwd_static_scratch(q, k, v, o, dout, lse, dq, dk, dv, scale: float, causal: bool = False,
                       causal_shift: int = 0, status=None, stream=None) -> int:
    """``fmha_bwd_static_scratch``: backward whose workspace is the 32 MiB area built into the
    library, for hosts that must not allocate device memory.  The caller passes every input and
    output (nothing is allocated here either) and gets the raw status code back."""
    _require_cuda_half(q, k, v, o, dout, dq, dk, dv)
    p = bwd_params(q, k, v, o, dout, lse, dq, dk, dv, scale, causal, causal_shift, None, None, 0, status)
    with torch.cuda.device(q.device):
        return int(load_library().fmha_bwd_static_scratch(ctypes.byref(p), _stream(stream)))


def bwd_convert_dq(workspace, dq, scale: float, stream=None):
    """dq (fp16 or bf16, strided) = scale * the fp32 dQ accumulator at the start of ``workspace``."""
    Z, N, H, D = dq.shape
    with torch.cuda.device(dq.device):
        _check(load_library().fmha_bwd_convert_dq(ctypes.c_void_p(workspace.data_ptr()), _ptr(dq),
                                                  _strides(dq), Z, H, N, D, float(scale),
                                                  _dtype_code(dq), _stream(stream)), "fmha_bwd_convert_dq")
    return dq


def merge(o_acc, lse_acc, o_part, lse_part, o_out=None, stream=None, row_offset: int = 0):
    """In-place LSE merge of (o_part fp16 / bf16, lse_part) into (o_acc fp32 contiguous, lse_acc).  The
    partial result covers rows [row_offset, row_offset + o_part.shape[1]) of the accumulators."""
    Z, N, H, D = o_part.shape
    acc_rows = o_acc.shape[1]
    if not (o_acc.is_contiguous() and lse_acc.is_contiguous() and lse_part.is_contiguous()):
        raise RuntimeError("o_acc, lse_acc and lse_part must be contiguous")
    if o_out is not None and not o_out.is_contiguous():
        raise RuntimeError("o_out must be contiguous")
    with torch.cuda.device(o_part.device):
        _check(load_library().fmha_merge_rows(_ptr(o_acc), _ptr(lse_acc), _ptr(o_part),
                                              _strides(o_part), _ptr(lse_part), _ptr(o_out), Z, H, N,
                                              acc_rows, int(row_offset), D, _dtype_code(o_part),
                                              _stream(stream)),
               "fmha_merge_rows")
    return o_acc, lse_acc


# ----------------------------------------------------------------------------------------------
# multi-GPU plumbing (CUDA IPC addresses, copy-engine copies, flags between GPUs)
# ----------------------------------------------------------------------------------------------
def ipc_export(t: torch.Tensor):
    """(64-byte handle, offset) that another process of this node can turn into an address of
    ``t``'s memory with ``ipc_open``."""
    handle = ctypes.create_string_buffer(64)
    offset = ctypes.c_int64(0)
    with torch.cuda.device(t.device):
        _check(load_library().fmha_ipc_export(ctypes.c_void_p(t.data_ptr()), handle, ctypes.byref(offset)),
               "fmha_ipc_export")
    return bytes(handle.raw), int(offset.value)


def ipc_open(handle: bytes, offset: int) -> int:
    """Address (int) in this process of memory another process exported."""
    out = ctypes.c_void_p(0)
    _check(load_library().fmha_ipc_open(ctypes.c_char_p(handle), offset, ctypes.byref(out)), "fmha_ipc_open")
    return int(out.value)


def ipc_close(addr: int, offset: int):
    _check(load_library().fmha_ipc_close(ctypes.c_void_p(addr), offset), "fmha_ipc_close")


def peer_copy(dst: int, src: int, nbytes: int, stream=None):
    _check(load_library().fmha_peer_copy(ctypes.c_void_p(dst), ctypes.c_void_p(src), nbytes, _stream(stream)),
           "fmha_peer_copy")


def peer_copy_2d(dst: int, dst_pitch: int, src: int, src_pitch: int, row_bytes: int, rows: int, stream=None):
    _check(load_library().fmha_peer_copy_2d(ctypes.c_void_p(dst), dst_pitch, ctypes.c_void_p(src), src_pitch,
                                            row_bytes, rows, _stream(stream)), "fmha_peer_copy_2d")


def counter_bump(word: torch.Tensor, stream=None):
    _check(load_library().fmha_counter_bump(ctypes.c_void_p(word.data_ptr()), _stream(stream)),
           "fmha_counter_bump")


def _addr_array(addrs):
    return (ctypes.c_void_p * len(addrs))(*[ctypes.c_void_p(a) for a in addrs])


def peer_signal(flag_addrs, value_addr: int, stream=None):
    if flag_addrs:
        _check(load_library().fmha_peer_signal(_addr_array(flag_addrs), len(flag_addrs),
                                               ctypes.c_void_p(value_addr), _stream(stream)), "fmha_peer_signal")


def peer_wait(flag_addrs, value_addr: int, status: Optional[torch.Tensor], timeout_ms: int, stream=None):
    if flag_addrs:
        _check(load_library().fmha_peer_wait(_addr_array(flag_addrs), len(flag_addrs), ctypes.c_void_p(value_addr),
                                             None if status is None else ctypes.c_void_p(status.data_ptr()),
                                             int(timeout_ms), _stream(stream)), "fmha_peer_wait")


def sum_partials(part_addrs, rows_per_part, out: torch.Tensor, stream=None):
    """out (Z, rows, H, D) 16-bit = sum of fp32 buffers (Z, rows, H, D), part s counting only its
    first rows_per_part[s] rows of every batch entry."""
    Z, rows, H, D = out.shape
    rp = (ctypes.c_int32 * len(rows_per_part))(*rows_per_part)
    with torch.cuda.device(out.device):
        _check(load_library().fmha_sum_partials(_addr_array(part_addrs), rp, len(part_addrs), _ptr(out),
                                                _strides(out), Z, H, rows, D, _dtype_code(out),
                                                _stream(stream)), "fmha_sum_partials")
    return out


def merge_parts(o_parts, lse_parts, row_offsets, o_out, lse_out, stream=None):
    """``fmha_merge_parts``: o_out (Z, rows, H, D) 16-bit, lse_out (Z, H, rows) fp32 = the LSE merge
    of the partial results (o_parts[s] (Z, rows_s, H, D), lse_parts[s] (Z, H, rows_s), both
    contiguous), part s covering the output rows from row_offsets[s] on."""
    Z, rows, H, D = o_out.shape
    for o, l in zip(o_parts, lse_parts):
        if not (o.is_contiguous() and l.is_contiguous()) or o.dtype != o_out.dtype:
            raise RuntimeError("partial results must be contiguous and of the output's type")
    if not (o_out.is_contiguous() and lse_out.is_contiguous()):
        raise RuntimeError("o_out and lse_out must be contiguous")
    n = len(o_parts)
    ro = (ctypes.c_int32 * n)(*[int(x) for x in row_offsets])
    rp = (ctypes.c_int32 * n)(*[int(o.shape[1]) for o in o_parts])
    with torch.cuda.device(o_out.device):
        _check(load_library().fmha_merge_parts(_addr_array([o.data_ptr() for o in o_parts]),
                                               _addr_array([l.data_ptr() for l in lse_parts]), ro, rp, n,
                                               _ptr(o_out), _ptr(lse_out), Z, H, rows, D,
                                               _dtype_code(o_out), _stream(stream)), "fmha_merge_parts")
    return o_out, lse_out
