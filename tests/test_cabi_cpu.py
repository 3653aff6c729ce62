"""CPU tests of the C-ABI library: it loads, exports every symbol the header declares, and
rejects bad parameters with status codes before touching a device (no compute here)."""
import ctypes
import os
import re

import pytest

from tests.conftest import ROOT


def _declared_functions():
    with open(os.path.join(ROOT, "include", "fmha_b200.h")) as f:
        text = f.read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmha_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(built_library):
    lib = ctypes.CDLL(built_library)
    names = _declared_functions()
    assert len(names) >= 8
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fmha_b200.h but not exported"


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header compiles as C99 (no C++ needed on the host side) and
    the parameter structs can be zero-initialised, which selects every default."""
    import subprocess

    src = tmp_path / "use_header.c"
    src.write_text('#include "fmha_b200.h"\n'
                   "int main(void) { FmhaFwdParams f = {0}; FmhaBwdParams b = {0};\n"
                   "  int (*fwd)(const FmhaFwdParams*, void*) = fmha_fwd; (void)fwd;\n"
                   "  return f.dtype + b.flags; }\n")
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-fsyntax-only",
                    "-I", os.path.join(ROOT, "include"), str(src)], check=True)


def test_binding_lists_the_same_symbols(built_library):
    from flash_attn_v100 import cabi

    assert sorted(cabi.EXPORTED_SYMBOLS) == _declared_functions()
    lib = cabi.load_library()
    assert lib.fmha_version().decode().count(".") == 2


def test_status_strings(built_library):
    from flash_attn_v100 import cabi

    assert cabi.status_string(0) == "ok"
    texts = {cabi.status_string(i) for i in range(0, 12)}
    assert len(texts) == 12 and "unknown status" not in texts
    assert cabi.status_string(999) == "unknown status"


def _fwd_params(cabi, **kw):
    p = cabi.FmhaFwdParams()
    for name in ("q", "k", "v", "o", "lse"):
        setattr(p, name, 0x1000)  # never dereferenced: validation fails first
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim = 1, 2, 64, 64, 128
    p.scale = 0.1
    for s in (p.q_strides, p.k_strides, p.v_strides, p.o_strides):
        s.batch, s.row, s.head = 64 * 2 * 128, 2 * 128, 128
    for k_, v_ in kw.items():
        setattr(p, k_, v_)
    return p


@pytest.mark.parametrize("change,status", [
    (dict(q=None), 1), (dict(lse=None), 1), (dict(head_dim=80), 2), (dict(head_dim=32), 2), (dict(head_dim=256), 2),
    (dict(batch=0), 3), (dict(seqlen_k=-5), 3), (dict(scale=0.0), 3), (dict(scale=float("nan")), 3),
    (dict(q=0x1008), 5), (dict(dtype=2), 11), (dict(dtype=-1), 11),
])
def test_forward_rejects_bad_parameters(built_library, change, status):
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    p = _fwd_params(cabi, **change)
    assert lib.fmha_fwd(ctypes.byref(p), None) == status


def test_forward_rejects_bad_strides(built_library):
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    p = _fwd_params(cabi)
    p.k_strides.row = 2 * 128 + 4  # not a multiple of 8 elements
    assert lib.fmha_fwd(ctypes.byref(p), None) == 4
    assert lib.fmha_fwd(None, None) == 1


def test_backward_workspace_size_and_validation(built_library):
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    # fp32 dQ accumulator (Z, N, H, D) + 2 x fp32 (Z, H, N padded to 128) + one int32 per (Z, H,
    # query tile), rounded up to 256 bytes
    assert cabi.bwd_workspace_bytes(2, 96, 3, 64) == 2 * 96 * 3 * 64 * 4 + 2 * 2 * 3 * 128 * 4 + 256
    assert cabi.bwd_workspace_bytes(8, 2048, 32, 128) == \
        8 * 2048 * 32 * 128 * 4 + 2 * 8 * 32 * 2048 * 4 + 8 * 32 * 16 * 4
    p = cabi.FmhaBwdParams()
    assert lib.fmha_bwd(ctypes.byref(p), None, 0, None) == 1
    for name in ("q", "k", "v", "o", "dout", "lse", "dq", "dk", "dv"):
        setattr(p, name, 0x1000)
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim, p.scale = 1, 1, 32, 32, 64, 1.0
    for s in (p.q_strides, p.k_strides, p.v_strides, p.o_strides, p.dout_strides, p.dq_strides,
              p.dk_strides, p.dv_strides):
        s.batch, s.row, s.head = 32 * 64, 64, 64
    assert lib.fmha_bwd(ctypes.byref(p), None, 0, None) == 6       # workspace missing
    assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 16, None) == 6    # workspace too small
    # "keep the workspace" and "only prepare the workspace" contradict each other
    p.flags = cabi.FMHA_BWD_KEEP_WORKSPACE | cabi.FMHA_BWD_PREPROCESS_ONLY
    assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 1 << 30, None) == 6
    p.flags = 0
    # q_row_begin: a multiple of the 128-row tile below seqlen_q, or 0
    p.seqlen_q = 512
    for bad in (64, 512, 640, -128):
        p.q_row_begin = bad
        assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 16, None) == 3, bad
    for good in (0, 128, 384):
        p.q_row_begin = good
        assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 16, None) == 6, good  # passes on to the workspace check
    p.q_row_begin, p.seqlen_q = 0, 32
    p.head_dim = 100
    assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 1 << 30, None) == 2


def test_backward_rejects_bad_accumulator_batch_stride(built_library):
    """dk_accum / dv_accum are added into with 16-byte accesses at accum + z * stride: a stride
    that would misalign them, overlap batch entries or is negative is a status code, not a GPU
    fault.  Validation returns before any CUDA call."""
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    p = cabi.FmhaBwdParams()
    for name in ("q", "k", "v", "o", "dout", "lse", "dq", "dk_accum", "dv_accum"):
        setattr(p, name, 0x1000)
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim, p.scale = 2, 2, 64, 32, 64, 1.0
    for s in (p.q_strides, p.o_strides, p.dout_strides, p.dq_strides):
        s.batch, s.row, s.head = 64 * 2 * 64, 2 * 64, 64
    for s in (p.k_strides, p.v_strides):
        s.batch, s.row, s.head = 32 * 2 * 64, 2 * 64, 64
    dense = 32 * 2 * 64
    for stride in (-dense, dense + 2, dense - 4, 4):
        p.accum_batch_stride = stride
        assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 1 << 30, None) == 4, stride
    # 0 (dense) and a larger multiple of 4 pass validation (the next check to fail is the
    # workspace, which is too small here)
    for stride in (0, dense, 2 * dense + 4):
        p.accum_batch_stride = stride
        assert lib.fmha_bwd(ctypes.byref(p), 0x2000, 16, None) == 6, stride


def test_static_scratch_refuses_flags_that_carry_state(built_library):
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    p = cabi.FmhaBwdParams()
    p.batch, p.heads, p.seqlen_q, p.seqlen_k, p.head_dim, p.scale = 1, 1, 32, 32, 64, 1.0
    for flag in (cabi.FMHA_BWD_KEEP_WORKSPACE, cabi.FMHA_BWD_SKIP_DQ_CONVERT, cabi.FMHA_BWD_PREPROCESS_ONLY):
        p.flags = flag
        assert lib.fmha_bwd_static_scratch(ctypes.byref(p), None) == 6, flag


def test_python_surface_matches_reference_names(built_library):
    """Same names as flash_attn_v100/flash_attn_interface.py and __init__.py of the reference."""
    import importlib.util
    import sys

    sys.path.insert(0, os.path.join(ROOT, "flash-attention-v100_b200"))
    import build as fmha_build

    fmha_build.build_extension()
    import inspect

    import flash_attn_v100
    from flash_attn_v100 import flash_attn_interface as fai

    assert flash_attn_v100.flash_attn_func is fai.flash_attn_func
    sig = inspect.signature(fai.flash_attn_func)
    assert list(sig.parameters) == ["q", "k", "v", "softmax_scale", "causal"]
    assert sig.parameters["softmax_scale"].default is None and sig.parameters["causal"].default is False
    for name in ("_flash_attn_forward", "_flash_attn_backward", "FlashAttnFunc"):
        assert hasattr(fai, name)
    assert hasattr(fai.flash_attn_cuda, "fwd") and hasattr(fai.flash_attn_cuda, "bwd")


def test_extension_raises_without_cuda_tensors(built_library):
    """No CPU fallback: CPU tensors are rejected with RuntimeError, like the reference's
    TORCH_CHECKs (kernel/fused_mha_api.cpp:31)."""
    import torch
    from flash_attn_v100 import flash_attn_func

    q = torch.zeros(1, 32, 1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="CUDA"):
        flash_attn_func(q, q, q)
