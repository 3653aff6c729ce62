"""GPU parity tests at the FULL sizes of the BASELINE configs, every (batch, head) compared.

The CPU oracle would take minutes to hours at these sizes, so the checker here is the blockwise
oracle (``oracle/attention_oracle_blockwise.py``: the same fp32 math path, evaluated chunk by
chunk with plain fp32 matmuls, TF32 off) running on the GPU; the first test ties it to the CPU
oracle on a row subset of the largest shape.  The kernels are called through the C ABI.
Tolerances (floating point) as everywhere: O <= 2e-3 max-abs, LSE <= 2e-3, dQ/dK/dV <= 1e-2
relative L2.
"""
import ctypes

import pytest
import torch

from oracle import attention_oracle as oracle
from oracle import attention_oracle_blockwise as blockwise
from tests import helpers

pytestmark = pytest.mark.gpu


def _device_inputs(Z, N, H, D, seed, n_k=None):
    """Seeded N(0,1) fp16 inputs drawn on the GPU (the CPU generator is slow at 67 M elements)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    n_k = N if n_k is None else n_k
    mk = lambda n: torch.randn((Z, n, H, D), generator=g, device="cuda", dtype=torch.float32).half()
    return mk(N), mk(n_k), mk(n_k), mk(N)


def _check(q, k, v, dout, scale, causal, what, shift=0):
    from flash_attn_v100 import cabi

    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = cabi.fwd(q, k, v, scale, causal, shift, status=status)
    dq, dk, dv = cabi.bwd(q, k, v, out, dout, lse, scale, causal, shift, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = blockwise.attention_fwd_bwd_blockwise(q, k, v, dout, scale, causal, shift)
    return helpers.check_against_oracle((out, lse, dq, dk, dv), ref, what)


def test_blockwise_gpu_oracle_agrees_with_the_cpu_oracle():
    """One (batch, head) of config 3's shape, causal: the blockwise oracle on the GPU against the
    CPU oracle (fp32 both; only the summation order of the dot products differs), plus a row
    subset against the same rows of the whole."""
    q, k, v, dout = oracle.make_inputs(1, 2048, 2, 128, seed=3)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, None, True)
    got = blockwise.attention_fwd_bwd_blockwise(q.cuda(), k.cuda(), v.cuda(), dout.cuda(), None, True,
                                                row_chunk=512, head_chunk=1)
    assert oracle.max_abs(got[0].cpu(), ref[0]) < 2e-5 and oracle.max_abs(got[1].cpu(), ref[1]) < 2e-5
    for a, b in zip(got[2:], ref[2:]):
        assert oracle.rel_l2(a.cpu(), b) < 1e-5
    rows = slice(1024, 1536)
    o_r, l_r, dq_r = blockwise.attention_rows_blockwise(q.cuda(), k.cuda(), v.cuda(), dout.cuda(), rows,
                                                        None, True)
    assert oracle.max_abs(o_r.cpu(), ref[0][:, rows]) < 2e-5
    assert oracle.rel_l2(dq_r.cpu(), ref[2][:, rows]) < 1e-5


@pytest.mark.parametrize("N", [2048, 2016])
@pytest.mark.parametrize("causal", [True, False])
def test_cfg3_full_size_every_head(N, causal):
    """BASELINE config 3 (Z=8, H=32, D=128) at N=2048 and its ragged variant N=2016, causal and
    non-causal, all 256 (batch, head) slices."""
    q, k, v, dout = _device_inputs(8, N, 32, 128, seed=0)
    _check(q, k, v, dout, 128 ** -0.5, causal, f"cfg3 N={N} causal={causal}")


def test_cfg4_slice_and_full_batch():
    """BASELINE config 4: the per-GPU slice at 8 GPUs (Z=8, H=16, N=512, D=64, non-causal) and
    the whole batch Z=64 that one GPU runs."""
    for Z in (8, 64):
        q, k, v, dout = _device_inputs(Z, 512, 16, 64, seed=Z)
        _check(q, k, v, dout, 0.125, False, f"cfg4 Z={Z}")


@pytest.mark.parametrize("n_q,n_k,causal", [(4096, 4096, True), (4096, 2048, False), (2048, 4096, False)])
def test_cfg5_ring_step_shapes(n_q, n_k, causal):
    """The three dense shapes a ring step of BASELINE config 5 runs at 8 GPUs (H=32, D=128,
    4096-row shards): the local causal block, all local queries against the first half of a
    received block, the second half of the local queries against a whole received block."""
    q, k, v, dout = _device_inputs(1, n_q, 32, 128, seed=n_q + n_k, n_k=n_k)
    _check(q, k, v, dout, 128 ** -0.5, causal, f"cfg5 step {n_q}x{n_k} causal={causal}")


def test_reference_shaped_launchers_by_ctypes():
    """``fmha_b200_forward`` / ``fmha_b200_backward``: the literal replacements of the
    reference's launchers (include/fused_mha.h:1-6; called at kernel/fused_mha_api.cpp:68-69
    and :158-160), bound by ctypes with raw pointers exactly as a host without torch extensions
    would, on the reference's own test shape scaled down (test.py:4: N=2048, D=128, causal,
    sm_scale 0.1, seed 20) and on a rectangular non-causal case."""
    from flash_attn_v100 import cabi

    lib = cabi.load_library()
    for (Z, H, m, n, D, causal, seed) in ((1, 5, 2048, 2048, 128, 1, 20), (2, 3, 160, 416, 64, 0, 21)):
        q, k, v, dout = oracle.make_inputs(Z, m, H, D, seed=seed, n_k=n)
        qd, kd, vd, dod = (t.cuda().contiguous() for t in (q, k, v, dout))
        out = torch.empty_like(qd)
        lse = torch.empty((Z, H, m), dtype=torch.float32, device="cuda")
        dq, dk, dv = torch.empty_like(qd), torch.empty_like(kd), torch.empty_like(vd)
        stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
        ptr = lambda t: ctypes.c_void_p(t.data_ptr())
        rc = lib.fmha_b200_forward(ptr(qd), ptr(kd), ptr(vd), ptr(out), ptr(lse), Z, H, m, n, D,
                                   ctypes.c_float(0.1), causal, stream)
        assert rc == 0, cabi.status_string(rc)
        ws_bytes = cabi.bwd_workspace_bytes(Z, m, H, D)
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device="cuda")
        rc = lib.fmha_b200_backward(ptr(qd), ptr(kd), ptr(vd), ptr(out), ptr(dod), ptr(lse), ptr(dq),
                                    ptr(dk), ptr(dv), ptr(ws), ws_bytes, Z, H, m, n, D,
                                    ctypes.c_float(0.1), causal, stream)
        assert rc == 0, cabi.status_string(rc)
        torch.cuda.synchronize()
        ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, bool(causal))
        helpers.check_against_oracle((out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()), ref,
                                     f"fmha_b200_forward/backward Z{Z} H{H} {m}x{n} D{D}")
        # a workspace one byte short is refused, nothing launched
        rc = lib.fmha_b200_backward(ptr(qd), ptr(kd), ptr(vd), ptr(out), ptr(dod), ptr(lse), ptr(dq),
                                    ptr(dk), ptr(dv), ptr(ws), ws_bytes - 1, Z, H, m, n, D,
                                    ctypes.c_float(0.1), causal, stream)
        assert rc == 6
