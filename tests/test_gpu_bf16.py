"""GPU parity tests with bf16 tensors (the reference is fp16 only, kernel/fused_mha_api.cpp:25-29,
and announces more types "in the future", :44): the same kernels with the tensor cores switched
to bf16 operands, against the oracle on the same bf16 inputs up-cast to fp32.

Tolerances (floating point, stated in tests/helpers.py): O <= 1.6e-2 max-abs (the output is
rounded to bf16: spacing 7.8e-3 in [1, 2)), LSE <= 2e-3 (fp32 either way), dQ/dK/dV <= 1e-2
relative L2."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16


def _check(got, ref, what):
    return helpers.check_against_oracle(got, ref, what, helpers.TOL_O_MAX_ABS_BF16,
                                        helpers.TOL_GRAD_REL_L2_BF16)


def _run(Z, N, H, D, causal, scale=None, seed=0, n_k=None, shift=0):
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed, n_k, dtype=BF16)
    scale = oracle.default_scale(D) if scale is None else scale
    got = helpers.gpu_fwd_bwd(q, k, v, dout, scale, causal, shift)
    assert got[0].dtype == BF16 and got[2].dtype == BF16
    ref = oracle.attention_fwd_bwd(q, k, v, dout, scale, causal, shift)
    return _check(got, ref, f"bf16 Z{Z} N{N}x{n_k or N} H{H} D{D} causal={causal} shift={shift}")


def test_cfg1_shape():
    _run(2, 128, 4, 64, False, 1.0 / 8.0)


@pytest.mark.parametrize("causal", [False, True])
def test_cfg2(causal):
    _run(4, 1024, 16, 64, causal, 0.125)


@pytest.mark.parametrize("causal", [True, False])
def test_cfg3_shape_reduced_batch_and_ragged(causal):
    _run(1, 2048, 4, 128, causal)
    _run(1, 2016, 2, 128, causal, seed=1)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("N", [32, 96, 160, 288])
def test_tile_edges(N, D):
    _run(2, N, 2, D, True, seed=N + D)
    _run(2, N, 2, D, False, seed=N + D + 1)


def test_rectangular_shifted_and_growing_scores():
    _run(1, 128, 2, 128, True, seed=3, n_k=256, shift=128)
    _run(1, 384, 2, 64, True, seed=4, n_k=128, shift=-256)
    # keys whose norm grows: the forward's lazy rescale path with bf16 P
    q, k, v, dout = oracle.make_inputs(1, 512, 2, 128, seed=31, dtype=BF16)
    ramp = (1.5 ** torch.arange(8, dtype=torch.float32)).repeat_interleave(64)
    k = (k.float() * ramp.view(1, 512, 1, 1)).to(BF16)
    got = helpers.gpu_fwd_bwd(q, k, v, dout, 128 ** -0.5, True)
    _check(got, oracle.attention_fwd_bwd(q, k, v, dout, 128 ** -0.5, True), "bf16 growing scores")


def test_flash_attn_func_autograd_bf16():
    """The public surface with bf16 tensors, written like the reference's test (test.py:33-37)."""
    from flash_attn_v100 import flash_attn_func

    qc, kc, vc, doc = oracle.make_inputs(2, 512, 4, 128, seed=20, dtype=BF16)
    q, k, v = (t.cuda().requires_grad_() for t in (qc, kc, vc))
    out = flash_attn_func(q, k, v, 0.1, True)
    out.backward(doc.cuda())
    assert out.dtype == BF16 and q.grad.dtype == BF16
    ref = oracle.attention_fwd_bwd(qc, kc, vc, doc, 0.1, True)
    assert oracle.max_abs(out.float().cpu(), ref[0]) <= helpers.TOL_O_MAX_ABS_BF16
    for a, b in ((q.grad, ref[2]), (k.grad, ref[3]), (v.grad, ref[4])):
        assert oracle.rel_l2(a.float().cpu(), b) <= helpers.TOL_GRAD_REL_L2_BF16
    # mixed types are refused
    with pytest.raises(RuntimeError, match="same data type"):
        flash_attn_func(q, k.half(), v)


def test_blockwise_backward_and_merge_bf16():
    """The ring-attention building blocks with bf16: two key blocks merged through LSE, dQ
    accumulated over two calls and converted at the end, dK/dV added into fp32 buffers."""
    from flash_attn_v100 import cabi

    Z, Nq, H, D, Nk = 2, 256, 2, 128, 384
    q, k, v, dout = oracle.make_inputs(Z, Nq, H, D, seed=6, n_k=Nk, dtype=BF16)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, False)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    o_acc = torch.zeros((Z, Nq, H, D), dtype=torch.float32, device="cuda")
    lse_acc = torch.full((Z, H, Nq), float("-inf"), device="cuda")
    out = torch.empty_like(qd)
    for lo, hi, last in ((0, 128, False), (128, 384, True)):
        o_p, l_p = cabi.fwd(qd, kd[:, lo:hi], vd[:, lo:hi], 0.1, False)
        cabi.merge(o_acc, lse_acc, o_p, l_p, o_out=out if last else None)
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, Nq, H, D), dtype=torch.uint8, device="cuda")
    dk_acc = torch.zeros((Z, Nk, H, D), dtype=torch.float32, device="cuda")
    dv_acc = torch.zeros_like(dk_acc)
    flags = cabi.FMHA_BWD_SKIP_DQ_CONVERT
    for lo, hi in ((0, 128), (128, 384)):
        cabi.bwd(qd, kd[:, lo:hi], vd[:, lo:hi], out, dod, lse_acc, 0.1, False, dq=None,
                 dk_accum=dk_acc[:, lo:hi], dv_accum=dv_acc[:, lo:hi], workspace=ws, flags=flags)
        flags |= cabi.FMHA_BWD_KEEP_WORKSPACE
    dq = cabi.bwd_convert_dq(ws, torch.empty_like(qd), 0.1)
    assert dq.dtype == BF16
    _check((out.cpu(), lse_acc.cpu(), dq.cpu(), dk_acc.cpu(), dv_acc.cpu()), ref, "bf16 blockwise")
