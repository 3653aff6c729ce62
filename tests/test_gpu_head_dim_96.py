"""GPU parity tests at head_dim 96 (the reference builds 128 only and announces more head
dimensions "in the future", kernel/fused_mha_api.cpp:44).  96 runs on the 128-wide kernels: the
tensor maps describe 96 columns, tile loads fill columns 96-127 with zeros and stores clip them.
Everything goes through the C ABI or the public Python API; the checker is the CPU oracle.
Tolerances as everywhere: O <= 2e-3 max-abs (bf16: 1.6e-2), LSE <= 2e-3, dQ/dK/dV <= 1e-2
relative L2."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu
D = 96


def _run(Z, N, H, causal, seed=0, n_k=None, shift=0, dtype=torch.float16):
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed, n_k, dtype=dtype)
    scale = oracle.default_scale(D)
    got = helpers.gpu_fwd_bwd(q, k, v, dout, scale, causal, shift)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, scale, causal, shift)
    bf16 = dtype == torch.bfloat16
    return helpers.check_against_oracle(
        got, ref, f"D96 Z{Z} N{N}x{n_k or N} H{H} causal={causal} shift={shift} {dtype}",
        helpers.TOL_O_MAX_ABS_BF16 if bf16 else helpers.TOL_O_MAX_ABS,
        helpers.TOL_GRAD_REL_L2_BF16 if bf16 else helpers.TOL_GRAD_REL_L2)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("N", [32, 128, 160, 416, 1024])
def test_tile_edges_and_a_long_row(N, causal):
    _run(2, N, 3, causal, seed=N)


@pytest.mark.parametrize("n_q,n_k,causal,shift", [(160, 416, False, 0), (256, 128, True, -64), (128, 384, True, 256)])
def test_rectangular_and_shifted_blocks(n_q, n_k, causal, shift):
    _run(1, n_q, 2, causal, seed=7, n_k=n_k, shift=shift)


@pytest.mark.parametrize("causal", [False, True])
def test_bf16(causal):
    _run(2, 288, 2, causal, seed=11, dtype=torch.bfloat16)


def test_many_heads_full_length():
    """A 7B-class layer shape with 96-wide heads, reduced batch: Z=1, H=8, N=2048, causal."""
    _run(1, 2048, 8, True, seed=3)


def test_columns_beyond_96_are_never_written():
    """q, k, v, dout and every output as 96-column views of 128-column buffers: the 32 columns
    behind each row keep their sentinel, in the outputs bit for bit (the stores clip), and the
    results equal those of dense tensors bit for bit (the loads never read them)."""
    from flash_attn_v100 import cabi

    Z, N, H = 2, 288, 3
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=21)
    dense = [t.cuda() for t in (q, k, v, dout)]

    def wide(t=None):
        buf = torch.full((Z, N, H, 128), 777.0, dtype=torch.float16, device="cuda")
        if t is not None:
            buf[..., :D] = t
        return buf

    bufs = [wide(t) for t in dense]
    qv, kv, vv, dov = (b[..., :D] for b in bufs)
    outs = [wide() for _ in range(4)]
    o_v, dq_v, dk_v, dv_v = (b[..., :D] for b in outs)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for causal in (True, False):
        o_d, lse_d = cabi.fwd(*dense[:3], 0.1, causal, status=status)
        dq_d, dk_d, dv_d = cabi.bwd(*dense[:3], o_d, dense[3], lse_d, 0.1, causal, status=status)
        _, lse_w = cabi.fwd(qv, kv, vv, 0.1, causal, out=o_v, status=status)
        cabi.bwd(qv, kv, vv, o_v, dov, lse_w, 0.1, causal, dq=dq_v, dk=dk_v, dv=dv_v, status=status)
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert torch.equal(lse_w, lse_d)
        for wide_out in outs:
            assert (wide_out[..., D:] == 777.0).all()
        # dQ sums fp32 partial tiles in the order the CTAs arrive: compare it by tolerance
        assert torch.equal(o_v, o_d) and torch.equal(dk_v, dk_d) and torch.equal(dv_v, dv_d)
        assert oracle.rel_l2(dq_v.float().cpu(), dq_d.float().cpu()) < 1e-3


def test_public_api_autograd():
    """flash_attn_func + backward at head_dim 96 (default scale 96^-0.5) against the oracle."""
    from flash_attn_v100 import flash_attn_func

    q, k, v, dout = oracle.make_inputs(2, 256, 4, D, seed=5)
    qd, kd, vd = (t.cuda().requires_grad_(True) for t in (q, k, v))
    out = flash_attn_func(qd, kd, vd, None, True)
    out.backward(dout.cuda())
    ref = oracle.attention_fwd_bwd(q, k, v, dout, None, True)
    assert oracle.max_abs(out.detach().float().cpu(), ref[0]) <= helpers.TOL_O_MAX_ABS
    for g, r in zip((qd.grad, kd.grad, vd.grad), ref[2:]):
        assert oracle.rel_l2(g.float().cpu(), r) <= helpers.TOL_GRAD_REL_L2


def test_deterministic_dq():
    """FMHA_BWD_DETERMINISTIC with three 32-column chunks per dQ row: the same bits twice, and
    inside the tolerance."""
    from flash_attn_v100 import cabi

    q, k, v, dout = oracle.make_inputs(2, 416, 3, D, seed=9)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = cabi.fwd(qd, kd, vd, 0.1, True, status=status)
    runs = [cabi.bwd(qd, kd, vd, out, dod, lse, 0.1, True, flags=cabi.FMHA_BWD_DETERMINISTIC, status=status)
            for _ in range(2)]
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert all(torch.equal(a, b) for a, b in zip(*runs))
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, True)
    helpers.check_against_oracle((out.cpu(), lse.cpu()) + tuple(t.cpu() for t in runs[0]), ref, "D96 deterministic")


def test_ring_building_blocks():
    """The pieces ring attention is made of, at head_dim 96: dK / dV into fp32 buffers (added and
    overwritten), dQ kept in the workspace over two calls and converted once, the LSE merge of
    two partial results, and the sum of fp32 partial results."""
    from flash_attn_v100 import cabi

    Z, N, H = 2, 256, 3
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=15)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, False)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    half = N // 2
    # forward: two key halves merged through LSE
    o_acc = torch.full((Z, N, H, D), float("nan"), dtype=torch.float32, device="cuda")  # never read while LSE = -inf
    lse_acc = torch.full((Z, H, N), float("-inf"), device="cuda")
    out16 = torch.empty((Z, N, H, D), dtype=torch.float16, device="cuda")
    for i, lo in enumerate((0, half)):
        o_p, l_p = cabi.fwd(qd, kd[:, lo:lo + half], vd[:, lo:lo + half], 0.1, False)
        cabi.merge(o_acc, lse_acc, o_p, l_p, o_out=out16 if i == 1 else None)
    assert oracle.max_abs(o_acc.cpu(), ref[0]) <= helpers.TOL_O_MAX_ABS
    assert oracle.max_abs(out16.float().cpu(), ref[0]) <= helpers.TOL_O_MAX_ABS
    assert oracle.max_abs(lse_acc.cpu(), ref[1]) <= helpers.TOL_LSE_MAX_ABS
    # backward: one call per key half, dQ kept in the workspace, dK / dV into fp32 buffers
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, N, H, D), dtype=torch.uint8, device="cuda")
    dk32 = torch.full((Z, N, H, D), float("nan"), device="cuda")
    dv32 = torch.full((Z, N, H, D), float("nan"), device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    for i, lo in enumerate((0, half)):
        flags = cabi.FMHA_BWD_SKIP_DQ_CONVERT | cabi.FMHA_BWD_ACCUM_OVERWRITE
        if i == 1:
            flags |= cabi.FMHA_BWD_KEEP_WORKSPACE
        cabi.bwd(qd, kd[:, lo:lo + half], vd[:, lo:lo + half], out16, dod, lse_acc, 0.1, False, dq=None,
                 dk_accum=dk32[:, lo:lo + half], dv_accum=dv32[:, lo:lo + half], workspace=ws, flags=flags,
                 status=status)
    # a second, adding pass over the first half doubles it
    cabi.bwd(qd, kd[:, :half], vd[:, :half], out16, dod, lse_acc, 0.1, False, dq=None,
             dk_accum=dk32[:, :half], dv_accum=dv32[:, :half], workspace=ws,
             flags=cabi.FMHA_BWD_SKIP_DQ_CONVERT | cabi.FMHA_BWD_KEEP_WORKSPACE,
             status=status)
    dq = torch.empty_like(qd)
    cabi.bwd_convert_dq(ws, dq, 0.1)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    dk32[:, :half] *= 0.5
    dv32[:, :half] *= 0.5
    assert oracle.rel_l2(dk32.cpu(), ref[3]) <= helpers.TOL_GRAD_REL_L2
    assert oracle.rel_l2(dv32.cpu(), ref[4]) <= helpers.TOL_GRAD_REL_L2
    # dQ saw the first key half twice: dQ = dQ(first half) * 2 + dQ(second half)
    q32, k32, v32, do32 = (t.float() for t in (q, k, v, dout))
    s = torch.einsum("zqhd,zkhd->zhqk", q32, k32) * 0.1
    p = torch.softmax(s, dim=-1)
    dp = torch.einsum("zqhd,zkhd->zhqk", do32, v32)
    delta = (do32 * ref[0]).sum(-1).permute(0, 2, 1).unsqueeze(-1)
    ds = p * (dp - delta) * 0.1
    ds[..., :half] *= 2.0
    dq_ref = torch.einsum("zhqk,zkhd->zqhd", ds, k32)
    assert oracle.rel_l2(dq.float().cpu(), dq_ref) <= helpers.TOL_GRAD_REL_L2
    # sum of fp32 partial results
    g = torch.Generator(device="cuda").manual_seed(3)
    parts = [torch.randn((Z, N, H, D), generator=g, device="cuda") for _ in range(3)]
    counts = [N, half, 0]
    want = torch.zeros((Z, N, H, D), device="cuda")
    for part, n in zip(parts, counts):
        want[:, :n] += part[:, :n]
    got = torch.empty((Z, N, H, D), dtype=torch.float16, device="cuda")
    cabi.sum_partials([t.data_ptr() for t in parts], counts, got)
    assert torch.equal(got, want.half())
