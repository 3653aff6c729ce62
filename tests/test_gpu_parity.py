"""GPU parity tests: the sm_100a kernels, called through the C ABI, against the CPU oracle
(fp32 math path) on the same seeded inputs, and against the golden fixtures made from the
reference's own math path.  Tolerances (floating point): O <= 2e-3 max-abs, LSE <= 2e-3,
dQ/dK/dV <= 1e-2 relative L2."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu


def _run(Z, N, H, D, causal, scale=None, seed=0, n_k=None, shift=0):
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed, n_k)
    scale = oracle.default_scale(D) if scale is None else scale
    got = helpers.gpu_fwd_bwd(q, k, v, dout, scale, causal, shift)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, scale, causal, shift)
    return helpers.check_against_oracle(got, ref, f"Z{Z} N{N}x{n_k or N} H{H} D{D} causal={causal} shift={shift}")


def test_cfg1_cpu_runnable_case():
    """BASELINE config 1: Z=2, H=4, N=128, D=64, scale 1/8, non-causal, seed 0."""
    _run(2, 128, 4, 64, False, 1.0 / 8.0, seed=0)


@pytest.mark.parametrize("name", helpers.golden_names())
def test_against_reference_math_path_fixtures(name):
    """Kernel vs the stored outputs of test.py:13-26, with the reference's own assertion
    (test.py:42-45): allclose(atol=1e-2, rtol=0) for out, dq, dk, dv."""
    g = helpers.load_golden(name)
    out, lse, dq, dk, dv = helpers.gpu_fwd_bwd(g["q"], g["k"], g["v"], g["dout"], g["scale"], g["causal"])
    for mine, ref, what in ((out, g["out"], "out"), (dq, g["dq"], "dq"), (dk, g["dk"], "dk"),
                            (dv, g["dv"], "dv")):
        assert torch.allclose(ref.float(), mine.float(), atol=helpers.TOL_REFERENCE_ATOL, rtol=0), \
            f"{name} {what}: max-abs {oracle.max_abs(mine.float(), ref.float()):.3e}"


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("N", [32, 64, 96, 128, 160, 256, 288, 416])
def test_tile_edges(N, D, causal):
    """Sequence lengths around the 128 / 256 tile sizes (multiples of 32, the reference's
    contract README.md:3); tails are masked inside the kernels."""
    _run(2, N, 2, D, causal, seed=N + D)


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
def test_growing_scores_exercise_the_lazy_rescale(D, causal):
    """Keys whose norm grows by 1.5x per block of 64: the running row maximum grows by more than
    2^8 at the late steps, the last one included, so the forward kernel has to rescale its
    output accumulator there (it does so only then), after waiting for the previous O += P V."""
    Z, N, H = 1, 512, 2
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=31)
    ramp = (1.5 ** torch.arange(N // 64, dtype=torch.float32)).repeat_interleave(64)
    k = (k.float() * ramp.view(1, N, 1, 1)).half()
    scale = oracle.default_scale(D)
    got = helpers.gpu_fwd_bwd(q, k, v, dout, scale, causal)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    helpers.check_against_oracle(got, ref, f"growing scores D{D} causal={causal}")


def test_long_sequence_many_steps_per_item():
    """N = 8192: 64 KV tiles per work item, i.e. 128 steps through the double-buffered S, the
    K/V ring and the Q ring of one persistent CTA, against the oracle on the whole problem."""
    _run(1, 8192, 1, 128, True, seed=21)


def test_many_items_per_cta_sampled_heads():
    """Z*H = 1184 heads of N = 512: every persistent forward CTA walks eight work items and the
    barrier phases run on across them; 6 heads, spread over the grid, are compared with the
    oracle (the oracle on all heads would take minutes)."""
    Z, N, H, D = 37, 512, 32, 64
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=22)
    scale = oracle.default_scale(D)
    out, lse, dq, dk, dv = helpers.gpu_fwd_bwd(q, k, v, dout, scale, True)
    for z, h in ((0, 0), (5, 31), (11, 7), (23, 16), (30, 1), (36, 31)):
        sl = (slice(z, z + 1), slice(None), slice(h, h + 1))
        ref = oracle.attention_fwd_bwd(q[sl], k[sl], v[sl], dout[sl], scale, True)
        got = (out[sl], lse[z:z + 1, h:h + 1], dq[sl], dk[sl], dv[sl])
        helpers.check_against_oracle(got, ref, f"head ({z},{h}) of Z{Z} H{H} N{N} D{D}")


@pytest.mark.parametrize("causal", [False, True])
def test_cfg2(causal):
    """BASELINE config 2: Z=4, H=16, N=1024, D=64, scale 0.125."""
    _run(4, 1024, 16, 64, causal, 0.125, seed=0)


@pytest.mark.parametrize("causal", [True, False])
def test_reference_test_shape_scaled_down(causal):
    """The reference's only test shape (test.py:4: H=40, N=2048, D=128, sm_scale 0.1, seed 20),
    with Z=1 and H=5 so that the CPU oracle stays in seconds."""
    _run(1, 2048, 5, 128, causal, 0.1, seed=20)


def test_ragged_tail_2016():
    """BASELINE config 3's ragged variant N=2016 (multiple of 32, not of 128), reduced batch."""
    _run(1, 2016, 4, 128, True, seed=0)


@pytest.mark.parametrize("n_q,n_k,causal,shift", [
    (128, 384, False, 0), (256, 128, False, 0), (128, 256, True, 128), (256, 256, True, -64),
    (256, 512, True, 256), (96, 160, True, 64), (384, 128, True, -256),
])
def test_rectangular_and_shifted_blocks(n_q, n_k, causal, shift):
    """Different query / key lengths and causal_shift, the block shapes ring attention feeds
    the same kernels; includes rows that see no key at all (O = 0, LSE = -inf)."""
    _run(1, n_q, 2, 128, causal, seed=n_q + n_k, n_k=n_k, shift=shift)
    _run(1, n_q, 2, 64, causal, seed=n_q + n_k + 1, n_k=n_k, shift=shift)


def test_strided_inputs_packed_qkv():
    """q, k, v as views of one packed (Z, N, 3, H, D) buffer: strides are honoured, no copy."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 2, 256, 3, 128
    g = torch.Generator().manual_seed(4)
    qkv = torch.randn((Z, N, 3, H, D), generator=g).half()
    dout = torch.randn((Z, N, H, D), generator=g).half()
    q, k, v = qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2]
    qkv_d = qkv.cuda()
    qd, kd, vd = qkv_d[:, :, 0], qkv_d[:, :, 1], qkv_d[:, :, 2]
    assert not qd.is_contiguous()
    out, lse = cabi.fwd(qd, kd, vd, 0.09, True)
    dq, dk, dv = cabi.bwd(qd, kd, vd, out, dout.cuda(), lse, 0.09, True)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.09, True)
    helpers.check_against_oracle((out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()), ref, "packed qkv")


def test_forward_is_deterministic_and_backward_dkdv_bitwise():
    from flash_attn_v100 import cabi

    q, k, v, dout = (t.cuda() for t in oracle.make_inputs(2, 512, 4, 128, seed=3))
    o1, l1 = cabi.fwd(q, k, v, 0.1, True)
    o2, l2 = cabi.fwd(q, k, v, 0.1, True)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    a = cabi.bwd(q, k, v, o1, dout, l1, 0.1, True)
    b = cabi.bwd(q, k, v, o1, dout, l1, 0.1, True)
    assert torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])  # dK, dV: no atomics
    assert oracle.rel_l2(a[0].float(), b[0].float()) < 1e-3     # dQ: fp32 reductions, order varies


@pytest.mark.parametrize("Z,N,H,D,causal,n_k,dtype", [
    (2, 1024, 4, 128, True, None, torch.float16), (2, 640, 3, 64, False, None, torch.float16),
    (1, 384, 2, 128, True, 896, torch.float16), (2, 512, 4, 128, True, None, torch.bfloat16),
])
def test_deterministic_dq_is_bitwise_reproducible(Z, N, H, D, causal, n_k, dtype):
    """FMHA_BWD_DETERMINISTIC: the partial sums of dQ are added in the order of the KV tiles, so
    three runs give the same bits (the default mode only promises the tolerance), and the result
    is as close to the oracle as the default mode's."""
    from flash_attn_v100 import cabi

    qc, kc, vc, doc = oracle.make_inputs(Z, N, H, D, seed=41, n_k=n_k, dtype=dtype)
    q, k, v, dout = qc.cuda(), kc.cuda(), vc.cuda(), doc.cuda()
    shift = 0 if n_k is None else n_k - N
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = cabi.fwd(q, k, v, 0.1, causal, shift)
    runs = [cabi.bwd(q, k, v, out, dout, lse, 0.1, causal, shift, flags=cabi.FMHA_BWD_DETERMINISTIC,
                     status=status) for _ in range(3)]
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    for other in runs[1:]:
        for a, b in zip(runs[0], other):
            assert torch.equal(a, b)
    ref = oracle.attention_fwd_bwd(qc, kc, vc, doc, 0.1, causal, shift)
    bf16 = dtype == torch.bfloat16
    helpers.check_against_oracle((out.cpu(), lse.cpu()) + tuple(t.cpu() for t in runs[0]), ref,
                                 f"deterministic Z{Z} N{N} H{H} D{D} causal={causal}",
                                 helpers.TOL_O_MAX_ABS_BF16 if bf16 else helpers.TOL_O_MAX_ABS)


def test_deterministic_dq_full_size_run_twice():
    """BASELINE config 3 at full size (4096 CTAs, 16 per head, far more than fit the GPU at once):
    the ordered reduction neither stalls nor changes between two runs."""
    from flash_attn_v100 import cabi

    g = torch.Generator(device="cuda").manual_seed(5)
    q, k, v, dout = (torch.randn((8, 2048, 32, 128), generator=g, device="cuda", dtype=torch.float32).half()
                     for _ in range(4))
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out, lse = cabi.fwd(q, k, v, 128 ** -0.5, True)
    a = cabi.bwd(q, k, v, out, dout, lse, 128 ** -0.5, True, flags=cabi.FMHA_BWD_DETERMINISTIC, status=status)
    b = cabi.bwd(q, k, v, out, dout, lse, 128 ** -0.5, True, flags=cabi.FMHA_BWD_DETERMINISTIC, status=status)
    c = cabi.bwd(q, k, v, out, dout, lse, 128 ** -0.5, True)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    assert oracle.rel_l2(a[0].float(), c[0].float()) < 1e-3


def test_linearity_in_v_and_dout_full_size():
    """Size-independent property at BASELINE config 3's full size (Z=8, H=32, N=2048, D=128,
    causal), where the CPU oracle is too slow: O is linear in V and dV is linear in dO, so
    f(2V) = 2 f(V) exactly in fp16 (a power of two), and O(V = const) = const."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 8, 2048, 32, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    q, k, v, dout = (torch.randn((Z, N, H, D), generator=g, device="cuda", dtype=torch.float32).half()
                     for _ in range(4))
    s = D ** -0.5
    o1, l1 = cabi.fwd(q, k, v, s, True)
    o2, l2 = cabi.fwd(q, k, 2 * v, s, True)
    # exact up to fp16 subnormals (2 * fp16(x) != fp16(2 * x) below 6.1e-5)
    assert (o2.float() - 2 * o1.float()).abs().max().item() <= 2.0 ** -23 and torch.equal(l1, l2)
    ones = torch.ones_like(v)
    o3, _ = cabi.fwd(q, k, ones, s, True)
    assert (o3.float() - 1).abs().max().item() < 2e-3
    dq1, dk1, dv1 = cabi.bwd(q, k, v, o1, dout, l1, s, True)
    dq2, dk2, dv2 = cabi.bwd(q, k, v, o1, 2 * dout, l1, s, True)
    assert (dv2.float() - 2 * dv1.float()).abs().max().item() <= 2.0 ** -23
    # dS = P o (dP - D) is rounded to fp16 before the dK / dQ MMAs: subnormal dS breaks exactness
    assert oracle.rel_l2(dk2.float(), 2 * dk1.float()) < 1e-4
    assert oracle.rel_l2(dq2.float(), 2 * dq1.float()) < 1e-3
    # against torch's own fp32 math on the GPU for one (batch, head) slice
    sl = lambda t: t[3:4, :, 7:8].cpu()
    ref = oracle.attention_fwd_bwd(sl(q), sl(k), sl(v), sl(dout), s, True)
    helpers.check_against_oracle((sl(o1), l1[3:4, 7:8].cpu(), sl(dq1), sl(dk1), sl(dv1)), ref, "cfg3 slice")


def test_status_word_stays_zero_and_negative_scale():
    from flash_attn_v100 import cabi

    q, k, v, dout = oracle.make_inputs(1, 256, 2, 64, seed=8)
    got = helpers.gpu_fwd_bwd(q, k, v, dout, -0.2, True)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, -0.2, True)
    helpers.check_against_oracle(got, ref, "negative scale")


def test_a_set_status_word_drains_the_kernels_without_touching_the_outputs():
    """A status word that is already non-zero (an earlier kernel gave up on a bounded wait) makes
    every CTA of the attention kernels return at once: the word keeps its value and the outputs
    keep their contents.  No wait is made to run out here: the word is set by the host."""
    from flash_attn_v100 import cabi

    q, k, v, dout = (t.cuda() for t in oracle.make_inputs(2, 256, 2, 128, seed=9))
    out_ok, lse = cabi.fwd(q, k, v, 0.1, True)
    status = torch.full((1,), 0x142, dtype=torch.int32, device="cuda")
    out = torch.full_like(q, 7.0)
    cabi.fwd(q, k, v, 0.1, True, out=out, lse=torch.empty_like(lse), status=status)
    dk, dv = torch.full_like(k, 7.0), torch.full_like(v, 7.0)
    cabi.bwd(q, k, v, out_ok, dout, lse, 0.1, True, dk=dk, dv=dv, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0x142
    assert bool((out == 7.0).all()) and bool((dk == 7.0).all()) and bool((dv == 7.0).all())
    # and with a clean word the same calls work again (nothing was left behind)
    status.zero_()
    out2, _ = cabi.fwd(q, k, v, 0.1, True, status=status)
    assert torch.equal(out2, out_ok) and int(status.item()) == 0


def test_forward_with_fewer_ctas_gives_the_same_bits():
    """sm_margin only changes how many persistent CTAs share the work list, never the result."""
    from flash_attn_v100 import cabi

    q, k, v, _ = (t.cuda() for t in oracle.make_inputs(4, 1024, 24, 128, seed=10))
    out0, lse0 = cabi.fwd(q, k, v, 0.09, True)
    for margin in (1, 47, 147, 1000):
        out1, lse1 = cabi.fwd(q, k, v, 0.09, True, sm_margin=margin)
        assert torch.equal(out0, out1) and torch.equal(lse0, lse1), f"sm_margin={margin}"
