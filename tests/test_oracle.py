"""CPU tests of the oracle: pinned against the reference math path's golden outputs, against
torch.autograd, and against an independent float64 numpy forward."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers


@pytest.mark.parametrize("name", helpers.golden_names())
def test_oracle_matches_reference_math_path(name):
    """The fp32 restatement agrees with the outputs of test.py:13-26 (fp16 matmuls, P rounded
    to fp16) within the reference's own tolerance, test.py:42-45: atol 1e-2."""
    g = helpers.load_golden(name)
    out, lse, dq, dk, dv = oracle.attention_fwd_bwd(g["q"], g["k"], g["v"], g["dout"], g["scale"],
                                                    g["causal"])
    for mine, ref, what in ((out, g["out"], "out"), (dq, g["dq"], "dq"), (dk, g["dk"], "dk"),
                            (dv, g["dv"], "dv")):
        err = oracle.max_abs(mine, ref.float())
        assert err <= helpers.TOL_REFERENCE_ATOL, f"{name} {what}: {err}"
    # and far inside it in the relative-L2 sense
    assert oracle.rel_l2(out, g["out"].float()) < 2e-3


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("D", [64, 128])
def test_closed_form_gradients_match_autograd(causal, D):
    q, k, v, dout = oracle.make_inputs(2, 96, 3, D, seed=5)
    out, lse, dq, dk, dv = oracle.attention_fwd_bwd(q, k, v, dout, None, causal, dtype=torch.float64)
    a_out, a_dq, a_dk, a_dv = oracle.attention_autograd(q, k, v, dout, None, causal, dtype=torch.float64)
    for mine, ref in ((out, a_out), (dq, a_dq), (dk, a_dk), (dv, a_dv)):
        assert oracle.max_abs(mine, ref) < 1e-10


def test_fp32_oracle_close_to_fp64():
    q, k, v, dout = oracle.make_inputs(1, 256, 2, 128, seed=7)
    r32 = oracle.attention_fwd_bwd(q, k, v, dout, None, True)
    r64 = oracle.attention_fwd_bwd(q, k, v, dout, None, True, dtype=torch.float64)
    assert oracle.max_abs(r32[0], r64[0]) < 1e-5
    for a, b in zip(r32[2:], r64[2:]):
        assert oracle.rel_l2(a, b) < 1e-5


@pytest.mark.parametrize("causal,shift", [(False, 0), (True, 0), (True, 32), (True, -40)])
def test_torch_forward_matches_numpy_f64(causal, shift):
    q, k, v, _ = oracle.make_inputs(1, 64, 2, 64, seed=11, n_k=96)
    out, lse = oracle.attention_forward(q, k, v, 0.2, causal, shift, dtype=torch.float64)
    n_out, n_lse = oracle.numpy_forward_f64(q, k, v, 0.2, causal, shift)
    assert oracle.max_abs(out, torch.from_numpy(n_out)) < 1e-12
    fin = torch.isfinite(lse)
    assert torch.equal(fin, torch.from_numpy(n_lse).isfinite())
    assert oracle.max_abs(lse[fin], torch.from_numpy(n_lse)[fin]) < 1e-12


def test_rows_without_visible_keys_give_zero_and_minus_inf():
    q, k, v, _ = oracle.make_inputs(1, 64, 1, 64, seed=2)
    out, lse = oracle.attention_forward(q, k, v, None, True, causal_shift=-16)
    assert torch.all(out[:, :16] == 0) and torch.all(torch.isinf(lse[:, :, :16]))
    assert torch.all(torch.isfinite(lse[:, :, 16:]))


def test_merge_of_key_halves_equals_full_attention():
    """Ring attention's merge: attention over keys [0, n/2) and [n/2, n) merged through LSE."""
    q, k, v, _ = oracle.make_inputs(2, 64, 2, 64, seed=9, n_k=128)
    full, lse_full = oracle.attention_forward(q, k, v, dtype=torch.float64)
    a, la = oracle.attention_forward(q, k[:, :64], v[:, :64], dtype=torch.float64)
    b, lb = oracle.attention_forward(q, k[:, 64:], v[:, 64:], dtype=torch.float64)
    merged, lse = oracle.merge_partials(a, la, b, lb)
    assert oracle.max_abs(merged, full) < 1e-12 and oracle.max_abs(lse, lse_full) < 1e-12


def test_flop_model():
    # forward 4*Z*H*N^2*D, halved when causal; backward 2.5x
    assert oracle.attention_flops(8, 32, 2048, 2048, 128, True) == pytest.approx(274.88e9, rel=1e-4)
    assert oracle.attention_flops(8, 32, 2048, 2048, 128, True, True) == pytest.approx(687.2e9, rel=1e-4)


def test_default_scale():
    assert oracle.default_scale(64) == 0.125


@pytest.mark.parametrize("causal,shift,n_k", [(False, 0, None), (True, 0, None), (True, 64, 224), (True, -32, 96)])
def test_blockwise_oracle_equals_the_plain_oracle(causal, shift, n_k):
    """The chunked form (one group of heads and one chunk of query rows at a time, used where the
    whole score matrix does not fit) is the same computation: identical up to fp32 summation
    order, rows that see no key included."""
    from oracle import attention_oracle_blockwise as blockwise

    q, k, v, dout = oracle.make_inputs(2, 160, 3, 64, seed=17, n_k=n_k)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.11, causal, shift)
    got = blockwise.attention_fwd_bwd_blockwise(q, k, v, dout, 0.11, causal, shift, row_chunk=48,
                                                head_chunk=2)
    assert torch.equal(torch.isfinite(got[1]), torch.isfinite(ref[1]))
    fin = torch.isfinite(ref[1])
    assert oracle.max_abs(got[1][fin], ref[1][fin]) < 1e-5
    for a, b in ((got[0], ref[0]), (got[2], ref[2]), (got[3], ref[3]), (got[4], ref[4])):
        assert oracle.max_abs(a, b) < 2e-5
    # a row subset keeps the rows' positions in the causal mask
    rows = slice(64, 128)
    o_r, l_r, dq_r = blockwise.attention_rows_blockwise(q, k, v, dout, rows, 0.11, causal, shift,
                                                        row_chunk=40)
    assert oracle.max_abs(o_r, ref[0][:, rows]) < 2e-5 and oracle.max_abs(dq_r, ref[2][:, rows]) < 2e-5
