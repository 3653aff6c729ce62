"""GPU parity tests of right-padded batches (``seqused_q`` / ``seqused_k``): every batch entry
has its own real length, the rest of its rows is padding.  The reference's contract is "the
caller pads to a multiple of 32" (README.md:3) and it computes the padding like real rows; here
padding keys are masked, padding tiles are skipped, and the padding rows of every output are
zero.  The oracle runs per batch entry on the real rows only."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu


def _oracle_padded(q, k, v, dout, scale, causal, sq, sk):
    """The oracle on each batch entry's real rows, zeros (LSE -inf) on the padding."""
    Z, Nq, H, D = q.shape
    Nk = k.shape[1]
    out = torch.zeros((Z, Nq, H, D)); dq = torch.zeros((Z, Nq, H, D))
    dk = torch.zeros((Z, Nk, H, D)); dv = torch.zeros((Z, Nk, H, D))
    lse = torch.full((Z, H, Nq), float("-inf"))
    for z in range(Z):
        a, b = sq[z], sk[z]
        if a == 0:
            continue
        if b == 0:
            continue  # no keys: O = 0, LSE = -inf, all gradients zero
        r = oracle.attention_fwd_bwd(q[z:z + 1, :a], k[z:z + 1, :b], v[z:z + 1, :b], dout[z:z + 1, :a],
                                     scale, causal)
        out[z, :a], lse[z, :, :a], dq[z, :a], dk[z, :b], dv[z, :b] = r[0][0], r[1][0], r[2][0], r[3][0], r[4][0]
    return out, lse, dq, dk, dv


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
def test_padded_batch_matches_per_entry_oracle(D, causal):
    from flash_attn_v100 import cabi

    Z, N, H = 5, 512, 3
    sq = [512, 300, 128, 1, 0]
    sk = sq if causal else [512, 77, 256, 512, 40]
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=51)
    # recognisable finite junk in the padding: it must not leak into any real row
    for z in range(Z):
        q[z, sq[z]:], dout[z, sq[z]:] = 3.0, -2.0
        k[z, sk[z]:], v[z, sk[z]:] = 5.0, 7.0
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    sq_d = torch.tensor(sq, dtype=torch.int32, device="cuda")
    sk_d = torch.tensor(sk, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    scale = oracle.default_scale(D)
    out, lse = cabi.fwd(qd, kd, vd, scale, causal, status=status, seqused_q=sq_d, seqused_k=sk_d)
    dq, dk, dv = cabi.bwd(qd, kd, vd, out, dod, lse, scale, causal, status=status, seqused_q=sq_d,
                          seqused_k=sk_d)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = _oracle_padded(q, k, v, dout, scale, causal, sq, sk)
    helpers.check_against_oracle((out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()), ref,
                                 f"padded D{D} causal={causal}")
    # the padding rows are exactly zero
    for z in range(Z):
        assert not out[z, sq[z]:].any() and not dq[z, sq[z]:].any()
        assert not dk[z, sk[z]:].any() and not dv[z, sk[z]:].any()


def test_padded_public_function_with_autograd_and_deterministic():
    from flash_attn_v100 import flash_attn_padded_func

    Z, N, H, D = 3, 384, 2, 128
    lens = [384, 200, 96]
    qc, kc, vc, doc = oracle.make_inputs(Z, N, H, D, seed=52)
    lens_d = torch.tensor(lens, dtype=torch.int32, device="cuda")
    grads = []
    for _ in range(2):
        q, k, v = (t.cuda().requires_grad_() for t in (qc, kc, vc))
        out = flash_attn_padded_func(q, k, v, lens_d, lens_d, None, True, deterministic=True)
        out.backward(doc.cuda())
        grads.append((out.detach(), q.grad, k.grad, v.grad))
    assert all(torch.equal(a, b) for a, b in zip(*grads))
    ref = _oracle_padded(qc, kc, vc, doc, oracle.default_scale(D), True, lens, lens)
    out, dq, dk, dv = grads[0]
    assert oracle.max_abs(out.float().cpu(), ref[0]) <= helpers.TOL_O_MAX_ABS
    for a, b in ((dq, ref[2]), (dk, ref[3]), (dv, ref[4])):
        assert oracle.rel_l2(a.float().cpu(), b) <= helpers.TOL_GRAD_REL_L2
    # without lengths it is flash_attn_func
    from flash_attn_v100 import flash_attn_func
    q, k, v = qc.cuda(), kc.cuda(), vc.cuda()
    assert torch.equal(flash_attn_padded_func(q, k, v, causal=True), flash_attn_func(q, k, v, None, True))


def test_padding_tiles_are_skipped_not_computed():
    """A batch whose entries are 1/8 full runs several times faster than the full batch: the
    padding is skipped tile-wise (the reference, and any caller that pads without lengths,
    pays for it in full)."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 8, 4096, 8, 128
    g = torch.Generator(device="cuda").manual_seed(1)
    q, k, v = (torch.randn((Z, N, H, D), generator=g, device="cuda", dtype=torch.float32).half() for _ in range(3))
    lens = torch.full((Z,), N // 8, dtype=torch.int32, device="cuda")
    out, lse = torch.empty_like(q), torch.empty((Z, H, N), dtype=torch.float32, device="cuda")

    def ms(**kw):
        for _ in range(2):
            cabi.fwd(q, k, v, 0.09, False, out=out, lse=lse, **kw)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(5):
            cabi.fwd(q, k, v, 0.09, False, out=out, lse=lse, **kw)
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1)

    full, padded = ms(), ms(seqused_q=lens, seqused_k=lens)
    assert padded < full / 4, (full, padded)
