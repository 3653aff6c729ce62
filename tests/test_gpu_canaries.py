"""GPU tests that stand in for a memory checker (compute-sanitizer is not available on the test
machines): every output of the kernels is a view into the middle of a larger buffer whose
surroundings hold a known pattern; after the kernels have run - on shapes whose tiles hang over
the end of the tensors - the surroundings must be untouched.  Also: two streams at once."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu
GUARD = 4096  # elements before and after every output


def _guarded(shape, dtype, fill):
    n = 1
    for s in shape:
        n *= s
    buf = torch.full((n + 2 * GUARD,), fill, dtype=dtype, device="cuda")
    return buf, buf[GUARD:GUARD + n].view(shape)


def _intact(buf, fill):
    return bool((buf[:GUARD] == fill).all()) and bool((buf[-GUARD:] == fill).all())


@pytest.mark.parametrize("Z,Nq,Nk,H,D,causal,shift", [
    (2, 96, 96, 3, 64, True, 0), (1, 160, 416, 2, 128, False, 0), (3, 288, 32, 2, 128, True, -64),
    (1, 2016, 2016, 2, 128, True, 0), (2, 32, 544, 1, 64, True, 512), (2, 160, 288, 3, 96, True, 0),
    (1, 416, 160, 2, 96, False, 0),
])
def test_outputs_do_not_write_outside_their_tensors(Z, Nq, Nk, H, D, causal, shift):
    from flash_attn_v100 import cabi

    q, k, v, dout = oracle.make_inputs(Z, Nq, H, D, seed=Nq + Nk, n_k=Nk)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    bo, out = _guarded((Z, Nq, H, D), torch.float16, 7.0)
    bl, lse = _guarded((Z, H, Nq), torch.float32, 7.0)
    bq, dq = _guarded((Z, Nq, H, D), torch.float16, 7.0)
    bk, dk = _guarded((Z, Nk, H, D), torch.float16, 7.0)
    bv, dv = _guarded((Z, Nk, H, D), torch.float16, 7.0)
    ws_bytes = cabi.bwd_workspace_bytes(Z, Nq, H, D)
    bw, ws = _guarded((ws_bytes,), torch.uint8, 0x5A)
    bak, dk_acc = _guarded((Z, Nk, H, D), torch.float32, 7.0)
    bav, dv_acc = _guarded((Z, Nk, H, D), torch.float32, 7.0)
    cabi.fwd(qd, kd, vd, 0.1, causal, shift, out=out, lse=lse)
    cabi.bwd(qd, kd, vd, out, dod, lse, 0.1, causal, shift, dq=dq, dk=dk, dv=dv, workspace=ws)
    # the same backward into fp32 buffers, overwritten, and once more with the ordered reduction
    cabi.bwd(qd, kd, vd, out, dod, lse, 0.1, causal, shift, dq=dq, dk_accum=dk_acc, dv_accum=dv_acc,
             workspace=ws, flags=cabi.FMHA_BWD_ACCUM_OVERWRITE | cabi.FMHA_BWD_DETERMINISTIC)
    torch.cuda.synchronize()
    for buf, fill, name in ((bo, 7.0, "out"), (bl, 7.0, "lse"), (bq, 7.0, "dq"), (bk, 7.0, "dk"), (bv, 7.0, "dv"),
                            (bw, 0x5A, "workspace"), (bak, 7.0, "dk_accum"), (bav, 7.0, "dv_accum")):
        assert _intact(buf, fill), f"{name}: a kernel wrote outside the tensor"
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, causal, shift)
    helpers.check_against_oracle((out.cpu(), lse.cpu(), dq.cpu(), dk.cpu(), dv.cpu()), ref, "guarded")
    assert oracle.rel_l2(dk_acc.cpu(), ref[3]) <= helpers.TOL_GRAD_REL_L2
    assert oracle.rel_l2(dv_acc.cpu(), ref[4]) <= helpers.TOL_GRAD_REL_L2


def test_two_streams_at_once_give_the_same_results():
    """The entry points keep no per-call state in the library: two forward + backward passes on two
    streams at the same time (own outputs, own workspaces) give the bits of the passes run alone."""
    from flash_attn_v100 import cabi

    cases = []
    for seed, (Z, N, H, D) in enumerate(((2, 1024, 8, 128), (4, 512, 8, 64))):
        q, k, v, dout = (t.cuda() for t in oracle.make_inputs(Z, N, H, D, seed=60 + seed))
        o, lse = cabi.fwd(q, k, v, 0.1, True)
        dq, dk, dv = cabi.bwd(q, k, v, o, dout, lse, 0.1, True)
        cases.append((q, k, v, dout, o, lse, dk, dv))
    torch.cuda.synchronize()
    streams = [torch.cuda.Stream(), torch.cuda.Stream()]
    got = []
    for _ in range(3):
        for s, (q, k, v, dout, *_r) in zip(streams, cases):
            with torch.cuda.stream(s):
                o, lse = cabi.fwd(q, k, v, 0.1, True, stream=s)
                dq, dk, dv = cabi.bwd(q, k, v, o, dout, lse, 0.1, True, stream=s)
                got.append((o, lse, dk, dv))
    torch.cuda.synchronize()
    for i, (o, lse, dk, dv) in enumerate(got):
        ref = cases[i % 2]
        assert torch.equal(o, ref[4]) and torch.equal(lse, ref[5])
        assert torch.equal(dk, ref[6]) and torch.equal(dv, ref[7])
