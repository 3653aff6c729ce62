"""GPU tests of the drop-in Python surface: flash_attn_func with autograd, written like the
reference's own test (test.py:4-45)."""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("Z,H,N,D,sm_scale", [(2, 4, 512, 128, 0.1), (2, 4, 128, 64, None)])
def test_flash_attn_func_autograd(Z, H, N, D, sm_scale, causal):
    from flash_attn_v100 import flash_attn_func

    qc, kc, vc, doc = oracle.make_inputs(Z, N, H, D, seed=20)
    q, k, v = (t.cuda().requires_grad_() for t in (qc, kc, vc))
    dout = doc.cuda()
    cuda_out = flash_attn_func(q, k, v, sm_scale, causal)   # test.py:33
    cuda_out.backward(dout)                                  # test.py:34
    dq, q.grad = q.grad.clone(), None
    dk, k.grad = k.grad.clone(), None
    dv, v.grad = v.grad.clone(), None
    ref_out, _, ref_dq, ref_dk, ref_dv = oracle.attention_fwd_bwd(qc, kc, vc, doc, sm_scale, causal)
    # the reference's assertions, test.py:42-45
    assert torch.allclose(ref_out, cuda_out.float().cpu(), atol=1e-2, rtol=0)
    assert torch.allclose(ref_dq, dq.float().cpu(), atol=1e-2, rtol=0)
    assert torch.allclose(ref_dk, dk.float().cpu(), atol=1e-2, rtol=0)
    assert torch.allclose(ref_dv, dv.float().cpu(), atol=1e-2, rtol=0)
    # and the build's tighter bar
    assert oracle.max_abs(cuda_out.float().cpu(), ref_out) <= helpers.TOL_O_MAX_ABS
    for a, b in ((dq, ref_dq), (dk, ref_dk), (dv, ref_dv)):
        assert oracle.rel_l2(a.float().cpu(), b) <= helpers.TOL_GRAD_REL_L2


def test_keyword_call_and_default_scale():
    from flash_attn_v100 import flash_attn_func

    qc, kc, vc, _ = oracle.make_inputs(1, 64, 2, 64, seed=1)
    q, k, v = qc.cuda(), kc.cuda(), vc.cuda()
    a = flash_attn_func(q, k, v)
    b = flash_attn_func(q, k, v, softmax_scale=64 ** -0.5, causal=False)
    assert torch.equal(a, b) and a.dtype == torch.float16 and a.shape == q.shape


def test_errors_like_the_reference():
    """RuntimeError from the extension's checks (kernel/fused_mha_api.cpp:23-47 style)."""
    from flash_attn_v100 import flash_attn_func

    q = torch.zeros(1, 64, 2, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(RuntimeError, match="fp16"):
        flash_attn_func(q.float(), q.float(), q.float())
    with pytest.raises(RuntimeError, match="head dimension"):
        flash_attn_func(q[..., :32], q[..., :32], q[..., :32])
    with pytest.raises(RuntimeError, match="multiples of 32"):
        flash_attn_func(q[:, :40], q[:, :40], q[:, :40])


def test_reference_extension_calling_convention():
    """The extension keeps the reference's positional fwd/bwd convention
    (flash_attn_interface.py:16-23,45-59): (max, sum) out, (D, sum, max) in."""
    import flash_attn_v100_cuda as ext

    qc, kc, vc, doc = oracle.make_inputs(1, 128, 2, 128, seed=6)
    q, k, v, dout = qc.cuda(), kc.cuda(), vc.cuda(), doc.cuda()
    out, softmax_max, softmax_sum = ext.fwd(q, k, v, None, 0.1, True)
    D = (out * dout).sum(-1)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    ext.bwd(dout, q, k, v, out, D, softmax_sum, softmax_max, dq, dk, dv, 0.1, True)
    ref = oracle.attention_fwd_bwd(qc, kc, vc, doc, 0.1, True)
    helpers.check_against_oracle((out.cpu(), softmax_max.cpu(), dq.cpu(), dk.cpu(), dv.cpu()), ref, "ext")


def test_registered_ops_and_torch_compile_fullgraph():
    """The extension calls are ``torch.library`` ops with fake implementations, so
    ``flash_attn_func`` compiles into one graph (the reference's glue,
    flash_attn_interface.py:62-99, calls pybind functions the compiler cannot trace).  The
    ``aot_eager`` backend traces forward and backward with fake tensors and runs the captured
    graph eagerly: same kernels, same bits as the uncompiled call."""
    from flash_attn_v100 import flash_attn_func

    qc, kc, vc, doc = oracle.make_inputs(2, 256, 3, 128, seed=14)
    dout = doc.cuda()

    def loss(q, k, v):
        return (flash_attn_func(q, k, v, 0.1, True).float() * dout.float()).sum()

    def grads(fn):
        q, k, v = (t.cuda().requires_grad_() for t in (qc, kc, vc))
        fn(q, k, v).backward()
        return q.grad, k.grad, v.grad

    eager = grads(loss)
    compiled = grads(torch.compile(loss, fullgraph=True, backend="aot_eager"))
    assert torch.equal(eager[1], compiled[1]) and torch.equal(eager[2], compiled[2])
    assert oracle.rel_l2(compiled[0].float().cpu(), eager[0].float().cpu()) < 1e-3  # dQ: fp32 add order
    ref = oracle.attention_fwd_bwd(qc, kc, vc, doc, 0.1, True)
    for a, b in zip(compiled, ref[2:]):
        assert oracle.rel_l2(a.float().cpu(), b) <= helpers.TOL_GRAD_REL_L2
    # schema, fake implementation and dispatch registration of both ops
    q, k, v = qc.cuda(), kc.cuda(), vc.cuda()
    torch.library.opcheck(torch.ops.flash_attn_v100.fwd.default, (q, k, v, 0.1, True),
                          test_utils=("test_schema", "test_faketensor"))
    out, lse = torch.ops.flash_attn_v100.fwd(q, k, v, 0.1, True)
    torch.library.opcheck(torch.ops.flash_attn_v100.bwd.default, (dout, q, k, v, out, lse, 0.1, True),
                          test_utils=("test_schema", "test_faketensor"))
