"""GPU test of ``fmha_bwd_static_scratch``, the backward entry point for hosts that cannot
allocate device memory when they need a backward pass (all HBM already given to their own
pool, a latency-critical section that must not hit cudaMalloc's device-wide synchronisation,
or a policy that forbids a library to allocate).  Its workspace is the 32 MiB area built into
the library, shared by every call on a device.

Collected last on purpose (file name): a run that stops at the first failure has then already
run every other test.  The checks: two calls in a row, of different sizes so that the second
finds the first one's leftovers in the shared area, each compared with the ordinary
caller-workspace entry point ``fmha_bwd`` within the tolerances the other tests use
(dK, dV bit-identical, dQ within the gradient tolerance; the fp32 dQ reduction order varies);
and the size limit is enforced without launching anything.
"""
import pytest
import torch

from oracle import attention_oracle as oracle
from tests import helpers

pytestmark = pytest.mark.gpu


def _both_ways(Z, N, H, D, causal, seed):
    from flash_attn_v100 import cabi

    q, k, v, dout = (t.cuda() for t in oracle.make_inputs(Z, N, H, D, seed))
    scale = oracle.default_scale(D)
    out, lse = cabi.fwd(q, k, v, scale, causal)
    ref_dq, ref_dk, ref_dv = cabi.bwd(q, k, v, out, dout, lse, scale, causal)
    # every buffer is made here, before the call: the entry point itself allocates nothing
    dq, dk, dv = torch.full_like(q, 7.0), torch.full_like(k, 7.0), torch.full_like(v, 7.0)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    rc = cabi.bwd_static_scratch(q, k, v, out, dout, lse, dq, dk, dv, scale, causal, status=status)
    torch.cuda.synchronize()
    assert rc == 0, cabi.status_string(rc)
    assert int(status.item()) == 0
    assert torch.equal(dk, ref_dk) and torch.equal(dv, ref_dv)
    assert oracle.rel_l2(dq.float(), ref_dq.float()) <= helpers.TOL_GRAD_REL_L2
    # and against the oracle, like every other parity test
    cpu = lambda t: t.cpu()
    ref = oracle.attention_fwd_bwd(cpu(q), cpu(k), cpu(v), cpu(dout), scale, causal)
    helpers.check_against_oracle((cpu(out), cpu(lse), cpu(dq), cpu(dk), cpu(dv)), ref,
                                 f"static scratch Z{Z} N{N} H{H} D{D} causal={causal}")


def test_two_calls_in_a_row_match_the_workspace_entry_point():
    _both_ways(2, 512, 4, 128, True, seed=11)   # 4 MiB of the area
    _both_ways(1, 160, 3, 64, False, seed=12)   # smaller: finds the first call's leftovers
    _both_ways(2, 512, 4, 128, True, seed=13)   # and back


def test_sizes_beyond_the_built_in_area_are_rejected():
    from flash_attn_v100 import cabi

    # BASELINE config 3 needs a 256 MiB accumulator: far beyond the 32 MiB area
    Z, N, H, D = 8, 2048, 32, 128
    assert cabi.bwd_workspace_bytes(Z, N, H, D) > cabi.STATIC_SCRATCH_BYTES
    q = torch.zeros((Z, N, H, D), dtype=torch.float16, device="cuda")
    lse = torch.zeros((Z, H, N), dtype=torch.float32, device="cuda")
    rc = cabi.bwd_static_scratch(q, q, q, q, q, lse, q, q, q, 0.1, True)
    assert rc == 10 and "exceeds" in cabi.status_string(rc)
    # a size that still fits (1 x 3968 x 16 x 128 fp32 + statistics + order words)
    assert cabi.bwd_workspace_bytes(1, 3968, 16, 128) <= cabi.STATIC_SCRATCH_BYTES
