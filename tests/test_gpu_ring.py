"""GPU tests of the multi-GPU layer's building blocks (1 GPU) and of ring attention itself
(2 GPUs, NCCL; skipped where fewer devices are visible)."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as oracle
from tests import helpers
from tests.conftest import PKG

pytestmark = pytest.mark.gpu
sys.path.insert(0, PKG)


def test_merge_kernel_matches_oracle_merge():
    """fmha_merge: two partial results over disjoint key halves merged through LSE equal the
    attention over all keys.  The accumulators start as LSE = -inf and an o_acc that is never
    read for such rows (NaN here): the first merge initialises them."""
    from flash_attn_v100 import cabi

    q, k, v, _ = oracle.make_inputs(2, 256, 3, 128, seed=5, n_k=512)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    o_acc = torch.full((2, 256, 3, 128), float("nan"), dtype=torch.float32, device="cuda")
    lse_acc = torch.full((2, 3, 256), float("-inf"), device="cuda")
    for lo in (0, 256):
        o_p, l_p = cabi.fwd(qd, kd[:, lo:lo + 256], vd[:, lo:lo + 256], 0.1, False)
        cabi.merge(o_acc, lse_acc, o_p, l_p)
    ref_o, ref_lse = oracle.attention_forward(q, k, v, 0.1, False)
    assert oracle.max_abs(o_acc.cpu(), ref_o) <= helpers.TOL_O_MAX_ABS
    assert oracle.max_abs(lse_acc.cpu(), ref_lse) <= helpers.TOL_LSE_MAX_ABS


@pytest.mark.parametrize("dtype,D", [(torch.float16, 128), (torch.bfloat16, 64), (torch.float16, 96)])
def test_merge_of_all_parts_in_one_pass(dtype, D):
    """fmha_merge_parts: three partial results (two over all query rows, one over the second half
    only, as in zig-zag ring attention) merged in one pass equal the attention over all keys the
    rows saw, and equal the step-by-step merge into fp32 accumulators."""
    from flash_attn_v100 import cabi

    Z, N, H = 2, 256, 3
    half = N // 2
    q, k, v, _ = oracle.make_inputs(Z, N, H, D, seed=41, n_k=3 * 128, dtype=dtype)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    blocks = [(slice(0, N), slice(0, 128)), (slice(half, N), slice(128, 256)), (slice(0, N), slice(256, 384))]
    parts_o, parts_l, offs = [], [], []
    o_acc = torch.empty((Z, N, H, D), dtype=torch.float32, device="cuda")
    lse_acc = torch.full((Z, H, N), float("-inf"), device="cuda")
    for qr, kr in blocks:
        o_p, l_p = cabi.fwd(qd[:, qr], kd[:, kr], vd[:, kr], 0.1, False)
        parts_o.append(o_p.contiguous())
        parts_l.append(l_p)
        offs.append(qr.start)
        cabi.merge(o_acc, lse_acc, o_p, l_p, row_offset=qr.start)
    out = torch.empty((Z, N, H, D), dtype=dtype, device="cuda")
    lse = torch.empty((Z, H, N), device="cuda")
    cabi.merge_parts(parts_o, parts_l, offs, out, lse)
    assert oracle.max_abs(lse.cpu(), lse_acc.cpu()) <= 1e-5
    tol = helpers.TOL_O_MAX_ABS_BF16 if dtype == torch.bfloat16 else helpers.TOL_O_MAX_ABS
    assert oracle.max_abs(out.float().cpu(), o_acc.cpu()) <= tol
    # against the oracle: the first half of the rows saw key blocks 0 and 2, the second half all
    keys_first = torch.cat([k[:, :128], k[:, 256:]], dim=1), torch.cat([v[:, :128], v[:, 256:]], dim=1)
    ref_a, lse_a = oracle.attention_forward(q[:, :half], keys_first[0], keys_first[1], 0.1, False)
    ref_b, lse_b = oracle.attention_forward(q[:, half:], k, v, 0.1, False)
    assert oracle.max_abs(out[:, :half].float().cpu(), ref_a) <= tol
    assert oracle.max_abs(out[:, half:].float().cpu(), ref_b) <= tol
    assert oracle.max_abs(lse[:, :, :half].cpu(), lse_a) <= helpers.TOL_LSE_MAX_ABS
    assert oracle.max_abs(lse[:, :, half:].cpu(), lse_b) <= helpers.TOL_LSE_MAX_ABS
    # rows whose parts are all empty (LSE = -inf): zeros and -inf, no NaN
    for l in parts_l:
        l[:, :, -1] = float("-inf")
    cabi.merge_parts(parts_o, parts_l, offs, out, lse)
    assert not out[:, -1].any() and bool(torch.isinf(lse[:, :, -1]).all()) and not torch.isnan(out.float()).any()


def test_merge_of_a_row_range_into_larger_accumulators():
    """fmha_merge_rows: a partial result for the second half of the query rows merged in place
    into full-height accumulators equals the merge of a compact copy of that row range."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 2, 256, 3, 128
    q, k, v, _ = oracle.make_inputs(Z, N, H, D, seed=13)
    qd, kd, vd = q.cuda(), k.cuda(), v.cuda()
    half = N // 2
    o_acc = torch.randn((Z, N, H, D), device="cuda")
    lse_acc = torch.randn((Z, H, N), device="cuda")
    o_p, l_p = cabi.fwd(qd[:, half:], kd, vd, 0.1, False)
    o_ref, l_ref = o_acc.clone(), lse_acc.clone()
    o_sub, l_sub = o_ref[:, half:].contiguous(), l_ref[:, :, half:].contiguous()
    cabi.merge(o_sub, l_sub, o_p, l_p)
    o_ref[:, half:], l_ref[:, :, half:] = o_sub, l_sub
    cabi.merge(o_acc, lse_acc, o_p, l_p, row_offset=half)
    assert torch.equal(o_acc, o_ref) and torch.equal(lse_acc, l_ref)


def test_backward_accumulates_over_key_blocks_into_fp32_buffers():
    """Ring-style backward on one GPU: two key blocks, dQ accumulated in one workspace over both
    calls, dK/dV added into row ranges of fp32 buffers (batch stride != dense), dQ converted at
    the end by fmha_bwd_convert_dq."""
    from flash_attn_v100 import cabi

    Z, Nq, H, D, Nk = 2, 256, 2, 64, 384
    q, k, v, dout = oracle.make_inputs(Z, Nq, H, D, seed=6, n_k=Nk)
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.15, False)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = cabi.fwd(qd, kd, vd, 0.15, False)
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, Nq, H, D), dtype=torch.uint8, device="cuda")
    dk_acc = torch.zeros((Z, Nk, H, D), dtype=torch.float32, device="cuda")
    dv_acc = torch.zeros_like(dk_acc)
    flags = cabi.FMHA_BWD_SKIP_DQ_CONVERT
    for lo, hi in ((0, 128), (128, 384)):
        cabi.bwd(qd, kd[:, lo:hi], vd[:, lo:hi], out, dod, lse, 0.15, False, dq=None,
                 dk_accum=dk_acc[:, lo:hi], dv_accum=dv_acc[:, lo:hi], workspace=ws, flags=flags)
        flags |= cabi.FMHA_BWD_KEEP_WORKSPACE
    dq = torch.empty_like(qd)
    cabi.bwd_convert_dq(ws, dq, 0.15)
    got = (out.cpu(), lse.cpu(), dq.cpu(), dk_acc.cpu(), dv_acc.cpu())
    helpers.check_against_oracle(got, ref, "blockwise backward")


def test_backward_overwrites_the_fp32_buffers_when_asked():
    """FMHA_BWD_ACCUM_OVERWRITE: dK / dV replace what dk_accum / dv_accum hold (NaN here), rows that
    no query row sees are written as zeros, so the buffers of ring attention's partial results
    need no clearing.  Rectangular causal case: the keys beyond the last query row are unseen."""
    from flash_attn_v100 import cabi

    for (Z, Nq, Nk, H, D, causal) in ((2, 128, 416, 2, 64, True), (1, 256, 256, 3, 128, False)):
        q, k, v, dout = oracle.make_inputs(Z, Nq, H, D, seed=16, n_k=Nk)
        ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.12, causal)
        qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
        out, lse = cabi.fwd(qd, kd, vd, 0.12, causal)
        # a row range of a larger buffer, like the half-block steps of the ring
        big_k = torch.full((Z, Nk + 64, H, D), float("nan"), dtype=torch.float32, device="cuda")
        big_v = torch.full_like(big_k, float("nan"))
        dq, _, _ = cabi.bwd(qd, kd, vd, out, dod, lse, 0.12, causal, dk_accum=big_k[:, :Nk], dv_accum=big_v[:, :Nk],
                            flags=cabi.FMHA_BWD_ACCUM_OVERWRITE)
        assert torch.isnan(big_k[:, Nk:]).all() and torch.isnan(big_v[:, Nk:]).all()  # untouched beyond
        got = (out.cpu(), lse.cpu(), dq.cpu(), big_k[:, :Nk].cpu(), big_v[:, :Nk].cpu())
        helpers.check_against_oracle(got, ref, f"overwrite Nq{Nq} Nk{Nk} D{D} causal={causal}")
        if causal:
            assert not big_k[:, Nq:Nk].any() and not big_v[:, Nq:Nk].any()  # unseen keys: zeros


def test_backward_over_a_row_range_of_the_queries_shares_the_workspace():
    """q_row_begin: query rows before it take no part.  (a) Alone: dQ of the excluded rows stays
    zero, dQ of the others and dK / dV equal those of an attention over the included rows only.
    (b) The way ring attention splits its local causal block: (second half of the queries) x
    (second half of the keys) first, all queries x (first half of the keys) second, one
    workspace, equals the causal backward in one call."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 2, 512, 3, 128
    half = N // 2
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=23)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    # (a) non-causal, rows [half, N) only
    out, lse = cabi.fwd(qd, kd, vd, 0.1, False, status=status)
    dq, dk, dv = cabi.bwd(qd, kd, vd, out, dod, lse, 0.1, False, q_row_begin=half, status=status)
    ref = oracle.attention_fwd_bwd(q[:, half:], k, v, dout[:, half:], 0.1, False)
    assert not dq[:, :half].any()
    for got, want in ((dq[:, half:], ref[2]), (dk, ref[3]), (dv, ref[4])):
        assert oracle.rel_l2(got.float().cpu(), want) <= helpers.TOL_GRAD_REL_L2
    # (b) the local causal block in two parts
    out, lse = cabi.fwd(qd, kd, vd, 0.1, True, status=status)
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, N, H, D), dtype=torch.uint8, device="cuda")
    dk32 = torch.full((Z, N, H, D), float("nan"), device="cuda")
    dv32 = torch.full((Z, N, H, D), float("nan"), device="cuda")
    base = cabi.FMHA_BWD_SKIP_DQ_CONVERT | cabi.FMHA_BWD_ACCUM_OVERWRITE
    cabi.bwd(qd, kd[:, half:], vd[:, half:], out, dod, lse, 0.1, True, -half, dq=None,
             dk_accum=dk32[:, half:], dv_accum=dv32[:, half:], workspace=ws, flags=base, status=status,
             q_row_begin=half)
    cabi.bwd(qd, kd[:, :half], vd[:, :half], out, dod, lse, 0.1, True, 0, dq=None,
             dk_accum=dk32[:, :half], dv_accum=dv32[:, :half], workspace=ws,
             flags=base | cabi.FMHA_BWD_KEEP_WORKSPACE, status=status)
    dq = torch.empty_like(qd)
    cabi.bwd_convert_dq(ws, dq, 0.1)
    torch.cuda.synchronize()
    assert int(status.item()) == 0
    ref = oracle.attention_fwd_bwd(q, k, v, dout, 0.1, True)
    helpers.check_against_oracle((out.cpu(), lse.cpu(), dq.cpu(), dk32.cpu(), dv32.cpu()), ref, "local block in two parts")
    # a begin that is no multiple of the tile, or beyond the rows, is refused
    for bad in (64, N, -128):
        with pytest.raises(RuntimeError):
            cabi.bwd(qd, kd, vd, out, dod, lse, 0.1, True, q_row_begin=bad)


def test_backward_in_three_separate_calls_matches_one_call():
    """Preprocess only, then the fused kernel on the kept workspace, then the dQ conversion: the
    same bits as one fmha_bwd call (dK/dV bitwise, dQ up to the order of its fp32 additions)."""
    from flash_attn_v100 import cabi

    Z, N, H, D = 2, 384, 3, 128
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=12)
    qd, kd, vd, dod = q.cuda(), k.cuda(), v.cuda(), dout.cuda()
    out, lse = cabi.fwd(qd, kd, vd, 0.09, True)
    dq1, dk1, dv1 = cabi.bwd(qd, kd, vd, out, dod, lse, 0.09, True)
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, N, H, D), dtype=torch.uint8, device="cuda")
    dk2, dv2 = torch.empty_like(kd), torch.empty_like(vd)
    cabi.bwd(qd, kd, vd, out, dod, lse, 0.09, True, dk=dk2, dv=dv2, workspace=ws,
             flags=cabi.FMHA_BWD_PREPROCESS_ONLY)
    cabi.bwd(qd, kd, vd, out, dod, lse, 0.09, True, dk=dk2, dv=dv2, workspace=ws,
             flags=cabi.FMHA_BWD_KEEP_WORKSPACE | cabi.FMHA_BWD_SKIP_DQ_CONVERT)
    dq2 = cabi.bwd_convert_dq(ws, torch.empty_like(qd), 0.09)
    assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
    assert oracle.rel_l2(dq2.cpu().float(), dq1.cpu().float()) <= 1e-3
    # the static-scratch entry point cannot keep state between calls and refuses the flag
    p = cabi.bwd_params(qd, kd, vd, out, dod, lse, dq2, dk2, dv2, 0.09, True, 0, None, None,
                        cabi.FMHA_BWD_PREPROCESS_ONLY, None)
    import ctypes
    assert cabi.load_library().fmha_bwd_static_scratch(ctypes.byref(p), None) == 6


def test_a_flag_wait_that_runs_out_sets_the_status_word_and_drains_the_kernels():
    """The bounded wait for another GPU's flag, made to run out on one GPU: nothing ever sets the
    flag, the wait gives up after its limit (200 ms here), writes its code to the status word, and
    an attention kernel queued behind it with that status word returns without touching its
    outputs.  With the word cleared and the flag set the same calls go through."""
    import time

    from flash_attn_v100 import cabi

    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    counter = torch.zeros(2, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    q, k, v, _ = (t.cuda() for t in oracle.make_inputs(1, 256, 2, 128, seed=2))
    out_ok, _ = cabi.fwd(q, k, v, 0.1, True)
    out = torch.full_like(q, 7.0)
    cabi.counter_bump(counter)  # iteration 1: the flag would have to reach 1
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    cabi.peer_wait([flag.data_ptr()], counter.data_ptr(), status, 200)
    cabi.fwd(q, k, v, 0.1, True, out=out, status=status)
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    assert 0.15 < waited < 5.0, waited
    assert int(status.item()) == 0x200 and bool((out == 7.0).all())
    # the producer's side of the hand-shake: a signal with the iteration number lets the wait pass
    status.zero_()
    cabi.peer_signal([flag.data_ptr()], counter.data_ptr())
    t0 = time.perf_counter()
    cabi.peer_wait([flag.data_ptr()], counter.data_ptr(), status, 200)
    cabi.fwd(q, k, v, 0.1, True, out=out, status=status)
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 0.15
    assert int(status.item()) == 0 and torch.equal(out, out_ok)
    assert counter.tolist() == [1, 0]
    # invalid limits are refused on the host
    lib = cabi.load_library()
    import ctypes
    arr = (ctypes.c_void_p * 1)(flag.data_ptr())
    assert lib.fmha_peer_wait(arr, 1, ctypes.c_void_p(counter.data_ptr()), None, 0, None) == 3
    assert lib.fmha_peer_wait(arr, 17, ctypes.c_void_p(counter.data_ptr()), None, 100, None) == 10


def test_sum_partials_kernel():
    """fmha_sum_partials: the owner's final dK / dV = the sum of the per-source fp32 partial
    results, each counting only its first rows."""
    from flash_attn_v100 import cabi

    Z, rows, H, D = 2, 96, 3, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    parts = [torch.randn((Z, rows, H, D), generator=g, device="cuda") for _ in range(5)]
    counts = [96, 48, 96, 0, 48]
    ref = torch.zeros((Z, rows, H, D), device="cuda")
    for p, n in zip(parts, counts):
        ref[:, :n] += p[:, :n]
    for dtype in (torch.float16, torch.bfloat16):
        out = torch.empty((Z, rows, H, D), dtype=dtype, device="cuda")
        cabi.sum_partials([p.data_ptr() for p in parts], counts, out)
        assert torch.equal(out, ref.to(dtype))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _ring_worker(rank, world, port, causal, out_dir, transport, Z, rows_per_rank, H, D, repeats, pair=False):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from flash_attn_v100 import distributed as fd
        from flash_attn_v100 import peer_ring

        N = rows_per_rank * world
        g = torch.Generator(device="cuda").manual_seed(9)  # every rank draws the same whole sequence
        q, k, v, dout = (torch.randn((Z, N, H, D), generator=g, device="cuda", dtype=torch.float32).half()
                         for _ in range(4))
        ring = None
        if transport == "peer":
            ring = peer_ring.PeerRing((Z, rows_per_rank, H, D), torch.float16, torch.device("cuda", rank),
                                      pair_steps=pair)
        for _ in range(repeats):  # more than once: buffers, flags and iteration numbers are reused
            ql, kl, vl, dol = (fd.zigzag_split(t, rank, world).requires_grad_(i < 3)
                               for i, t in enumerate((q, k, v, dout)))
            if ring is None:
                out = fd.ring_flash_attn_func(ql, kl, vl, 0.1, causal)
            else:
                out = peer_ring.peer_ring_flash_attn_func(ring, ql, kl, vl, 0.1, causal)
            out.backward(dol)
        torch.cuda.synchronize()
        if ring is not None:
            ring.check()
            ring.close()
        torch.save(dict(out=out.detach().cpu(), dq=ql.grad.cpu(), dk=kl.grad.cpu(), dv=vl.grad.cpu()),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _visible_world():
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1


def _run_ring(tmp_path, causal, transport, Z, rows_per_rank, H, D, repeats=1, pair=False):
    from flash_attn_v100 import distributed as fd
    from oracle import attention_oracle_blockwise as blockwise

    world = _visible_world()
    mp.spawn(_ring_worker, args=(world, _free_port(), causal, str(tmp_path), transport, Z, rows_per_rank, H, D,
                                 repeats, pair), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    N = rows_per_rank * world
    g = torch.Generator(device="cuda").manual_seed(9)
    q, k, v, dout = (torch.randn((Z, N, H, D), generator=g, device="cuda", dtype=torch.float32).half()
                     for _ in range(4))
    ref_out, _, ref_dq, ref_dk, ref_dv = (t.cpu() for t in blockwise.attention_fwd_bwd_blockwise(
        q, k, v, dout, 0.1, causal))
    got = {key: fd.zigzag_merge([p[key] for p in parts]) for key in ("out", "dq", "dk", "dv")}
    assert oracle.max_abs(got["out"].float(), ref_out) <= helpers.TOL_O_MAX_ABS
    for key, ref in (("dq", ref_dq), ("dk", ref_dk), ("dv", ref_dv)):
        assert oracle.rel_l2(got[key].float(), ref) <= helpers.TOL_GRAD_REL_L2, key


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("transport", ["nccl", "peer"])
def test_ring_attention_on_gpus(transport, causal, tmp_path):
    """Zig-zag ring attention against the oracle on the full sequence, with the K/V blocks passed
    on by NCCL send/recv ("nccl") or pulled from their owners by the copy engines, gradients
    pushed to theirs ("peer").  World size = visible GPUs (2, 4 or 8); world size 1 exercises the
    same code path without a peer.  Two passes in a row: the second reuses every buffer and flag."""
    _run_ring(tmp_path, causal, transport, Z=2, rows_per_rank=512, H=4, D=128, repeats=2)


@pytest.mark.parametrize("causal", [True, False])
def test_ring_attention_shards_whose_half_is_no_multiple_of_the_tile(causal, tmp_path):
    """320 rows per rank: half a shard (160 rows) is no multiple of the 128-row tile, so the steps
    over the second half of the queries run on sliced tensors with a workspace of their own
    instead of q_row_begin."""
    _run_ring(tmp_path, causal, "peer", Z=2, rows_per_rank=320, H=2, D=64, repeats=2)


def test_ring_attention_with_paired_steps(tmp_path):
    """``pair_steps``: two steps over first halves of blocks in one kernel call (ranks 2 and up
    have such pairs, so this takes 3 or more GPUs to mean anything; with fewer it is the plain
    schedule).  Two passes in a row."""
    _run_ring(tmp_path, True, "peer", Z=2, rows_per_rank=512, H=4, D=128, repeats=2, pair=True)


@pytest.mark.parametrize("transport", ["nccl", "peer"])
def test_ring_attention_cfg5_shaped_shards(transport, tmp_path):
    """Shards shaped like BASELINE config 5's at 8 GPUs (Z=1, H=32, D=128, 4096 rows per rank),
    causal, checked against the blockwise oracle."""
    _run_ring(tmp_path, True, transport, Z=1, rows_per_rank=4096, H=32, D=128)
