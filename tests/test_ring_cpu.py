"""CPU (gloo, world_size 2 and 4) tests of the ring-attention schedule: zig-zag sharding, the
K/V rotation, the three block shapes per step, the LSE merge and the travelling dK/dV
accumulators, with the oracle standing in for the CUDA kernels as the per-block backend."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import attention_oracle as oracle
from tests.conftest import PKG

sys.path.insert(0, PKG)


class OracleBackend:
    """Per-block compute by the CPU oracle (fp32), same interface as distributed.CudaBackend."""

    def fwd(self, q, k, v, scale, causal, overlap=False):
        return oracle.attention_forward(q, k, v, scale, causal)

    def new_accumulators(self, q):
        Z, N, H, D = q.shape
        return torch.zeros((Z, N, H, D)), torch.full((Z, H, N), float("-inf"))

    def merge(self, o_acc, lse_acc, o_part, lse_part, rows):
        o, l = oracle.merge_partials(o_acc[:, rows], lse_acc[:, :, rows], o_part.float(), lse_part)
        o_acc[:, rows] = o
        lse_acc[:, :, rows] = l

    def finish(self, o_acc, lse_acc, dtype):
        return o_acc, lse_acc  # keep fp32 for a tight comparison

    def new_bwd_state(self, q):
        return {"dq": torch.zeros(q.shape)}

    def bwd_step(self, state, which, q, k, v, o, dout, lse, scale, causal, dk_acc, dv_acc):
        dq, dk, dv = oracle.attention_backward(q, k, v, o, lse, dout, scale, causal)
        if which == "full":
            state["dq"] += dq
        else:
            state["dq"][:, state["dq"].shape[1] // 2:] += dq
        dk_acc += dk
        dv_acc += dv

    def bwd_finish(self, state, q, k, v, o, dout, lse, scale):
        return state["dq"]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, causal, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from flash_attn_v100 import distributed as fd

        Z, N, H, D = 2, 32 * world, 2, 64
        q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=3)
        ql, kl, vl, dol = (fd.zigzag_split(t, rank, world) for t in (q, k, v, dout))
        be = OracleBackend()
        out, lse = fd.ring_attention_forward(ql, kl, vl, 0.2, causal, None, be)
        dq, dk, dv = fd.ring_attention_backward(ql, kl, vl, out, lse, dol, 0.2, causal, None, be)
        torch.save(dict(out=out, lse=lse, dq=dq, dk=dk.float(), dv=dv.float()),
                   os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("world", [2, 4])
def test_ring_schedule_matches_full_attention(world, causal, tmp_path):
    from flash_attn_v100 import distributed as fd

    mp.spawn(_worker, args=(world, _free_port(), causal, str(tmp_path)), nprocs=world, join=True)
    parts = [torch.load(os.path.join(tmp_path, f"rank{r}.pt")) for r in range(world)]
    Z, N, H, D = 2, 32 * world, 2, 64
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=3)
    ref_out, ref_lse, ref_dq, ref_dk, ref_dv = oracle.attention_fwd_bwd(q, k, v, dout, 0.2, causal)
    got = {key: fd.zigzag_merge([p[key] for p in parts], dim=2 if key == "lse" else 1)
           for key in ("out", "lse", "dq", "dk", "dv")}
    assert oracle.max_abs(got["out"], ref_out) < 1e-5
    assert oracle.max_abs(got["lse"], ref_lse) < 1e-5
    # dK / dV went round the ring as fp32 and were cast to the fp16 of k / v at the end
    assert oracle.rel_l2(got["dq"], ref_dq) < 1e-5
    assert oracle.rel_l2(got["dk"], ref_dk) < 1e-3
    assert oracle.rel_l2(got["dv"], ref_dv) < 1e-3


def test_zigzag_split_roundtrip_and_batch_shard():
    from flash_attn_v100 import distributed as fd

    x = torch.arange(2 * 16 * 3).reshape(2, 16, 3)
    parts = [fd.zigzag_split(x, r, 4) for r in range(4)]
    assert parts[0][0, :, 0].tolist() == [0, 3, 42, 45]  # chunks 0 and 7 of 8 (2 rows each)
    assert torch.equal(fd.zigzag_merge(parts), x)
    assert torch.equal(torch.cat([fd.shard_batch(x, r, 2) for r in range(2)]), x)
    with pytest.raises(ValueError):
        fd.zigzag_split(x, 0, 3)
    with pytest.raises(ValueError):
        fd.shard_batch(x, 0, 3)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("world", [1, 2, 3, 8])
def test_pull_push_schedule_adds_up_to_full_attention(world, causal):
    """The schedule of the copy-engine transport (``peer_ring.PeerRing``), which has no gloo
    form because it moves data with CUDA IPC copies: every rank's per-step blocks
    (``ring_step_shapes``) and the rows each source contributes to an owner's dK/dV
    (``ring_grad_rows``) are played through for all ranks in one process, the oracle standing in
    for the kernels and plain tensor copies for the transport.  Outputs merged through LSE and
    gradients summed at the owners must equal attention over the whole sequence."""
    from flash_attn_v100 import distributed as fd

    Z, H, D = 1, 2, 64
    rows = 32  # per rank
    N = rows * world
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=7)
    ref_out, ref_lse, ref_dq, ref_dk, ref_dv = oracle.attention_fwd_bwd(q, k, v, dout, 0.2, causal)
    shard = lambda t, r: fd.zigzag_split(t, r, world)
    outs, lses, dqs = [], [], []
    # slots[owner][source] = (dk, dv) partial, and how many rows of it the source wrote
    slots = [[None] * world for _ in range(world)]
    for r in range(world):
        ql, dol = shard(q, r).float(), shard(dout, r).float()
        o_acc = torch.zeros((Z, rows, H, D))
        lse_acc = torch.full((Z, H, rows), float("-inf"))
        plan = fd.ring_step_shapes(r, world, causal, rows)
        assert [s[0] for s in plan] == [(r - t) % world for t in range(world)]
        for src, q_rows, kv_rows, causal_block in plan:
            kb, vb = shard(k, src)[:, kv_rows].float(), shard(v, src)[:, kv_rows].float()
            o_p, l_p = oracle.attention_forward(ql[:, q_rows], kb, vb, 0.2, causal_block)
            o, l = oracle.merge_partials(o_acc[:, q_rows], lse_acc[:, :, q_rows], o_p, l_p)
            o_acc[:, q_rows], lse_acc[:, :, q_rows] = o, l
        outs.append(o_acc), lses.append(lse_acc)
        dq = torch.zeros((Z, rows, H, D))
        for src, q_rows, kv_rows, causal_block in plan:
            kb, vb = shard(k, src)[:, kv_rows].float(), shard(v, src)[:, kv_rows].float()
            g = oracle.attention_backward(ql[:, q_rows], kb, vb, o_acc[:, q_rows], lse_acc[:, :, q_rows],
                                          dol[:, q_rows], 0.2, causal_block)
            dq[:, q_rows] += g[0]
            slots[src][r] = (g[1], g[2], kv_rows.stop)
        dqs.append(dq)
    dks, dvs = [], []
    for owner in range(world):
        expect = fd.ring_grad_rows(owner, world, causal, rows)
        dk, dv = torch.zeros((Z, rows, H, D)), torch.zeros((Z, rows, H, D))
        for source in range(world):
            part_dk, part_dv, n = slots[owner][source]
            assert n == expect[source], (owner, source)  # what the owner adds is what the source sent
            dk[:, :n] += part_dk
            dv[:, :n] += part_dv
        dks.append(dk), dvs.append(dv)
    assert oracle.max_abs(fd.zigzag_merge(outs), ref_out) < 1e-5
    assert oracle.max_abs(fd.zigzag_merge(lses, dim=2), ref_lse) < 1e-5
    for got, ref in ((dqs, ref_dq), (dks, ref_dk), (dvs, ref_dv)):
        assert oracle.max_abs(fd.zigzag_merge(got), ref) < 1e-4


@pytest.mark.parametrize("world", [1, 2, 3, 4, 8])
def test_paired_calls_add_up_to_full_attention(world):
    """``ring_calls``: the steps grouped into kernel calls, two first halves of blocks behind each
    other in one buffer where the causal schedule allows it.  Played through for all ranks with
    the oracle as the kernel: outputs merged through LSE over the calls and gradients split back
    to the blocks' owners must equal attention over the whole sequence, every step must appear in
    exactly one call, and a pair must be two first halves seen by all local queries."""
    from flash_attn_v100 import distributed as fd

    Z, H, D = 1, 2, 64
    rows = 32
    half = rows // 2
    N = rows * world
    q, k, v, dout = oracle.make_inputs(Z, N, H, D, seed=9)
    ref_out, ref_lse, ref_dq, ref_dk, ref_dv = oracle.attention_fwd_bwd(q, k, v, dout, 0.2, True)
    shard = lambda t, r: fd.zigzag_split(t, r, world)
    outs, dqs = [], []
    dks = [torch.zeros((Z, rows, H, D)) for _ in range(world)]
    dvs = [torch.zeros((Z, rows, H, D)) for _ in range(world)]
    pairs = 0
    for r in range(world):
        calls = fd.ring_calls(r, world, True, rows)
        steps = fd.ring_step_shapes(r, world, True, rows)
        assert sorted(t for c in calls for (t, _, _, _) in c.parts) == list(range(world))
        ql, dol = shard(q, r).float(), shard(dout, r).float()
        o_acc, lse_acc = torch.zeros((Z, rows, H, D)), torch.full((Z, H, rows), float("-inf"))
        buffers = []
        for c in calls:
            kb, vb = torch.zeros((Z, rows, H, D)), torch.zeros((Z, rows, H, D))
            for (t, src, src_rows, first_row) in c.parts:
                assert (src, c.q_rows if len(c.parts) == 1 else steps[t][1], src_rows) == \
                       (steps[t][0], steps[t][1], steps[t][2])
                n = src_rows.stop
                kb[:, first_row:first_row + n] = shard(k, src)[:, src_rows].float()
                vb[:, first_row:first_row + n] = shard(v, src)[:, src_rows].float()
            if len(c.parts) == 2:
                pairs += 1
                assert c.kv_stop == rows and c.q_rows == slice(0, rows) and not c.causal_block
                assert [p[2].stop for p in c.parts] == [half, half] and [p[3] for p in c.parts] == [0, half]
            buffers.append((kb[:, :c.kv_stop], vb[:, :c.kv_stop]))
            o_p, l_p = oracle.attention_forward(ql[:, c.q_rows], *buffers[-1], 0.2, c.causal_block)
            o, l = oracle.merge_partials(o_acc[:, c.q_rows], lse_acc[:, :, c.q_rows], o_p, l_p)
            o_acc[:, c.q_rows], lse_acc[:, :, c.q_rows] = o, l
        outs.append(o_acc)
        dq = torch.zeros((Z, rows, H, D))
        for c, (kb, vb) in zip(calls, buffers):
            g = oracle.attention_backward(ql[:, c.q_rows], kb, vb, o_acc[:, c.q_rows], lse_acc[:, :, c.q_rows],
                                          dol[:, c.q_rows], 0.2, c.causal_block)
            dq[:, c.q_rows] += g[0]
            for (t, src, src_rows, first_row) in c.parts:
                n = src_rows.stop
                dks[src][:, :n] += g[1][:, first_row:first_row + n]
                dvs[src][:, :n] += g[2][:, first_row:first_row + n]
        dqs.append(dq)
    assert pairs == sum(r // 2 for r in range(world))  # rank r has r blocks of earlier ranks
    assert oracle.max_abs(fd.zigzag_merge(outs), ref_out) < 1e-5
    for got, ref in ((dqs, ref_dq), (dks, ref_dk), (dvs, ref_dv)):
        assert oracle.max_abs(fd.zigzag_merge(got), ref) < 1e-4
    # without a causal mask every step needs a whole block: no pairs
    assert all(len(c.parts) == 1 for c in fd.ring_calls(world - 1, world, False, rows))


def _missing_peer_worker(rank, world, port, out_dir):
    """Rank 1 leaves between steps without ever joining the exchange; rank 0 must get an error on
    the host within the process group's (short) time-out, not hang."""
    import datetime
    import time

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from flash_attn_v100 import distributed as fd

    q, k, v, _ = oracle.make_inputs(1, 64, 1, 64, seed=1)
    ql, kl, vl = (fd.zigzag_split(t, rank, world) for t in (q, k, v))
    if rank == 1:
        return  # the peer that never shows up (no collective of its in flight)
    t0 = time.perf_counter()
    try:
        fd.ring_attention_forward(ql, kl, vl, 0.2, True, None, OracleBackend())
        outcome = "no error"
    except Exception as exc:  # noqa: BLE001 - any host-side error is the point
        outcome = f"error after {time.perf_counter() - t0:.1f} s: {type(exc).__name__}"
    with open(os.path.join(out_dir, "rank0.txt"), "w") as f:
        f.write(outcome)


def test_a_missing_peer_is_an_error_on_the_host_not_a_hang(tmp_path):
    """Failure detection without a GPU: the exchange with a rank that has gone away ends with an
    exception on the surviving rank once the process group's time-out (5 s here) has passed."""
    mp.spawn(_missing_peer_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    outcome = open(os.path.join(tmp_path, "rank0.txt")).read()
    assert outcome.startswith("error after"), outcome
    assert float(outcome.split()[2]) < 60.0, outcome
