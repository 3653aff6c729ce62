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
