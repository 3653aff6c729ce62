"""Multi-GPU layer of the B200 attention library (one process per GPU, torch.distributed).

The reference is single-GPU (kernel/fused_mha_api.cpp:61 guards one device and there is no
collective anywhere in it); this module adds the two ways its hot path shards:

1. ``shard_batch`` - independent (batch, head) slices: every rank runs ``flash_attn_func`` on
   its own slice of the batch, no communication (the reference's kernels already treat each
   (batch, head) independently, kernel/fused_mha_kernel.cu:53-54).

2. ``ring_attention_forward`` / ``ring_attention_backward`` / ``RingAttnFunc`` - sequence
   sharding for long contexts.  The sequence is cut into 2G chunks and rank r holds chunks r
   and 2G-1-r ("zig-zag"), which balances causal work.  K/V blocks travel round the ring with
   point-to-point send/recv (NCCL over NVLink on GPUs) while the local kernels run; partial
   results are merged through their log-sum-exp.  In the backward the K/V block travels
   together with its fp32 dK/dV accumulator and arrives home after G hops.
   With zig-zag sharding every step is one of three dense shapes, none of which needs a mask
   other than the ordinary causal one:
       step 0                 local Q x local K/V, causal
       block from a rank < r  all local Q x first half of the block, not causal
       block from a rank > r  second half of local Q x the whole block, not causal
   Received blocks land in this GPU's own memory and are then read by ordinary TMA loads.

The compute backend is the C ABI (``flash_attn_v100.cabi``); it is injected as an object so
that the communication schedule can be exercised on CPU ranks (gloo) by tests that supply
their own backend.  The default backend needs the CUDA library and a GPU: there is no CPU
path in the product.
"""
from __future__ import annotations

from typing import NamedTuple, List, Optional, Tuple

import torch
import torch.distributed as dist


# ----------------------------------------------------------------------------------------------
# sharding helpers
# ----------------------------------------------------------------------------------------------
def shard_batch(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank's contiguous slice of the batch dimension (dim 0); the batch must divide evenly."""
    if x.shape[0] % world != 0:
        raise ValueError(f"batch {x.shape[0]} is not divisible by world size {world}")
    per = x.shape[0] // world
    return x[rank * per:(rank + 1) * per]


def zigzag_split(x: torch.Tensor, rank: int, world: int, dim: int = 1) -> torch.Tensor:
    """Chunks ``rank`` and ``2*world-1-rank`` of ``x`` cut into 2*world equal chunks along
    ``dim``, concatenated in that (ascending) order."""
    n = x.shape[dim]
    if n % (2 * world) != 0:
        raise ValueError(f"sequence length {n} is not divisible by 2 * world size ({2 * world})")
    chunks = x.chunk(2 * world, dim=dim)
    return torch.cat([chunks[rank], chunks[2 * world - 1 - rank]], dim=dim).contiguous()


def zigzag_merge(parts: List[torch.Tensor], dim: int = 1) -> torch.Tensor:
    """Inverse of ``zigzag_split`` given every rank's shard (rank order)."""
    world = len(parts)
    chunks: List[Optional[torch.Tensor]] = [None] * (2 * world)
    for r, p in enumerate(parts):
        a, b = p.chunk(2, dim=dim)
        chunks[r], chunks[2 * world - 1 - r] = a, b
    return torch.cat(chunks, dim=dim)


def ring_step_shapes(rank: int, world: int, causal: bool, rows: int):
    """The dense block rank ``rank`` computes at every step of zig-zag ring attention over local
    shards of ``rows`` rows: a list of ``(src, q_rows, kv_rows, causal_block)`` where ``src`` is
    the rank that owns the K/V block, ``q_rows`` the slice of the local query rows that takes
    part, ``kv_rows`` the slice of the block's rows that is needed, and ``causal_block`` whether
    the block carries the ordinary causal mask (only the local one does)."""
    half = rows // 2
    full = slice(0, rows)
    steps = []
    for t in range(world):
        src = (rank - t) % world
        if t == 0:
            steps.append((src, full, full, causal))
        elif not causal:
            steps.append((src, full, full, False))
        elif src < rank:
            steps.append((src, full, slice(0, half), False))  # all local Q x first half of the block
        else:
            steps.append((src, slice(half, rows), full, False))  # second half of local Q x whole block
    return steps


class RingCall(NamedTuple):
    """One kernel call of the copy-engine ring: the blocks it works on and the dense shape."""
    parts: tuple        # of (step t, src rank, rows of the src's block needed, first row in the local buffer)
    q_rows: slice       # local query rows that take part
    kv_stop: int        # rows [0, kv_stop) of the local buffer hold the keys / values of the call
    causal_block: bool


def ring_calls(rank: int, world: int, causal: bool, rows: int, pair: bool = True):
    """``ring_step_shapes`` grouped into kernel calls.  Two consecutive steps that need only the
    first half of their block (under a causal mask: blocks of ranks before this one) share one
    call: the two half blocks sit behind each other in one buffer, which is then as long as a
    whole block, and all local queries see all of it.  A step's grid of 128-row tiles then fills
    the SMs in twice as many rounds, i.e. more evenly, and there are fewer launches and partial
    results.  Every other step is a call of its own."""
    half = rows // 2
    steps = ring_step_shapes(rank, world, causal, rows)
    calls, t = [], 0
    while t < len(steps):
        src, q_rows, kv_rows, causal_block = steps[t]
        halved = t >= 1 and kv_rows.stop == half and q_rows.start == 0
        if pair and halved and t + 1 < len(steps) and steps[t + 1][2].stop == half and steps[t + 1][1].start == 0:
            calls.append(RingCall(((t, src, kv_rows, 0), (t + 1, steps[t + 1][0], steps[t + 1][2], half)),
                                  q_rows, rows, False))
            t += 2
        else:
            calls.append(RingCall(((t, src, kv_rows, 0),), q_rows, kv_rows.stop, causal_block))
            t += 1
    return calls


def ring_grad_rows(owner: int, world: int, causal: bool, rows: int):
    """For the K/V block owned by ``owner``: how many of its rows (always a prefix) every source
    rank contributes dK/dV for.  Ranks behind the owner in the sequence only ever see the first
    half of the block."""
    return [rows if (p == owner or not causal or p < owner) else rows // 2 for p in range(world)]


# ----------------------------------------------------------------------------------------------
# compute backend
# ----------------------------------------------------------------------------------------------
class CudaBackend:
    """The product backend: the sm_100a kernels through the C ABI."""

    def __init__(self, sm_margin: int = 0):
        from flash_attn_v100 import cabi  # raises if the library is not built

        self.cabi = cabi
        # SMs the persistent forward kernel leaves to the NCCL kernels of the exchange posted
        # just before it.  Off by default: measured on 2 B200 with hops of 0.15 ms of attention,
        # 32 free SMs shorten the ring forward by 10 % and 8 or 16 by nothing, while on long hops
        # every SM given away is attention throughput lost.
        self.sm_margin = sm_margin
        # optional device status word handed to every attention kernel (a bounded wait that ran
        # out anywhere makes the kernels behind it return at once)
        self.status = None

    def comm_name(self, world: int) -> str:
        return "NCCL send/recv" if world > 1 else "one rank, no exchange"

    def fwd(self, q, k, v, scale, causal, overlap: bool = False):
        return self.cabi.fwd(q, k, v, scale, causal, sm_margin=self.sm_margin if overlap else 0,
                             status=self.status)

    def new_accumulators(self, q):
        Z, N, H, D = q.shape
        # rows start with LSE = -inf, for which the merge does not read o_acc: no zero fill
        o_acc = torch.empty((Z, N, H, D), dtype=torch.float32, device=q.device)
        lse_acc = torch.full((Z, H, N), float("-inf"), dtype=torch.float32, device=q.device)
        return o_acc, lse_acc

    def merge(self, o_acc, lse_acc, o_part, lse_part, rows: slice, o_out=None):
        """Merge a partial result for query rows ``rows`` into the accumulators, in place; with
        ``o_out`` the merged rows are also written in the tensors' 16-bit type."""
        self.cabi.merge(o_acc, lse_acc, o_part, lse_part, o_out=o_out, row_offset=rows.start or 0)

    def finish(self, o_acc, lse_acc, dtype):
        return o_acc.to(dtype), lse_acc

    def new_bwd_state(self, q, device=None, half: bool = True):
        """Workspaces of a ring backward: one for steps over all query rows and (``half``) one
        for steps over the second half of them given as a tensor of its own."""
        Z, N, H, D = q.shape
        device = q.device if device is None else device
        nbytes = self.cabi.bwd_workspace_bytes
        return {
            "full": torch.empty(nbytes(Z, N, H, D), dtype=torch.uint8, device=device),
            "half": torch.empty(nbytes(Z, N // 2, H, D) if half else 0, dtype=torch.uint8, device=device),
            "full_used": False, "half_used": False,
        }

    def bwd_step(self, state, which, q, k, v, o, dout, lse, scale, causal, dk_acc, dv_acc,
                 overwrite: bool = False, causal_shift: int = 0, q_row_begin: int = 0):
        """Accumulate this block's dQ into the workspace ``which`` ('full' or 'half' query rows)
        and its dK/dV into the fp32 buffers (``overwrite``: in place of what they hold).
        ``q_row_begin``: the query rows before it take no part (q, o, dout, lse are those of all
        rows, the workspace is 'full')."""
        c = self.cabi
        flags = c.FMHA_BWD_SKIP_DQ_CONVERT | (c.FMHA_BWD_KEEP_WORKSPACE if state[which + "_used"] else 0)
        if overwrite:
            flags |= c.FMHA_BWD_ACCUM_OVERWRITE
        c.bwd(q, k, v, o, dout, lse, scale, causal, causal_shift, dq=None, dk_accum=dk_acc, dv_accum=dv_acc,
              workspace=state[which], flags=flags, status=self.status, q_row_begin=q_row_begin)
        state[which + "_used"] = True

    def bwd_finish(self, state, q, k, v, o, dout, lse, scale):
        """Convert the accumulated dQ to fp16 (full rows, plus the second-half rows' extra)."""
        c = self.cabi
        Z, N, H, D = q.shape
        half = N // 2
        # the conversion of the 'full' workspace writes every row of dq
        dq = torch.empty_like(q) if state["full_used"] else torch.zeros_like(q)
        if state["full_used"]:
            self._convert(state["full"], dq, scale, q.shape)
        if state["half_used"]:
            dq_half = torch.empty_like(q[:, half:])
            self._convert(state["half"], dq_half, scale, (Z, half, H, D))
            dq[:, half:] += dq_half
        return dq

    def _convert(self, ws, dq, scale, shape):
        self.cabi.bwd_convert_dq(ws, dq, scale)


# ----------------------------------------------------------------------------------------------
# ring plumbing
# ----------------------------------------------------------------------------------------------
def _exchange(tensors: List[torch.Tensor], group, rank: int, world: int, comm: bool = True):
    """Post sends of ``tensors`` to rank+1 and receives of same-shaped buffers from rank-1;
    returns (requests, received buffers).  The caller waits before touching the buffers.
    ``comm=False`` (measurements only) leaves the exchange out: the "received" buffers are the
    tensors themselves, so that the same kernels run on the same shapes with nothing sent."""
    if not comm:
        return [], list(tensors)
    dst = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    src = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    bufs = [torch.empty_like(t) for t in tensors]
    ops = []
    for t, b in zip(tensors, bufs):
        ops.append(dist.P2POp(dist.isend, t, dst, group))
        ops.append(dist.P2POp(dist.irecv, b, src, group))
    return dist.batch_isend_irecv(ops), bufs


def _wait(reqs):
    for r in reqs:
        r.wait()


def ring_attention_forward(q, k, v, scale: float, causal: bool, group=None, backend=None,
                           comm: bool = True) -> Tuple[torch.Tensor, torch.Tensor]:
    """Forward over a zig-zag-sharded sequence: returns this rank's (out, lse) shard.

    q, k, v: (Z, 2c, H, D) local shards (``zigzag_split``).  K/V blocks rotate rank -> rank+1;
    the transfer for the next step is posted before this step's kernel is launched."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    half = q.shape[1] // 2
    o_acc, lse_acc = backend.new_accumulators(q)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    for step in range(world):
        reqs = None
        if step + 1 < world:
            reqs, (k_nxt, v_nxt) = _exchange([k_cur, v_cur], group, rank, world, comm)
        src = (rank - step) % world
        ov = reqs is not None  # an exchange is in flight beside this step's kernel
        if step == 0:
            o_p, l_p = backend.fwd(q, k_cur, v_cur, scale, causal, ov)
            backend.merge(o_acc, lse_acc, o_p, l_p, slice(0, None))
        elif not causal:
            o_p, l_p = backend.fwd(q, k_cur, v_cur, scale, False, ov)
            backend.merge(o_acc, lse_acc, o_p, l_p, slice(0, None))
        elif src < rank:
            o_p, l_p = backend.fwd(q, k_cur[:, :half], v_cur[:, :half], scale, False, ov)
            backend.merge(o_acc, lse_acc, o_p, l_p, slice(0, None))
        else:
            o_p, l_p = backend.fwd(q[:, half:], k_cur, v_cur, scale, False, ov)
            backend.merge(o_acc, lse_acc, o_p, l_p, slice(half, None))
        if reqs is not None:
            _wait(reqs)
            k_cur, v_cur = k_nxt, v_nxt
    return backend.finish(o_acc, lse_acc, q.dtype)


def ring_attention_backward(q, k, v, out, lse, dout, scale: float, causal: bool, group=None,
                            backend=None, comm: bool = True):
    """Backward over the same sharding: returns this rank's (dq, dk, dv) shards.

    The K/V block and its fp32 (dK, dV) accumulator travel together; after ``world`` hops the
    accumulator is back at the rank that owns the block."""
    backend = backend or CudaBackend()
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    half = q.shape[1] // 2
    state = backend.new_bwd_state(q)
    k_cur, v_cur = k.contiguous(), v.contiguous()
    dk_cur = torch.zeros(k.shape, dtype=torch.float32, device=k.device)
    dv_cur = torch.zeros(v.shape, dtype=torch.float32, device=v.device)
    lse_half = lse[:, :, half:].contiguous()
    for step in range(world):
        # the next block's K/V can travel while this step computes; dK/dV follow afterwards
        reqs_kv = None
        if step + 1 < world:
            reqs_kv, (k_nxt, v_nxt) = _exchange([k_cur, v_cur], group, rank, world, comm)
        src = (rank - step) % world
        if step == 0:
            backend.bwd_step(state, "full", q, k_cur, v_cur, out, dout, lse, scale, causal, dk_cur, dv_cur)
        elif not causal:
            backend.bwd_step(state, "full", q, k_cur, v_cur, out, dout, lse, scale, False, dk_cur, dv_cur)
        elif src < rank:
            backend.bwd_step(state, "full", q, k_cur[:, :half], v_cur[:, :half], out, dout, lse, scale,
                             False, dk_cur[:, :half], dv_cur[:, :half])
        else:
            backend.bwd_step(state, "half", q[:, half:], k_cur, v_cur, out[:, half:], dout[:, half:],
                             lse_half, scale, False, dk_cur, dv_cur)
        # hand the accumulators on (also after the last step: that hop brings them home)
        reqs_g, (dk_nxt, dv_nxt) = _exchange([dk_cur, dv_cur], group, rank, world, comm)
        if reqs_kv is not None:
            _wait(reqs_kv)
            k_cur, v_cur = k_nxt, v_nxt
        _wait(reqs_g)
        dk_cur, dv_cur = dk_nxt, dv_nxt
    dq = backend.bwd_finish(state, q, k, v, out, dout, lse, scale)
    return dq, dk_cur.to(k.dtype), dv_cur.to(v.dtype)


class RingAttnFunc(torch.autograd.Function):
    """Autograd wrapper: ``RingAttnFunc.apply(q, k, v, softmax_scale, causal, group)`` on
    zig-zag shards, same calling shape as ``flash_attn_func``."""

    @staticmethod
    def forward(ctx, q, k, v, softmax_scale, causal, group):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, lse = ring_attention_forward(q, k, v, softmax_scale, causal, group)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.softmax_scale, ctx.causal, ctx.group = softmax_scale, causal, group
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ring_attention_backward(q, k, v, out, lse, dout.contiguous(), ctx.softmax_scale,
                                             ctx.causal, ctx.group)
        return dq, dk, dv, None, None, None


def ring_flash_attn_func(q, k, v, softmax_scale=None, causal=False, group=None):
    """Sequence-parallel counterpart of ``flash_attn_func`` for zig-zag shards."""
    return RingAttnFunc.apply(q, k, v, softmax_scale, causal, group)
