"""Ring attention over NVLink without a collective library in the data path.

The reference is single-GPU (kernel/fused_mha_api.cpp:61); ``distributed.py`` adds sequence
sharding with K/V blocks passed from rank to rank by NCCL send/recv.  On an NVSwitch node every
GPU reaches every other at full bandwidth, so nothing has to be *passed round*: this module
shards the same way (zig-zag, see ``distributed.py``) but

* every rank PULLS the K/V block it needs next straight from the rank that owns it, with the
  copy engines (``cudaMemcpyAsync`` from an address mapped through CUDA IPC), two steps ahead,
  on a stream of its own, while the attention kernel of the current step runs on all SMs;
* in the backward pass every rank PUSHES its fp32 dK/dV contribution for a visiting block to
  a slot at the block's owner, again with the copy engines while the next step computes; the
  owner adds up the slots once at the end (``fmha_sum_partials``).  No accumulator travels and
  nothing waits for a gradient hop;
* readiness of a buffer is a flag in the consumer's memory set by the producer
  (``fmha_peer_signal``) and awaited on the consumer's stream (``fmha_peer_wait``, bounded: a
  wait that runs out sets the status word and the attention kernels behind it return at once).
  Flags carry an iteration number kept on the device; there is no host synchronisation and no
  allocation in a step.

The attention kernels only ever read this GPU's own memory: a pulled block lands in a local
buffer first.  torch.distributed is used once, to exchange the IPC handles.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

# rows of the flag matrix (one column per peer)
_READY_F, _ACK_F, _READY_B, _ACK_B, _GRAD_READY, _GRAD_FREE, _N_FLAGS = 0, 1, 2, 3, 4, 5, 6
# receive buffers per direction: a block is fetched _DEPTH - 1 calls before the call that uses it
# (FMHA_RING_DEPTH, 2..6, overrides for tuning experiments)
_DEPTH = min(6, max(2, int(os.environ.get("FMHA_RING_DEPTH", "3"))))


class _KVSide:
    """Export buffer, the receive buffers and the iteration words of one direction (fwd or bwd)."""

    def __init__(self, shape, dtype, device, ready_row, ack_row):
        self.export = torch.empty((2,) + shape, dtype=dtype, device=device)
        self.recv = [torch.empty((2,) + shape, dtype=dtype, device=device) for _ in range(_DEPTH)]
        self.it = torch.zeros(2, dtype=torch.int32, device=device)  # [this iteration, the previous]
        self.ready_row, self.ack_row = ready_row, ack_row


class PeerRing:
    """Buffers, peer mappings and streams for ring attention on local shards of one shape.

    Create it once per (shard shape, dtype) on every rank of ``group`` (collective: the IPC
    handles are exchanged here), then call ``forward`` / ``backward`` any number of times, all
    ranks in the same order."""

    def __init__(self, shard_shape, dtype, device, group=None, timeout_ms: int = 10000, sm_margin: int = 2,
                 pair_steps: Optional[bool] = None):
        from flash_attn_v100 import cabi, distributed as fd

        self.cabi = cabi
        self.fd = fd
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 16:
            raise ValueError("PeerRing supports up to 16 ranks on one node")
        self.shape = tuple(shard_shape)
        self.dtype, self.device = dtype, torch.device(device)
        Z, rows, H, D = self.shape
        if rows % 2:
            raise ValueError("a zig-zag shard has an even number of rows")
        self.timeout_ms = int(timeout_ms)
        # two steps over first halves of blocks in one kernel call (distributed.ring_calls)
        # Off by default: at 8 GPUs the kernels of a step get 3-4 % faster (a paired call fills
        # the SMs in 6.9 rounds of tiles instead of 3.46) but the step does not, its time then
        # being set by the hand-shakes, and it varies more from step to step (same box, three
        # regions of five steps: 4.85-5.28 ms without, 4.86-5.43 ms with).  FMHA_RING_PAIR=1
        # switches it on for experiments.
        if pair_steps is None:
            pair_steps = os.environ.get("FMHA_RING_PAIR", "0") != "0"
        self.pair_steps = bool(pair_steps)
        self.backend = fd.CudaBackend(sm_margin=sm_margin if self.world > 1 else 0)
        with torch.cuda.device(self.device):
            self.fwd_side = _KVSide(self.shape, dtype, self.device, _READY_F, _ACK_F)
            self.bwd_side = _KVSide(self.shape, dtype, self.device, _READY_B, _ACK_B)
            self.flags = torch.zeros((_N_FLAGS, self.world), dtype=torch.int32, device=self.device)
            self.grad_it = torch.zeros(2, dtype=torch.int32, device=self.device)
            self.slots = torch.empty((self.world, 2) + self.shape, dtype=torch.float32, device=self.device)
            self.part = [torch.empty((2,) + self.shape, dtype=torch.float32, device=self.device) for _ in range(2)]
            self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
            self.backend.status = self.status
            # Steps in which only the second half of the queries sees a block run on all rows'
            # tensors with q_row_begin (a multiple of the 128-row tile) and share the one
            # workspace; shards too short for that fall back to a workspace of their own.
            self.row_begin_ok = (rows // 2) % 128 == 0
            self.bwd_state = self.backend.new_bwd_state(torch.empty(self.shape, dtype=dtype, device="meta"),
                                                        device=self.device, half=not self.row_begin_ok)
            self.pull_stream = torch.cuda.Stream(device=self.device, priority=-1)
            self.push_stream = torch.cuda.Stream(device=self.device, priority=-1)
            torch.cuda.synchronize(self.device)
        # ---- exchange the addresses (CUDA IPC): my export buffers, slots and flags for every peer.
        # Every rank takes part in every collective of this set-up whether or not its own local
        # steps worked, and all ranks agree on the outcome, so that a failure on one rank (IPC not
        # permitted, no peer access) is an exception on all of them and never a hang.
        def all_ok(ok: bool) -> bool:
            t = torch.tensor([1 if ok else 0], dtype=torch.int32, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
            return bool(t.item())

        self._opened = {}
        mine, error = None, None
        try:
            mine = {name: cabi.ipc_export(t) for name, t in (
                ("kv_f", self.fwd_side.export), ("kv_b", self.bwd_side.export), ("slots", self.slots),
                ("flags", self.flags))}
        except Exception as exc:  # noqa: BLE001 - reported on every rank below
            error = exc
        exported = all_ok(error is None)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, mine, group=group)
        own = {"kv_f": self.fwd_side.export.data_ptr(), "kv_b": self.bwd_side.export.data_ptr(),
               "slots": self.slots.data_ptr(), "flags": self.flags.data_ptr()}
        self.peer = []
        if exported:
            try:
                with torch.cuda.device(self.device):
                    for p in range(self.world):
                        if p == self.rank:
                            self.peer.append(own)
                            continue
                        entry = {}
                        for name, (handle, offset) in everyone[p].items():
                            key = (p, handle)
                            if key not in self._opened:
                                self._opened[key] = cabi.ipc_open(handle, 0)
                            entry[name] = self._opened[key] + offset
                        self.peer.append(entry)
            except Exception as exc:  # noqa: BLE001
                error = exc
        if not all_ok(exported and error is None):
            raise RuntimeError("PeerRing: CUDA IPC set-up failed on at least one rank"
                               + (f" (here: {error})" if error is not None else ""))
        dist.barrier(group=group)

    # ---- addresses
    def _flag(self, owner: int, row: int, col: int) -> int:
        return self.peer[owner]["flags"] + 4 * (row * self.world + col)

    def _others(self) -> List[int]:
        return [p for p in range(self.world) if p != self.rank]

    def close(self):
        """Unmap the peers' memory (collective: nobody may still be copying)."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for addr in self._opened.values():
                self.cabi.ipc_close(addr, 0)
        self._opened = {}

    def check(self):
        """Host check of the status word (synchronises): raises if a peer wait ran out."""
        code = int(self.status.item())
        if code != 0:
            raise RuntimeError(f"ring attention: a bounded wait gave up (status {code:#x})")

    # ---- K/V side shared by forward and backward
    def _publish(self, side: _KVSide, k, v, cs, exchange: bool):
        """This rank's K/V into the export buffer, once the peers have finished reading the
        previous iteration's; then tell them.  Returns the address of the iteration word."""
        c = self.cabi
        cur, prev = side.it.data_ptr(), side.it.data_ptr() + 4
        if self.world == 1:
            return cur
        if exchange:
            others = self._others()
            c.counter_bump(side.it, cs)
            c.peer_wait([self._flag(self.rank, side.ack_row, p) for p in others], prev, self.status,
                        self.timeout_ms, cs)
        side.export[0].copy_(k)
        side.export[1].copy_(v)
        if exchange:
            c.peer_signal([self._flag(p, side.ready_row, self.rank) for p in others], cur, cs)
        return cur

    def _pull(self, side: _KVSide, kv_name: str, ci: int, call, cur: int, ev_free, ev_ready, exchange: bool):
        """Fetch the block(s) of call ``ci`` (>= 1) into receive buffer ci % _DEPTH on the pull
        stream: a whole block, or the first halves of one or two blocks behind each other."""
        c = self.cabi
        Z, rows, H, D = self.shape
        buf = side.recv[ci % _DEPTH]
        esize = buf.element_size()
        entry = rows * H * D * esize  # one tensor of one batch entry
        with torch.cuda.stream(self.pull_stream):
            if ci >= _DEPTH + 1:
                # the kernels of call ci - _DEPTH are done with the buffer
                self.pull_stream.wait_event(ev_free[ci % _DEPTH])
            for (_t, src, kv_rows, first_row) in call.parts:
                if exchange:
                    c.peer_wait([self._flag(self.rank, side.ready_row, src)], cur, self.status,
                                self.timeout_ms, self.pull_stream)
                    src_addr = self.peer[src][kv_name]
                else:
                    src_addr = side.export.data_ptr()  # measurements: same bytes, local source
                if kv_rows.stop < rows:
                    # only the first half of the block is needed; it goes to rows first_row.. here
                    c.peer_copy_2d(buf.data_ptr() + first_row * H * D * esize, entry, src_addr, entry,
                                   entry // 2, 2 * Z, self.pull_stream)
                else:
                    c.peer_copy(buf.data_ptr(), src_addr, 2 * Z * entry, self.pull_stream)
                if exchange:
                    c.peer_signal([self._flag(src, side.ack_row, self.rank)], cur, self.pull_stream)
            ev_ready[ci % _DEPTH].record(self.pull_stream)

    # ---- forward
    def forward(self, q, k, v, scale: float, causal: bool, exchange: bool = True
                ) -> Tuple[torch.Tensor, torch.Tensor]:
        """This rank's (out, lse) shard; q, k, v are the local zig-zag shards."""
        be, world, rank = self.backend, self.world, self.rank
        cs = torch.cuda.current_stream(self.device)
        side = self.fwd_side
        self.pull_stream.wait_stream(cs)  # earlier work on the receive buffers is behind us
        cur = self._publish(side, k, v, cs, exchange)
        ev_ready = [torch.cuda.Event() for _ in range(_DEPTH)]
        ev_free = [torch.cuda.Event() for _ in range(_DEPTH)]
        Z, rows, H, D = self.shape
        calls = self.fd.ring_calls(rank, world, causal, rows, self.pair_steps)
        if world > 1:
            self.pull_stream.wait_stream(cs)
            for ci in range(1, min(_DEPTH, len(calls))):
                self._pull(side, "kv_f", ci, calls[ci], cur, ev_free, ev_ready, exchange)
        # every call leaves its partial (O, LSE) in buffers of its own; ONE pass merges them all
        # at the end (fmha_merge_parts) instead of a read-modify-write pass over fp32
        # accumulators after every step
        parts_o, parts_l, offsets = [], [], []
        for ci, call in enumerate(calls):
            if ci == 0:
                kb, vb = k, v
            else:
                cs.wait_event(ev_ready[ci % _DEPTH])
                kb, vb = side.recv[ci % _DEPTH][0], side.recv[ci % _DEPTH][1]
            if ci >= 1 and ci + _DEPTH - 1 < len(calls):
                self._pull(side, "kv_f", ci + _DEPTH - 1, calls[ci + _DEPTH - 1], cur, ev_free, ev_ready, exchange)
            q_rows = call.q_rows
            n_q = q_rows.stop - q_rows.start
            o_p = torch.empty((Z, n_q, H, D), dtype=q.dtype, device=self.device)
            l_p = torch.empty((Z, H, n_q), dtype=torch.float32, device=self.device)
            self.cabi.fwd(q[:, q_rows], kb[:, :call.kv_stop], vb[:, :call.kv_stop], scale, call.causal_block,
                          out=o_p, lse=l_p, status=self.status,
                          sm_margin=be.sm_margin if ci + 1 < len(calls) else 0)
            parts_o.append(o_p)
            parts_l.append(l_p)
            offsets.append(q_rows.start)
            if ci >= 1:
                ev_free[ci % _DEPTH].record(cs)
        if world == 1:
            out, lse = parts_o[0], parts_l[0]
        else:
            out = torch.empty_like(q)
            lse = torch.empty((Z, H, rows), dtype=torch.float32, device=self.device)
            self.cabi.merge_parts(parts_o, parts_l, offsets, out, lse, cs)
        cs.wait_stream(self.pull_stream)  # nothing of this call is left on the side stream
        return out, lse

    # ---- backward
    def backward(self, q, k, v, out, lse, dout, scale: float, causal: bool, exchange: bool = True):
        """This rank's (dq, dk, dv) shards."""
        c, be, world, rank = self.cabi, self.backend, self.world, self.rank
        cs = torch.cuda.current_stream(self.device)
        side = self.bwd_side
        Z, rows, H, D = self.shape
        half = rows // 2
        others = self._others() if exchange else []
        self.pull_stream.wait_stream(cs)
        self.push_stream.wait_stream(cs)
        cur = self._publish(side, k, v, cs, exchange)
        # my slots may be written for this iteration: everything of my previous backward is
        # behind this point of the stream
        gcur = self.grad_it.data_ptr()
        if others:
            c.counter_bump(self.grad_it, cs)
            c.peer_signal([self._flag(p, _GRAD_FREE, rank) for p in others], gcur, cs)
        state = self.bwd_state
        state["full_used"] = state["half_used"] = False
        ev_ready = [torch.cuda.Event() for _ in range(_DEPTH)]
        ev_free = [torch.cuda.Event() for _ in range(_DEPTH)]
        ev_part = [torch.cuda.Event(), torch.cuda.Event()]
        ev_pushed = [torch.cuda.Event(), torch.cuda.Event()]
        begin_ok = self.row_begin_ok
        lse_half = None if begin_ok else lse[:, :, half:].contiguous()
        calls = self.fd.ring_calls(rank, world, causal, rows, self.pair_steps)
        if world > 1:
            self.pull_stream.wait_stream(cs)
            for ci in range(1, min(_DEPTH, len(calls))):
                self._pull(side, "kv_b", ci, calls[ci], cur, ev_free, ev_ready, exchange)
        slot_bytes = 2 * Z * rows * H * D * 4
        entry = rows * H * D * 4
        mine = self.slots[rank]  # my own contribution goes straight into my slot

        def second_half_step(kb, vb, kv_rows, causal_block, target, shift=0):
            """dQ of the second half of the query rows, dK / dV of key rows ``kv_rows``."""
            if begin_ok:
                be.bwd_step(state, "full", q, kb[:, kv_rows], vb[:, kv_rows], out, dout, lse, scale,
                            causal_block, target[0][:, kv_rows], target[1][:, kv_rows], overwrite=True,
                            causal_shift=shift, q_row_begin=half)
            else:
                be.bwd_step(state, "half", q[:, half:], kb[:, kv_rows], vb[:, kv_rows], out[:, half:],
                            dout[:, half:], lse_half, scale, causal_block, target[0][:, kv_rows],
                            target[1][:, kv_rows], overwrite=True, causal_shift=shift + (half if causal_block else 0))

        # The local block is done in two parts, a short one first and the long one last, so that
        # the first pull of a visiting block and the last push of a partial result both have a
        # kernel running beside them: (second half of the queries) x (second half of the keys)
        # now, all queries x (first half of the keys) after the last visiting block.  Each part
        # overwrites its own key rows of my slot.  With a causal mask the local block is causal
        # over the local row numbers (the second chunk of a zig-zag shard is later in the
        # sequence than the first); without one the two parts are simply two key halves.
        split_local = world > 1
        lo, hi = slice(0, half), slice(half, rows)
        if not split_local:
            be.bwd_step(state, "full", q, k, v, out, dout, lse, scale, causal, mine[0], mine[1], overwrite=True)
        elif causal:
            # key j (local number) is visible to query i iff j <= i: with the keys given from
            # row `half` on that is j' <= i - half
            second_half_step(k, v, hi, True, mine, shift=-half)
        else:
            be.bwd_step(state, "full", q, k[:, hi], v[:, hi], out, dout, lse, scale, False,
                        mine[0][:, hi], mine[1][:, hi], overwrite=True)
        for ci, call in enumerate(calls):
            if ci == 0:
                continue
            cs.wait_event(ev_ready[ci % _DEPTH])
            kb, vb = side.recv[ci % _DEPTH][0], side.recv[ci % _DEPTH][1]
            target = self.part[ci % 2]
            if ci >= 3:
                cs.wait_event(ev_pushed[ci % 2])  # the pushes of call ci - 2 have read the buffer
            if ci + _DEPTH - 1 < len(calls):
                self._pull(side, "kv_b", ci + _DEPTH - 1, calls[ci + _DEPTH - 1], cur, ev_free, ev_ready, exchange)
            kv_rows = slice(0, call.kv_stop)
            if call.q_rows.start == 0:
                be.bwd_step(state, "full", q, kb[:, kv_rows], vb[:, kv_rows], out, dout, lse, scale,
                            call.causal_block, target[0][:, kv_rows], target[1][:, kv_rows], overwrite=True)
            else:
                second_half_step(kb, vb, kv_rows, call.causal_block, target)
            ev_free[ci % _DEPTH].record(cs)
            ev_part[ci % 2].record(cs)
            if exchange:
                with torch.cuda.stream(self.push_stream):
                    ps = self.push_stream
                    ps.wait_event(ev_part[ci % 2])
                    for (_t, src, src_rows, first_row) in call.parts:
                        c.peer_wait([self._flag(rank, _GRAD_FREE, src)], gcur, self.status, self.timeout_ms, ps)
                        dst = self.peer[src]["slots"] + rank * slot_bytes
                        if src_rows.stop < rows:
                            # the first half of src's block: rows first_row.. of my buffer
                            c.peer_copy_2d(dst, entry, target.data_ptr() + first_row * H * D * 4, entry,
                                           entry // 2, 2 * Z, ps)
                        else:
                            c.peer_copy(dst, target.data_ptr(), slot_bytes, ps)
                        c.peer_signal([self._flag(src, _GRAD_READY, rank)], gcur, ps)
                    ev_pushed[ci % 2].record(ps)
        if split_local:
            be.bwd_step(state, "full", q, k[:, lo], v[:, lo], out, dout, lse, scale, causal,
                        mine[0][:, lo], mine[1][:, lo], overwrite=True)
        # every other rank's contribution to my block has arrived; add them up
        c.peer_wait([self._flag(rank, _GRAD_READY, p) for p in others], gcur, self.status, self.timeout_ms, cs)
        sources = list(range(world)) if exchange else [rank]
        all_rows = self.fd.ring_grad_rows(rank, world, causal, rows)
        rows_per = [all_rows[p] for p in sources]
        dk, dv = torch.empty_like(k), torch.empty_like(v)
        base = self.slots.data_ptr()
        c.sum_partials([base + p * slot_bytes for p in sources], rows_per, dk, cs)
        c.sum_partials([base + p * slot_bytes + slot_bytes // 2 for p in sources], rows_per, dv, cs)
        cs.wait_stream(self.push_stream)
        cs.wait_stream(self.pull_stream)
        dq = be.bwd_finish(state, q, k, v, out, dout, lse, scale)
        return dq, dk, dv


class PeerRingAttnFunc(torch.autograd.Function):
    """``PeerRingAttnFunc.apply(ring, q, k, v, softmax_scale, causal)`` on zig-zag shards."""

    @staticmethod
    def forward(ctx, ring: PeerRing, q, k, v, softmax_scale, causal):
        if softmax_scale is None:
            softmax_scale = q.shape[-1] ** (-0.5)
        out, lse = ring.forward(q, k, v, softmax_scale, causal)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.ring, ctx.softmax_scale, ctx.causal = ring, softmax_scale, causal
        return out

    @staticmethod
    def backward(ctx, dout):
        q, k, v, out, lse = ctx.saved_tensors
        dq, dk, dv = ctx.ring.backward(q, k, v, out, lse, dout.contiguous(), ctx.softmax_scale, ctx.causal)
        return None, dq, dk, dv, None, None


def peer_ring_flash_attn_func(ring: PeerRing, q, k, v, softmax_scale=None, causal=False):
    """Sequence-parallel counterpart of ``flash_attn_func`` over ``ring`` (see ``PeerRing``)."""
    return PeerRingAttnFunc.apply(ring, q, k, v, softmax_scale, causal)
