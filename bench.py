"""Benchmark of the attention hot path (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

One "step" = one forward + one backward of the workload's batch.  The default workload is
BASELINE config 3, the shape the metric is quoted on: Z=8, H=32, N=2048, D=128, fp16, causal,
N(0,1) inputs from seed 0 (synthetic; the reference uses the same distribution, test.py:5-10).
With N > 1 GPUs (one process per GPU under torch.distributed.run) every rank runs its own
batch of that shape with no data-path collective: independent (batch, head) slices shard
without communication, so the scaling is "weak".

Prints ONE JSON line (rank 0):
  value        whole-job fwd+bwd TFLOP/s with inputs resident in HBM, algorithmic FLOPs
               (fwd 4*Z*H*N^2*D, halved when causal; bwd 2.5x), CUDA-event time, max over ranks
  e2e          the same metric through the public API flash_attn_func (+ autograd backward)
               with pinned HOST buffers (placed on the GPU's NUMA node where sysfs tells it):
               H2D of q, k, v, dout and D2H of out, dq, dk, dv inside the timed region
  roofline     the dominant kernel (fused dK/dV/dQ backward) against the measured dense 16-bit
               tensor peak from MEASURED_PEAKS.json (fallback 1590 TF/s), timed in place with CUDA
               events; `traffic` is DRAM bytes per launch from the committed ncu capture (null
               when the kernel source has changed since the capture)
  cpu_baseline the oracle (fp32 math path) timed on this box's host cores on a bounded sample
  kernels      per-kernel device times (medians): forward, preprocess (HBM-bound, GB/s),
               backward main, dQ convert
  regions      the timed region is repeated back to back; ms_per_step is the median region
  sharded      (default workload only) BASELINE's two sharded configs measured in the same run
               on the same ranks: config 4 (Z=64 split over the GPUs, no communication) with its
               speed-up over one GPU, and config 5 (ring attention over one 32768-token causal
               sequence) with its exposed communication; both with parity against the oracle

--impl reference times the reference's own math path (test.py:13-26 restated in fp32: the
oracle) on the host cores; the reference's CUDA kernel cannot run here (sm_70 only, needs an
un-vendored CUTLASS 3.x).
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.join(ROOT, "flash-attention-v100_b200")
for _p in (ROOT, PKG):
    if _p not in sys.path:
        sys.path.insert(0, _p)

WORKLOADS = {
    # name: (Z, H, N, D, causal, scale)
    "cfg3_causal": (8, 32, 2048, 128, True, 128 ** -0.5),
    "cfg3_noncausal": (8, 32, 2048, 128, False, 128 ** -0.5),
    "cfg3_ragged2016_causal": (8, 32, 2016, 128, True, 128 ** -0.5),
    "cfg2_causal": (4, 16, 1024, 64, True, 0.125),
    "cfg2_noncausal": (4, 16, 1024, 64, False, 0.125),
    "cfg4_per_gpu_z8": (8, 16, 512, 64, False, 0.125),
    "cfg4_full_z64": (64, 16, 512, 64, False, 0.125),
    "ref_test_shape": (2, 40, 2048, 128, True, 0.1),
    # head_dim 96 (runs on the 128-wide kernels)
    "cfg3_shape_d96_causal": (8, 32, 2048, 96, True, 96 ** -0.5),
    # BASELINE config 5: the whole sequence is sharded over the GPUs (zig-zag ring attention)
    "cfg5_ring_causal": (1, 32, 32768, 128, True, 128 ** -0.5),
}
DEFAULT_WORKLOAD = "cfg3_causal"
METRIC = "attention fwd+bwd TFLOPS (algorithmic), whole job"


def flops(Z, H, N, D, causal, backward):
    f = 4.0 * Z * H * N * N * D * (0.5 if causal else 1.0)
    return f * (2.5 if backward else 1.0)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(tflops=float(d["bf16_tflops"]), tflops_sustained=float(d["bf16_tflops_sustained"]),
                    hbm_gbs=float(d["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def cpu_baseline(workload, target_seconds=12.0, threads=None):
    """The oracle (reference math path in fp32) on the host cores, forward + backward, on a
    (batch=1, heads=h) sample of the workload sized for roughly `target_seconds`."""
    import torch

    from oracle import attention_oracle as oracle

    Z, H, N, D, causal, scale = WORKLOADS[workload]
    threads = threads or os.cpu_count() or 1
    torch.set_num_threads(threads)
    q, k, v, dout = oracle.make_inputs(1, N, 1, D, seed=0)
    oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)  # warm-up
    t0 = time.perf_counter()
    oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    per_head = max(time.perf_counter() - t0, 1e-6)
    heads = int(max(1, min(H, target_seconds / per_head)))
    q, k, v, dout = oracle.make_inputs(1, N, heads, D, seed=0)
    best = float("inf")
    for _ in range(2):
        t0 = time.perf_counter()
        oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
        best = min(best, time.perf_counter() - t0)
    fl = flops(1, heads, N, D, causal, False) + flops(1, heads, N, D, causal, True)
    return {"value": fl / best / 1e12, "unit": "TFLOPS", "cores": threads, "kind": "port",
            "sample": f"fwd+bwd of Z=1, H={heads} of {workload} (N={N}, D={D}, causal={causal}), "
                      f"best of 2, {best:.2f} s; algorithmic FLOPs"}


def run_reference(args):
    """Reference arm: the reference's math path on the host cores (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    Z, H, N, D, causal, scale = WORKLOADS[args.workload]
    import torch

    from oracle import attention_oracle as oracle

    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    # a bounded sample per step: as many heads of one batch element as fit ~3 s
    q, k, v, dout = oracle.make_inputs(1, N, 1, D, seed=0)
    oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    t0 = time.perf_counter()
    oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    per_head = max(time.perf_counter() - t0, 1e-6)
    heads = int(max(1, min(H, 3.0 / per_head)))
    q, k, v, dout = oracle.make_inputs(1, N, heads, D, seed=0)
    for _ in range(args.warmup):
        oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        oracle.attention_fwd_bwd(q, k, v, dout, scale, causal)
    dt = (time.perf_counter() - t0) / args.steps
    fl = flops(1, heads, N, D, causal, False) + flops(1, heads, N, D, causal, True)
    value = fl / dt / 1e12
    sample = (f"each step = fwd+bwd of Z=1, H={heads} of {args.workload} on {threads} host threads "
              f"(torch fp32 math path)")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "Z": Z, "H": H, "N": N, "D": D, "causal": causal,
                   "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def cpus_near_gpu(torch, dev):
    """The CPUs of the NUMA node the GPU hangs off (its PCI device's local_cpulist in sysfs),
    restricted to those this process may run on; None when that cannot be told."""
    try:
        props = torch.cuda.get_device_properties(dev)
        path = "/sys/bus/pci/devices/%04x:%02x:%02x.0/local_cpulist" % (
            props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(path) as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        return cpus or None
    except (AttributeError, OSError, ValueError, RuntimeError):
        return None


class near_gpu:
    """Context: the calling thread runs on the GPU's own NUMA node, so that pinned host buffers
    allocated inside are placed in the memory the GPU's PCIe root port reaches without crossing
    sockets.  The previous affinity is put back on exit.  Does nothing when the node is unknown."""

    def __init__(self, torch, dev):
        self.cpus = cpus_near_gpu(torch, dev)
        self.old = None

    def __enter__(self):
        if self.cpus:
            try:
                self.old = os.sched_getaffinity(0)
                os.sched_setaffinity(0, self.cpus)
            except OSError:
                self.old = None
        return self

    def __exit__(self, *exc):
        if self.old is not None:
            os.sched_setaffinity(0, self.old)
        return False


def time_events(fn, iters, torch):
    """Average device milliseconds of fn() over `iters` back-to-back calls (CUDA events on the
    current stream, synchronised on both sides)."""
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    start.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def median(xs):
    xs = sorted(xs)
    return xs[len(xs) // 2]


def timed_regions(fn, steps, regions, torch, dist, world, dev):
    """`regions` timed regions of exactly `steps` calls each, back to back, every one bracketed by
    a barrier + synchronize; per region the MAX over ranks.  Returns the list (ms per step)."""
    out = []
    for _ in range(regions):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        out.append(time_events(fn, steps, torch))
    t = torch.tensor(out, dtype=torch.float64, device=dev)
    if world > 1:
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return [float(x) for x in t.tolist()]


def region_stats(regs):
    return {"count": len(regs), "first_ms": regs[0], "min_ms": min(regs), "median_ms": median(regs),
            "max_ms": max(regs)}


def recorded_traffic(kernel_file, workload):
    """DRAM bytes per launch of the dominant kernel from the committed ncu summary, or None when
    the summary was captured from another version of the kernel source (it records the SHA-256 of
    the source file it was taken from) or for another workload."""
    import hashlib
    import re

    path = os.path.join(ROOT, "profiles", "bwd_kernel_cfg3_causal.md")
    if workload != "cfg3_causal" or not os.path.exists(path):
        return None
    text = open(path).read()
    m_sha = re.search(r"kernel_source_sha256:\s*([0-9a-f]{64})", text)
    m_bytes = re.search(r"dram_bytes_per_launch:\s*([0-9.eE+]+)", text)
    if not (m_sha and m_bytes):
        return None
    with open(kernel_file, "rb") as f:
        if hashlib.sha256(f.read()).hexdigest() != m_sha.group(1):
            return None
    return float(m_bytes.group(1))


# ------------------------------------------------------------------------------------------------
# sharded configs of BASELINE (4: batch split, 5: ring attention), measured in the same run
# ------------------------------------------------------------------------------------------------
def parity_figures(got, ref, torch, dist, world, dev):
    """max-abs O and relative-L2 of the gradients against the oracle, MAX over ranks."""
    from oracle import attention_oracle as oracle

    out, dq, dk, dv = got
    r_out, r_dq, r_dk, r_dv = ref
    vals = [oracle.max_abs(out.float(), r_out)] + [oracle.rel_l2(a.float(), b) for a, b in
                                                    ((dq, r_dq), (dk, r_dk), (dv, r_dv))]
    t = torch.tensor(vals, dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e_o, e_dq, e_dk, e_dv = (float(x) for x in t.tolist())
    return {"max_abs_O": e_o, "rel_l2_dq": e_dq, "rel_l2_dk": e_dk, "rel_l2_dv": e_dv,
            "within_tolerance": bool(e_o <= 2e-3 and max(e_dq, e_dk, e_dv) <= 1e-2),
            "checker": "blockwise fp32 oracle on the GPU (TF32 off), outside the timed region"}


def graph_of(step, torch):
    """The step captured in a CUDA graph (the short configs are launch-bound from Python), or None."""
    try:
        cap = torch.cuda.Stream()
        cap.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(cap):
            step()
            torch.cuda.synchronize()
            with torch.cuda.graph(graph, stream=cap):
                step()
        torch.cuda.current_stream().wait_stream(cap)
        torch.cuda.synchronize()
        graph.replay()
        torch.cuda.synchronize()
        return graph
    except Exception as exc:  # capture refused: time the plain launches, and say so
        print(f"CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        return None


def measure_cfg4(args, torch, dist, world, rank, dev):
    """BASELINE config 4: Z=64 split evenly over the GPUs, no communication (strong scaling).
    Rank 0 first times the whole batch alone (the 1-GPU reference of the speed-up), then every
    rank runs its slice; every rank's slice is compared with the oracle."""
    from flash_attn_v100 import cabi
    from oracle import attention_oracle_blockwise as blockwise

    Z, H, N, D, causal, scale = WORKLOADS["cfg4_full_z64"]
    steps, regions = max(args.steps, 20), 7

    def build(z_count, z_first):
        g = torch.Generator(device=dev).manual_seed(1000)
        full = [torch.randn((Z, N, H, D), generator=g, device=dev, dtype=torch.float32).half() for _ in range(4)]
        q, k, v, dout = (t[z_first:z_first + z_count].contiguous() for t in full)
        del full
        out = torch.empty_like(q)
        lse = torch.empty((z_count, H, N), dtype=torch.float32, device=dev)
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        ws = torch.empty(cabi.bwd_workspace_bytes(z_count, N, H, D), dtype=torch.uint8, device=dev)

        def step():
            cabi.fwd(q, k, v, scale, causal, out=out, lse=lse)
            cabi.bwd(q, k, v, out, dout, lse, scale, causal, dq=dq, dk=dk, dv=dv, workspace=ws)

        return step, (q, k, v, dout), (out, dq, dk, dv)

    ms_one = None
    if world > 1:
        if rank == 0:
            step1, _, _ = build(Z, 0)
            for _ in range(3):
                step1()
            g1 = graph_of(step1, torch)
            fn1 = g1.replay if g1 is not None else step1
            regs1 = [time_events(fn1, steps, torch) for _ in range(regions)]
            ms_one = median(regs1)
            del step1, g1, fn1
        dist.barrier()
    per = Z // world
    step, ins, outs = build(per, rank * per)
    for _ in range(3):
        step()
    graph = graph_of(step, torch)
    fn = graph.replay if graph is not None else step
    regs = timed_regions(fn, steps, regions, torch, dist, world, dev)
    ms = median(regs)
    ref = blockwise.attention_fwd_bwd_blockwise(*ins, scale, causal)
    parity = parity_figures(outs, (ref[0], ref[2], ref[3], ref[4]), torch, dist, world, dev)
    fl = flops(Z, H, N, D, causal, False) + flops(Z, H, N, D, causal, True)
    if world == 1:
        ms_one = ms
    res = {"workload": "cfg4_full_z64", "scaling": "strong", "Z_total": Z, "Z_per_gpu": per, "H": H, "N": N,
           "D": D, "causal": causal, "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms,
           "regions": region_stats(regs), "steps": steps,
           "launch": "CUDA graph replay of one step" if graph is not None else "four launches per step",
           "parallelism": f"batch split x{world}, no collective", "parity": parity}
    if rank == 0 and ms_one is not None:
        res["ms_per_step_1gpu_same_run"] = ms_one
        res["speedup_vs_n1"] = ms_one / ms
    return res


def measure_ring(args, torch, dist, world, rank, dev, steps=None):
    """BASELINE config 5: one long causal sequence sharded over all ranks (zig-zag), K/V blocks
    rotating between the GPUs, partial results merged through LSE (strong scaling: the total work
    is fixed).  Also: the same schedule with the exchanges left out (what the kernels alone take,
    from which the exposed communication per hop follows), and parity on sampled heads."""
    from flash_attn_v100 import distributed as fd
    from oracle import attention_oracle_blockwise as blockwise

    Z, H, N, D, causal, scale = WORKLOADS["cfg5_ring_causal"]
    steps = steps or max(3, min(args.steps, 5))
    c = N // (2 * world)
    g = torch.Generator(device=dev).manual_seed(rank)
    ql, kl, vl, dol = (torch.randn((Z, 2 * c, H, D), generator=g, device=dev, dtype=torch.float32).half()
                       for _ in range(4))
    from flash_attn_v100 import peer_ring

    be = fd.CudaBackend()
    # the copy-engine transport needs CUDA IPC between the ranks; where that is not to be had the
    # NCCL send/recv ring is measured instead (the set-up fails or succeeds on all ranks together)
    try:
        ring = peer_ring.PeerRing((Z, 2 * c, H, D), torch.float16, dev)
        product = "peer"
    except RuntimeError as exc:
        print(f"copy-engine ring unavailable ({exc}); measuring the NCCL send/recv ring", file=sys.stderr)
        ring, product = None, "nccl"
    res_holder = {}

    def make_step(comm, transport):
        def step():
            if transport == "peer":
                out, lse = ring.forward(ql, kl, vl, scale, causal, exchange=comm)
                grads = ring.backward(ql, kl, vl, out, lse, dol, scale, causal, exchange=comm)
            else:
                out, lse = fd.ring_attention_forward(ql, kl, vl, scale, causal, None, be, comm=comm)
                grads = fd.ring_attention_backward(ql, kl, vl, out, lse, dol, scale, causal, None, be, comm=comm)
            res_holder["last"] = (out,) + tuple(grads)
        return step

    # the product path: blocks pulled / gradients pushed by the copy engines.  With many ranks a
    # hop is short (0.15 ms of forward kernels at 8 GPUs) and the Python loop that issues it would
    # be what is timed: the whole step (kernels, copies, flag kernels, events on three streams) is
    # captured in a CUDA graph once and replayed; the flags carry an iteration number that lives
    # on the device, so a replay is a new iteration.
    step = make_step(True, product)
    for _ in range(3):
        step()
    graph = graph_of(step, torch) if (args.graph != "off" and product == "peer") else None
    graphed = graph is not None
    t = torch.tensor([1 if graphed else 0], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MIN)  # replay only if every rank captured
    graphed = bool(t.item())
    timed = graph.replay if graphed else step
    regs = timed_regions(timed, steps, 3, torch, dist, world, dev)
    ms = median(regs)
    got = res_holder["last"]
    if ring is not None:
        # a bounded wait for a peer's flag that ran out leaves a code in the status word of the
        # rank it happened on; all ranks agree on the outcome before any of them gives up
        st = ring.status.clone()
        if world > 1:
            dist.all_reduce(st, op=dist.ReduceOp.MAX)
        if int(st.item()) != 0:
            ring.close()
            return {"workload": "cfg5_ring_causal",
                    "error": f"a bounded wait for a peer's flag gave up (status {int(st.item()):#x}); no number reported"}
    ms_nocomm = ms_nccl = None
    if world > 1:
        quiet = make_step(False, product)
        quiet()
        qgraph = graph_of(quiet, torch) if graphed else None
        t = torch.tensor([1 if qgraph is not None else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        quiet_timed = qgraph.replay if bool(t.item()) else quiet
        ms_nocomm = median(timed_regions(quiet_timed, steps, 3, torch, dist, world, dev))
        # for comparison: the same schedule with NCCL send/recv passing the blocks round
        if product == "peer":
            nccl = make_step(True, "nccl")
            nccl()
            ms_nccl = median(timed_regions(nccl, steps, 2, torch, dist, world, dev))
        else:
            ms_nccl = ms

    # parity on two sampled heads: gather them from every rank, rebuild the whole sequence, run
    # the oracle on it, compare this rank's shard
    heads = [0, H - 1]
    def gather_full(local):
        part = local[:, :, heads].contiguous()
        if world == 1:
            parts = [part]
        else:
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
        return fd.zigzag_merge(parts)
    qf, kf, vf, dof = (gather_full(t) for t in (ql, kl, vl, dol))
    ref = blockwise.attention_fwd_bwd_blockwise(qf, kf, vf, dof, scale, causal, row_chunk=2048, head_chunk=1)
    mine = lambda t: fd.zigzag_split(t, rank, world)
    parity = parity_figures(tuple(t[:, :, heads] for t in got),
                            (mine(ref[0]), mine(ref[2]), mine(ref[3]), mine(ref[4])), torch, dist, world, dev)
    parity["sampled_heads"] = heads
    del qf, kf, vf, dof, ref

    fl = flops(Z, H, N, D, causal, False) + flops(Z, H, N, D, causal, True)
    kv_hop = 2 * Z * 2 * c * H * D * 2
    res = {"workload": "cfg5_ring_causal", "scaling": "strong", "Z": Z, "H": H, "N": N, "D": D,
           "causal": causal, "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "ms_per_step": ms,
           "regions": region_stats(regs), "steps": steps,
           "per_gpu_tflops": fl / (ms * 1e-3) / 1e12 / world,
           "parallelism": f"zig-zag ring attention x{world} (" + (
               "K/V pulled from their owners and dK/dV pushed to theirs by the copy engines over NVLink; "
               "flags in peer memory" if product == "peer" else "NCCL send/recv") + ")",
           "launch": "CUDA graph replay of one ring step" if graphed else "launches issued from Python",
           "rows_per_gpu": 2 * c, "kv_bytes_per_hop": kv_hop, "dkdv_bytes_per_hop": 2 * kv_hop,
           "parity": parity}
    if ms_nocomm is not None:
        hops = (world - 1) + world  # forward K/V hops + backward hops of a step
        res["ms_per_step_without_exchange"] = ms_nocomm
        res["exposed_comm_ms_per_hop"] = max(0.0, ms - ms_nocomm) / hops
        res["exposed_comm_frac_of_step"] = max(0.0, ms - ms_nocomm) / ms
        res["ms_per_step_nccl_send_recv"] = ms_nccl  # launches issued from Python, not replayed
    if ring is not None:
        ring.close()
    return res


def run_ring(args):
    """`--workload cfg5_ring_causal`: the ring measurement as the line's headline."""
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    res = measure_ring(args, torch, dist, world, rank, dev, steps=args.steps)
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        peaks = measured_peaks()
        line = {"metric": METRIC, "value": res["value"], "unit": "TFLOPS", "n_gpus": world,
                "steps": res["steps"], "warmup": 3, "ms_per_step": res["ms_per_step"],
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
                "config": {k: res[k] for k in ("workload", "Z", "H", "N", "D", "causal", "parallelism",
                                               "rows_per_gpu", "kv_bytes_per_hop", "dkdv_bytes_per_hop")},
                "ring": res, "per_gpu_frac_of_sustained_peak": res["per_gpu_tflops"] / peaks["tflops_sustained"],
                "gpu_launches": None, "clocks": clocks}
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    want_sharded = args.workload == DEFAULT_WORKLOAD and not args.no_sharded
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    elif want_sharded:
        # the ring measurement runs through torch.distributed also on one rank (no peer)
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)

    from flash_attn_v100 import cabi, flash_attn_func
    from oracle import attention_oracle as oracle

    Z, H, N, D, causal, scale = WORKLOADS[args.workload]
    # BASELINE config 4 fixes the total batch (Z=64) and splits it over the GPUs: strong scaling
    strong = args.workload == "cfg4_full_z64" and world > 1
    if strong:
        Z //= world
    # every rank draws its own batch (seed = rank): no communication
    host_inputs = oracle.make_inputs(Z, N, H, D, seed=rank)
    with near_gpu(torch, dev) as placement:
        hq, hk, hv, hdo = (t.pin_memory() for t in host_inputs)
    q, k, v, dout = (t.to(dev) for t in (hq, hk, hv, hdo))
    out = torch.empty_like(q)
    lse = torch.empty((Z, H, N), dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = torch.empty(cabi.bwd_workspace_bytes(Z, N, H, D), dtype=torch.uint8, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def fwd():
        cabi.fwd(q, k, v, scale, causal, out=out, lse=lse, status=status)

    def bwd(flags=0):
        cabi.bwd(q, k, v, out, dout, lse, scale, causal, dq=dq, dk=dk, dv=dv, workspace=ws,
                 flags=flags, status=status)

    def step():
        fwd()
        bwd()

    # ---- resident-in-HBM timing of whole steps
    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    # A step is four kernel launches.  Where the kernels are short (cfg-2, cfg-4 split over many
    # GPUs) the launches, issued from Python, would be what is timed: there the step is captured
    # once in a CUDA graph and the graph is replayed (same kernels, same arguments, same stream
    # order).
    timed_step, graphed = step, False
    if args.graph != "off":
        probe_ms = time_events(step, 5, torch)
        if args.graph == "on" or probe_ms < 0.6:
            graph = graph_of(step, torch)
            if graph is not None:
                timed_step, graphed = graph.replay, True
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    # `regions` timed regions of exactly `steps` steps each, back to back.  The first starts on a
    # GPU that has been idle for the set-up and runs at boost clocks; from the second or third on
    # both attention kernels sit at the 1000 W power cap and a step takes 10-20 % longer.  The
    # line reports the MEDIAN region (the steady state) and keeps the first beside it.
    regs = timed_regions(timed_step, args.steps, args.regions, torch, dist, world, dev)
    ms_step = median(regs)
    assert int(status.item()) == 0, f"kernel status word {int(status.item()):#x}"

    # ---- per-kernel timing, in place: the four kernels of a step in their normal order, an
    # event between each two (timed alone in a loop of its own a kernel runs at another SM clock
    # under the power cap, and the parts would not add up to the step); medians over the loop
    iters = args.kernel_iters
    both = cabi.FMHA_BWD_KEEP_WORKSPACE | cabi.FMHA_BWD_SKIP_DQ_CONVERT

    def instrumented(n_iters):
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(n_iters)]
        torch.cuda.synchronize()
        for e in ev:
            e[0].record()
            fwd()
            e[1].record()
            bwd(cabi.FMHA_BWD_PREPROCESS_ONLY)
            e[2].record()
            bwd(both)
            e[3].record()
            cabi.bwd_convert_dq(ws, dq, scale)
            e[4].record()
        torch.cuda.synchronize()
        return [median([e[i].elapsed_time(e[i + 1]) for e in ev]) for i in range(4)] + [
            median([e[0].elapsed_time(e[4]) for e in ev])]

    ms_fwd, ms_pre, ms_bwd_main, ms_cvt, ms_parts = instrumented(iters)
    ms_bwd = ms_pre + ms_bwd_main + ms_cvt
    # the same plain steps once more, right behind the instrumented loop: what the events between
    # the kernels cost, and how far the GPU has drifted since the timed regions
    regs_after = timed_regions(timed_step, args.steps, 3, torch, dist, world, dev)
    clocks_kernels = sampler.stop() if sampler else None
    # and the same instrumented loop, short, after the GPU has been left idle for a second: the
    # kernels at boost clocks, before the power cap bites (what a burst peak is measured like)
    time.sleep(1.0)
    idle = instrumented(8)

    # ---- end to end through the public API with host buffers.  Every step copies its own inputs
    # from pinned host memory and its own results back; the copies of neighbouring steps overlap
    # with each other and with the kernels (PCIe is full duplex): inputs of step i+1 go up while
    # step i computes and the results of step i-1 come down, through two sets of device buffers.
    with near_gpu(torch, dev):
        h_out, h_dq, h_dk, h_dv = (torch.empty_like(hq).pin_memory() for _ in range(4))
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
    sets = [{"in": [torch.empty_like(q) for _ in range(4)], "res": None,
             "up": torch.cuda.Event(), "done": torch.cuda.Event(), "down": torch.cuda.Event()}
            for _ in range(2)]

    def e2e_run(n_steps):
        main = torch.cuda.current_stream()
        for i in range(n_steps):
            b = sets[i % 2]
            with torch.cuda.stream(s_up):
                s_up.wait_event(b["done"])   # the buffers' previous user (step i-2) has computed
                for dst, src in zip(b["in"], (hq, hk, hv, hdo)):
                    dst.copy_(src, non_blocking=True)
                b["up"].record(s_up)
            main.wait_event(b["up"])
            main.wait_event(b["down"])       # the previous results of this set have gone down
            q2, k2, v2 = (t.detach().requires_grad_() for t in b["in"][:3])
            o2 = flash_attn_func(q2, k2, v2, scale, causal)
            o2.backward(b["in"][3])
            b["res"] = (o2.detach(), q2.grad, k2.grad, v2.grad)
            b["done"].record(main)
            with torch.cuda.stream(s_down):
                s_down.wait_event(b["done"])
                for dst, src in zip((h_out, h_dq, h_dk, h_dv), b["res"]):
                    dst.copy_(src, non_blocking=True)
                b["down"].record(s_down)
        main.wait_stream(s_down)
        main.wait_stream(s_up)

    e2e_run(2)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    # enough steps that filling and draining the three-stage pipeline (one step without an
    # upload beside it, one without a download) is a few per cent of the region
    e2e_iters = max(30, args.steps)
    ms_e2e = time_events(lambda: e2e_run(e2e_iters), 1, torch) / e2e_iters
    t = torch.tensor([ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())

    # ---- the sharded configs BASELINE names (4: batch split, 5: ring attention), same run
    sharded = None
    if want_sharded:
        sharded = {}
        for name, fn in (("cfg4_batch_split", measure_cfg4), ("cfg5_ring", measure_ring)):
            try:
                sharded[name] = fn(args, torch, dist, world, rank, dev)
            except Exception as exc:  # keep the headline: report what failed instead of dying
                sharded[name] = {"error": f"{type(exc).__name__}: {exc}"[:400]}
                if world > 1:
                    raise

    if rank == 0:
        peaks = measured_peaks()
        f_fwd = flops(Z, H, N, D, causal, False)
        f_bwd = flops(Z, H, N, D, causal, True)
        elem = Z * N * H * D
        tensor_bytes = elem * 2
        achieved = f_bwd / (ms_bwd_main * 1e-3) / 1e12
        pre_bytes = 2 * tensor_bytes + elem * 4 + 3 * Z * H * N * 4  # read O, dO; zero dq_acc; lse, lse2, delta
        mhz = (clocks_kernels or {}).get("sm_mhz")
        kernel_file = os.path.join(PKG, "csrc", "bwd_kernel.cuh")
        line = {
            "metric": METRIC,
            "value": world * (f_fwd + f_bwd) / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "Z_per_gpu": Z, "H": H, "N": N, "D": D, "causal": causal,
                       "scale": scale, "parallelism": f"batch-sharded x{world}, no collective",
                       "launch": "CUDA graph replay of one step" if graphed else "four launches per step",
                       "timing": f"median of {args.regions} back-to-back regions of {args.steps} steps (steady state "
                                 "under the power cap); regions.first_ms is the first region, from an idle GPU",
                       "l2": "working set 1.3 GB per step (q,k,v,dout,out,dq,dk,dv + fp32 dq accumulator) > 126 MB L2"},
            "regions": region_stats(regs),
            "kernels": {
                "iterations": iters, "statistic": "median, timed in place inside the step",
                "fwd_ms": ms_fwd, "fwd_tflops": f_fwd / ms_fwd / 1e9,
                "fwd_frac_of_measured_peak": f_fwd / ms_fwd / 1e9 / peaks["tflops"],
                "fwd_frac_of_sustained_peak": f_fwd / ms_fwd / 1e9 / peaks["tflops_sustained"],
                "bwd_ms": ms_bwd, "bwd_tflops": f_bwd / ms_bwd / 1e9,
                "bwd_frac_of_measured_peak": f_bwd / ms_bwd / 1e9 / peaks["tflops"],
                "bwd_frac_of_sustained_peak": f_bwd / ms_bwd / 1e9 / peaks["tflops_sustained"],
                "bwd_main_ms": ms_bwd_main, "bwd_preprocess_ms": ms_pre,
                "bwd_preprocess_gbs": pre_bytes / ms_pre / 1e6,
                "bwd_preprocess_frac_of_measured_hbm": pre_bytes / ms_pre / 1e6 / peaks["hbm_gbs"],
                "bwd_convert_ms": ms_cvt,
                "sum_of_parts_ms": ms_parts, "sum_of_parts_over_step": ms_parts / ms_step,
                "plain_step_ms_right_after": median(regs_after),
                "sum_of_parts_over_step_right_after": ms_parts / median(regs_after),
                "ms_x_sm_mhz": None if not mhz else {"fwd": ms_fwd * mhz, "bwd_preprocess": ms_pre * mhz,
                                                    "bwd_main": ms_bwd_main * mhz, "bwd_convert": ms_cvt * mhz,
                                                    "sm_mhz": mhz},
                "frac_of_nominal_2250": {"fwd": f_fwd / ms_fwd / 1e9 / 2250.0, "bwd": f_bwd / ms_bwd / 1e9 / 2250.0},
                "from_idle": {
                    "what": "the same loop, 8 iterations, after one second of idle (boost clocks, no power cap yet)",
                    "fwd_ms": idle[0], "bwd_preprocess_ms": idle[1], "bwd_main_ms": idle[2],
                    "bwd_convert_ms": idle[3], "bwd_ms": idle[1] + idle[2] + idle[3],
                    "fwd_frac_of_measured_peak": f_fwd / idle[0] / 1e9 / peaks["tflops"],
                    "bwd_frac_of_measured_peak": f_bwd / (idle[1] + idle[2] + idle[3]) / 1e9 / peaks["tflops"],
                    "bwd_main_frac_of_measured_peak": f_bwd / idle[2] / 1e9 / peaks["tflops"]},
            },
            # the fused backward kernel is timed inside a long back-to-back loop, under the power
            # cap: the like-for-like denominator is the SUSTAINED measured peak; the burst figure
            # (and the kernel's own time from an idle GPU) are given beside it
            "roofline": {"kernel": f"fmha_bwd_kernel<{128 if D > 64 else 64}> (fused dK/dV/dQ)", "bound": "tensor",
                         "achieved": achieved, "peak": peaks["tflops_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops_sustained"],
                         "peak_source": peaks["source"] + " (sustained: the kernel is timed inside a long loop)",
                         "frac_of_burst_peak": achieved / peaks["tflops"], "burst_peak": peaks["tflops"],
                         "from_idle": {"achieved": f_bwd / idle[2] / 1e9,
                                       "frac_of_burst_peak": f_bwd / idle[2] / 1e9 / peaks["tflops"]},
                         "algorithmic_flops_per_launch": f_bwd,
                         "traffic": recorded_traffic(kernel_file, args.workload)},
            "e2e": {"value": world * (f_fwd + f_bwd) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOPS",
                    "ms_per_step": ms_e2e, "h2d_bytes_per_step": 4 * tensor_bytes,
                    "d2h_bytes_per_step": 4 * tensor_bytes, "api": "flash_attn_v100.flash_attn_func + backward",
                    "overlap": "copies of neighbouring steps overlap (two buffer sets, three streams)",
                    "pcie_gbs_each_way": 4 * tensor_bytes / (ms_e2e * 1e-3) / 1e9,
                    "host_buffers": ("pinned, allocated from the GPU's NUMA node (%d CPUs)" % len(placement.cpus))
                    if placement.cpus else "pinned, placement left to the OS"},
            "gpu_launches": 4 * args.steps,  # fwd, bwd preprocess, bwd main, bwd convert per step of a region
            "clocks": clocks_kernels,
        }
        if sharded is not None:
            line["sharded"] = sharded
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true",
                    help="skip the batch-split and ring-attention measurements that follow the headline")
    ap.add_argument("--kernel-iters", type=int, default=50,
                    help="iterations of the instrumented loop that times the kernels of a step one by one")
    ap.add_argument("--regions", type=int, default=15,
                    help="timed regions of --steps steps each, back to back; the median is reported")
    ap.add_argument("--graph", default="auto", choices=["auto", "on", "off"],
                    help="replay the step from a CUDA graph (auto: when a step is shorter than 0.6 ms)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload.startswith("cfg5_ring"):
        run_ring(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
