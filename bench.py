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
               with pinned HOST buffers: H2D of q, k, v, dout and D2H of out, dq, dk, dv inside
               the timed region
  roofline     the dominant kernel (fused dK/dV/dQ backward) against the measured dense 16-bit
               tensor peak from MEASURED_PEAKS.json (fallback 1590 TF/s), timed alone with CUDA
               events; `traffic` is DRAM bytes per launch from the committed ncu capture
  cpu_baseline the oracle (fp32 math path) timed on this box's host cores on a bounded sample
  kernels      per-kernel device times: forward, preprocess (HBM-bound, GB/s), backward main,
               dQ convert

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
    # BASELINE config 5: the whole sequence is sharded over the GPUs (zig-zag ring attention)
    "cfg5_ring_causal": (1, 32, 32768, 128, True, 128 ** -0.5),
}
DEFAULT_WORKLOAD = "cfg3_causal"
METRIC = "attention fwd+bwd TFLOPS (algorithmic), whole job"
# DRAM bytes per launch of the backward main kernel at cfg3_causal, from the ncu capture
# summarised in profiles/ (dram__bytes_read.sum + dram__bytes_write.sum)
NCU_TRAFFIC_BYTES = {"cfg3_causal": 1.302e9}


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


def run_ring(args):
    """BASELINE config 5: one long causal sequence sharded over all ranks (zig-zag), K/V blocks and
    fp32 dK/dV rotating over NCCL send/recv, merged through LSE.  Strong scaling: the total work
    is fixed, value = whole-sequence algorithmic FLOPs / max-over-ranks device time."""
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
    from flash_attn_v100 import distributed as fd

    Z, H, N, D, causal, scale = WORKLOADS[args.workload]
    c = N // (2 * world)
    g = torch.Generator(device=dev).manual_seed(rank)
    ql, kl, vl, dol = (torch.randn((Z, 2 * c, H, D), generator=g, device=dev, dtype=torch.float32).half()
                       for _ in range(4))
    be = fd.CudaBackend()

    def step():
        out, lse = fd.ring_attention_forward(ql, kl, vl, scale, causal, None, be)
        fd.ring_attention_backward(ql, kl, vl, out, lse, dol, scale, causal, None, be)

    for _ in range(max(args.warmup, 3)):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    ms = time_events(step, args.steps, torch)
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    clocks = sampler.stop() if sampler else None
    if rank == 0:
        fl = flops(Z, H, N, D, causal, False) + flops(Z, H, N, D, causal, True)
        peaks = measured_peaks()
        kv_hop = 2 * Z * 2 * c * H * D * 2
        print(json.dumps({
            "metric": METRIC, "value": fl / (ms * 1e-3) / 1e12, "unit": "TFLOPS", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "Z": Z, "H": H, "N": N, "D": D, "causal": causal,
                       "parallelism": f"zig-zag ring attention x{world} (NCCL send/recv)",
                       "rows_per_gpu": 2 * c, "kv_bytes_per_hop": kv_hop,
                       "dkdv_bytes_per_hop": 2 * kv_hop},
            "per_gpu_tflops": fl / (ms * 1e-3) / 1e12 / world,
            "per_gpu_frac_of_measured_peak": fl / (ms * 1e-3) / 1e12 / world / peaks["tflops_sustained"],
            "gpu_launches": None, "clocks": clocks}), flush=True)
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
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from flash_attn_v100 import cabi, flash_attn_func
    from oracle import attention_oracle as oracle

    Z, H, N, D, causal, scale = WORKLOADS[args.workload]
    # BASELINE config 4 fixes the total batch (Z=64) and splits it over the GPUs: strong scaling
    strong = args.workload == "cfg4_full_z64" and world > 1
    if strong:
        Z //= world
    # every rank draws its own batch (seed = rank): no communication
    hq, hk, hv, hdo = (t.pin_memory() for t in oracle.make_inputs(Z, N, H, D, seed=rank))
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
                timed_step, graphed = graph.replay, True
            except Exception as exc:  # capture refused: time the plain launches, and say so
                print(f"CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
                torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    if world > 1:
        dist.barrier()
    if sampler:
        sampler.start()
    torch.cuda.synchronize()
    ms_step = time_events(timed_step, args.steps, torch)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([ms_step], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item())
    assert int(status.item()) == 0, f"kernel status word {int(status.item()):#x}"

    # ---- per-kernel timing, in place: the four kernels of a step in their normal order, an
    # event between each two (timed alone in a loop of its own a kernel runs at another SM clock
    # under the power cap, and the parts would not add up to the step)
    iters = 10
    both = cabi.FMHA_BWD_KEEP_WORKSPACE | cabi.FMHA_BWD_SKIP_DQ_CONVERT
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(5)] for _ in range(iters)]
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
    ms_fwd, ms_pre, ms_bwd_main, ms_cvt = (
        sum(e[i].elapsed_time(e[i + 1]) for e in ev) / iters for i in range(4))
    ms_bwd = ms_pre + ms_bwd_main + ms_cvt

    # ---- end to end through the public API with host buffers.  Every step copies its own inputs
    # from pinned host memory and its own results back; the copies of neighbouring steps overlap
    # with each other and with the kernels (PCIe is full duplex): inputs of step i+1 go up while
    # step i computes and the results of step i-1 come down, through two sets of device buffers.
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
    e2e_iters = max(4, min(args.steps, 10))
    ms_e2e = time_events(lambda: e2e_run(e2e_iters), 1, torch) / e2e_iters
    t = torch.tensor([ms_e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_e2e = float(t.item())
    clocks = sampler.stop() if sampler else None

    if rank == 0:
        peaks = measured_peaks()
        f_fwd = flops(Z, H, N, D, causal, False)
        f_bwd = flops(Z, H, N, D, causal, True)
        elem = Z * N * H * D
        tensor_bytes = elem * 2
        achieved = f_bwd / (ms_bwd_main * 1e-3) / 1e12
        pre_bytes = 2 * tensor_bytes + elem * 4 + 3 * Z * H * N * 4  # read O, dO; zero dq_acc; lse, lse2, delta
        line = {
            "metric": METRIC,
            "value": world * (f_fwd + f_bwd) / (ms_step * 1e-3) / 1e12,
            "unit": "TFLOPS", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if strong else "weak", "vs_baseline": None,
            "dtype": "f16 (fp32 accumulate)", "data": "synthetic",
            "config": {"workload": args.workload, "Z_per_gpu": Z, "H": H, "N": N, "D": D, "causal": causal,
                       "scale": scale, "parallelism": f"batch-sharded x{world}, no collective",
                       "launch": "CUDA graph replay of one step" if graphed else "four launches per step",
                       "l2": "working set 1.3 GB per step (q,k,v,dout,out,dq,dk,dv + fp32 dq accumulator) > 126 MB L2"},
            "kernels": {
                "fwd_ms": ms_fwd, "fwd_tflops": f_fwd / ms_fwd / 1e9,
                "fwd_frac_of_measured_peak": f_fwd / ms_fwd / 1e9 / peaks["tflops"],
                "bwd_ms": ms_bwd, "bwd_tflops": f_bwd / ms_bwd / 1e9,
                "bwd_frac_of_measured_peak": f_bwd / ms_bwd / 1e9 / peaks["tflops"],
                "bwd_main_ms": ms_bwd_main, "bwd_preprocess_ms": ms_pre,
                "bwd_preprocess_gbs": pre_bytes / ms_pre / 1e6,
                "bwd_preprocess_frac_of_measured_hbm": pre_bytes / ms_pre / 1e6 / peaks["hbm_gbs"],
                "bwd_convert_ms": ms_cvt,
                "frac_of_nominal_2250": {"fwd": f_fwd / ms_fwd / 1e9 / 2250.0, "bwd": f_bwd / ms_bwd / 1e9 / 2250.0},
            },
            "roofline": {"kernel": f"fmha_bwd_kernel<{D}> (fused dK/dV/dQ)", "bound": "tensor",
                         "achieved": achieved, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["tflops"], "peak_source": peaks["source"] + " (burst)",
                         "frac_of_sustained_peak": achieved / peaks["tflops_sustained"],
                         "traffic": NCU_TRAFFIC_BYTES.get(args.workload)},
            "e2e": {"value": world * (f_fwd + f_bwd) / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOPS",
                    "ms_per_step": ms_e2e, "h2d_bytes_per_step": 4 * tensor_bytes,
                    "d2h_bytes_per_step": 4 * tensor_bytes, "api": "flash_attn_v100.flash_attn_func + backward",
                    "overlap": "copies of neighbouring steps overlap (two buffer sets, three streams)"},
            "gpu_launches": 4 * args.steps,  # fwd, bwd preprocess, bwd main, bwd convert per step
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.workload)
        print(json.dumps(line), flush=True)
    if world > 1:
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
