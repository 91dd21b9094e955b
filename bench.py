#!/usr/bin/env python
"""Benchmark of the INT8 flash-attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--scaling strong|weak]
                    [--impl ours|reference] [--no-e2e] [--no-cpu] [--no-extras]

One "step" is one forward pass over one batch of synthetic int8 Q,K,V (seeded; the reference
project ships no dataset).  The default workload is C3 (B=8,H=32,S=2048,D=128), the shape the
throughput target is quoted on.

With N > 1 (launched under torchrun, one rank per GPU) ONE workload is partitioned: rank r takes
the heads [r*BH/N, (r+1)*BH/N) of the flattened batch*head axis, holds only that slice of Q,K,V,O
plus the whole mask, and calls FMHAInferI8Slice.  The path shards with no exchange step, so there
is no collective on the data path; NCCL carries the barrier, the max-over-ranks of the device time
and, after the timed region, the gather that checks the slices bit for bit against a run of the
whole problem on rank 0.  `--scaling weak` (every rank runs the whole workload) is also measured
and printed in the same line as `weak_replicas`.

Prints ONE JSON line on rank 0:
  value          effective INT8 TOPS = 4*B*H*S^2*D / t (t = slowest rank), inputs resident in HBM,
                 CUDA-event timed
  e2e            the same metric through the host-buffer entry point: pinned HOST buffers in and
                 out, host<->device copies inside the timed region
  roofline       dominant kernel against the dense-INT8 tensor peak (2 x the measured dense bf16
                 cuBLAS rate of this pool's B200s; kind::i8 runs at twice the bf16 rate)
  parity         distance of the timed output from the quantised CPU oracle on a row sample, and
                 the reference's own acceptance figure against the fp32 golden
  ref_gpu_baseline   the reference project's own CUDA kernel, rebuilt unchanged for sm_100a, on
                 the same inputs (context: its output is checked against the oracle beside it)
  other_configs  the other benchmark shapes, timed the same way (1 GPU only)
  sustained      the same step back to back for at least a second, with the sampled SM clock
  cpu_baseline   the reference project's CPU path (oracle/_ref) on a bounded sample of heads

--impl reference times the reference project's own CPU implementation of the path instead.
"""
import argparse
import ctypes
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "effective INT8 TOPS (4*B*H*S^2*D / t) per job"
L2_BYTES = 126 * 1024 * 1024
UNIT = "TOPS"


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"bf16_tflops": float(p["bf16_tflops"]), "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.samples = []
        self._stop = threading.Event()
        self._thread = None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                parts = [x.strip() for x in out.strip().split(",")]
                if len(parts) >= 6:
                    self.samples.append(parts)
            except Exception:
                pass
            self._stop.wait(0.05)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        self._thread.join(timeout=6)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        mhz = sorted(float(s[0]) for s in self.samples)
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": float(self.samples[0][1]), "reasons": reasons,
                "samples": len(self.samples)}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        ids = [x for x in vis.split(",") if x != ""]
        if local_rank < len(ids) and ids[local_rank].isdigit():
            return int(ids[local_rank])
    return local_rank


def bind_host_thread_near_gpu(torch, local_rank):
    """Moves this process onto the CPUs of the NUMA node the GPU hangs off, before any pinned host buffer
    is allocated (pages are placed where they are first touched), so that with several ranks per host the
    end-to-end copies do not all cross the socket interconnect.  Best effort: returns the node number, or
    None when the topology cannot be read or no allowed CPU sits on that node."""
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bdf = "%04x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return None
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if not allowed:
            return None
        os.sched_setaffinity(0, allowed)
        return node
    except Exception:
        return None


def cpu_baseline(workload, seconds_hint=10.0, threads=0):
    """The reference project's fp32 CPU path (its unchanged templates, one single-slice call chain per
    head, heads spread over all host threads) on a bounded sample of whole heads of `workload`."""
    import numpy as np
    import __graft_entry__ as ge
    oracle = ge.load_oracle()
    cores = threads if threads > 0 else oracle.n_threads_default()
    w = workload
    per_head_ops = 4.0 * w.S * w.S * w.D
    est_rate = 1.5e9  # ops/s/thread, the order of magnitude of the unvectorised triple loop
    heads = max(1, min(w.B * w.H, int(round(seconds_hint * est_rate * cores / per_head_ops))))
    if heads >= cores:
        heads = (heads // cores) * cores       # whole rounds of one head per thread
    rng = np.random.default_rng(2023)
    q, k, v = (rng.standard_normal((1, heads, w.S, w.D), dtype=np.float32) for _ in range(3))
    mask = np.zeros((1, w.S), np.int8)
    if w.valid_choices is not None:
        mask[0, min(w.valid_choices):] = 1
    if oracle.ref_cpu_available(native=True):
        kind = "reference"
        t0 = time.perf_counter()
        oracle.ref_fp32_attention(q, k, v, mask, batched=False, threads=cores, native=True)
        dt = time.perf_counter() - t0
    else:
        kind = "port"
        t0 = time.perf_counter()
        oracle.fp32_attention(q, k, v, mask, threads=cores)
        dt = time.perf_counter() - t0
    return {"value": heads * per_head_ops / dt / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
            "sample": f"{heads} of {w.B * w.H} heads of {w.name} (S={w.S}, D={w.D}), fp32 cpuGEMM/cpuSoftmax path, "
                      f"{dt:.2f} s, -O3 -march=x86-64-v3",
            "seconds": dt, "heads": heads}


def run_reference_arm(args, workload):
    """--impl reference: the reference's CPU implementation of the path, all host threads."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import numpy as np
    import __graft_entry__ as ge
    oracle = ge.load_oracle()
    cores = args.cpu_threads if args.cpu_threads > 0 else oracle.n_threads_default()
    w = workload
    per_head_ops = 4.0 * w.S * w.S * w.D
    heads = min(w.B * w.H, cores)          # one whole head per host thread and step
    rng = np.random.default_rng(2023)
    q, k, v = (rng.standard_normal((1, heads, w.S, w.D), dtype=np.float32) for _ in range(3))
    mask = np.zeros((1, w.S), np.int8)
    if w.valid_choices is not None:
        mask[0, min(w.valid_choices):] = 1
    native = oracle.ref_cpu_available(native=True)
    kind = "reference" if native else "port"

    def step():
        if native:
            oracle.ref_fp32_attention(q, k, v, mask, batched=False, threads=cores, native=True)
        else:
            oracle.fp32_attention(q, k, v, mask, threads=cores)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / max(args.steps, 1)
    value = heads * per_head_ops / dt / 1e12
    sample = (f"each step = {heads} of {w.B * w.H} heads of {w.name} (S={w.S}, D={w.D}), one head per host thread, "
              f"reference fp32 cpuGEMM/cpuSoftmax path")
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"{w.name}: B={w.B} H={w.H} S={w.S} D={w.D}", "sampled_heads_per_step": heads},
            "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def run_quantize_bench(args, pkg, w, dev, rank, world):
    """HBM-bound producer in front of the attention call: fp32 [B,H,S,D] -> amax + int8.
    Algorithmic bytes per element: 4 (abs-max pass) + 4 + 1 (quantise pass) = 9."""
    import torch
    n = w.B * w.H * w.S * w.D
    g = torch.Generator(device=dev)
    g.manual_seed(args.seed)
    x = torch.randn(n, generator=g, device=dev, dtype=torch.float32)
    out = torch.empty(n, dtype=torch.int8, device=dev)
    amax = torch.zeros(1, dtype=torch.float32, device=dev)
    stream = torch.cuda.current_stream()
    for _ in range(max(args.warmup, 3)):
        pkg.quantize_f32(stream, x, out, amax)
    torch.cuda.synchronize()
    l0 = pkg.launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(args.steps):
        pkg.quantize_f32(stream, x, out, amax)
    ev1.record(stream)
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / args.steps
    peaks = read_peaks()
    gbs = 9.0 * n / (ms * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({"metric": "quantise producer throughput (9 B/element algorithmic)", "value": gbs, "unit": "GB/s", "n_gpus": 1,
                          "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "dtype": "f32->int8",
                          "data": "synthetic", "config": {"workload": f"quantize one {w.name} tensor: {n} elements", "l2": "input larger than L2"},
                          "gpu_launches": pkg.launch_count() - l0,
                          "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": gbs / peaks["hbm_gbs"],
                                       "traffic": None, "kernel": "quant_absmax_kernel + quant_apply_kernel"}}), flush=True)


# ------------------------------------------------------------------------------------------------ timing helpers
def time_steps(torch, stream, step, steps, flush_l2, dev):
    """Device time of `steps` calls of step(), in ms (total).  With flush_l2 every step is timed on its own with
    the L2 overwritten in between; otherwise the steps run back to back between one pair of events."""
    if flush_l2:
        scratch = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b in evs:
            scratch.fill_(1)
            a.record(stream)
            step()
            b.record(stream)
        torch.cuda.synchronize()
        total = sum(a.elapsed_time(b) for a, b in evs)
        del scratch
        return total
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record(stream)
    for _ in range(steps):
        step()
    ev1.record(stream)
    torch.cuda.synchronize()
    return ev0.elapsed_time(ev1)


def make_problem(torch, wl, w, seed, dev):
    """Inputs generated and quantised on the device; o_amax calibrated from an fp32 attention there.
    Returns (data dict with q8,k8,v8,mask,amax, o_fp32 or None, o_amax)."""
    data = wl.make_int8_torch(w, seed, dev, want_fp32=True)
    o_fp32, o_amax = wl.fp32_attention_torch(data["q"], data["k"], data["v"], data["mask"])
    for n in ("q", "k", "v"):
        del data[n]
    torch.cuda.empty_cache()
    return data, o_fp32, o_amax


def parity_block(torch, oracle, w, data, o8_whole, o_fp32, o_amax, rows_per_head=8, seed=0):
    """Distance of an int8 output [B,H,S,D] from the quantised CPU oracle (tier C) on a row sample, and the
    reference's own acceptance figure (mean relative deviation from the fp32 golden, inc/utils.hpp:59-89)
    on the same rows."""
    import numpy as np
    rng = np.random.default_rng(seed)
    BH = w.B * w.H
    rows = []
    for bh in range(BH):
        fixed = {0, w.S - 1}
        extra = rng.integers(0, w.S, max(rows_per_head - len(fixed), 0))
        rows.extend(bh * w.S + r for r in sorted(fixed | set(int(x) for x in extra)))
    rows = np.asarray(rows, np.int64)
    q8, k8, v8, mask = (data[n].cpu().numpy() for n in ("q8", "k8", "v8", "mask"))
    amax = (*data["amax"], o_amax)
    want = oracle.q128(q8, k8, v8, mask, amax, rows=rows)
    idx = torch.from_numpy(rows).to(o8_whole.device)
    got = o8_whole.reshape(-1, w.D).index_select(0, idx).cpu().numpy()
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    out = {"rows_checked": int(rows.size), "elements": int(d.size), "exact_pct": 100.0 * float((d == 0).mean()),
           "within_1_lsb_pct": 100.0 * float((d <= 1).mean()), "max_lsb": int(d.max()),
           "against": "quantised tile-128 CPU oracle (tier C), pinned to the reference kernel's bytes through its emulation"}
    if o_fp32 is not None:
        gold = o_fp32.reshape(-1, w.D).index_select(0, idx).float().cpu().numpy()
        out["mean_rel_deviation_pct_vs_fp32_golden"] = float(oracle.mean_rel_deviation(got, gold, o_amax))
        out["oracle_mean_rel_deviation_pct_vs_fp32_golden"] = float(oracle.mean_rel_deviation(want, gold, o_amax))
        out["reference_acceptance_threshold_pct"] = 20.0
    return out, rows, want


def ref_gpu_block(torch, oracle, w, data, o_amax, rows, want, o_fp32, steps=5):
    """The reference project's CUDA kernel rebuilt for sm_100a on the same inputs: time per launch and how far its
    output is from the oracle and from its own fp32 golden (it serves as context, not as an oracle)."""
    import numpy as np
    if not oracle.ref_gpu_available():
        return {"available": False, "why": "oracle/_ref/libref_gpu.so not built"}
    R = oracle.ref_gpu()
    if R.ref_gpu_shape_ok(w.S, w.D) != 1:
        return {"available": False, "why": f"the reference has no instantiation for S={w.S}, D={w.D} (src/fmha_i8.cu:39-155)"}
    out = torch.zeros_like(data["q8"])
    a5 = (ctypes.c_float * 5)(*data["amax"], o_amax, 1.0)
    d4 = (ctypes.c_int * 4)(w.B, w.S, w.H, w.D)

    def step():
        rc = R.ref_gpu_fmha(None, a5, d4, data["q8"].data_ptr(), data["k8"].data_ptr(), data["v8"].data_ptr(),
                            data["mask"].data_ptr(), out.data_ptr())
        if rc != 0:
            raise RuntimeError(f"reference kernel launch failed: {rc}")

    torch.cuda.synchronize()
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    torch.cuda.synchronize()
    ms = ev0.elapsed_time(ev1) / steps
    idx = torch.from_numpy(rows).to(out.device)
    got = out.reshape(-1, w.D).index_select(0, idx).cpu().numpy()
    d = np.abs(got.astype(np.int32) - want.astype(np.int32))
    res = {"available": True, "ms_per_launch": ms, "value": w.ops / (ms * 1e-3) / 1e12, "unit": UNIT, "steps": steps,
           "kernel": "gpuImpl::kernel::FMHAInferKernel (WMMA m16n16k16), built with -O3 for sm_100a, default stream, back to back",
           "within_1_lsb_pct_vs_oracle": 100.0 * float((d <= 1).mean()), "max_lsb_vs_oracle": int(d.max()),
           "note": "its P relayout drops and doubles keys (see tests/test_gpu_d_reference_kernel.py), so its output is far from "
                   "its own fp32 golden on anything but near-uniform attention: timing context, not an oracle"}
    if o_fp32 is not None:
        gold = o_fp32.reshape(-1, w.D).index_select(0, idx).float().cpu().numpy()
        res["mean_rel_deviation_pct_vs_fp32_golden"] = float(oracle.mean_rel_deviation(got, gold, o_amax))
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="C3")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size of the workload (profiling)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="strong (default): one workload partitioned over the ranks; weak: every rank runs the whole workload")
    ap.add_argument("--seed", type=int, default=2023)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip parity, reference-GPU baseline, other configs, sustained run")
    ap.add_argument("--e2e-steps", type=int, default=0)
    ap.add_argument("--sustain-seconds", type=float, default=1.2)
    ap.add_argument("--cpu-threads", type=int, default=0,
                    help="host threads of the CPU baseline and of --impl reference (0 = all the box has)")
    ap.add_argument("--check", action="store_true",
                    help="exit with status 3 when the parity block misses the tolerance (>= 99.9 %% within 1 LSB, none beyond 2)")
    ap.add_argument("--path", default="attention", choices=["attention", "quantize"],
                    help="attention = the forward pass (default); quantize = the device-side abs_max + int8 producer")
    args = ap.parse_args()

    import __graft_entry__ as ge
    pkg = ge.load_package()
    import importlib
    wl = importlib.import_module("int8_fmha_b200.workloads")
    part = importlib.import_module("int8_fmha_b200.partition")
    w = wl.CONFIGS[args.config]
    if args.batch:
        w = w.with_batch(args.batch)

    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    import torch
    import torch.distributed as dist

    check_failed = False
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n_gpus = max(world, 1)
    args.warmup = max(args.warmup, 3)

    pkg.lib()  # fails loudly if the CUDA library is missing
    host_numa = bind_host_thread_near_gpu(torch, local_rank) if world > 1 else None
    if args.path == "quantize":
        run_quantize_bench(args, pkg, w, dev, rank, world)
        return
    oracle = ge.load_oracle()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_ranks(x):
        t = torch.tensor([float(x)], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- the problem: the same on every rank (same seed); each rank then keeps its slice of heads
    data, o_fp32, o_amax = make_problem(torch, wl, w, args.seed, dev)
    o_amax = max_ranks(o_amax)
    BH = w.B * w.H
    param = pkg.FMHAParamI8(*data["amax"], o_amax, 1.0)
    desc = pkg.AttnDataDescriptor(w.B, w.S, w.H, w.D)
    stream = torch.cuda.current_stream()
    mask = data["mask"]
    weak = args.scaling == "weak" or world == 1
    begin, count = (0, BH) if weak else part.slice_bounds(BH, rank, world)
    head_elems = w.S * w.D

    def head_slice(t):
        return t.reshape(BH, w.S, w.D)[begin:begin + count].contiguous()

    q8s, k8s, v8s = head_slice(data["q8"]), head_slice(data["k8"]), head_slice(data["v8"])
    o8s = torch.empty_like(q8s)
    keep_whole = (rank == 0)       # rank 0 keeps the whole problem for the checks after the timed region
    if not keep_whole and not weak:
        for n in ("q8", "k8", "v8"):
            del data[n]
        o_fp32 = None
        torch.cuda.empty_cache()

    def step():
        pkg.FMHAInferI8Slice(stream, param, desc, q8s, k8s, v8s, mask, o8s, begin, count)

    for _ in range(args.warmup):
        step()
    barrier()
    st, words = pkg.device_status()
    if st != pkg.OK:
        raise RuntimeError(f"device status after warm-up: {words}")

    # The timed region is a few milliseconds, shorter than one nvidia-smi poll, so the clock sampler
    # brackets it with the same steps, untimed, for a quarter of a second on each side.
    clocks = ClockSampler(physical_gpu_index(local_rank))
    clocks.__enter__()

    def soak(seconds):
        t_end = time.perf_counter() + seconds
        while time.perf_counter() < t_end:
            for _ in range(8):
                step()
            torch.cuda.synchronize()

    soak(0.25)
    launches0 = pkg.launch_count()
    # A slice whose tensors would stay resident in the 126 MB L2 is timed step by step with the L2
    # overwritten in between; a larger one back to back (every step streams more than L2 holds).
    slice_bytes = 4.0 * count * head_elems + w.B * w.S
    flush_l2 = slice_bytes < 2 * L2_BYTES
    barrier()
    ms_total = time_steps(torch, stream, step, args.steps, flush_l2, dev)
    barrier()
    launches = pkg.launch_count() - launches0
    # the same steps once more with an event pair around each, for the spread (not part of `value`)
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in pairs:
        a.record(stream)
        step()
        b.record(stream)
    torch.cuda.synchronize()
    per_launch = sorted(a.elapsed_time(b) for a, b in pairs)
    soak(0.25)
    clocks.__exit__(None, None, None)
    ms_step = max_ranks(ms_total) / args.steps
    st, words = pkg.device_status()
    if st != pkg.OK:
        raise RuntimeError(f"device status after the timed region: {words}")
    job_ops = w.ops * (n_gpus if (weak and world > 1) else 1)
    value = job_ops / (ms_step * 1e-3) / 1e12

    # ---- roofline of the dominant (only) kernel: one launch per step, this rank's share of the work
    peaks = read_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    local_ms_launch = ms_total / max(launches, 1)
    slice_ops = w.ops * count / BH
    achieved = slice_ops / (local_ms_launch * 1e-3) / 1e12
    traffic, traffic_note = None, None
    tpath = os.path.join(ROOT, "profiles", "fmha_fwd_d128_c3_b4_traffic.json")
    if w.D == 128 and w.S == 2048 and w.H == 32 and os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        # measured on a smaller batch of the same shape; DRAM traffic of this kernel is proportional to the heads
        traffic = (tj["dram_bytes_read_per_launch"] + tj["dram_bytes_write_per_launch"]) * count / (tj["captured_batch"] * w.H)
        traffic_note = ("bytes per launch: ncu dram read+write of a B=4 capture scaled by the heads of this launch; reads equal Q+K+V, "
                        "the write part is a LOWER bound (the capture nearly fits the L2, part of O had not been written back)")
    live_tiles = int((~(mask != 0).view(w.B, -1, 128).all(dim=2)).sum().item()) if w.S % 128 == 0 else None
    ops_executed = None if live_tiles is None else 4.0 * w.H * w.S * 128.0 * live_tiles * w.D
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
                "traffic": traffic, "traffic_unit": traffic_note,
                "algorithmic_bytes": slice_bytes, "kernel": f"fmha_fwd_kernel<{w.D}>",
                "peak_source": f"2 x {peaks['source']} dense bf16 ({peaks['bf16_tflops']} TFLOP/s, burst): kind::i8 issues at twice the bf16 rate",
                "hbm_gbs_achieved": slice_bytes / (local_ms_launch * 1e-3) / 1e9, "hbm_gbs_peak": peaks["hbm_gbs"],
                "hbm_frac": slice_bytes / (local_ms_launch * 1e-3) / 1e9 / peaks["hbm_gbs"],
                "ops_executed_frac_of_algorithmic": None if ops_executed is None else ops_executed / w.ops}

    # ---- the slices, put together on rank 0, against one run of the whole problem there (outside the timed region)
    partition_check = None
    o8_whole = None
    if not weak:
        whole, cov = part.assemble_on_rank0(o8s, begin, count, True, BH)
        if rank == 0:
            o_ref = torch.empty_like(data["q8"])
            pkg.FMHAInferI8(stream, param, desc, data["q8"], data["k8"], data["v8"], mask, o_ref, True)
            torch.cuda.synchronize()
            same = bool(torch.equal(whole.reshape(o_ref.shape), o_ref))
            partition_check = {"slices_equal_whole_problem_run": same, "coverage": cov,
                               "heads_per_rank": [part.slice_bounds(BH, r, world)[1] for r in range(world)]}
            o8_whole = o_ref
    elif rank == 0:
        o8_whole = o8s.reshape(w.B, w.H, w.S, w.D)

    # ---- every rank running the whole workload (replicas), for comparison with the partitioned run
    weak_replicas = None
    if world > 1 and not weak and not args.no_extras:
        full = wl.make_int8_torch(w, args.seed, dev) if not keep_whole else data
        o_full = torch.empty_like(full["q8"])

        def step_whole():
            pkg.FMHAInferI8(stream, param, desc, full["q8"], full["k8"], full["v8"], mask, o_full, True)

        for _ in range(3):
            step_whole()
        barrier()
        ms_w = time_steps(torch, stream, step_whole, args.steps, w.bytes < 2 * L2_BYTES, dev)
        barrier()
        ms_w = max_ranks(ms_w) / args.steps
        weak_replicas = {"value": n_gpus * w.ops / (ms_w * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_w,
                         "what": f"{n_gpus} x the whole workload, one replica per GPU"}
        if full is not data:
            del full
        del o_full
        torch.cuda.empty_cache()

    # ---- end to end through the host-buffer entry point (pinned host memory, copies inside)
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hm = (x.cpu().pin_memory() for x in (q8s, k8s, v8s, mask))
        ho = torch.empty_like(hq).pin_memory()
        n_e2e = args.e2e_steps or max(3, min(args.steps, 10))
        for _ in range(2):
            pkg.FMHAInferI8HostSlice(param, desc, hq, hk, hv, hm, ho, begin, count)
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            pkg.FMHAInferI8HostSlice(param, desc, hq, hk, hv, hm, ho, begin, count)
        dt = max_ranks((time.perf_counter() - t0) / n_e2e)
        same = bool(torch.equal(ho, o8s.cpu()))
        e2e = {"value": job_ops / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(3 * q8s.numel() + mask.numel()),
               "d2h_bytes_per_step": int(o8s.numel()), "ms_per_step": dt * 1e3, "steps": n_e2e,
               "bytes_are": "per rank", "matches_device_resident_result": same}
        del hq, hk, hv, ho

    # ---- the same step back to back for at least a second, with the clocks of that second
    sustained = None
    if not args.no_extras:
        n_sus = max(args.steps, int(args.sustain_seconds / max(ms_total / args.steps * 1e-3, 1e-6)))
        n_sus = min(n_sus, 200000)
        barrier()
        with ClockSampler(physical_gpu_index(local_rank)) as cs:
            ms_s = time_steps(torch, stream, step, n_sus, False, dev)
        ms_s = max_ranks(ms_s) / n_sus
        sustained = {"value": job_ops / (ms_s * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": ms_s, "steps": n_sus,
                     "seconds": ms_s * n_sus * 1e-3, "clocks": cs.summary(),
                     "frac_of_int8_peak_sustained": (slice_ops / (ms_s * 1e-3) / 1e12) / (2.0 * peaks["bf16_tflops_sustained"]),
                     "note": "back to back, L2 not flushed; denominator 2 x the sustained dense bf16 figure"}

    parity = ref_gpu = others = cpu = None
    if rank == 0 and not args.no_extras and o8_whole is not None:
        try:
            parity, rows, want = parity_block(torch, oracle, w, data, o8_whole, o_fp32, o_amax)
            if n_gpus == 1:
                ref_gpu = ref_gpu_block(torch, oracle, w, data, o_amax, rows, want, o_fp32)
        except Exception as exc:  # reported extras never cost the GPU numbers
            parity = parity or {"error": repr(exc)}
    # the other benchmark shapes, 1 GPU only
    if rank == 0 and n_gpus == 1 and not args.no_extras:
        del data, o_fp32, q8s, k8s, v8s
        torch.cuda.empty_cache()
        others = {}
        for name in ("C2", "C3", "C4", "C5"):
            if name == w.name:
                continue
            try:
                w2 = wl.CONFIGS[name]
                d2, of2, oa2 = make_problem(torch, wl, w2, args.seed, dev)
                p2 = pkg.FMHAParamI8(*d2["amax"], oa2, 1.0)
                desc2 = pkg.AttnDataDescriptor(w2.B, w2.S, w2.H, w2.D)
                o2 = torch.empty_like(d2["q8"])

                def step2():
                    pkg.FMHAInferI8(stream, p2, desc2, d2["q8"], d2["k8"], d2["v8"], d2["mask"], o2, True)

                for _ in range(3):
                    step2()
                torch.cuda.synchronize()
                fl = w2.bytes < 2 * L2_BYTES
                n2 = 10
                ms2 = time_steps(torch, stream, step2, n2, fl, dev) / n2
                par2, _, _ = parity_block(torch, oracle, w2, d2, o2, of2, oa2, rows_per_head=2 if w2.B * w2.H > 1024 else 4)
                tops2 = w2.ops / (ms2 * 1e-3) / 1e12
                gbs2 = w2.bytes / (ms2 * 1e-3) / 1e9
                others[name] = {"workload": f"B={w2.B} H={w2.H} S={w2.S} D={w2.D}", "ms_per_step": ms2, "value": tops2, "unit": UNIT,
                                "frac_of_int8_peak": tops2 / int8_peak, "hbm_gbs": gbs2, "hbm_frac": gbs2 / peaks["hbm_gbs"],
                                "l2": "flushed between steps" if fl else "inputs larger than L2", "steps": n2,
                                "within_1_lsb_pct": par2["within_1_lsb_pct"], "exact_pct": par2["exact_pct"], "max_lsb": par2["max_lsb"]}
                del d2, of2, o2
                torch.cuda.empty_cache()
            except Exception as exc:
                others[name] = {"error": repr(exc)}
    if rank == 0 and n_gpus == 1 and not args.no_cpu:
        try:
            cpu = cpu_baseline(w, threads=args.cpu_threads)
        except Exception as exc:  # the baseline is a reported extra, never a reason to lose the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "unavailable", "sample": repr(exc)}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak" if (weak and world > 1) else "strong",
                "vs_baseline": None, "dtype": "int8", "data": "synthetic",
                "config": {"workload": f"{w.name}: B={w.B} H={w.H} S={w.S} D={w.D}", "mask": "none" if w.valid_choices is None else f"valid lengths {w.valid_choices}",
                           "l2": ("L2 overwritten between steps (this rank's Q,K,V,O = %.0f MB)" if flush_l2 else "this rank's inputs larger than L2 (Q,K,V,O = %.0f MB)") % (slice_bytes / 1e6),
                           "seed": args.seed,
                           "parallelism": (f"{n_gpus} x whole workload, no collective" if (weak and world > 1) else
                                           f"heads of one workload partitioned over {n_gpus} GPU(s), {count} of {BH} heads on rank 0, no collective on the data path"),
                           "host_numa_node_of_rank0": host_numa},
                "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "cpu_baseline": cpu, "pct_of_int8_peak": 100.0 * achieved / int8_peak,
                "per_launch_ms": {"median": per_launch[len(per_launch) // 2], "min": per_launch[0], "max": per_launch[-1],
                                  "note": "separate pass, one event pair per launch, L2 warm for slices that fit in it"},
                "partition_check": partition_check, "weak_replicas": weak_replicas, "sustained": sustained,
                "parity": parity, "ref_gpu_baseline": ref_gpu, "other_configs": others}
        print(json.dumps(line), flush=True)
        if args.check:
            checked = [parity] + [v for v in (others or {}).values() if isinstance(v, dict)]
            checked = [c for c in checked if c and "within_1_lsb_pct" in c]
            bad = [c for c in checked if c["within_1_lsb_pct"] < 99.9 or c["max_lsb"] > 2]
            if bad or not checked:
                print("bench.py --check: " + ("no parity block was computed (do not combine with --no-extras)" if not checked
                                               else f"parity outside the tolerance: {bad}"), file=sys.stderr, flush=True)
                check_failed = True
    if world > 1:
        dist.destroy_process_group()
    if check_failed:
        sys.exit(3)


if __name__ == "__main__":
    main()
