#!/usr/bin/env python
"""Benchmark of the INT8 flash-attention forward path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--impl ours|reference]

One "step" is one forward pass over one batch of synthetic int8 Q,K,V (seeded; the reference
project ships no dataset).  The default workload is C3 (B=8,H=32,S=2048,D=128), the shape the
throughput target is quoted on.  With N > 1 (launched under torchrun, one rank per GPU) every rank
runs the whole workload on its own GPU -- the path shards over batch*head with no exchange step,
so there is no collective on the data path ("weak" scaling); NCCL is used only for the barrier and
the max-over-ranks of the device time.

Prints ONE JSON line on rank 0:
  value      effective INT8 TOPS = N * 4*B*H*S^2*D / t, inputs resident in HBM, CUDA-event timed
  e2e        the same metric through fmha_i8_sm100_infer_host: pinned HOST buffers in and out,
             host<->device copies inside the timed region
  roofline   dominant kernel against the dense-INT8 tensor peak (2 x the measured dense bf16
             cuBLAS rate of this pool's B200s; kind::i8 runs at twice the bf16 rate)
  cpu_baseline  the reference project's CPU path (oracle/_ref) on a bounded sample of heads

--impl reference times the reference project's own CPU implementation of the path instead.
"""
import argparse
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
        return {"bf16_tflops": float(p["bf16_tflops"]), "hbm_gbs": float(p["hbm_gbs"]), "source": "measured"}
    return {"bf16_tflops": 1590.0, "hbm_gbs": 6650.0, "source": "fallback"}


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


def cpu_baseline(workload, seconds_hint=10.0):
    """The reference project's fp32 CPU path (its unchanged templates, one single-slice call chain per
    head, heads spread over all host threads) on a bounded sample of whole heads of `workload`."""
    import numpy as np
    import __graft_entry__ as ge
    oracle = ge.load_oracle()
    cores = oracle.n_threads_default()
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
    cores = oracle.n_threads_default()
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
            "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--config", default="C3")
    ap.add_argument("--batch", type=int, default=0, help="override the batch size of the workload (profiling)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--seed", type=int, default=2023)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--e2e-steps", type=int, default=0)
    ap.add_argument("--path", default="attention", choices=["attention", "quantize"],
                    help="attention = the forward pass (default); quantize = the device-side abs_max + int8 producer")
    args = ap.parse_args()

    import __graft_entry__ as ge
    pkg = ge.load_package()
    import importlib
    wl = importlib.import_module("int8_fmha_b200.workloads")
    w = wl.CONFIGS[args.config]
    if args.batch:
        w = w.with_batch(args.batch)

    if args.impl == "reference":
        run_reference_arm(args, w)
        return

    import torch
    import torch.distributed as dist

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
    # ---- inputs: generated and quantised on the device, o_amax calibrated from an fp32 attention
    data = wl.make_int8_torch(w, args.seed + 101 * rank, dev, want_fp32=True)
    _, o_amax = wl.fp32_attention_torch(data["q"], data["k"], data["v"], data["mask"])
    for n in ("q", "k", "v"):
        del data[n]
    torch.cuda.empty_cache()
    q8, k8, v8, mask = data["q8"], data["k8"], data["v8"], data["mask"]
    o8 = torch.empty_like(q8)
    param = pkg.FMHAParamI8(*data["amax"], o_amax, 1.0)
    desc = pkg.AttnDataDescriptor(w.B, w.S, w.H, w.D)
    stream = torch.cuda.current_stream()

    def step():
        pkg.FMHAInferI8(stream, param, desc, q8, k8, v8, mask, o8, True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

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
    # Workloads whose tensors would stay resident in the 126 MB L2 are timed step by step with the L2
    # overwritten in between; larger ones are timed back to back (every step streams more than L2 holds).
    flush_l2 = w.bytes < 2 * L2_BYTES
    barrier()
    if flush_l2:
        scratch = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device=dev)
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
        for a, b in evs:
            scratch.fill_(1)
            a.record(stream)
            step()
            b.record(stream)
        barrier()
        ms_total = sum(a.elapsed_time(b) for a, b in evs)
        del scratch
    else:
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        barrier()
        ms_total = ev0.elapsed_time(ev1)
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
    t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    st, words = pkg.device_status()
    if st != pkg.OK:
        raise RuntimeError(f"device status after the timed region: {words}")
    value = n_gpus * w.ops / (ms_step * 1e-3) / 1e12

    # ---- roofline of the dominant (only) kernel: one launch per step
    peaks = read_peaks()
    int8_peak = 2.0 * peaks["bf16_tflops"]
    local_ms_launch = ms_total / max(launches, 1)
    achieved = w.ops / (local_ms_launch * 1e-3) / 1e12
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "fmha_fwd_d128_c3_b4_traffic.json")
    if w.D == 128 and w.S == 2048 and w.H == 32 and os.path.exists(tpath):
        with open(tpath) as f:
            tj = json.load(f)
        # measured on a smaller batch of the same shape; DRAM traffic of this kernel is proportional to the batch
        traffic = (tj["dram_bytes_read_per_launch"] + tj["dram_bytes_write_per_launch"]) * w.B / tj["captured_batch"]
    # key tiles that hold at least one unmasked key are the ones the kernel executes; the headline counts all
    live_tiles = int((~(mask != 0).view(w.B, -1, 128).all(dim=2)).sum().item()) if w.S % 128 == 0 else None
    ops_executed = None if live_tiles is None else 4.0 * w.H * w.S * 128.0 * live_tiles * w.D
    roofline = {"bound": "tensor", "achieved": achieved, "peak": int8_peak, "unit": "TOP/s", "frac": achieved / int8_peak,
                "traffic": traffic, "traffic_unit": "bytes per launch (ncu dram read+write, scaled from the B=4 capture)",
                "algorithmic_bytes": w.bytes, "kernel": f"fmha_fwd_kernel<{w.D}>",
                "peak_source": f"2 x {peaks['source']} dense bf16 ({peaks['bf16_tflops']} TFLOP/s): kind::i8 issues at twice the bf16 rate",
                "hbm_gbs_achieved": w.bytes / (local_ms_launch * 1e-3) / 1e9, "hbm_gbs_peak": peaks["hbm_gbs"],
                "ops_executed_frac_of_algorithmic": None if ops_executed is None else ops_executed / w.ops}

    # ---- end to end through the host-buffer entry point (pinned host memory, copies inside)
    e2e = None
    if not args.no_e2e:
        hq, hk, hv, hm = (x.cpu().pin_memory() for x in (q8, k8, v8, mask))
        ho = torch.empty_like(hq).pin_memory()
        n_e2e = args.e2e_steps or max(3, min(args.steps, 10))
        for _ in range(2):
            pkg.FMHAInferI8Host(param, desc, hq, hk, hv, hm, ho)
        barrier()
        t0 = time.perf_counter()
        for _ in range(n_e2e):
            pkg.FMHAInferI8Host(param, desc, hq, hk, hv, hm, ho)
        dt = (time.perf_counter() - t0) / n_e2e
        tt = torch.tensor([dt], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        dt = float(tt.item())
        same = bool(torch.equal(ho, o8.cpu()))
        e2e = {"value": n_gpus * w.ops / dt / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(3 * q8.numel() + mask.numel()),
               "d2h_bytes_per_step": int(o8.numel()), "ms_per_step": dt * 1e3, "steps": n_e2e,
               "matches_device_resident_result": same}

    cpu = None
    if rank == 0 and n_gpus == 1 and not args.no_cpu:
        try:
            cpu = cpu_baseline(w)
        except Exception as exc:  # the baseline is a reported extra, never a reason to lose the GPU numbers
            cpu = {"value": None, "unit": UNIT, "cores": None, "kind": "unavailable", "sample": repr(exc)}

    if rank == 0:
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8",
                "data": "synthetic",
                "config": {"workload": f"{w.name}: B={w.B} H={w.H} S={w.S} D={w.D} per GPU", "mask": "none" if w.valid_choices is None else f"valid lengths {w.valid_choices}",
                           "l2": ("L2 overwritten between steps (Q,K,V,O = %.0f MB)" if flush_l2 else "inputs larger than L2 (Q,K,V,O = %.0f MB)") % (w.bytes / 1e6),
                           "seed": args.seed,
                           "parallelism": f"{n_gpus} x whole workload, no collective",
                           "host_numa_node_of_rank0": host_numa},
                "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches), "roofline": roofline,
                "cpu_baseline": cpu, "pct_of_int8_peak": 100.0 * achieved / int8_peak,
                "per_launch_ms": {"median": per_launch[len(per_launch) // 2], "min": per_launch[0], "max": per_launch[-1],
                                  "note": "separate pass, one event pair per launch, L2 warm for workloads that fit in it"}}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
