#!/usr/bin/env python
"""Benchmark of the mops hot path on B200: forward + VJP of the five sparse operations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload all|hpe|sap|opsa|opsa_f32|opsaw|sasaw] [--no-cpu-baseline]

A step is one pass of the hot path over one batch of synthetic input: forward and VJP of
every selected operation at its large configuration (per GPU):

    hpe      f64  I=2^20, N=100, J=2000, K=4   (the reference's HPE table, batch scaled up)
    sap      f64  I=2^22, 20x6 -> 50, 1000 triplets
    opsa     f64  J=2^24 entries, 13x20, 2^18 output rows
    opsa_f32 f32  the same draws cast to f32
    opsaw    f64  E=2^22 edges, 13x32, 2^16 nodes   (the reference's OPSAW shape, scaled up)
    sasaw    f64  E=2^22 edges, 9x32, 2^16 nodes, 500 coupling entries

Metric: algorithmic GB/s (bytes each call must move, every input read once and every output
written once, divided by device time), summed over all calls of a step and all GPUs. The
per-operation numbers are in ``per_op``. ``e2e`` is the same pass starting and ending in
HOST memory: every step copies each case's inputs from pinned host buffers to the device,
calls forward and VJP through the public API (``mops_b200``) and copies every result back
to pinned host buffers, all inside the timed region (copy-in, compute and copy-out streams
chained by events, so copies in both directions and kernels overlap). With N > 1 every rank works on its own shard of the same size (weak scaling; rows
and output-segment ranges are independent, so there is no collective on the data path
except the all-reduce of grad_W for OPSAW/SASAW, whose W is replicated).

``--impl reference`` times the reference's own CPU implementation (oracle/_ref/libmops_ref.so,
built from the unmodified reference sources; the C restatement if that is absent) on all
host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from mops_b200 import workloads  # noqa: E402

FALLBACK_HBM_GBS = 6650.0

# name -> (op, dtype, generator kwargs for the full per-GPU size, CPU sample divisor)
CASES = {
    "hpe": ("hpe", np.float64, dict(I=1 << 20), 8),
    "sap": ("sap", np.float64, dict(I=1 << 22), 16),
    "opsa": ("opsa", np.float64, dict(J=1 << 24, nO=1 << 18), 8),
    "opsa_f32": ("opsa", np.float32, dict(J=1 << 24, nO=1 << 18), 8),
    "opsaw": ("opsaw", np.float64, dict(E=1 << 22, n=1 << 16), 8),
    "sasaw": ("sasaw", np.float64, dict(E=1 << 22, n=1 << 16), 64),
}
BATCH_KEYS = {"hpe": ("I",), "sap": ("I",), "opsa": ("J", "nO"), "opsaw": ("E", "n"),
              "sasaw": ("E", "n")}
# kernels of this library launched by one forward / one VJP call of every case (sorted input,
# waiting calls): a table builder (plan, segment offsets, coupling) + the main kernel; the f32
# OPSA VJP needs no table, the SASAW forward builds two
LAUNCHES = {"hpe": (2, 2), "sap": (2, 2), "opsa": (2, 2), "opsa_f32": (2, 1), "opsaw": (2, 2),
            "sasaw": (3, 2)}
# DRAM traffic per launch of the main kernel (dram__bytes_read.sum + dram__bytes_write.sum of
# one ncu capture), by case and level. Captured with every batch dimension divided by 8 (the
# full-size step is too large for a multi-pass capture) and multiplied by 8 here: all
# operands and results of these kernels scale with the batch. The summaries under profiles/
# hold the captured figures.
MEASURED_TRAFFIC = {
    ("hpe", "fwd"): 8 * 108.6e6, ("hpe", "vjp"): 8 * 193.5e6,
    ("sap", "fwd"): 8 * 432.9e6, ("sap", "vjp"): 8 * 407.4e6,
    ("opsa", "fwd"): 8 * 614.0e6, ("opsa", "vjp"): 8 * 1138.3e6,
    ("opsa_f32", "fwd"): 8 * 304.7e6, ("opsa_f32", "vjp"): 8 * 554.5e6,
    ("opsaw", "fwd"): 8 * 212.0e6, ("opsaw", "vjp"): 8 * 372.9e6,
    ("sasaw", "fwd"): 8 * 209.2e6, ("sasaw", "vjp"): 8 * 409.8e6,
}


def traffic(name, level):
    t = MEASURED_TRAFFIC.get((name, level))
    return None if t is None else t / SCALE


def selected_cases(which):
    return list(CASES) if which == "all" else [which]


SCALE = 1  # --scale N divides every batch dimension by N (small cases for ncu captures)


def generate(name, rank, divisor=1):
    op, dtype, kw, _ = CASES[name]
    divisor *= SCALE
    kw = {k: (v // divisor if k in BATCH_KEYS[op] else v) for k, v in kw.items()}
    seed = workloads.SEEDS[op] + 1000 * rank
    if name == "opsa_f32":
        seed = workloads.SEEDS["opsa"] + 1000 * rank
    return workloads.GENERATORS[op](dtype=dtype, seed=seed, **kw)


# ------------------------------------------------------------------------------ call shapes
def fwd_args(op, d):
    if op == "hpe":
        return (d["A"], d["C"], d["indices_A"])
    if op == "sap":
        return (d["A"], d["B"], d["C"], d["indices_A"], d["indices_B"], d["indices_output"],
                d["output_size"])
    if op == "opsa":
        return (d["A"], d["B"], d["indices_output"], d["output_size"])
    if op == "opsaw":
        return (d["A"], d["B"], d["W"], d["indices_W"], d["indices_output"])
    return (d["A"], d["B"], d["C"], d["W"], d["indices_A"], d["indices_W_1"], d["indices_W_2"],
            d["indices_output_1"], d["indices_output_2"], d["output_size"])


def vjp_args(op, d):
    a = fwd_args(op, d)
    if op in ("sap", "opsa", "sasaw"):
        a = a[:-1]  # no output_size
    return (d["grad_output"],) + a


def api(op):
    import mops_b200 as M
    f = {"hpe": "homogeneous_polynomial_evaluation", "sap": "sparse_accumulation_of_products",
         "opsa": "outer_product_scatter_add", "opsaw": "outer_product_scatter_add_with_weights",
         "sasaw": "sparse_accumulation_scatter_add_with_weights"}[op]
    return getattr(M, f), getattr(M, f + "_vjp")


def tensor_bytes(args):
    import torch
    return sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor))


# ------------------------------------------------------------------------------ clocks
class ClockSampler(threading.Thread):
    """Reads SM clock, max clock and clock-event reasons every 200 ms (NVML, read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self._stop_event = threading.Event()
        self.enabled = False

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
        except Exception:
            return
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
                 0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks"}
        while not self._stop_event.is_set():
            if self.enabled:
                try:
                    self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                    for bit, n in names.items():
                        if r & bit:
                            self.reasons.add(n)
                except Exception:
                    pass
            self._stop_event.wait(0.2 if self.enabled else 0.02)

    def stop(self):
        self._stop_event.set()

    def summary(self):
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ------------------------------------------------------------------------------ CPU arm
def cpu_impl():
    from oracle import mops_oracle as mo
    if mo.have_reference():
        return mo.Reference(), "reference"
    return mo.Oracle(), "port"


def cpu_pass(impl, name, d):
    """Forward + VJP of one case on the CPU implementation; returns seconds (fwd, vjp)."""
    op = CASES[name][0]
    t0 = time.perf_counter()
    if op == "hpe":
        impl.hpe(d["A"], d["C"], d["indices_A"])
        t1 = time.perf_counter()
        impl.hpe_vjp(d["grad_output"], d["A"], d["C"], d["indices_A"])
    elif op == "sap":
        idx = (d["indices_A"], d["indices_B"], d["indices_output"])
        impl.sap(d["A"], d["B"], d["C"], *idx, d["output_size"])
        t1 = time.perf_counter()
        impl.sap_vjp(d["grad_output"], d["A"], d["B"], d["C"], *idx)
    elif op == "opsa":
        impl.opsa(d["A"], d["B"], d["indices_output"], d["output_size"])
        t1 = time.perf_counter()
        impl.opsa_vjp(d["grad_output"], d["A"], d["B"], d["indices_output"])
    elif op == "opsaw":
        impl.opsaw(d["A"], d["B"], d["W"], d["indices_W"], d["indices_output"])
        t1 = time.perf_counter()
        impl.opsaw_vjp(d["grad_output"], d["A"], d["B"], d["W"], d["indices_W"], d["indices_output"])
    else:
        idx = (d["indices_A"], d["indices_W_1"], d["indices_W_2"], d["indices_output_1"],
               d["indices_output_2"])
        impl.sasaw(d["A"], d["B"], d["C"], d["W"], *idx, d["output_size"])
        t1 = time.perf_counter()
        impl.sasaw_vjp(d["grad_output"], d["A"], d["B"], d["C"], d["W"], *idx)
    t2 = time.perf_counter()
    return t1 - t0, t2 - t1


def cpu_run(names, steps, warmup):
    """Times the CPU implementation on a bounded sample (a 1/divisor-size draw of every case)."""
    impl, kind = cpu_impl()
    cores = os.cpu_count() or 1
    os.environ.setdefault("OMP_NUM_THREADS", str(cores))
    data, nbytes, sample = {}, 0, []
    for n in names:
        op, _, _, div = CASES[n]
        data[n] = generate(n, 0, divisor=div)
        nbytes += workloads.algorithmic_bytes(op, "fwd", data[n]) + \
            workloads.algorithmic_bytes(op, "vjp", data[n])
        sample.append(f"{n}: 1/{div}")
    per_op = {n: [0.0, 0.0] for n in names}
    total = 0.0
    for s in range(warmup + steps):
        t_step = 0.0
        for n in names:
            f, v = cpu_pass(impl, n, data[n])
            if s >= warmup:
                per_op[n][0] += f
                per_op[n][1] += v
            t_step += f + v
        if s >= warmup:
            total += t_step
    ms = total / steps * 1e3
    out_per_op = {}
    for n in names:
        op = CASES[n][0]
        bf = workloads.algorithmic_bytes(op, "fwd", data[n])
        bv = workloads.algorithmic_bytes(op, "vjp", data[n])
        out_per_op[n] = {"fwd_ms": per_op[n][0] / steps * 1e3, "vjp_ms": per_op[n][1] / steps * 1e3,
                         "fwd_GBps": bf / (per_op[n][0] / steps) / 1e9,
                         "vjp_GBps": bv / (per_op[n][1] / steps) / 1e9}
    return {"value": nbytes / (total / steps) / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
            "sample": "same generators at reduced batch: " + ", ".join(sample),
            "ms_per_step": ms, "per_op": out_per_op}


# ------------------------------------------------------------------------------ main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="all", choices=["all"] + list(CASES))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-spread", action="store_true",
                    help="skip the per-call median / p10 / p90 measurement (also skipped with "
                         "--no-e2e)")
    ap.add_argument("--scale", type=int, default=1,
                    help="divide every batch dimension by this (small cases for profiling)")
    args = ap.parse_args()
    # stdout carries exactly one JSON line: everything libraries print there (NCCL's version
    # banner, for one) is sent to stderr, and the line is written to the original descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    global SCALE
    SCALE = max(1, args.scale)
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    names = selected_cases(args.workload)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "fwd+vjp of " + ",".join(names) + " at the scaled per-GPU sizes" +
              (f" divided by {SCALE}" if SCALE > 1 else ""),
              "cases": {n: {**{k: int(v) // (SCALE if k in BATCH_KEYS[CASES[n][0]] else 1)
                               for k, v in CASES[n][2].items()},
                            "dtype": np.dtype(CASES[n][1]).name} for n in names},
              "sharding": "independent shard per rank (batch rows / output-segment ranges)",
              "cache": "inputs larger than L2 (126 MB) for every case"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        r = cpu_run(names, args.steps, max(args.warmup, 1))
        line = {"impl": "reference", "metric": "algorithmic_GBps_fwd_plus_vjp", "value": r["value"],
                "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": config,
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "per_op": r["per_op"], "gpu_launches": 0}
        emit(line)
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (no CPU fallback exists)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # keep stdout for the one JSON line: NCCL's version / debug lines go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- data: pinned host copies (e2e source) and device-resident copies
    host, devd, nbytes = {}, {}, {}
    for n in names:
        op = CASES[n][0]
        d = generate(n, rank)
        nbytes[n] = (workloads.algorithmic_bytes(op, "fwd", d),
                     workloads.algorithmic_bytes(op, "vjp", d))
        host[n] = {k: (torch.from_numpy(v).pin_memory() if isinstance(v, np.ndarray) else v)
                   for k, v in d.items()}
        devd[n] = {k: (v.to(dev) if isinstance(v, torch.Tensor) else v) for k, v in host[n].items()}
        del d
    reduce_gw = world > 1

    def run_case(n, data, timers=None):
        op = CASES[n][0]
        fwd, vjp = api(op)
        if timers is not None:
            timers[0].record()
        out = fwd(*fwd_args(op, data))
        if timers is not None:
            timers[1].record()
        grads = vjp(*vjp_args(op, data))
        if reduce_gw and op in ("opsaw", "sasaw") and grads[2].is_cuda:
            dist.all_reduce(grads[2])
        if timers is not None:
            timers[2].record()
        return out, grads

    # ---- device-resident timing
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    for _ in range(args.warmup):
        for n in names:
            run_case(n, devd[n])
    barrier()
    events = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in names]
              for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.enabled = True
    start.record()
    for s in range(args.steps):
        for i, n in enumerate(names):
            run_case(n, devd[n], events[s][i])
    stop.record()
    barrier()
    sampler.enabled = False
    t_ms = start.elapsed_time(stop)
    per_op_ms = {n: [statistics.mean(events[s][i][0].elapsed_time(events[s][i][1])
                                     for s in range(args.steps)),
                     statistics.mean(events[s][i][1].elapsed_time(events[s][i][2])
                                     for s in range(args.steps))] for i, n in enumerate(names)}
    if world > 1:
        t = torch.tensor([t_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        t_ms = float(t.item())
    step_bytes = sum(sum(nbytes[n]) for n in names)
    value = step_bytes * world * args.steps / (t_ms / 1e3) / 1e9

    # ---- spread of every call: the same calls again, each one between its own pair of events
    # (outside the timed step; rank 0's view)
    spread = {}
    if not (args.no_spread or args.no_e2e):  # quick / profiling runs skip it with the e2e leg
        reps = 20
        for n in names:
            ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(reps)]
            for r in range(reps):
                run_case(n, devd[n], ev[r])
            torch.cuda.synchronize()
            f = sorted(e[0].elapsed_time(e[1]) for e in ev)
            v = sorted(e[1].elapsed_time(e[2]) for e in ev)
            q = lambda xs, p: xs[min(len(xs) - 1, int(p * len(xs)))]
            spread[n] = {"reps": reps, "fwd_ms_median": q(f, 0.5), "fwd_ms_p10": q(f, 0.1),
                         "fwd_ms_p90": q(f, 0.9), "vjp_ms_median": q(v, 0.5),
                         "vjp_ms_p10": q(v, 0.1), "vjp_ms_p90": q(v, 0.9)}

    # ---- end to end: every step copies each case's inputs from pinned host memory to the
    # device, calls forward and VJP through the public API and copies all results back into
    # pinned host buffers. Three CUDA streams (copy in, compute, copy out) chained by events:
    # the copies of different cases overlap each other (PCIe is full duplex) and the kernels.
    e2e = None
    if not args.no_e2e:
        s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
        host_out = {}

        def e2e_step():
            staged, keep = [], []
            with torch.cuda.stream(s_in):
                for n in names:
                    data = {k: (v.to(dev, non_blocking=True) if isinstance(v, torch.Tensor) else v)
                            for k, v in host[n].items()}
                    ready = torch.cuda.Event()
                    ready.record(s_in)
                    staged.append((n, data, ready))
            for n, data, ready in staged:
                s_run.wait_event(ready)
                with torch.cuda.stream(s_run):
                    out, grads = run_case(n, data)
                    done = torch.cuda.Event()
                    done.record(s_run)
                results = (out,) + tuple(grads if isinstance(grads, tuple) else (grads,))
                if n not in host_out:
                    host_out[n] = [torch.empty(r.shape, dtype=r.dtype, pin_memory=True)
                                   for r in results]
                s_out.wait_event(done)
                with torch.cuda.stream(s_out):
                    for r, h in zip(results, host_out[n]):
                        h.copy_(r, non_blocking=True)
                keep.append((data, results))  # device buffers stay alive until the step ends
            s_out.synchronize()
            s_run.synchronize()

        torch.cuda.synchronize()
        for _ in range(3):
            e2e_step()
        h2d = sum(tensor_bytes(tuple(v for v in host[n].values() if isinstance(v, torch.Tensor)))
                  for n in names)
        d2h = sum(tensor_bytes(tuple(host_out[n])) for n in names)
        barrier()
        t0 = time.perf_counter()
        e2e_steps = max(1, min(args.steps, 3))
        for _ in range(e2e_steps):
            e2e_step()
        torch.cuda.synchronize()
        t_e2e = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([t_e2e], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            t_e2e = float(t.item())
        e2e = {"value": step_bytes * world * e2e_steps / t_e2e / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": t_e2e / e2e_steps * 1e3}
    sampler.stop()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    per_op = {}
    dominant = None
    for n in names:
        f_ms, v_ms = per_op_ms[n]
        bf, bv = nbytes[n]
        items = devd[n]["A"].shape[0]
        per_op[n] = {"fwd_ms": f_ms, "vjp_ms": v_ms, "fwd_GBps": bf / f_ms / 1e6,
                     "vjp_GBps": bv / v_ms / 1e6, "fwd_frac_of_hbm": bf / f_ms / 1e6 / peak,
                     "vjp_frac_of_hbm": bv / v_ms / 1e6 / peak,
                     "fwd_items_per_s": items / f_ms * 1e3, "vjp_items_per_s": items / v_ms * 1e3,
                     "fwd_bytes": bf, "vjp_bytes": bv, **spread.get(n, {}),
                     "fwd_traffic": traffic(n, "fwd"), "vjp_traffic": traffic(n, "vjp")}
        for lvl, ms, b in (("fwd", f_ms, bf), ("vjp", v_ms, bv)):
            if dominant is None or ms > dominant[2]:
                dominant = (n, lvl, ms, b)
    dn, dl, dms, db = dominant
    roofline = {"bound": "hbm", "kernel": f"{dn} {dl}", "achieved": db / dms / 1e6, "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": db / dms / 1e6 / peak,
                "traffic": traffic(dn, dl)}
    launches = sum(sum(LAUNCHES[n]) for n in names) * args.steps
    line = {"metric": "algorithmic_GBps_fwd_plus_vjp", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64" if names != ["opsa_f32"] else "f32",
            "data": "synthetic", "config": config, "roofline": roofline, "per_op": per_op,
            "clocks": sampler.summary(), "gpu_launches": launches, "peak_hbm_GBps": peak}
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        r = cpu_run(names, 1, 1)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["cpu_baseline"]["per_op"] = r["per_op"]
    emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
