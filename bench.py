#!/usr/bin/env python
"""Benchmark of the mops hot path on B200: forward + VJP of the five sparse operations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload all|hpe|sap|opsa|opsa_f32|opsaw|sasaw]
                    [--no-cpu-baseline] [--no-e2e] [--no-verify] [--no-small] [--no-strong]
                    [--scale D [--keep-rows]]

A step is one pass of the hot path over one batch of synthetic input: forward and VJP of
every selected operation at its large configuration (per GPU):

    hpe      f64  I=2^20, N=100, J=2000, K=4   (the reference's HPE table, batch scaled up)
    sap      f64  I=2^22, 20x6 -> 50, 1000 triplets
    opsa     f64  J=2^24 entries, 13x20, 2^18 output rows
    opsa_f32 f32  the same draws cast to f32
    opsaw    f64  E=2^22 edges, 13x32, 2^16 nodes   (the reference's OPSAW shape, scaled up)
    sasaw    f64  E=2^22 edges, 9x32, 2^16 nodes, 500 coupling entries

``value``: algorithmic GB/s (bytes each call must move, every input read once and every
output written once, divided by device time), summed over all calls of a step and all GPUs;
inputs resident in HBM, CUDA events on the launching stream. ``per_op``: each operation's
forward and VJP time, GB/s, fraction of the measured HBM peak, the resource that bounds it
and the fraction of that resource, measured DRAM traffic (profiles/traffic.json).

``e2e``: the same pass starting and ending in HOST memory through the package's public API:
inside ``with mops_b200.HostQueue()`` every step calls forward and VJP of every case on
pinned host arrays; the queue copies the operands in, runs the kernels and copies every
result back to pinned host memory on three streams, all inside the timed region.

``verified``: after timing, the very buffers that were timed are compared with the CPU
oracle on sub-ranges (tests/subrange.py), outside the timed region.

``small_configs``: call latency (median / p10 / p90 of >= 100 synchronous calls through the
C ABI) at the five small configurations the reference's own benchmark programs run
(mops/benchmarks/*.cpp: the generators' defaults); no roofline for these.

With N > 1 every rank first runs its own problem of the full per-GPU size (weak scaling, the
headline), then all ranks split rank 0's problem (``strong``: batch rows / output-segment
ranges cut by mops_b200.sharding, grad_W all-reduced) and report T(1)/T(N) per operation.

``--impl reference`` times the reference's own CPU implementation (oracle/_ref/libmops_ref.so,
built from the unmodified reference sources; the C restatement if that is absent) with all
host threads on the same configuration at its full size; because one such step takes many
seconds it times at most 3 steps after 1 warm-up and says so in the line.
"""
import argparse
import ctypes
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
FP64_FLOP_PER_CLK_PER_SM = 128  # 64 DFMA lanes (or the same rate as DMMA) x 2

# name -> (op, dtype, generator kwargs for the full per-GPU size, CPU sample divisor)
CASES = {
    "hpe": ("hpe", np.float64, dict(I=1 << 20), 8),
    "sap": ("sap", np.float64, dict(I=1 << 22), 16),
    "opsa": ("opsa", np.float64, dict(J=1 << 24, nO=1 << 18), 8),
    "opsa_f32": ("opsa", np.float32, dict(J=1 << 24, nO=1 << 18), 8),
    "opsaw": ("opsaw", np.float64, dict(E=1 << 22, n=1 << 16), 8),
    "sasaw": ("sasaw", np.float64, dict(E=1 << 22, n=1 << 16), 64),
}
# the configurations of the reference's benchmark programs (the generators' defaults):
# latency cases
SMALL_CASES = {
    "hpe": ("hpe", np.float64), "sap": ("sap", np.float64), "opsa": ("opsa", np.float64),
    "opsa_f32": ("opsa", np.float32), "opsaw": ("opsaw", np.float64),
    "sasaw": ("sasaw", np.float64),
}
BATCH_KEYS = {"hpe": ("I",), "sap": ("I",), "opsa": ("J", "nO"), "opsaw": ("E", "n"),
              "sasaw": ("E", "n")}
ROW_KEYS = ("nO", "n")
# what bounds each case on the SM: HBM bytes, shared-memory
# wavefronts (every operand is a gather with a run-time index), or FP64 throughput. SASAW also
# reports the DRAM traffic it really causes (`*_traffic_frac_of_hbm`): its W table (151 MB at
# the benchmark size) does not fit L2, so the gathered W rows and the grad_W additions of every
# edge go to DRAM and the kernels move 4 to 7 times their algorithmic bytes.
BOUND = {"hpe": "smem", "sap": "smem", "opsa": "hbm", "opsa_f32": "hbm", "opsaw": "hbm",
         "sasaw": "fp64"}
# kernels of this library launched by one forward / one VJP call of every case (sorted input,
# waiting calls, no plan bound): a table builder (HPE / SAP plan, segment offsets) + the main
# kernel; SASAW builds two tables (segment offsets and the grouped coupling) in either call.
# profiles/launch_list_full_bench.md counts the same 26 launches per step.
LAUNCHES = {"hpe": (2, 2), "sap": (2, 2), "opsa": (2, 2), "opsa_f32": (2, 2), "opsaw": (2, 2),
            "sasaw": (3, 3)}

OP_NAMES = {"hpe": "homogeneous_polynomial_evaluation", "sap": "sparse_accumulation_of_products",
            "opsa": "outer_product_scatter_add", "opsaw": "outer_product_scatter_add_with_weights",
            "sasaw": "sparse_accumulation_scatter_add_with_weights"}
# C-ABI argument order (include/mops.h): outputs, grad_output, inputs, indices
ABI = {
    "hpe": (("output", "A", "C", "indices_A"),
            ("grad_A", "grad_output", "A", "C", "indices_A")),
    "sap": (("output", "A", "B", "C", "indices_A", "indices_B", "indices_output"),
            ("grad_A", "grad_B", "grad_output", "A", "B", "C", "indices_A", "indices_B",
             "indices_output")),
    "opsa": (("output", "A", "B", "indices_output"),
             ("grad_A", "grad_B", "grad_output", "A", "B", "indices_output")),
    "opsaw": (("output", "A", "B", "W", "indices_W", "indices_output"),
              ("grad_A", "grad_B", "grad_W", "grad_output", "A", "B", "W", "indices_W",
               "indices_output")),
    "sasaw": (("output", "A", "B", "C", "W", "indices_A", "indices_W_1", "indices_W_2",
               "indices_output_1", "indices_output_2"),
              ("grad_A", "grad_B", "grad_W", "grad_output", "A", "B", "C", "W", "indices_A",
               "indices_W_1", "indices_W_2", "indices_output_1", "indices_output_2")),
}

SCALE = 1          # --scale N divides every batch dimension by N (small cases for ncu captures)
KEEP_ROWS = False  # --keep-rows: --scale leaves the number of output rows / nodes alone


def selected_cases(which):
    return list(CASES) if which == "all" else [which]


def case_sizes(name, divisor=1):
    op, _, kw, _ = CASES[name]
    div = divisor * SCALE
    return {k: (v // (1 if (KEEP_ROWS and k in ROW_KEYS) else div) if k in BATCH_KEYS[op] else v)
            for k, v in kw.items()}


def generate(name, rank, divisor=1):
    op, dtype, _, _ = CASES[name]
    seed = workloads.SEEDS[op] + 1000 * rank
    return workloads.GENERATORS[op](dtype=dtype, seed=seed, **case_sizes(name, divisor))


def output_shape(op, d):
    if op == "hpe":
        return (d["A"].shape[0],)
    if op == "sap":
        return (d["A"].shape[0], d["output_size"])
    if op == "opsa":
        return (d["output_size"], d["A"].shape[1], d["B"].shape[1])
    if op == "opsaw":
        return (d["W"].shape[0], d["A"].shape[1], d["B"].shape[1])
    return (d["W"].shape[0], d["output_size"], d["B"].shape[1])


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
    return getattr(M, OP_NAMES[op]), getattr(M, OP_NAMES[op] + "_vjp")


def named_results(op, out, grads):
    grads = grads if isinstance(grads, tuple) else (grads,)
    names = [n for n in ABI[op][1] if n.startswith("grad_") and n != "grad_output"]
    res = {"output": out}
    res.update(dict(zip(names, grads)))
    return res


def tensor_bytes(args):
    import torch
    return sum(a.numel() * a.element_size() for a in args if isinstance(a, torch.Tensor))


def quantiles(xs):
    xs = sorted(xs)
    q = lambda p: xs[min(len(xs) - 1, int(p * len(xs)))]
    return q(0.5), q(0.1), q(0.9)


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


def bind_to_gpu_numa_node(pci_bus_id):
    """Runs this process on the CPUs of the NUMA node the GPU hangs off, so that the pinned
    host buffers of the end-to-end leg (allocated afterwards) are local to the GPU's PCIe root
    and the copies do not cross the socket interconnect. Best effort; returns the node or None."""
    try:
        dev = pci_bus_id.lower()
        node = int(open(f"/sys/bus/pci/devices/{dev}/numa_node").read().strip())
        if node < 0:
            return None
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            a, _, b = part.partition("-")
            cpus.update(range(int(a), int(b or a) + 1))
        cpus &= set(os.sched_getaffinity(0))
        if not cpus:
            return None
        os.sched_setaffinity(0, cpus)
        return node
    except (OSError, ValueError, AttributeError):
        return None


def physical_gpu_index(local):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local])
        except (ValueError, IndexError):
            return local
    return local


# ------------------------------------------------------------------------------ CPU arm
def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def cpu_impl():
    """The CPU implementation and the number of OpenMP threads it will really use. The thread
    count is set explicitly (a launcher may have exported OMP_NUM_THREADS=1) both in the
    environment, before the library loads, and through the OpenMP runtime it is linked to."""
    want = host_threads()
    os.environ["OMP_NUM_THREADS"] = str(want)
    from oracle import mops_oracle as mo
    impl, kind = (mo.Reference(), "reference") if mo.have_reference() else (mo.Oracle(), "port")
    threads = want
    try:
        gomp = ctypes.CDLL("libgomp.so.1")
        gomp.omp_set_num_threads(ctypes.c_int(want))
        threads = int(gomp.omp_get_max_threads())
    except OSError:
        pass
    return impl, kind, threads


def cpu_pass(impl, name, d):
    """Forward + VJP of one case on the CPU implementation; returns seconds (fwd, vjp)."""
    op = CASES[name][0] if name in CASES else name
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


def cpu_run(impl, kind, threads, names, steps, warmup, full):
    """Times the CPU implementation on every case: at the full configured size (``full``) or
    on a bounded sample (a 1/divisor-size draw of every case)."""
    nbytes, sample = 0, []
    per_op = {n: [0.0, 0.0] for n in names}
    total = 0.0
    # one case at a time, so that only one case's arrays are alive
    for n in names:
        op, _, _, div = CASES[n]
        div = 1 if full else div
        d = generate(n, 0, divisor=div)
        nbytes += workloads.algorithmic_bytes(op, "fwd", d) + workloads.algorithmic_bytes(op, "vjp", d)
        sample.append(f"{n}: 1/{div}")
        for s in range(warmup + steps):
            f, v = cpu_pass(impl, n, d)
            if s >= warmup:
                per_op[n][0] += f
                per_op[n][1] += v
                total += f + v
        per_op[n] += [workloads.algorithmic_bytes(op, "fwd", d), workloads.algorithmic_bytes(op, "vjp", d)]
        del d
    out_per_op = {}
    for n in names:
        f, v, bf, bv = per_op[n]
        out_per_op[n] = {"fwd_ms": f / steps * 1e3, "vjp_ms": v / steps * 1e3,
                         "fwd_GBps": bf / (f / steps) / 1e9, "vjp_GBps": bv / (v / steps) / 1e9}
    what = "the full configured size of every case" if full else \
        "same generators at reduced batch: " + ", ".join(sample)
    return {"value": nbytes / (total / steps) / 1e9, "unit": "GB/s", "cores": threads,
            "kind": kind, "sample": what + f"; {steps} timed step(s) after {warmup} warm-up",
            "ms_per_step": total / steps * 1e3, "per_op": out_per_op}


def cpu_small_configs(impl, kind, names):
    """Call latency of the CPU implementation at the small configurations (full config, as
    of the reference's benchmark programs), through the reference's C ABI on preallocated arrays;
    repetitions sized to about two seconds per call kind."""
    out = {}
    for n in names:
        op, dtype = SMALL_CASES[n]
        d = workloads.GENERATORS[op](dtype=dtype)
        arrays = dict(d)
        arrays["output"] = np.empty(output_shape(op, d), dtype)
        for k in ("A", "B", "W"):
            if k in d:
                arrays["grad_" + k] = np.empty_like(d[k])
        res = {}
        for level, tag in ((0, "fwd"), (1, "vjp")):
            if kind == "reference":
                call = impl.prepared(op, "_vjp" if level else "", dtype,
                                     *[arrays[k] for k in ABI[op][level]])
            else:
                call = (lambda: cpu_pass(impl, op, d))  # the port: forward and VJP together
            call()
            t0 = time.perf_counter()
            call()
            once = time.perf_counter() - t0
            reps = int(max(5, min(100, 2.0 / max(once, 1e-6))))
            ts = []
            for _ in range(reps):
                t0 = time.perf_counter()
                call()
                ts.append((time.perf_counter() - t0) * 1e6)
            m, p10, p90 = quantiles(ts)
            res.update({f"{tag}_us_median": m, f"{tag}_us_p10": p10, f"{tag}_us_p90": p90,
                        f"{tag}_reps": reps})
        out[n] = res
    return out


# ------------------------------------------------------------------------------ GPU, C ABI
def abi_structs(op, level, tensors):
    """ctypes structs of one C-ABI call on CUDA tensors (prototype order)."""
    from mops_b200 import _lib
    return [_lib.make_struct(tensors[k].data_ptr(), tensors[k].shape) for k in ABI[op][level]]


def gpu_small_configs(names, dev):
    """Call latency through the C ABI (mops_cuda_*: device pointers, complete on return) at
    the small configurations: wall-clock time of >= 100 synchronous calls each."""
    import torch
    import mops_b200 as M
    from mops_b200 import _lib
    lib = _lib.library()
    out = {}
    for n in names:
        op, dtype = SMALL_CASES[n]
        d = workloads.GENERATORS[op](dtype=dtype)
        t = {k: torch.from_numpy(v).to(dev) for k, v in d.items() if isinstance(v, np.ndarray)}
        tdt = t["A"].dtype
        t["output"] = torch.empty(output_shape(op, d), dtype=tdt, device=dev)
        for k in ("A", "B", "W"):
            if k in t:
                t["grad_" + k] = torch.empty_like(t[k])
        suffix = "f32" if dtype == np.float32 else "f64"
        res = {}
        for level, tag in ((0, "fwd"), (1, "vjp")):
            fn = getattr(lib, f"mops_cuda_{OP_NAMES[op]}{'_vjp' if level else ''}_{suffix}")
            structs = abi_structs(op, level, t)
            fn.restype, fn.argtypes = ctypes.c_int, [type(s) for s in structs]
            for _ in range(10):
                _lib.check_status(fn(*structs))
            torch.cuda.synchronize()
            ts = []
            for _ in range(200):
                t0 = time.perf_counter()
                status = fn(*structs)
                ts.append((time.perf_counter() - t0) * 1e6)
                _lib.check_status(status)
            m, p10, p90 = quantiles(ts)
            res.update({f"{tag}_us_median": m, f"{tag}_us_p10": p10, f"{tag}_us_p90": p90,
                        f"{tag}_kernels": _lib.last_kernels()})
            # the same calls with a plan bound: tables are built by the first call only
            with M.Plan() as plan:
                for _ in range(10):
                    _lib.check_status(fn(*structs))
                ts = []
                for _ in range(200):
                    t0 = time.perf_counter()
                    status = fn(*structs)
                    ts.append((time.perf_counter() - t0) * 1e6)
                    _lib.check_status(status)
                m, p10, p90 = quantiles(ts)
                res.update({f"{tag}_planned_us_median": m, f"{tag}_planned_us_p10": p10,
                            f"{tag}_planned_us_p90": p90, f"{tag}_plan_tables": plan.tables})
            plan.close()
        res["reps"] = 200
        out[n] = res
    return out


# ------------------------------------------------------------------------------ traffic
def load_traffic():
    path = os.path.join(ROOT, "profiles", "traffic.json")
    return json.load(open(path)) if os.path.exists(path) else {}


def measured(traffic, name, level, launched):
    """(DRAM bytes per launch, shared-memory wavefronts per launch) of the captured kernel,
    scaled to this run's size, or (None, None, why) when the capture is of another
    instantiation than the one this run launched."""
    e = traffic.get(f"{name}/{level}")
    if e is None:
        return None, None, "no capture"
    if not any(e["kernel"] in k for k in launched):
        return None, None, f"capture is of {e['kernel']}, this run launched {'; '.join(launched)}"
    if bool(e.get("keep_rows", False)) != KEEP_ROWS and SCALE != 1:
        return None, None, "capture and run scale their output rows differently"
    f = e["scale"] / SCALE
    wf = e.get("smem_wavefronts")
    return (e["dram_read_bytes"] + e["dram_write_bytes"]) * f, None if wf is None else wf * f, \
        e.get("note")


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
    ap.add_argument("--no-verify", action="store_true",
                    help="skip the oracle check of the timed buffers")
    ap.add_argument("--no-small", action="store_true", help="skip the small-config latencies")
    ap.add_argument("--no-strong", action="store_true",
                    help="with N > 1: skip the strong-scaling leg")
    ap.add_argument("--no-spread", action="store_true",
                    help="skip the per-call median / p10 / p90 measurement")
    ap.add_argument("--quick", action="store_true",
                    help="device-resident timing only (profiling runs)")
    ap.add_argument("--scale", type=int, default=1,
                    help="divide every batch dimension by this (small cases for profiling)")
    ap.add_argument("--keep-rows", action="store_true",
                    help="--scale leaves the number of output rows / nodes alone")
    args = ap.parse_args()
    if args.quick:
        args.no_cpu_baseline = args.no_e2e = args.no_verify = args.no_small = True
        args.no_strong = args.no_spread = True
    # stdout carries exactly one JSON line: everything libraries print there (NCCL's version
    # banner, for one) is sent to stderr, and the line is written to the original descriptor.
    sys.stdout.flush()
    json_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(line):
        sys.stdout.flush()
        os.write(json_fd, (json.dumps(line) + "\n").encode())

    global SCALE, KEEP_ROWS
    SCALE, KEEP_ROWS = max(1, args.scale), args.keep_rows
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    names = selected_cases(args.workload)
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    config = {"workload": "fwd+vjp of " + ",".join(names) + " at the scaled per-GPU sizes" +
              (f" divided by {SCALE}" + (" (rows kept)" if KEEP_ROWS else "") if SCALE > 1 else ""),
              "cases": {n: {**{k: int(v) for k, v in case_sizes(n).items()},
                            "dtype": np.dtype(CASES[n][1]).name} for n in names},
              "sharding": "independent shard per rank (batch rows / output-segment ranges)",
              "cache": "inputs larger than L2 (126 MB) for every case"}

    if args.impl == "reference":
        if rank != 0:
            return 0
        impl, kind, threads = cpu_impl()
        steps, warm = max(1, min(args.steps, 3)), max(1, min(args.warmup, 1))
        r = cpu_run(impl, kind, threads, names, steps, warm, full=(SCALE == 1))
        line = {"impl": "reference", "metric": "algorithmic_GBps_fwd_plus_vjp", "value": r["value"],
                "unit": "GB/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
                "steps_requested": args.steps, "warmup_requested": args.warmup,
                "note": "one step of the CPU implementation at these sizes takes many seconds: "
                        "at most 3 timed steps after 1 warm-up, whatever was requested",
                "ms_per_step": r["ms_per_step"], "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": "f64", "data": "synthetic", "config": config,
                "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
                "e2e": {"value": r["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0},
                "per_op": r["per_op"], "gpu_launches": 0}
        if not args.no_small:
            line["small_configs"] = cpu_small_configs(impl, kind, names)
        emit(line)
        return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py --impl ours needs a CUDA device (no CPU fallback exists)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    props = torch.cuda.get_device_properties(dev)
    try:
        pci = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
    except (AttributeError, TypeError):
        pci = ""
    numa_node = bind_to_gpu_numa_node(pci)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # keep stdout for the one JSON line: NCCL's version / debug lines go to stderr
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        dist.init_process_group("nccl", device_id=dev)
    from mops_b200 import _lib, sharding
    import mops_b200 as M

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- data: pinned host copies (e2e source, checker input) and device-resident copies
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
    launched = {}

    def run_case(n, data, timers=None, reduce=reduce_gw):
        op = CASES[n][0]
        fwd, vjp = api(op)
        if timers is not None:
            timers[0].record()
        out = fwd(*fwd_args(op, data))
        if timers is not None:
            timers[1].record()
            launched[(n, "fwd")] = _lib.last_kernels()
        grads = vjp(*vjp_args(op, data))
        if timers is not None:
            launched[(n, "vjp")] = _lib.last_kernels()
        if reduce and op in ("opsaw", "sasaw") and grads[2].is_cuda:
            # the one exchange step of the path: started here, joined at the end of the step,
            # so that it overlaps the calls that follow (nothing in the step reads grad_W)
            pending.append((dist.all_reduce(grads[2], async_op=True), grads[2]))
        if timers is not None:
            timers[2].record()
        return out, grads

    pending = []

    def join_reductions():
        for work, _ in pending:
            work.wait()
        pending.clear()

    # ---- device-resident timing
    sampler = ClockSampler(physical_gpu_index(local))
    sampler.start()
    for _ in range(args.warmup):
        for n in names:
            run_case(n, devd[n])
        join_reductions()
    barrier()
    events = [[[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in names]
              for _ in range(args.steps)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.enabled = True
    start.record()
    last = {}
    for s in range(args.steps):
        for i, n in enumerate(names):
            run_case(n, devd[n], events[s][i])
        join_reductions()
    stop.record()
    barrier()
    sampler.enabled = False
    t_ms = max_over_ranks(start.elapsed_time(stop))
    per_op_ms = {n: [statistics.mean(events[s][i][0].elapsed_time(events[s][i][1])
                                     for s in range(args.steps)),
                     statistics.mean(events[s][i][1].elapsed_time(events[s][i][2])
                                     for s in range(args.steps))] for i, n in enumerate(names)}
    step_bytes = sum(sum(nbytes[n]) for n in names)
    value = step_bytes * world * args.steps / (t_ms / 1e3) / 1e9

    # ---- parity, outside the timed region: one more (untimed) pass over the very input buffers
    # that were timed, one case at a time, its results checked against the CPU oracle. (Keeping
    # the timed steps' own results alive would make the allocator fetch new memory inside the
    # timed region.)
    verified = {}
    if not args.no_verify and rank == 0 and SCALE == 1:
        for n in names:
            last[n] = None
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import subrange
        from oracle.mops_oracle import Oracle
        oracle = Oracle()
        for n in names:
            op = CASES[n][0]
            d = {k: (v.numpy() if isinstance(v, torch.Tensor) else v) for k, v in host[n].items()}
            last[n] = run_case(n, devd[n], reduce=False)
            results = named_results(op, *last[n])

            def library_vjp(sub, op=op):
                t = {k: (torch.from_numpy(np.ascontiguousarray(v)).to(dev)
                         if isinstance(v, np.ndarray) else v) for k, v in sub.items()}
                return api(op)[1](*vjp_args(op, t))[2]

            try:
                report = subrange.check_case(oracle, op, d, results, inputs=devd[n],
                                             library_vjp=library_vjp)
                worst = max((r["max_abs_err"] / max(r["scale"], 1e-300) for r in report
                             if r["n"] > 1), default=0.0)
                verified[n] = {"verified": True, "comparisons": len(report),
                               "worst_rel_to_max": worst}
            except subrange.Mismatch as e:
                verified[n] = {"verified": False, "error": str(e)}
            last[n] = None
            del results
    last.clear()

    # ---- spread of every call: the same calls again, each one between its own pair of events
    # (outside the timed step; rank 0's view)
    spread = {}
    if not args.no_spread:
        reps = 20
        for n in names:
            ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(reps)]
            for r in range(reps):
                run_case(n, devd[n], ev[r], reduce=False)
            torch.cuda.synchronize()
            fm, f10, f90 = quantiles([e[0].elapsed_time(e[1]) for e in ev])
            vm, v10, v90 = quantiles([e[1].elapsed_time(e[2]) for e in ev])
            spread[n] = {"reps": reps, "fwd_ms_median": fm, "fwd_ms_p10": f10, "fwd_ms_p90": f90,
                         "vjp_ms_median": vm, "vjp_ms_p10": v10, "vjp_ms_p90": v90}

    # ---- strong scaling: all ranks split rank 0's problem
    strong = None
    if world > 1 and not args.no_strong:
        strong = {}
        for n in names:
            op = CASES[n][0]
            # rank 0's device-resident operands go to every rank over NCCL
            full = {}
            meta = [None]
            if rank == 0:
                meta = [{k: ((tuple(v.shape), str(v.dtype)) if isinstance(v, torch.Tensor) else v)
                         for k, v in devd[n].items()}]
            dist.broadcast_object_list(meta, src=0)
            for k, m in meta[0].items():
                if isinstance(m, tuple):
                    if rank == 0:
                        full[k] = devd[n][k]
                    else:
                        full[k] = torch.empty(m[0], dtype=getattr(torch, m[1].replace("torch.", "")),
                                              device=dev)
                    dist.broadcast(full[k], src=0)
                else:
                    full[k] = m
            # cut: batch rows (HPE, SAP) or output-row ranges that balance the entries
            if op in ("hpe", "sap"):
                a, b = sharding.batch_range(full["A"].shape[0], world, rank)
                per_row = ("A", "B", "grad_output")
                shard = {k: (v[a:b].clone() if k in per_row and isinstance(v, torch.Tensor)
                             else v) for k, v in full.items()}
            else:
                key = "indices_output_1" if op == "sasaw" else "indices_output"
                n_rows = full["output_size"] if op == "opsa" else full["W"].shape[0]
                cuts = [None]
                if rank == 0:
                    cuts = [sharding.segment_cuts(host[n][key].numpy(), n_rows, world)]
                dist.broadcast_object_list(cuts, src=0)
                rho, eps = cuts[0]
                lo, hi = eps[rank], eps[rank + 1]
                per_entry = ("A", "B", key, "indices_W", "indices_W_1")
                # every rank holds its shard in buffers of its own (a slice of the full array
                # may start at an address that is no multiple of 16 bytes, which the streaming
                # kernels' bulk copies do not take: such views run on the slower kernels)
                shard = {k: (v[lo:hi].clone() if k in per_entry and isinstance(v, torch.Tensor)
                             else v) for k, v in full.items()}
                if op == "opsa":  # the output is sharded by rows: rebase the scatter index
                    shard[key] = shard[key] - rho[rank]
                    shard["output_size"] = rho[rank + 1] - rho[rank]
                    shard["grad_output"] = full["grad_output"][rho[rank]:rho[rank + 1]].clone()
            del full
            for _ in range(2):
                run_case(n, shard, reduce=False)
            barrier()
            ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
            for s in range(args.steps):
                run_case(n, shard, ev[s], reduce=False)
            torch.cuda.synchronize()
            f = max_over_ranks(statistics.mean(e[0].elapsed_time(e[1]) for e in ev))
            v = max_over_ranks(statistics.mean(e[1].elapsed_time(e[2]) for e in ev))
            entry = {"fwd_ms_max_over_ranks": f, "vjp_ms_max_over_ranks": v}
            if op in ("opsaw", "sasaw"):
                # the one exchange step: the partial grad_W of every rank, summed
                _, grads = run_case(n, shard, reduce=False)
                barrier()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                dist.all_reduce(grads[2])
                e1.record()
                torch.cuda.synchronize()
                entry["grad_W_allreduce_ms"] = max_over_ranks(e0.elapsed_time(e1))
                entry["grad_W_bytes"] = grads[2].numel() * grads[2].element_size()
            strong[n] = entry
            del shard
        barrier()

    # ---- end to end: the public API on pinned host arrays inside a HostQueue
    e2e = None
    if not args.no_e2e:
        def e2e_step():
            keep = []
            with M.HostQueue():
                for n in names:
                    keep.append(run_case(n, host[n], reduce=False))
            return keep

        torch.cuda.synchronize()
        for _ in range(3):
            res = e2e_step()
        h2d = sum(tensor_bytes(tuple(v for v in host[n].values() if isinstance(v, torch.Tensor)))
                  for n in names)
        d2h = sum(tensor_bytes((out,) + tuple(g if isinstance(g, tuple) else (g,)))
                  for out, g in res)
        del res
        barrier()
        t0 = time.perf_counter()
        e2e_steps = max(1, args.steps)
        each = []
        for _ in range(e2e_steps):
            t1 = time.perf_counter()
            e2e_step()  # returns when every result is in host memory
            each.append((time.perf_counter() - t1) * 1e3)
        torch.cuda.synchronize()
        t_e2e = max_over_ranks(time.perf_counter() - t0)
        e2e = {"value": step_bytes * world * e2e_steps / t_e2e / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": t_e2e / e2e_steps * 1e3, "steps": e2e_steps,
               "ms_per_step_median_rank0": statistics.median(each),
               "ms_per_step_max_rank0": max(each),
               "api": "mops_b200.<op>(pinned host arrays) inside mops_b200.HostQueue",
               "host_numa_node": numa_node}
    sampler.stop()

    small = None
    if not args.no_small and rank == 0 and SCALE == 1:
        small = gpu_small_configs(names, dev)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return 0

    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    else:
        peak, peak_src = FALLBACK_HBM_GBS, "fallback"
    clocks = sampler.summary()
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    clk_hz = (clocks["sm_mhz"] or clocks["sm_max_mhz"] or 1965.0) * 1e6
    traffic = load_traffic()
    per_op = {}
    dominant = None
    for n in names:
        op = CASES[n][0]
        f_ms, v_ms = per_op_ms[n]
        bf, bv = nbytes[n]
        items = devd[n]["A"].shape[0]
        entry = {"fwd_ms": f_ms, "vjp_ms": v_ms, "fwd_GBps": bf / f_ms / 1e6,
                 "vjp_GBps": bv / v_ms / 1e6, "fwd_frac_of_hbm": bf / f_ms / 1e6 / peak,
                 "vjp_frac_of_hbm": bv / v_ms / 1e6 / peak,
                 "fwd_items_per_s": items / f_ms * 1e3, "vjp_items_per_s": items / v_ms * 1e3,
                 "fwd_bytes": bf, "vjp_bytes": bv, "bound": BOUND[n], **spread.get(n, {})}
        for lvl, ms, b in (("fwd", f_ms, bf), ("vjp", v_ms, bv)):
            k = launched.get((n, lvl), [])
            entry[f"{lvl}_kernels"] = k
            dram, wavefronts, note = measured(traffic, n, lvl, k)
            entry[f"{lvl}_traffic"] = dram
            if note:
                entry[f"{lvl}_traffic_note"] = note
            if dram is not None:
                entry[f"{lvl}_traffic_frac_of_hbm"] = dram / ms / 1e6 / peak
            if BOUND[n] == "hbm":
                entry[f"{lvl}_frac_of_bound"] = b / ms / 1e6 / peak
            elif BOUND[n] == "smem":
                # one shared-memory wavefront per clock per SM
                entry[f"{lvl}_frac_of_bound"] = None if wavefronts is None else \
                    wavefronts / (sms * clk_hz * ms / 1e3)
            else:
                hd = {k2: (v.numpy() if isinstance(v, torch.Tensor) else v)
                      for k2, v in host[n].items()}
                flops = workloads.useful_flops(op, lvl, hd)
                entry[f"{lvl}_useful_GFLOP"] = flops / 1e9
                entry[f"{lvl}_frac_of_bound"] = flops / (ms / 1e3) / \
                    (sms * FP64_FLOP_PER_CLK_PER_SM * clk_hz)
            if dominant is None or ms > dominant[2]:
                dominant = (n, lvl, ms, b)
        if n in verified:
            entry.update(verified[n])
        if strong is not None and n in strong:
            s = strong[n]
            entry["strong"] = {**s, "n_gpus": world,
                               "fwd_speedup_vs_1gpu": f_ms / s["fwd_ms_max_over_ranks"],
                               "vjp_speedup_vs_1gpu": v_ms / s["vjp_ms_max_over_ranks"]}
        per_op[n] = entry
    dn, dl, dms, db = dominant
    roofline = {"bound": "hbm", "kernel": f"{dn} {dl}: " + "; ".join(launched.get((dn, dl), [])),
                "achieved": db / dms / 1e6, "peak": peak,
                "peak_source": peak_src, "unit": "GB/s", "frac": db / dms / 1e6 / peak,
                "traffic": per_op[dn][f"{dl}_traffic"],
                "binding_resource": BOUND[dn],
                "frac_of_binding_resource": per_op[dn][f"{dl}_frac_of_bound"]}
    launches = sum(sum(LAUNCHES[n]) for n in names) * args.steps
    line = {"metric": "algorithmic_GBps_fwd_plus_vjp", "value": value, "unit": "GB/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": t_ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f64" if names != ["opsa_f32"] else "f32",
            "data": "synthetic", "config": config, "roofline": roofline, "per_op": per_op,
            "clocks": clocks, "gpu_launches": launches, "peak_hbm_GBps": peak,
            "fp64_peak_TFLOPs": sms * FP64_FLOP_PER_CLK_PER_SM * clk_hz / 1e12}
    if verified:
        line["verified"] = all(v["verified"] for v in verified.values())
    if e2e is not None:
        line["e2e"] = e2e
    if small is not None:
        line["small_configs"] = small
    if world == 1 and not args.no_cpu_baseline:
        impl, kind, threads = cpu_impl()
        r = cpu_run(impl, kind, threads, names, 1, 1, full=False)
        line["cpu_baseline"] = {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")}
        line["cpu_baseline"]["per_op"] = r["per_op"]
    emit(line)
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
