#!/usr/bin/env python
"""Headline benchmark: HBM streaming bandwidth (8 GiB read / copy / triad) on N B200s.

A *step* is one pass of the three STREAM kernels over 8 GiB fp32 buffers:
read (8 GiB), copy (16 GiB), triad a = b + 1.5*c (24 GiB) -> 48 GiB of
algorithmic HBM traffic per step.  `value` is whole-job GB/s with the buffers
resident in HBM; `e2e` is the same three kernels driven through the C ABI from
pinned HOST buffers (H2D of b and c and a D2H of the read checksum inside the
timed region).  The tensor-core and GEMM rows of the same backend are measured
after the timed region and reported under "rows" (they explain the headline
metric's "TFLOPS/TOPS per dtype" part; each carries its own roofline fraction).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Multi-GPU (launched by torch.distributed.run, one rank per GPU): every rank runs
the identical, independent workload on its own buffers -- replicas only, no
data-path collective; torch.distributed is used for the start barrier and the
max-over-ranks of the device-timed duration.

`e2e_plugin` wall-clocks the product's own plugin call, `clpeak_launch --cuda
--global-memory-bandwidth` in libclpeak_ffi.so (allocation, seeded fills, kernels, the backend's
host checks, result rows), on rank 0; with N > 1 it names all N GPUs, which runs the C++
thread-per-GPU driver while the other ranks idle.

The oracle (oracle/) appears here in two roles only: as the CPU baseline, and as the checker
of results this file times (sampled GEMM elements, the config-1b sums, the pointer-chase walk).
It is never the thing measured.

--impl reference times the reference project's own CPU implementation of the
same metric (its native-CPU backend's global_memory_bandwidth read/copy/triad,
built unchanged into oracle/_ref/clpeak_ref) on the host cores; when that
binary is absent it falls back to the oracle's C port of the three passes.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import re
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

GIB = 1 << 30
METRIC = "global_memory_bandwidth (HBM stream read+copy+triad)"
UNIT = "GB/s"
SPEC = {  # NVIDIA HGX B200 datasheet, per GPU, dense (the 8-GPU figures divided by 8)
    "hbm_gbs": 8000.0, "bf16_tflops": 2250.0, "fp16_tflops": 2250.0, "fp8_tflops": 4500.0,
    "int8_tops": 4500.0, "fp4_tflops": 9000.0,
}


def measured_peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic(kernel: str):
    """Per-launch DRAM bytes of `kernel` from the committed ncu summary (None if not captured)."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    return json.loads(p.read_text()).get(kernel)


# ---------------------------------------------------------------------------------
# clock sampling during the timed region
# ---------------------------------------------------------------------------------

class ClockSampler:
    """SM clock, power and throttle reasons sampled DURING the timed region: an NVML thread (10 ms period),
    or `nvidia-smi -lms 100` where the NVML binding is missing.  Reading only; nothing is set."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # nvmlClocksEventReason* bits
    BITS = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}

    def __init__(self, gpu_index: int, uuid: str | None = None):
        self.gpu = gpu_index
        self.uuid = uuid
        self.proc = None
        self.lines: list[str] = []
        self.samples: list[tuple] = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = None
            if self.uuid:
                try:
                    h = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + self.uuid).encode() if not self.uuid.startswith("GPU-") else self.uuid.encode())
                except Exception:
                    h = None
            if h is None:
                h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.nvml = (pynvml, h)
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _poll(self):
        nv, h = self.nvml
        smax = None
        while not self.stop_flag.is_set():
            try:
                if smax is None:
                    smax = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
                sm = nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)
                pw = nv.nvmlDeviceGetPowerUsage(h) / 1000.0
                try:
                    rs = nv.nvmlDeviceGetCurrentClocksEventReasons(h)
                except Exception:
                    rs = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                self.samples.append((float(sm), float(smax), pw, int(rs)))
            except Exception:
                pass
            time.sleep(0.01)

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        sm, smax, reasons, power = [], [], set(), []
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            for a, b, c, r in self.samples:
                sm.append(a); smax.append(b); power.append(c)
                for name, bit in self.BITS.items():
                    if r & bit:
                        reasons.add(name)
            source = "nvml, 10 ms period"
        elif self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            for ln in self.lines:
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); smax.append(float(f[2])); power.append(float(f[3]))
                except ValueError:
                    continue
                for name, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            source = "nvidia-smi -lms 100"
        else:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no NVML binding and no nvidia-smi"]}
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "reasons": sorted(reasons),
                "source": source}


# ---------------------------------------------------------------------------------
# reference arm / CPU baseline
# ---------------------------------------------------------------------------------

def harmonic_stream(read, copy, triad):
    """Aggregate GB/s of one read+copy+triad pass over equal arrays (1:2:3 bytes)."""
    return 6.0 / (1.0 / read + 2.0 / copy + 3.0 / triad)


def run_reference_cpu(max_time_ms: int):
    """The reference's own CPU backend (built unchanged by oracle/Makefile `ref`)."""
    exe = ROOT / "oracle" / "_ref" / "clpeak_ref"
    if not exe.exists():
        return None
    with tempfile.TemporaryDirectory() as td:
        xml = Path(td) / "ref.xml"
        t0 = time.time()
        r = subprocess.run([str(exe), "--cpu", "--global-memory-bandwidth", "--max-time-cpu", str(max_time_ms),
                            "--xml-file", str(xml)], capture_output=True, text=True, timeout=600)
        wall = time.time() - t0
        if r.returncode != 0 or not xml.exists():
            return None
        txt = xml.read_text()
    vals = {}
    for name in ("read", "copy", "triad"):
        m = re.search(rf'<metric name="{name}"[^>]*>([0-9.]+)</metric>', txt)
        if not m:
            return None
        vals[name] = float(m.group(1))
    cores = re.search(r'<prop name="Cores" value="([^"]*)"', txt)
    return {"rows": vals, "value": harmonic_stream(vals["read"], vals["copy"], vals["triad"]),
            "cores": os.cpu_count(), "cores_prop": cores.group(1) if cores else "", "wall_s": wall,
            "kind": "reference",
            "sample": f"reference CPU backend global_memory_bandwidth read/copy/triad on its own array sizing "
                      f"(<=512 MiB per array), all logical cores, --max-time-cpu {max_time_ms} ms, gcc build"}


def run_reference_cpu_pairs(max_time_ms: int):
    """The reference CPU backend's rows that pair with configs 1a / 2b: fp32 compute and memory latency."""
    exe = ROOT / "oracle" / "_ref" / "clpeak_ref"
    if not exe.exists():
        return None
    with tempfile.TemporaryDirectory() as td:
        xml = Path(td) / "ref.xml"
        r = subprocess.run([str(exe), "--cpu", "--single-precision-compute", "--memory-latency", "--max-time-cpu",
                            str(max_time_ms), "--xml-file", str(xml)], capture_output=True, text=True, timeout=600)
        if r.returncode != 0 or not xml.exists():
            return None
        txt = xml.read_text()
    out = {}
    for test, metrics in re.findall(r'<test name="([^"]+)"[^>]*>(.*?)</test>', txt, flags=re.S):
        for name, val in re.findall(r'<metric name="([^"]+)"[^>]*>([0-9.]+)</metric>', metrics):
            out[f"{test}/{name}"] = float(val)
    return out


def run_reference_cuda_kernels(budget_us: int, row_filter: str = ""):
    """The reference's own CUDA kernels on this GPU.

    `make -C oracle refcuda` compiles the reference's src/cuda/cuda_kernels/*.cu (unchanged, from the reference
    checkout) to sm_100a cubins and builds oracle/ref_cuda_runner.cpp, a launcher that follows the reference
    host side's geometry, calibration and accounting.  Returns {"test/label": value} in the reference's units,
    or None when the prebuilt files are not there.
    """
    exe = ROOT / "oracle" / "_ref" / "ref_cuda_runner"
    cubins = ROOT / "oracle" / "_ref" / "cuda"
    if not exe.exists() or not cubins.is_dir():
        return None
    try:
        cmd = [str(exe), str(cubins), "--budget-us", str(budget_us)] + (["--filter", row_filter] if row_filter else [])
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    except (OSError, subprocess.TimeoutExpired):
        return None
    if r.returncode != 0:
        return {"error": r.stderr.strip()[-300:]}
    out = {}
    for ln in r.stdout.splitlines():
        try:
            row = json.loads(ln)
        except ValueError:
            continue
        key = f"{row['test']}/{row['label']}"
        out[key] = row.get("value", row.get("skipped"))
    out["unit_note"] = ("gbps / gflops / gops / tflops / tops / us as the reference reports each row; its kernels, "
                        f"compiled for sm_100a, launched with its geometry; {budget_us} us timed per row")
    return out


def run_port_cpu(seconds: float):
    """Fallback: the oracle's C port of the three passes on 256 MiB arrays."""
    import numpy as np
    from oracle import binding as ob
    n = (256 << 20) // 4
    threads = os.cpu_count() or 1
    a = np.zeros(n, dtype=np.float32)
    b = ob.fill_f32(n, 101, 0)
    c = ob.fill_f32(n, 102, 0)
    rows = {}
    t0 = time.time()
    for kind, name, mult in ((0, "read", 1), (1, "copy", 2), (2, "triad", 3)):
        sec = ob.lib().orc_stream_pass_mt(kind, ob.ptr(a), ob.ptr(b), ob.ptr(c), n, threads, 1, None)
        passes = max(1, int(seconds / 3.0 / max(sec, 1e-6)))
        sec = ob.lib().orc_stream_pass_mt(kind, ob.ptr(a), ob.ptr(b), ob.ptr(c), n, threads, passes, None)
        rows[name] = mult * n * 4 / sec / 1e9
    return {"rows": rows, "value": harmonic_stream(rows["read"], rows["copy"], rows["triad"]), "cores": threads,
            "wall_s": time.time() - t0, "kind": "port",
            "sample": "oracle C port of read/copy/triad, 256 MiB arrays, one pthread per logical core"}


def run_plugin(N, devices, extra):
    """One blocking clpeak_launch through libclpeak_ffi.so; returns rc, wall seconds and the metric events."""
    lib = N.ffi()
    events = []

    def cb(_ud, ptr):
        events.append(json.loads(C.string_at(ptr).decode()))
        lib.clpeak_free_string(ptr)                 # the callee owns the event string

    keep = N.EVENT_CALLBACK(cb)
    argv = ["clpeak", "--cuda", "--cuda-device", ",".join(str(d) for d in devices)] + list(extra)
    arr = (C.c_char_p * len(argv))(*[a.encode() for a in argv])
    t0 = time.time()
    rc = lib.clpeak_launch(len(argv), arr, C.cast(keep, C.c_void_p), None)
    wall = time.time() - t0
    per_device = {}
    for e in events:
        if e.get("t") == "metric":
            per_device.setdefault(e["device"], {})[f"{e['test']}/{e['metric']}"] = (
                e["value"] if e["status"] == "ok" else f"{e['status']}: {e['reason']}")
    return {"rc": rc, "wall_s": wall, "argv": " ".join(argv[1:]), "devices": per_device,
            "notes": [e["message"].strip() for e in events if e.get("t") == "note"]}


def plugin_leg(N, world):
    """clpeak_launch --cuda --global-memory-bandwidth on the real GPU(s), wall-clocked."""
    out = run_plugin(N, list(range(world)), ["--global-memory-bandwidth", "--max-time", "200"])
    names = list(out["devices"])
    key = "global_memory_bandwidth/"
    if names:
        first = out["devices"][names[0]]
        try:
            out["value"] = harmonic_stream(first[key + "read"], first[key + "copy"], first[key + "triad"])
            out["unit"] = UNIT
        except (KeyError, TypeError):
            out["value"] = None
    if world > 1 and len(names) == world + 1:
        agg = out["devices"][names[-1]]
        singles = [out["devices"][n] for n in names[:-1]]
        out["box_aggregate_over_sum_of_gpus"] = {
            m.split("/")[1]: agg[m] / sum(d[m] for d in singles)
            for m in (key + "read", key + "copy", key + "triad")
            if isinstance(agg.get(m), float) and all(isinstance(d.get(m), float) for d in singles)}
    return out


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    per_step_ms = 400
    vals, t_steps = [], []
    res = None
    for i in range(args.warmup + args.steps):
        t0 = time.time()
        res = run_reference_cpu(per_step_ms) or run_port_cpu(per_step_ms * 3 / 1000.0)
        if i >= args.warmup:
            vals.append(res["value"]); t_steps.append(time.time() - t0)
    value = sum(vals) / len(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * sum(t_steps) / len(t_steps),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "hbm_stream_read_copy_triad (reference CPU backend arrays, host DRAM)",
                   "note": "CPU run of the same metric; array size is the reference's own (<=512 MiB)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": res["cores"], "kind": res["kind"],
                         "sample": res["sample"]},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "rows_last_step": res["rows"],
        "reference_cuda_kernels_on_this_gpu": run_reference_cuda_kernels(200000, "global_memory_bandwidth"),
    }
    print(json.dumps(line), flush=True)
    return 0


# ---------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--size-gib", type=float, default=8.0, help="bytes per array (default: the 8 GiB of the config)")
    ap.add_argument("--no-rows", action="store_true", help="skip the tensor-core / GEMM rows")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        return reference_arm(args)

    import numpy as np
    import torch
    from clpeak_b200 import native as N

    from clpeak_b200.replicas import Replicas

    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    reps = Replicas("nccl", torch.device("cuda", local))
    rank, world = reps.rank, reps.world
    K = N.kernels()                      # raises if the CUDA library is missing
    K.clpk_set_device(local)
    stream = torch.cuda.current_stream().cuda_stream

    n_bytes = int(args.size_gib * GIB) // 4096 * 4096
    n_floats = n_bytes // 4
    a, b, c = (torch.empty(n_floats, dtype=torch.float32, device="cuda") for _ in range(3))
    for i, t in enumerate((a, b, c)):
        K.clpk_fill_f32(t.data_ptr(), n_floats, 100 + i, N.DIST_UNIFORM01, 0.0, 1.0, stream)

    grids = {}
    for v in N.STREAM_VARIANTS:
        g = C.c_int(0)
        K.clpk_stream_read_grid(v, C.byref(g))
        grids[v] = g.value
    parts = torch.empty(max(grids.values()), dtype=torch.int32, device="cuda")

    ops = {
        "read": lambda v: K.clpk_stream_read(v, b.data_ptr(), n_bytes, parts.data_ptr(), stream),
        "copy": lambda v: K.clpk_stream_copy(v, a.data_ptr(), c.data_ptr(), n_bytes, stream),
        "triad": lambda v: K.clpk_stream_triad(v, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.5, n_floats, stream),
    }
    alg_bytes = {"read": n_bytes, "copy": 2 * n_bytes, "triad": 3 * n_bytes}

    def ev():
        return torch.cuda.Event(enable_timing=True)

    def time_once(fn, reps=3):
        fn(); torch.cuda.synchronize()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    # pick the faster flavour of each kernel once, outside the timed region
    variant = {}
    for name, fn in ops.items():
        t = {v: time_once(lambda v=v: fn(v)) for v in N.STREAM_VARIANTS}
        variant[name] = min(t, key=t.get)
    vname = {N.STREAM_LDG: "ldg", N.STREAM_TMA: "tma", N.STREAM_WIDE: "wide"}

    def step(events=None):
        for i, name in enumerate(("read", "copy", "triad")):
            if events is not None:
                events[i].record()
            ops[name](variant[name])
        if events is not None:
            events[3].record()

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    st = C.c_uint32(0)
    K.clpk_stream_status(C.byref(st), stream)

    try:
        uuid = str(torch.cuda.get_device_properties(local).uuid)
    except Exception:
        uuid = None
    sampler = ClockSampler(local, uuid)
    if rank == 0:
        sampler.start()
    per_step_events = [[ev() for _ in range(4)] for _ in range(args.steps)]
    reps.barrier()
    torch.cuda.synchronize()
    for k in range(args.steps):
        step(per_step_events[k])
    torch.cuda.synchronize()
    reps.barrier()
    total_ms = per_step_events[0][0].elapsed_time(per_step_events[-1][3])
    clocks = sampler.stop() if rank == 0 else None
    K.clpk_stream_status(C.byref(st), stream)      # raises on a device-side timeout

    kern_ms = {name: sum(e[i].elapsed_time(e[i + 1]) for e in per_step_events) / args.steps
               for i, name in enumerate(("read", "copy", "triad"))}
    bytes_per_step = sum(alg_bytes.values())
    value, total_ms = reps.whole_job_rate(bytes_per_step * args.steps, total_ms)
    value /= 1e9
    ms_per_step = total_ms / args.steps

    # checksum of the step's result vs a second, independent pass (copy then read-back XOR)
    read_xor = int(np.bitwise_xor.reduce(parts[:grids[variant["read"]]].cpu().numpy().view(np.uint32)))

    # ---- the timed kernels' results at full size, against torch's own elementwise kernels (untimed) ----
    def xor_words(t):
        x = t.view(torch.int64)
        while x.numel() > 1:
            h = x.numel() // 2
            y = x[:h] ^ x[h:2 * h]
            if x.numel() & 1:
                y[0] ^= x[-1]
            x = y
        w = int(x.item()) & 0xFFFFFFFFFFFFFFFF
        return (w ^ (w >> 32)) & 0xFFFFFFFF

    checks = {"read_checksum_equals_xor_of_b": read_xor == xor_words(b)}
    ops["copy"](variant["copy"])
    torch.cuda.synchronize()
    checks["copy_equals_source_bitwise"] = bool(torch.equal(a.view(torch.int32), c.view(torch.int32)))
    ops["triad"](variant["triad"])
    torch.cuda.synchronize()
    ok = True
    piece = 1 << 28                                   # 1 GiB of floats at a time
    for off in range(0, n_floats, piece):
        t = c[off:off + piece] * 1.5                  # separate multiply and add, as the kernel and the oracle do
        t += b[off:off + piece]
        ok = ok and bool(torch.equal(t.view(torch.int32), a[off:off + piece].view(torch.int32)))
        del t
    checks["triad_equals_b_plus_s_times_c_bitwise"] = ok
    checks["elements_per_array"] = n_floats
    failed = reps.max_over_ranks(0.0 if all(v for k, v in checks.items() if k != "elements_per_array") else 1.0)
    checks["all_ranks"] = failed == 0.0
    torch.cuda.empty_cache()

    # ---- end to end: host buffers through the C ABI -------------------------------------------
    e2e = None
    if not args.no_e2e:
        avail_kb = 0
        for ln in open("/proc/meminfo"):
            if ln.startswith("MemAvailable"):
                avail_kb = int(ln.split()[1])
        local_world = reps.local_world
        budget = avail_kb * 1024 // (6 * max(local_world, 1))     # per pinned array, per rank
        chunk = min(n_bytes, max(256 << 20, budget // (1 << 20) * (1 << 20)))
        hb = torch.empty(chunk // 4, dtype=torch.float32).pin_memory()
        hc = torch.empty(chunk // 4, dtype=torch.float32).pin_memory()
        hb.copy_(b[:chunk // 4]); hc.copy_(c[:chunk // 4])
        hparts = torch.empty(parts.numel(), dtype=torch.int32).pin_memory()

        def e2e_step():
            off = 0
            while off < n_bytes:
                m = min(chunk, n_bytes - off)
                K.clpk_memcpy_h2d(b.data_ptr() + off, hb.data_ptr(), m, stream)
                K.clpk_memcpy_h2d(c.data_ptr() + off, hc.data_ptr(), m, stream)
                off += m
            step()
            K.clpk_memcpy_d2h(hparts.data_ptr(), parts.data_ptr(), parts.numel() * 4, stream)
            K.clpk_stream_sync(stream)

        e2e_steps = max(3, min(args.steps, 10))
        e2e_step()
        reps.barrier()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(e2e_steps):
            e2e_step()
        e1.record(); torch.cuda.synchronize()
        e2e_rate, e2e_ms = reps.whole_job_rate(bytes_per_step * e2e_steps, e0.elapsed_time(e1))
        e2e = {"value": e2e_rate / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": 2 * n_bytes, "d2h_bytes_per_step": parts.numel() * 4,
               "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
               "host_buffer": "pinned, full size" if chunk == n_bytes else f"pinned {chunk >> 20} MiB chunk reused"}
        del hb, hc

    # ---- the other rows of the metric (per-dtype tensor peaks, GEMM) -----------------------------
    # Every replica runs them at the same moment (barrier before each timing, slowest replica's time), so at
    # N > 1 a row is the per-GPU rate with all GPUs of the box busy, and "box" = N x that.
    rows = None
    if not args.no_rows:
        del a, c
        torch.cuda.empty_cache()

        def time_together(fn, reps_=3):
            fn(); torch.cuda.synchronize()
            reps.barrier()
            e0, e1 = ev(), ev()
            e0.record()
            for _ in range(reps_):
                fn()
            e1.record(); torch.cuda.synchronize()
            return reps.max_over_ranks(e0.elapsed_time(e1) / reps_)

        def clocked(fn, est_ms, seconds):
            """A loop of at least `seconds` with the SM clock sampled under it: (ms per launch, median MHz)."""
            n = max(5, int(seconds * 1e3 / max(est_ms, 1e-3)))
            smp = ClockSampler(local, uuid)
            smp.start()
            ms = time_together(fn, n)
            c = smp.stop()
            return ms, c.get("sm_mhz"), c.get("reasons")

        rows = measure_rows(K, N, torch, stream, lambda fn, reps=3: time_together(fn, reps), world, clocked,
                            all_ranks_ok=lambda ok: reps.max_over_ranks(0.0 if ok else 1.0) == 0.0)
        if world == 1:
            rows.update(measure_small_rows(K, N, torch, stream, time_once))

    # ---- the plugin call itself (rank 0; the other ranks have freed their buffers and wait) ----------------
    plugin = None
    if not args.no_e2e:
        del b, parts
        torch.cuda.empty_cache()
        reps.barrier()
        torch.cuda.synchronize()
        if rank == 0:
            try:
                plugin = plugin_leg(N, world)
            except Exception as e:                      # a missing library is an error of the build, say so
                plugin = {"error": repr(e)[:300]}
        reps.host_barrier()                             # a CPU-side wait: an NCCL barrier would spin on the other GPUs

    if rank != 0:
        reps.close()
        return 0

    peaks = measured_peaks()
    dom = max(kern_ms, key=kern_ms.get)
    kernel_symbol = f"stream_{dom}_{vname[variant[dom]]}"
    achieved = alg_bytes[dom] / (kern_ms[dom] * 1e6)
    cpu = (run_reference_cpu(2000) or run_port_cpu(12.0)) if world == 1 else None
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"hbm_stream_read_copy_triad_{args.size_gib:g}GiB_fp32 (configs[1](a) of the benchmark definition)",
                   "bytes_per_array": n_bytes, "algorithmic_bytes_per_step": bytes_per_step,
                   "variants": {k: vname[v] for k, v in variant.items()},
                   "l2": "inputs (3 x %.0f GiB) far exceed the 126 MB L2; no flush needed" % args.size_gib,
                   "parallelism": f"replicas x{world}, no collective"},
        "kernels": {k: {"ms": kern_ms[k], "GBps": alg_bytes[k] / (kern_ms[k] * 1e6),
                        "frac_of_spec_8TBps": alg_bytes[k] / (kern_ms[k] * 1e6) / SPEC["hbm_gbs"]} for k in kern_ms},
        "roofline": {"bound": "hbm", "kernel": kernel_symbol, "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "peak_source": f"of {peaks['source']}", "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "frac_of_spec": achieved / SPEC["hbm_gbs"], "traffic": ncu_traffic(kernel_symbol)},
        "cpu_baseline": ({"value": cpu["value"], "unit": UNIT, "cores": cpu["cores"], "kind": cpu["kind"],
                          "sample": cpu["sample"], "rows": cpu["rows"],
                          "other_reference_cpu_rows": (run_reference_cpu_pairs(500) if not args.no_rows else None),
                          # the same baseline leg also times the reference's own CUDA kernels on this GPU
                          "reference_cuda_kernels_on_this_gpu": (run_reference_cuda_kernels(200000)
                                                                 if not args.no_rows else None)}
                         if cpu else None),
        "e2e": e2e, "e2e_plugin": plugin, "gpu_launches": 3 * args.steps, "clocks": clocks, "read_checksum": read_xor, "verified_at_full_size": checks,
        "rows": rows, "spec_peaks_per_gpu": SPEC,
    }
    print(json.dumps(line), flush=True)
    reps.close()
    return 0


def measure_small_rows(K, N, torch, stream, time_once):
    """Configs 1a, 1b, 2b, 2c on this GPU (rank 0, one GPU): chain, read-and-sum, pointer chase, launch roundtrip.
    The results of 1b and 2b are compared exactly with the oracle's replay at the full configured size."""
    import numpy as np
    from oracle import binding as orc            # checker only
    rows = {}
    items = 1 << 20
    out = torch.empty(items, dtype=torch.float32, device="cuda")
    ms = time_once(lambda: K.clpk_mad_chain(out.data_ptr(), items, 0, 0.999, 4096, stream), reps=20)
    rows["mad_chain_2^20x4096"] = {"GFLOPS": items * 4 * 4096 * 2 / ms / 1e6, "ms": ms}

    # config 1b: float4 read-and-sum over 256 MiB of uniform[0,1) (seed 1), 16 repeats, sums and checksum exact
    n = (256 << 20) // 4
    src = torch.empty(n, dtype=torch.float32, device="cuda")
    K.clpk_fill_f32(src.data_ptr(), n, 1, N.DIST_UNIFORM01, 0.0, 1.0, stream)
    dst = torch.empty(n // 64, dtype=torch.float32, device="cuda")
    ms = time_once(lambda: K.clpk_global_bandwidth(4, src.data_ptr(), dst.data_ptr(), n, stream), reps=16)
    g = C.c_int(0)
    K.clpk_stream_read_grid(N.STREAM_LDG, C.byref(g))
    parts = torch.zeros(g.value, dtype=torch.int32, device="cuda")
    K.clpk_stream_read(N.STREAM_LDG, src.data_ptr(), n * 4, parts.data_ptr(), stream)
    torch.cuda.synchronize()
    host = orc.fill_f32(n, 1, 0)
    sums_exact = bool(np.array_equal(dst.cpu().numpy().view(np.uint32), orc.global_bandwidth(4, host).view(np.uint32)))
    xor_exact = int(np.bitwise_xor.reduce(parts.cpu().numpy().view(np.uint32))) == orc.xor_words(host)
    rows["read_sum_float4_256MiB"] = {"GBps": n * 4 / ms / 1e6, "ms": ms, "repeats": 16,
                                      "sums_equal_cpu_replay_bitwise": sums_exact,
                                      "xor_checksum_equals_cpu": bool(xor_exact), "checked": sums_exact and bool(xor_exact),
                                      "note": "256 MiB is about twice the L2: partly L2-resident between repeats"}
    del src, dst, parts, host

    # config 2b: 2^28 x uint32 (1 GiB) single cycle, 2^24 dependent hops; the walk is replayed on the host
    n_idx, hops = 1 << 28, 1 << 24
    host_next = np.empty(n_idx, dtype=np.uint32)
    K.clpk_build_chase_cycle(host_next.ctypes.data, n_idx, 0xC0FFEE)
    nxt = torch.from_numpy(host_next.view(np.int32)).cuda()
    res = torch.zeros(4, dtype=torch.int32, device="cuda")
    K.clpk_pointer_chase(nxt.data_ptr(), 0, 1 << 16, res.data_ptr(), stream)        # warm the TLBs a little
    K.clpk_pointer_chase(nxt.data_ptr(), 0, hops, res.data_ptr(), stream)
    torch.cuda.synchronize()
    r = res.cpu().numpy().view(np.uint32)
    ns = (int(r[2]) | (int(r[3]) << 32)) / hops
    want_final, want_xor = orc.chase(host_next, 0, hops)
    rows["pointer_chase_1GiB"] = {"ns_per_hop": ns, "hops": hops, "final_index": int(r[0]), "xor_of_indices": int(r[1]),
                                  "final_index_equals_cpu_replay": int(r[0]) == want_final,
                                  "xor_equals_cpu_replay": int(r[1]) == want_xor,
                                  "checked": int(r[0]) == want_final and int(r[1]) == want_xor}
    del nxt, host_next
    # pinned host <-> device copies of the reference's transfer size (512 MiB, src/cuda/transfer_bandwidth.cpp:43-95)
    nb = 512 << 20
    hbuf = torch.empty(nb, dtype=torch.uint8).pin_memory()
    hbuf.copy_(torch.arange(nb, dtype=torch.int64).to(torch.uint8))
    hback = torch.empty(nb, dtype=torch.uint8).pin_memory()
    dbuf = torch.empty(nb, dtype=torch.uint8, device="cuda")
    h2d = time_once(lambda: K.clpk_memcpy_h2d(dbuf.data_ptr(), hbuf.data_ptr(), nb, stream), reps=5)
    d2h = time_once(lambda: K.clpk_memcpy_d2h(hback.data_ptr(), dbuf.data_ptr(), nb, stream), reps=5)
    rows["transfer_pinned_512MiB"] = {"h2d_GBps": nb / h2d / 1e6, "d2h_GBps": nb / d2h / 1e6,
                                      "checked": bool(torch.equal(hbuf, hback))}
    del hbuf, hback, dbuf
    mean_us = C.c_double(0.0)
    K.clpk_launch_latency(100000, 200, C.byref(mean_us), stream)
    rows["launch_roundtrip"] = {"us": mean_us.value, "launches": 100000}
    try:        # additive readings: a kernel node of a replayed CUDA graph; the texture path in tiled order
        K.clpk_graph_launch_latency(1000, 50, 3, C.byref(mean_us), stream)
        rows["launch_graph_node"] = {"us": mean_us.value, "nodes_per_graph": 1000, "graph_launches": 50}
        img = C.c_void_p()
        K.clpk_image_create(C.byref(img), 4096, 4096, 5, stream)
        threads = 4096 * 4096 // 16
        out = torch.empty(threads, dtype=torch.float32, device="cuda")
        for name, fn in (("texture_float4_reference_order", K.clpk_image_bandwidth),
                         ("texture_float4_tiled", K.clpk_image_bandwidth_tiled)):
            ms = time_once(lambda: fn(img, out.data_ptr(), threads // 256, stream), reps=20)
            rows[name] = {"GBps": 4096 * 4096 * 16 / ms / 1e6, "ms": ms}
        K.clpk_image_destroy(img)
        del out
    except Exception as e:
        rows["additive_rows_error"] = repr(e)[:200]
    torch.cuda.empty_cache()
    return rows


def check_gemm_samples(torch, N, dt, m, A, B, Cc, sfs, alpha, row_bytes, n_samples=64):
    """A fixed seeded sample of C elements against the oracle's fp64 dot product of the same quantised operand
    rows (fetched by D2H).  Tolerance: fp32 accumulation over K terms, K * 2^-23 * sum|a||b|, plus the rounding
    of the bf16 output, 2^-8 * |c|.  Returns (ok, worst error / tolerance)."""
    import numpy as np
    from oracle import binding as orc            # checker only
    rng = np.random.default_rng(77)
    ii, jj = rng.integers(0, m, n_samples), rng.integers(0, m, n_samples)
    sf_row = m // (32 if dt == N.DT_MXF4 else 16) if sfs[0] is not None else 0        # scale bytes per row
    worst = 0.0
    c16 = Cc.view(torch.int16)
    for i, j in zip(ii.tolist(), jj.tolist()):
        ra = A[i * row_bytes:(i + 1) * row_bytes].cpu().numpy()
        rb = B[j * row_bytes:(j + 1) * row_bytes].cpu().numpy()
        sa = sfs[0][i * sf_row:(i + 1) * sf_row].cpu().numpy() if sf_row else None
        sb = sfs[1][j * sf_row:(j + 1) * sf_row].cpu().numpy() if sf_row else None
        want, s_abs = orc.gemm_element(dt, ra, rb, m, 0, 0, sa, sb)
        want *= alpha
        s_abs *= alpha
        got = float(np.array([(int(c16[i * m + j].item()) & 0xFFFF) << 16], dtype=np.uint32).view(np.float32)[0])
        tol = m * 2.0 ** -23 * s_abs + 2.0 ** -8 * abs(want) + 1e-30
        worst = max(worst, abs(got - want) / tol)
    return worst <= 1.0, worst


def compare_alternating(mine, lib, time_once, rounds=6, reps=5):
    """Ours and the library, the same number of rounds each, the order swapped every round (both sit at the power
    cap, so whoever runs second inherits the other's heat).  Returns the two lists of per-launch milliseconds."""
    ours_ms, lib_ms = [], []
    for r in range(rounds):
        if r % 2 == 0:
            ours_ms.append(time_once(mine, reps=reps))
            lib_ms.append(time_once(lib, reps=reps))
        else:
            lib_ms.append(time_once(lib, reps=reps))
            ours_ms.append(time_once(mine, reps=reps))
    return ours_ms, lib_ms


def median(xs):
    xs = sorted(xs)
    n = len(xs)
    return xs[n // 2] if n % 2 else 0.5 * (xs[n // 2 - 1] + xs[n // 2])


def measure_rows(K, N, torch, stream, time_once, world=1, clocked=None, all_ranks_ok=lambda ok: ok):
    """Tensor-core peak per dtype (config 3/4) and GEMM (config 5) on this GPU, after the timed region.

    Every tensor row is given twice: `burst` (5 launches on a GPU that has just idled) and `sustained` (a loop of
    at least 0.5 s, GEMMs 2 s, with the SM clock sampled under it).  ms x MHz = cycles separates what the kernel
    does per clock from what the 1000 W cap leaves of the clock: a peak probe at the hardware rate reads 128
    cycles per instruction (one 128x256xK instruction per 128 clocks per SM)."""
    import numpy as np
    peaks = measured_peaks()
    sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    rows = {}
    spec_of = {N.MMA_F16: "fp16_tflops", N.MMA_BF16: "bf16_tflops", N.MMA_E4M3: "fp8_tflops",
               N.MMA_E5M2: "fp8_tflops", N.MMA_I8: "int8_tops", N.MMA_MXF4: "fp4_tflops", N.MMA_NVF4: "fp4_tflops"}
    # 2:4 sparse kinds: rate counted at the logical K, against twice the dense figure
    sparse_spec = {N.MMA_E4M3_SP: "fp8_tflops", N.MMA_I8_SP: "int8_tops", N.MMA_MXF4_SP: "fp4_tflops",
                   N.MMA_NVF4_SP: "fp4_tflops"}
    ctas_per_sm = 4
    grid, n_mma = ctas_per_sm * sms, 1 << 14
    ta = torch.zeros(128 * 32, dtype=torch.uint8, device="cuda")
    tb = torch.zeros(256 * 64, dtype=torch.uint8, device="cuda")
    # selector bytes: groups alternate "keep slots 0,1" (nibble 0x4) and "keep slots 2,3" (nibble 0xE)
    meta = torch.full((128 * 8,), 0xE4, dtype=torch.uint8, device="cuda")
    # operands: seeded values converted on the device (bit patterns do not change the rate check here;
    # the parity tests own the numerics)
    f = torch.empty(256 * 128, dtype=torch.float32, device="cuda")
    sf = torch.full((256 * 4,), 0x38, dtype=torch.uint8, device="cuda")
    chk = torch.empty(grid, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    clk = torch.zeros(2, dtype=torch.int64, device="cuda")       # CTA 0's {SM cycles, ns} of the last launch
    # fp64 tensor cores (warp-level DMMA; tcgen05 has no fp64 kind): successor of the reference's wmma_fp64 row.
    # Measured first: this pipe runs at the full SM clock, which a GPU that has just run the tcgen05 rows at its
    # power cap does not offer for the next second or so
    try:
        da = torch.tensor(np.floor(np.linspace(-1, 0.99, 32) * 256) / 256, dtype=torch.float64, device="cuda")
        db = torch.tensor(np.floor(np.linspace(0.97, -1, 32) * 256) / 256, dtype=torch.float64, device="cuda")
        dgrid, dn = 8 * sms, 1 << 13
        launch = lambda: K.clpk_dmma_peak(da.data_ptr(), db.data_ptr(), dn, dgrid, 0, None, None, stream)
        ms = time_once(launch, reps=5)
        tf = 512.0 * dn * 64 * dgrid / ms / 1e9
        rows["dmma_fp64"] = {"TFLOPS": tf, "ms": ms, "frac_of_spec_37TF": tf / 37.0, "box_TFLOPS": world * tf}
    except Exception as e:
        rows["dmma_fp64"] = {"error": repr(e)[:200]}

    for kind, name in N.MMA_KIND_NAMES.items():
        if kind not in spec_of and kind not in sparse_spec:
            continue
        K.clpk_fill_f32(f.data_ptr(), f.numel(), 2, N.DIST_UNIFORM_PM1, 0.0, 1.0, stream)
        if kind in (N.MMA_E4M3_SP, N.MMA_I8_SP):
            if kind == N.MMA_I8_SP:
                K.clpk_fill_i8(ta.data_ptr(), 128 * 32, 2, stream)
                K.clpk_fill_i8(tb.data_ptr(), 256 * 64, 3, stream)
            else:
                K.clpk_convert_f32(ta.data_ptr(), f.data_ptr(), 128 * 32, N.DT_E4M3, stream)
                K.clpk_convert_f32(tb.data_ptr(), f.data_ptr(), 256 * 64, N.DT_E4M3, stream)
        elif kind in (N.MMA_MXF4_SP, N.MMA_NVF4_SP):
            mx = kind == N.MMA_MXF4_SP
            K.clpk_quantize_fp4(ta.data_ptr(), sf.data_ptr(), f.data_ptr(), 128, 64,
                                N.DT_MXF4 if mx else N.DT_NVF4, 1.0, stream)
            K.clpk_quantize_fp4(tb.data_ptr(), sf.data_ptr(), f.data_ptr(), 256, 128,
                                N.DT_MXF4_B64 if mx else N.DT_NVF4_B32, 1.0, stream)
        elif kind in (N.MMA_F16, N.MMA_BF16, N.MMA_E4M3, N.MMA_E5M2):
            dt = {N.MMA_F16: N.DT_F16, N.MMA_BF16: N.DT_BF16, N.MMA_E4M3: N.DT_E4M3, N.MMA_E5M2: N.DT_E5M2}[kind]
            K.clpk_convert_f32(ta.data_ptr(), f.data_ptr(), 128 * K.raw("clpk_mma_kind_k")(kind), dt, stream)
            K.clpk_convert_f32(tb.data_ptr(), f.data_ptr(), 256 * K.raw("clpk_mma_kind_k")(kind), dt, stream)
        elif kind == N.MMA_I8:
            K.clpk_fill_i8(ta.data_ptr(), ta.numel(), 2, stream)
            K.clpk_fill_i8(tb.data_ptr(), tb.numel(), 3, stream)
        else:
            dt = N.DT_MXF4 if kind == N.MMA_MXF4 else N.DT_NVF4
            K.clpk_quantize_fp4(ta.data_ptr(), sf.data_ptr(), f.data_ptr(), 128, 64, dt, 1.0, stream)
            K.clpk_quantize_fp4(tb.data_ptr(), sf.data_ptr(), f.data_ptr(), 256, 64, dt, 1.0, stream)
        args = N.MmaPeakArgs(kind=kind, d_a=ta.data_ptr(), d_b=tb.data_ptr(), d_sfa=sf.data_ptr(),
                             d_sfb=sf.data_ptr(), d_meta=meta.data_ptr() if kind in sparse_spec else None, n_mma=n_mma, grid=grid, n_out_tiles=0, d_out=None,
                             d_checksum=chk.data_ptr(), d_status=status.data_ptr(), d_clock=clk.data_ptr())
        launch = lambda: K.clpk_mma_peak(C.byref(args), stream)
        ms = time_once(launch, reps=5)
        if int(status.item()) != 0:
            rows[f"mma_{name}"] = {"error": "device-side wait timed out"}
            continue
        same = bool((chk == chk[0]).all().item())
        per_ms = K.raw("clpk_mma_flops_per_instr")(kind) * n_mma * grid / 1e9
        tf = per_ms / ms
        spec = 2 * SPEC[sparse_spec[kind]] if kind in sparse_spec else SPEC[spec_of[kind]]
        row = {"T(FL)OPS": tf, "ms": ms, "frac_of_spec": tf / spec, "all_ctas_same_checksum": same,
               "box_T(FL)OPS": world * tf, "timing": "burst: 5 launches"}
        if clocked is not None:
            sms_ms, mhz, reasons = clocked(launch, ms, 0.5)
            cyc, ns = (int(v) for v in clk.cpu().tolist())
            true_mhz = cyc / ns * 1e3 if ns else None
            row["sustained"] = {"T(FL)OPS": per_ms / sms_ms, "ms": sms_ms, "frac_of_spec": per_ms / sms_ms / spec,
                                "seconds": 0.5, "sm_mhz_nvml_median": mhz, "reasons": reasons,
                                # clock64 / %globaltimer of CTA 0 inside the last launch: the clock the kernel really had
                                "sm_mhz_in_kernel": true_mhz,
                                "cycles_per_instruction": (sms_ms * 1e-3 * true_mhz * 1e6 / (n_mma * ctas_per_sm)) if true_mhz else None,
                                "rate_at_max_clock_T(FL)OPS": (per_ms / sms_ms * 1965.0 / true_mhz) if true_mhz else None}
        rows[f"mma_{name}"] = row

    # the reference's fp32 and fp64 GEMM rows (CUDA cores / DMMA), 8192^3, with the library beside them
    for dt, tdt, name, spec_tf in ((N.DT_F32, torch.float32, "fp32", 75.0), (N.DT_F64, torch.float64, "fp64", 37.0)):
        try:
            m = 8192
            a = torch.empty(m * m, dtype=torch.float32, device="cuda")
            K.clpk_fill_f32(a.data_ptr(), m * m, 40, N.DIST_NORMAL, 0.0, 0.02, stream)
            b = torch.empty(m * m, dtype=torch.float32, device="cuda")
            K.clpk_fill_f32(b.data_ptr(), m * m, 41, N.DIST_NORMAL, 0.0, 0.02, stream)
            a, b = a.to(tdt).view(m, m), b.to(tdt).view(m, m)
            c = torch.empty(m, m, dtype=tdt, device="cuda")
            o = torch.empty(m, m, dtype=tdt, device="cuda")
            ga = N.GemmArgs(dtype=dt, m=m, n=m, k=m, d_a=a.data_ptr(), d_b=b.data_ptr(), d_c=c.data_ptr(), alpha=1.0,
                            d_status=status.data_ptr())
            mine = lambda: K.clpk_gemm(C.byref(ga), stream)
            tf32_was = torch.backends.cuda.matmul.allow_tf32
            torch.backends.cuda.matmul.allow_tf32 = False
            lib = lambda: torch.matmul(a, b.t(), out=o)
            ours_ms, lib_ms = compare_alternating(mine, lib, time_once, rounds=4, reps=3)
            torch.backends.cuda.matmul.allow_tf32 = tf32_was
            flop = 2.0 * m ** 3
            # both sides accumulate K products in the operand type; they agree to rounding
            err = float((c - o).abs().max().item())
            scale = float(o.abs().max().item())
            tol = m * (2.0 ** -23 if dt == N.DT_F32 else 2.0 ** -52) * scale * 4
            rows[f"gemm_{name}_{m}"] = {"TFLOPS": flop / median(ours_ms) / 1e9, "ms_rounds": ours_ms,
                                        "frac_of_spec": flop / median(ours_ms) / 1e9 / spec_tf,
                                        "vs_cublas_median": median(lib_ms) / median(ours_ms),
                                        "checked": err <= tol, "max_abs_difference_from_library": err}
            rows[f"library_cublas_{name}_{m}"] = {"TFLOPS_median": flop / median(lib_ms) / 1e9, "ms_rounds": lib_ms}
            del a, b, c, o
        except Exception as e:
            rows[f"gemm_{name}_8192"] = {"error": repr(e)[:200]}
        torch.cuda.empty_cache()

    # GEMM (config 5): M = N = K in {4096, 8192, 16384}; bf16, fp8 e4m3, NVFP4
    order = 0
    for dt, name, spec in ((N.DT_BF16, "bf16", "bf16_tflops"), (N.DT_E4M3, "fp8_e4m3", "fp8_tflops"),
                           (N.DT_NVF4, "nvf4_e2m1", "fp4_tflops")):
        for m in (4096, 8192, 16384):
            nv = dt == N.DT_NVF4
            row_bytes = m // 2 if nv else (2 * m if dt == N.DT_BF16 else m)
            A = torch.empty(m * row_bytes, dtype=torch.uint8, device="cuda")
            B = torch.empty(m * row_bytes, dtype=torch.uint8, device="cuda")
            Cc = torch.empty(m * m, dtype=torch.int16, device="cuda")
            tmp = torch.empty(m * m, dtype=torch.float32, device="cuda")
            sfs = [torch.empty(m * m // 16, dtype=torch.uint8, device="cuda") for _ in range(2)] if nv else [None, None]
            tscale = 2.0 ** -15      # N(0, 0.02) operands: keeps x / scale / 6 inside ue4m3's range
            for buf, sfbuf, seed in ((A, sfs[0], 40), (B, sfs[1], 41)):
                K.clpk_fill_f32(tmp.data_ptr(), m * m, seed, N.DIST_NORMAL, 0.0, 0.02, stream)
                if nv:
                    K.clpk_quantize_fp4(buf.data_ptr(), sfbuf.data_ptr(), tmp.data_ptr(), m, m, dt, tscale, stream)
                else:
                    K.clpk_convert_f32(buf.data_ptr(), tmp.data_ptr(), m * m, dt, stream)
            del tmp
            ws = None
            ws_bytes = C.c_size_t(0)
            if nv:
                K.clpk_gemm_workspace_bytes(dt, m, m, m, C.byref(ws_bytes))
                ws = torch.empty(max(ws_bytes.value, 16), dtype=torch.uint8, device="cuda")
            alpha = tscale * tscale if nv else 1.0
            ga = N.GemmArgs(dtype=dt, m=m, n=m, k=m, d_a=A.data_ptr(), d_b=B.data_ptr(), d_c=Cc.data_ptr(),
                            d_sfa=sfs[0].data_ptr() if nv else None, d_sfb=sfs[1].data_ptr() if nv else None,
                            alpha=alpha, d_workspace=ws.data_ptr() if nv else None,
                            workspace_bytes=ws_bytes.value, d_status=status.data_ptr())
            ms_with_pack = None
            if nv:
                # one call that also puts the scale arrays in tile order, then the steady state: packed once,
                # multiplied many times (what the library's caller has to do as well)
                ms_with_pack = time_once(lambda: K.clpk_gemm(C.byref(ga), stream), reps=5)
                K.clpk_gemm_pack_scales(C.byref(ga), stream)
                ga.d_sfa = None
                ga.d_sfb = None
            mine = lambda: K.clpk_gemm(C.byref(ga), stream)
            flop = 2.0 * m * m * m
            ms = time_once(mine, reps=5)
            row = {"TFLOPS": flop / ms / 1e9, "ms": ms, "frac_of_spec": flop / ms / 1e9 / SPEC[spec],
                   "status": int(status.item()), "box_TFLOPS": world * flop / ms / 1e9, "timing": "burst: 5 launches",
                   # 1: cooperative launch with the per-wave producer meeting; 0: plain launch (small problem or no co-residency)
                   "producers_aligned": K.raw("clpk_gemm_last_launch_aligned")()}
            if ms_with_pack is not None:
                row["ms_including_scale_repack"] = ms_with_pack
            if dt == N.DT_BF16:
                row["frac_of_measured_cublas_burst"] = flop / ms / 1e9 / peaks["bf16_tflops"]
            # every replica checks the C it has just timed; the row is "checked" only if all of them agree
            Cc.fill_(0x7FC0)                                        # bf16 NaN canary under the result that is checked
            mine()
            torch.cuda.synchronize()
            ok, worst = check_gemm_samples(torch, N, dt, m, A, B, Cc, sfs, alpha, row_bytes)
            row["checked"] = all_ranks_ok(bool(ok) and int(status.item()) == 0)
            row["check"] = {"samples": 64, "worst_error_over_tolerance": worst, "replicas": world,
                            "tolerance": "K*2^-23*sum|a||b| + 2^-8*|c|, vs fp64 dot of the quantised operands"}
            rows[f"gemm_{name}_{m}"] = row
            # The vendor library on the very same operand buffers (same data, same thermal state); for comparison
            # only, never on the product path.  The reference's GEMM rows call cuBLASLt
            # (src/cuda/cuda_blas.cpp:264-394, :435-551), which is what torch dispatches to here.
            try:
                lib_out = torch.empty((m, m), dtype=torch.bfloat16, device="cuda")
                if dt == N.DT_BF16:
                    x, y = A.view(torch.bfloat16).view(m, m), B.view(torch.bfloat16).view(m, m)
                    lib, what = (lambda: torch.matmul(x, y.t(), out=lib_out)), "torch.matmul (cuBLAS), bf16 in / bf16 out, TN"
                elif dt == N.DT_E4M3:
                    x, y = A.view(torch.float8_e4m3fn).view(m, m), B.view(torch.float8_e4m3fn).view(m, m)
                    one = torch.ones((), dtype=torch.float32, device="cuda")
                    lib = lambda: torch._scaled_mm(x, y.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16, out=lib_out)
                    what = "torch._scaled_mm (cuBLASLt), e4m3 in, per-tensor scale, bf16 out, TN"
                else:
                    x = A.view(torch.float4_e2m1fn_x2).view(m, m // 2)
                    y = B.view(torch.float4_e2m1fn_x2).view(m, m // 2)
                    sx, sy = sfs[0].view(torch.float8_e4m3fn), sfs[1].view(torch.float8_e4m3fn)
                    lib = lambda: torch._scaled_mm(x, y.t(), scale_a=sx, scale_b=sy, out_dtype=torch.bfloat16, out=lib_out)
                    what = ("torch._scaled_mm (cuBLASLt), NVFP4: e2m1 + ue4m3 per 16, bf16 out, TN; the same scale "
                            "bytes read in the library's blocked order (timing only)")
                try:
                    lib()
                except TypeError:                   # a torch without out= on this entry point
                    if dt == N.DT_E4M3:
                        lib = lambda: torch._scaled_mm(x, y.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
                    elif nv:
                        lib = lambda: torch._scaled_mm(x, y.t(), scale_a=sx, scale_b=sy, out_dtype=torch.bfloat16)
                    what += "; output allocated per call by torch's caching allocator"
                ours_ms, lib_ms = compare_alternating(mine, lib, time_once)
                lrow = {"TFLOPS_best": flop / min(lib_ms) / 1e9, "TFLOPS_median": flop / median(lib_ms) / 1e9,
                        "ms_rounds": lib_ms, "note": what}
                row["ms_rounds"] = ours_ms
                row["TFLOPS_best_of_rounds"] = flop / min(ours_ms) / 1e9
                row["TFLOPS_median_of_rounds"] = flop / median(ours_ms) / 1e9
                row["vs_cublas_median"] = median(lib_ms) / median(ours_ms)
                row["vs_cublas_best"] = min(lib_ms) / min(ours_ms)
                row["vs_cublas_note"] = ("6 alternating rounds of 5 launches on each side, order swapped every round; "
                                         "ratio of medians and of bests (library time / our time)")
                if clocked is not None:
                    # >= 2 s of each, clock sampled under the loop; which side goes first alternates per row
                    first_ours = order % 2 == 0
                    order += 1
                    res = {}
                    for who in (("ours", "lib") if first_ours else ("lib", "ours")):
                        fn, est = (mine, median(ours_ms)) if who == "ours" else (lib, median(lib_ms))
                        sms_ms, mhz, reasons = clocked(fn, est, 2.0)
                        res[who] = {"TFLOPS": flop / sms_ms / 1e9, "ms": sms_ms, "sm_mhz_median": mhz, "reasons": reasons,
                                    "mega_cycles": sms_ms * 1e-3 * mhz if mhz else None}
                        if who == "ours":
                            cyc, ns = C.c_ulonglong(0), C.c_ulonglong(0)
                            K.clpk_gemm_last_clock(C.byref(cyc), C.byref(ns), stream)
                            if ns.value:
                                res[who]["sm_mhz_in_kernel"] = cyc.value / ns.value * 1e3
                    row["sustained"] = dict(res["ours"], seconds=2.0, ran="first" if first_ours else "second")
                    lrow["sustained"] = dict(res["lib"], seconds=2.0, ran="second" if first_ours else "first")
                    row["vs_cublas_sustained"] = res["lib"]["ms"] / res["ours"]["ms"]
                    if res["ours"]["mega_cycles"] and res["lib"]["mega_cycles"]:
                        row["vs_cublas_sustained_in_cycles"] = res["lib"]["mega_cycles"] / res["ours"]["mega_cycles"]
                rows[f"library_cublaslt_{name}_{m}"] = lrow
            except Exception as e:          # a torch build without that path: report, do not fail the bench
                rows[f"library_cublaslt_{name}_{m}"] = {"error": repr(e)[:200]}
            x = y = sx = sy = lib = lib_out = None
            del A, B, Cc, sfs, ws
            torch.cuda.empty_cache()

    # MXFP4 (e2m1 with one ue8m0 factor per 32): the reference's cuBLASLt "mxf4_e2m1" row.  Timed and checked like
    # the rows above, without a library side (torch's block-scaled entry point takes another scale layout).
    for m in (8192, 16384):
        try:
            dt = N.DT_MXF4
            A = torch.empty(m * m // 2, dtype=torch.uint8, device="cuda")
            B = torch.empty(m * m // 2, dtype=torch.uint8, device="cuda")
            Cc = torch.empty(m * m, dtype=torch.int16, device="cuda")
            tmp = torch.empty(m * m, dtype=torch.float32, device="cuda")
            sfs = [torch.empty(m * m // 32, dtype=torch.uint8, device="cuda") for _ in range(2)]
            for buf, sfbuf, seed in ((A, sfs[0], 40), (B, sfs[1], 41)):
                K.clpk_fill_f32(tmp.data_ptr(), m * m, seed, N.DIST_NORMAL, 0.0, 0.02, stream)
                K.clpk_quantize_fp4(buf.data_ptr(), sfbuf.data_ptr(), tmp.data_ptr(), m, m, dt, 1.0, stream)
            del tmp
            ws_bytes = C.c_size_t(0)
            K.clpk_gemm_workspace_bytes(dt, m, m, m, C.byref(ws_bytes))
            ws = torch.empty(max(ws_bytes.value, 16), dtype=torch.uint8, device="cuda")
            ga = N.GemmArgs(dtype=dt, m=m, n=m, k=m, d_a=A.data_ptr(), d_b=B.data_ptr(), d_c=Cc.data_ptr(),
                            d_sfa=sfs[0].data_ptr(), d_sfb=sfs[1].data_ptr(), alpha=1.0, d_workspace=ws.data_ptr(),
                            workspace_bytes=ws_bytes.value, d_status=status.data_ptr())
            K.clpk_gemm_pack_scales(C.byref(ga), stream)
            ga.d_sfa = None
            ga.d_sfb = None
            mine = lambda: K.clpk_gemm(C.byref(ga), stream)
            flop = 2.0 * m * m * m
            torch.cuda.synchronize()
            time.sleep(3.0)                          # the rows above end in 2 s loops at the power cap
            ms_rounds = [time_once(mine, reps=5) for _ in range(3)]
            ms = median(ms_rounds)
            Cc.fill_(0x7FC0)
            mine()
            torch.cuda.synchronize()
            ok, worst = check_gemm_samples(torch, N, dt, m, A, B, Cc, sfs, 1.0, m // 2)
            rows[f"gemm_mxf4_e2m1_{m}"] = {
                "TFLOPS": flop / ms / 1e9, "ms": ms, "ms_rounds": ms_rounds, "frac_of_spec": flop / ms / 1e9 / SPEC["fp4_tflops"],
                "status": int(status.item()), "box_TFLOPS": world * flop / ms / 1e9, "timing": "median of 3 bursts of 5 launches after 3 s idle",
                "checked": all_ranks_ok(bool(ok) and int(status.item()) == 0),
                "check": {"samples": 64, "worst_error_over_tolerance": worst, "replicas": world}}
            del A, B, Cc, sfs, ws
        except Exception as e:
            rows[f"gemm_mxf4_e2m1_{m}"] = {"error": repr(e)[:200]}
            all_ranks_ok(False)                      # keep the ranks' collectives in step
        torch.cuda.empty_cache()
    return rows


if __name__ == "__main__":
    sys.exit(main())
