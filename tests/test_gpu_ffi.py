"""The product's own plugin API on the real GPU: libclpeak_ffi.so is loaded with ctypes and
`clpeak_launch` drives CudaPeak::runAll, the timing harness, every kernel and the in-product
host checks end to end.  Restates the reference's contract test
(app/test/ffi_integration_test.dart:27-105): rc 0, a final `done`, ok metrics with value > 0,
an XML file that loads back through clpeak_load_result_file_json; `--bogus-flag` -> -1;
cancel -> -2; the backend catalog names the device.

A row is `ok` only if the backend's own check of that row's result against the host passed
(host_check.hpp), so "every supported row is ok" is the parity statement for the C++ host.
The row table is the CUDA run of the reference's saved result file
(results/Nvidia/GeForce_RTX_5060.xml:8-124): the same test tags, metric labels and units must
come out of this backend."""
import ctypes as C
import json
import xml.etree.ElementTree as ET

import pytest

from clpeak_b200 import native as N
from tests.gpu_util import dev_empty, stream_ptr, sync

pytestmark = pytest.mark.gpu

# (category, test tag, unit, metric labels) of the reference's CUDA backend
REFERENCE_ROWS = [
    ("fp_compute", "single_precision_compute", "gflops", ["float"]),
    ("fp_compute", "half_precision_compute", "gflops", ["half", "half2"]),
    ("fp_compute", "double_precision_compute", "gflops", ["double"]),
    ("fp_compute", "mixed_precision_compute", "gflops", ["mp"]),
    ("fp_compute", "bfloat16_compute", "gflops", ["bf16"]),
    ("fp_compute", "wmma_fp16", "tflops", ["wmma_fp16"]),
    ("fp_compute", "wmma_fp16_f16", "tflops", ["fp16_f16acc"]),
    ("fp_compute", "wmma_bf16", "tflops", ["wmma_bf16"]),
    ("fp_compute", "wmma_tf32", "tflops", ["wmma_tf32"]),
    ("fp_compute", "wmma_fp64", "tflops", ["wmma_fp64"]),
    ("fp_compute", "wmma_fp8_e4m3", "tflops", ["fp8_e4m3"]),
    ("fp_compute", "wmma_fp8_e5m2", "tflops", ["fp8_e5m2"]),
    ("fp_compute", "wmma_fp4_e2m1", "tflops", ["fp4_e2m1"]),
    ("fp_compute", "wmma_mxf4_e2m1", "tflops", ["mxf4_e2m1"]),
    ("fp_compute", "wmma_nvf4_e2m1", "tflops", ["nvf4_e2m1"]),
    ("fp_compute", "wmma_mxf4_sparse", "tflops", ["mxf4_sparse"]),
    ("fp_compute", "wmma_nvf4_sparse", "tflops", ["nvf4_sparse"]),
    ("fp_compute", "cublas-fp", "tflops", ["fp32", "fp64", "tf32", "fp16", "bf16", "fp8_e4m3", "fp8_e5m2", "mxf4_e2m1",
                                          "nvf4_e2m1"]),
    ("int_compute", "integer_compute", "gops", ["int"]),
    ("int_compute", "integer_compute_int8_dp", "gops", ["int8_dp", "int8_dp2", "int8_dp4", "int8_dp8"]),
    ("int_compute", "wmma_int8", "tops", ["wmma_int8"]),
    ("int_compute", "wmma_int8_k32", "tops", ["int8_k32"]),
    ("int_compute", "wmma_int8_sparse", "tops", ["int8_sparse"]),
    ("int_compute", "wmma_int4", "tops", ["int4"]),
    ("int_compute", "cublas-int", "tops", ["int8", "int4"]),
    ("bandwidth", "global_memory_bandwidth", "gbps", ["float", "float2", "float4"]),
    ("bandwidth", "local_memory_bandwidth", "gbps", ["float", "float2", "float4"]),
    ("bandwidth", "image_memory_bandwidth", "gbps", ["float4"]),
    ("bandwidth", "transfer_bandwidth", "gbps", ["h2d_pinned", "d2h_pinned"]),
    ("latency", "kernel_launch_latency", "us", ["dispatch", "roundtrip"]),
]

# Rows this backend answers "unsupported" on a B200, with the reason: the legacy 16x16x16 int8
# row is superseded by the tcgen05 int8_k32 row, sm_100 has no int4 tensor path (the reference
# skips it above sm_89 too), and CUDA has no host/device clock for a one-way dispatch time (the
# reference reports the same row unsupported, src/cuda/kernel_latency.cpp:66-67).
EXPECTED_UNSUPPORTED = {("wmma_int8", "wmma_int8"), ("wmma_int4", "int4"), ("cublas-int", "int4"),
                        ("kernel_launch_latency", "dispatch")}

# Additive rows of this backend (not in the reference's file) that a full run must also report ok.
ADDED_ROWS = [("single_precision_compute", "float4_seeded"), ("wmma_fp8_e4m3_sparse", "fp8_e4m3_sparse"),
              ("global_memory_bandwidth", "read"), ("global_memory_bandwidth", "copy"),
              ("global_memory_bandwidth", "triad"), ("image_memory_bandwidth", "float4_tiled"),
              ("memory_latency", "L2"), ("memory_latency", "HBM"), ("kernel_launch_latency", "graph_node")]

# plausibility windows on a B200 (loose: they catch a wrong unit or a row that timed nothing)
BOUNDS = {
    ("single_precision_compute", "float"): (20e3, 90e3),
    ("double_precision_compute", "double"): (10e3, 45e3),
    ("wmma_bf16", "wmma_bf16"): (800, 2300),
    ("wmma_fp64", "wmma_fp64"): (10, 45),
    ("wmma_fp8_e4m3", "fp8_e4m3"): (1500, 4600),
    ("wmma_nvf4_e2m1", "nvf4_e2m1"): (3000, 9200),
    ("wmma_int8_k32", "int8_k32"): (1500, 4600),
    ("cublas-fp", "bf16"): (600, 2300),
    ("cublas-fp", "fp32"): (10, 80),
    ("cublas-fp", "fp64"): (5, 45),
    ("cublas-fp", "nvf4_e2m1"): (1500, 9200),
    ("global_memory_bandwidth", "float4"): (3000, 8200),
    ("global_memory_bandwidth", "read"): (5000, 8200),
    ("global_memory_bandwidth", "copy"): (5000, 8200),
    ("global_memory_bandwidth", "triad"): (5000, 8200),
    ("transfer_bandwidth", "h2d_pinned"): (5, 130),       # PCIe gen4 x16 floor .. gen6 x16 ceiling
    ("transfer_bandwidth", "d2h_pinned"): (5, 130),
    ("memory_latency", "L2"): (50, 1000),
    ("memory_latency", "HBM"): (200, 2000),
    ("kernel_launch_latency", "roundtrip"): (1, 200),
}


class Ffi:
    def __init__(self):
        self.lib = N.ffi()

    def take(self, p):
        if not p:
            return None
        s = C.string_at(p).decode()
        self.lib.clpeak_free_string(p)
        return s

    def launch(self, argv, on_event=None):
        events = []

        def cb(_ud, p):
            ev = json.loads(self.take(p))           # ownership of the string passes to the callee
            events.append(ev)
            if on_event:
                on_event(ev)

        args = [b"clpeak"] + [a.encode() for a in argv]
        arr = (C.c_char_p * len(args))(*args)
        keep = N.EVENT_CALLBACK(cb)
        rc = self.lib.clpeak_launch(len(args), arr, C.cast(keep, C.c_void_p), None)
        return rc, events


@pytest.fixture(scope="module")
def ffi(cuda):
    return Ffi()


@pytest.fixture(scope="module")
def full_run(ffi, tmp_path_factory):
    xml = tmp_path_factory.mktemp("ffi") / "b200.xml"
    rc, events = ffi.launch(["--cuda", "--cuda-device", "0", "--max-time", "50", "--xml-file", str(xml)])
    return rc, events, xml


def test_version_and_catalog_name_the_real_device(ffi):
    assert ffi.lib.clpeak_version().decode().startswith("2.")
    cat = json.loads(ffi.take(ffi.lib.clpeak_copy_backend_catalog_json()))
    (cuda_b,) = [b for b in cat["backends"] if b["name"] == "CUDA"]
    assert cuda_b["available"] is True
    dev = cuda_b["platforms"][0]["devices"][0]
    assert dev["index"] == 0 and dev["type"] == "sm_100" and "B200" in dev["name"]


def test_full_run_ends_ok_and_in_order(full_run):
    rc, ev, _ = full_run
    kinds = [e["t"] for e in ev]
    assert rc == 0, [e for e in ev if e["t"] == "note"]
    assert ev[-1] == {"t": "done", "status": 0, "cancelled": False}
    assert kinds[0] == "backend_begin" and kinds[-2] == "backend_end"
    assert kinds.count("device") == 1 and kinds.count("test_begin") == kinds.count("test_end")
    dev = next(e for e in ev if e["t"] == "device")
    props = {p["k"]: p["v"] for p in dev["props"]}
    assert list(props) == ["Arch", "Toolkit", "SMs", "VRAM"]           # src/cuda/cuda_peak.cpp:153-158
    assert props["Arch"] == "sm_100" and int(props["SMs"]) >= 100 and "B200" in dev["device"]
    order = [e["category"] for e in ev if e["t"] == "metric"]
    assert order.index("fp_compute") < order.index("int_compute") < order.index("bandwidth") < order.index("latency")


def test_every_reference_row_is_present_with_its_tag_label_and_unit(full_run):
    _, ev, _ = full_run
    by = {(m["test"], m["metric"]): m for m in ev if m["t"] == "metric"}
    for category, test, unit, labels in REFERENCE_ROWS:
        for label in labels:
            assert (test, label) in by, f"row {test}/{label} is missing"
            m = by[(test, label)]
            assert m["unit"] == unit and m["category"] == category, m


def test_every_supported_row_passed_its_host_check(full_run):
    _, ev, _ = full_run
    metrics = [m for m in ev if m["t"] == "metric"]
    bad = [(m["test"], m["metric"], m["status"], m["reason"]) for m in metrics
           if m["status"] != "ok" and (m["test"], m["metric"]) not in EXPECTED_UNSUPPORTED]
    assert not bad, bad
    for key in EXPECTED_UNSUPPORTED:
        m = next(x for x in metrics if (x["test"], x["metric"]) == key)
        assert m["status"] == "unsupported" and m["reason"] and m["value"] == 0
    ok = {(m["test"], m["metric"]): m["value"] for m in metrics if m["status"] == "ok"}
    assert all(v > 0 for v in ok.values())
    for key in ADDED_ROWS:
        assert key in ok, f"additive row {key} missing or not ok"
    for key, (lo, hi) in BOUNDS.items():
        assert lo <= ok[key] <= hi, f"{key}: {ok[key]} outside [{lo}, {hi}]"
    for m in metrics:                                                    # every reading is described for the GUI
        assert m["desc"] or m["status"] != "ok", m


def test_result_file_round_trips_through_the_loader(ffi, full_run):
    _, ev, xml = full_run
    metrics = [m for m in ev if m["t"] == "metric"]
    root = ET.parse(xml).getroot()
    assert root.tag == "clpeak" and root.get("format_version") == "2"
    (run,) = root.findall("run")
    assert run.get("backend") == "CUDA" and "B200" in run.get("device")
    assert [c.get("name") for c in run.findall("category")] == ["fp_compute", "int_compute", "bandwidth", "latency"]
    doc = json.loads(ffi.take(ffi.lib.clpeak_load_result_file_json(str(xml).encode())))
    assert doc["format_version"] == 2 and len(doc["entries"]) == len(metrics)
    assert doc["devices"][0]["props"][0] == {"k": "Arch", "v": "sm_100"}
    entries = {(e["test"], e["metric"]): e for e in doc["entries"]}
    assert len(entries) == len(metrics)
    for m in metrics:
        e = entries[(m["test"], m["metric"])]
        if m["status"] == "ok":
            assert "status" not in e and abs(e["value"] - m["value"]) <= 1e-3 * max(1.0, abs(m["value"]))
        else:
            assert "value" not in e and e["status"] == m["status"] and e["reason"]


def test_bad_flag_is_refused(ffi):
    rc, ev = ffi.launch(["--bogus-flag"])
    assert rc == -1
    assert [e["t"] for e in ev] == ["note", "done"] and "--bogus-flag" in ev[0]["message"]
    assert ev[1] == {"t": "done", "status": -1, "cancelled": False}


def test_cancel_and_busy_on_the_gpu(ffi):
    seen = {}

    def on_event(ev):
        if ev["t"] == "test_begin" and "busy" not in seen:
            seen["busy"] = ffi.launch(["--kernel-launch-latency"])       # a second launch while one runs
            ffi.lib.clpeak_request_cancel()

    rc, ev = ffi.launch(["--cuda", "--cuda-device", "0", "--fp-compute", "--no-cublas", "--max-time", "20"], on_event)
    assert seen["busy"] == (-3, [])
    assert rc == -2 and ev[-1] == {"t": "done", "status": -2, "cancelled": True}
    assert [e["t"] for e in ev].count("test_begin") < 6
    rc, ev = ffi.launch(["--cuda", "--cuda-device", "0", "--kernel-launch-latency", "-i", "200"])
    assert rc == 0 and ev[-1]["cancelled"] is False                      # the flag resets at the next launch
    (m,) = [e for e in ev if e["t"] == "metric" and e["metric"] == "roundtrip"]
    assert m["status"] == "ok" and m["value"] > 0


def test_forced_iterations_and_selection_on_the_gpu(ffi):
    """-i / -w reach the timing harness (src/cuda/cuda_peak.cpp:64-107) and the allow-list picks the tests."""
    rc, ev = ffi.launch(["--cuda", "--cuda-device", "0", "--global-memory-bandwidth", "--memory-latency",
                         "--transfer-bandwidth", "-i", "3", "-w", "1"])
    assert rc == 0
    assert sorted({e["test"] for e in ev if e["t"] == "test_begin"}) == ["global_memory_bandwidth", "memory_latency",
                                                                         "transfer_bandwidth"]
    assert all(m["status"] == "ok" for m in ev if m["t"] == "metric")


def test_two_gpus_through_the_thread_per_gpu_driver(ffi, cuda):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rc, ev = ffi.launch(["--cuda", "--cuda-device", "0,1", "--global-memory-bandwidth", "--wmma", "--no-int-compute",
                         "--max-time", "50"])
    assert rc == 0 and not [e for e in ev if e["t"] == "note"], [e for e in ev if e["t"] == "note"]
    devs = [e["device_index"] for e in ev if e["t"] == "device"]
    assert devs == [0, 1, -1]
    per = {}
    for m in ev:
        if m["t"] == "metric" and m["status"] == "ok":
            per.setdefault(m["device"], {})[(m["test"], m["metric"])] = m["value"]
    names = list(per)
    agg = per[names[2]]
    for key in (("global_memory_bandwidth", "read"), ("wmma_bf16", "wmma_bf16")):
        singles = [per[names[0]][key], per[names[1]][key]]
        assert 1.6 * min(singles) <= agg[key] <= 2.02 * max(singles), (key, singles, agg[key])


def test_transfer_bandwidth_bytes_arrive_intact(K, cuda):
    """Pinned host <-> device copies of the reference's transfer size (512 MiB,
    src/cuda/transfer_bandwidth.cpp:43-95) through the shim calls the backend times."""
    import numpy as np
    n = 512 << 20
    stream = C.c_void_p(None)
    K.clpk_stream_create(C.byref(stream))
    h_src, h_dst, d = C.c_void_p(None), C.c_void_p(None), C.c_void_p(None)
    K.clpk_malloc_host(C.byref(h_src), n)
    K.clpk_malloc_host(C.byref(h_dst), n)
    K.clpk_malloc(C.byref(d), n)
    try:
        src = np.ctypeslib.as_array(C.cast(h_src, C.POINTER(C.c_uint8)), shape=(n,))
        dst = np.ctypeslib.as_array(C.cast(h_dst, C.POINTER(C.c_uint8)), shape=(n,))
        src[:] = np.random.default_rng(5).integers(0, 256, n, dtype=np.uint8)
        dst[:] = 0
        K.clpk_memcpy_h2d(d, h_src, n, stream)
        K.clpk_memcpy_d2h(h_dst, d, n, stream)
        K.clpk_stream_sync(stream)
        assert np.array_equal(src, dst)
    finally:
        K.clpk_free(d)
        K.clpk_free_host(h_src)
        K.clpk_free_host(h_dst)
        K.clpk_stream_destroy(stream)


def test_device_info_describes_a_b200(K, cuda):
    """clpk_device_info / clpk_device_count behind CudaDevice::init and CudaPeak::enumerate
    (src/cuda/cuda_device.cpp:40-120, src/cuda/cuda_peak.cpp:221-275) against what torch reports."""
    n = C.c_int(0)
    K.clpk_device_count(C.byref(n))
    assert n.value == cuda.cuda.device_count() >= 1
    info = N.DeviceInfo()
    K.clpk_device_info(0, C.byref(info))
    props = cuda.cuda.get_device_properties(0)
    assert info.name.decode() == props.name and "B200" in props.name
    assert (info.cc_major, info.cc_minor) == (10, 0) == (props.major, props.minor)
    assert info.num_sms == props.multi_processor_count >= 100
    assert info.total_mem_bytes == props.total_memory > 100 << 30
    assert info.smem_optin_bytes >= 227 * 1024 and info.l2_bytes >= 64 << 20
    assert info.sm_clock_khz >= 1_000_000 and info.mem_bus_bits >= 4096
    assert info.driver_version >= 12000 and info.runtime_version >= 12000
    with pytest.raises(N.ClpkError):
        K.clpk_device_info(n.value, C.byref(info))                # one past the last device
    # a failure that has been reported does not come back at the next launch
    d = dev_empty(4, cuda.float32)
    K.clpk_fill_f32(d.data_ptr(), 4, 1, N.DIST_UNIFORM01, 0.0, 1.0, stream_ptr())
    sync()
