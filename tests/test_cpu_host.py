"""The C++ host side (options, multi-device driver, logger, FFI event stream,
result files) run end to end on the CPU against the test double of the kernel
shim.  Mirrors what the reference's GUI tests expect of the ABI
(app/test/ffi_integration_test.dart:27-105, app/test/models_test.dart)."""
import json
import os
import subprocess
import threading
import xml.etree.ElementTree as ET
from pathlib import Path

import pytest

from tests.host_fake import FakeFfi

ROOT = Path(__file__).resolve().parent.parent
REF_RESULTS = Path(os.environ.get("CLPEAK_REFERENCE_DIR", "/root/reference")) / "results"
FAST = ["-i", "1", "-w", "0"]


@pytest.fixture(scope="module")
def ffi():
    return FakeFfi()


@pytest.fixture()
def one_device(monkeypatch):
    monkeypatch.setenv("CLPK_FAKE_DEVICES", "1")


def kinds(events):
    return [e["t"] for e in events]


def test_version_and_catalog(ffi, one_device):
    assert ffi.lib.clpeak_version().decode().startswith("2.")
    cat = json.loads(ffi.take(ffi.lib.clpeak_copy_backend_catalog_json()))
    (cuda,) = [b for b in cat["backends"] if b["name"] == "CUDA"]
    assert cuda["available"] is True
    dev = cuda["platforms"][0]["devices"][0]
    assert dev["index"] == 0 and dev["type"] == "sm_100" and "B200" in dev["name"]


def test_launch_streams_events_and_writes_xml(ffi, one_device, tmp_path):
    xml = tmp_path / "run.xml"
    rc, ev = ffi.launch(["--cuda", "--wmma", "--kernel-launch-latency", *FAST, "--xml-file", str(xml)])
    assert rc == 0
    k = kinds(ev)
    assert k[0] == "backend_begin" and k[-1] == "done" and k[-2] == "backend_end"
    assert ev[-1] == {"t": "done", "status": 0, "cancelled": False}
    assert k.count("device") == 1 and k.count("test_begin") == k.count("test_end") > 5
    dev = next(e for e in ev if e["t"] == "device")
    assert dev["device_index"] == 0 and dev["platform_index"] == -1
    assert [p["k"] for p in dev["props"]] == ["Arch", "Toolkit", "SMs", "VRAM"]
    metrics = [e for e in ev if e["t"] == "metric"]
    okm = [m for m in metrics if m["status"] == "ok"]
    assert okm and all(m["value"] > 0 for m in okm)
    assert all(set(m) >= {"category", "test", "display", "metric", "unit", "value", "status", "reason", "sub", "desc",
                          "minfo"} for m in metrics)
    by = {(m["test"], m["metric"]): m for m in metrics}
    assert by[("wmma_bf16", "wmma_bf16")]["unit"] == "tflops" and by[("wmma_bf16", "wmma_bf16")]["category"] == "fp_compute"
    assert by[("wmma_int8_k32", "int8_k32")]["unit"] == "tops" and by[("wmma_int8_k32", "int8_k32")]["category"] == "int_compute"
    assert by[("wmma_int4", "int4")]["status"] == "unsupported" and by[("wmma_int4", "int4")]["value"] == 0
    assert by[("wmma_fp64", "wmma_fp64")]["status"] == "ok" and by[("wmma_fp64", "wmma_fp64")]["unit"] == "tflops"
    # the 2:4 sparse rows prune on the host, run, and pass the host's own tile check (exact for int8)
    for key, unit, cat in ((("wmma_int8_sparse", "int8_sparse"), "tops", "int_compute"),
                           (("wmma_mxf4_sparse", "mxf4_sparse"), "tflops", "fp_compute"),
                           (("wmma_nvf4_sparse", "nvf4_sparse"), "tflops", "fp_compute"),
                           (("wmma_fp8_e4m3_sparse", "fp8_e4m3_sparse"), "tflops", "fp_compute")):
        assert by[key]["status"] == "ok", by[key]
        assert by[key]["unit"] == unit and by[key]["category"] == cat and by[key]["value"] > 0
    assert by[("kernel_launch_latency", "dispatch")]["status"] == "unsupported"
    assert by[("kernel_launch_latency", "roundtrip")]["category"] == "latency"
    # fp rows come before int rows, which come before latency (the reference's phase order)
    order = [m["category"] for m in metrics]
    assert order.index("int_compute") > order.index("fp_compute") and order.index("latency") > order.index("int_compute")

    root = ET.parse(xml).getroot()
    assert root.tag == "clpeak" and root.get("format_version") == "2" and root.get("os")
    (run,) = root.findall("run")
    assert run.get("backend") == "CUDA" and run.get("platform") == "CUDA"
    assert [p.get("name") for p in run.findall("prop")] == ["Arch", "Toolkit", "SMs", "VRAM"]
    cats = [c.get("name") for c in run.findall("category")]
    assert cats == ["fp_compute", "int_compute", "latency"]
    m = run.find("./category[@name='int_compute']/test[@name='wmma_int4']/metric")
    assert m.get("status") == "unsupported" and m.text is None

    # round trip through the loader export, descriptions intact
    doc = json.loads(ffi.take(ffi.lib.clpeak_load_result_file_json(str(xml).encode())))
    assert doc["format_version"] == 2 and len(doc["entries"]) == len(metrics)
    assert doc["devices"][0]["props"][0] == {"k": "Arch", "v": "sm_100"}
    e = next(x for x in doc["entries"] if x["test"] == "wmma_bf16")
    assert "value" in e and "status" not in e and e["description"] and e["metric_description"]
    bad = next(x for x in doc["entries"] if x["metric"] == "int4")
    assert "value" not in bad and bad["status"] == "unsupported" and bad["reason"]


def test_bad_arguments(ffi, one_device):
    rc, ev = ffi.launch(["--bogus-flag"])
    assert rc == -1
    assert kinds(ev) == ["note", "done"] and "--bogus-flag" in ev[0]["message"]
    assert ev[1] == {"t": "done", "status": -1, "cancelled": False}
    for argv in (["--help"], ["--version"], ["--iters"], ["-i", "0"], ["--cuda-device", "0,,1"], ["--max-time", "x"],
                 ["--vulkan"]):
        rc, ev = ffi.launch(argv)
        assert rc == -1 and ev[-1]["t"] == "done", argv


def test_selection_grammar(ffi, one_device):
    def tests_run(argv):
        rc, ev = ffi.launch(argv + FAST)
        assert rc == 0
        return sorted({e["test"] for e in ev if e["t"] == "test_begin"})

    only_latency = tests_run(["--kernel-launch-latency"])
    assert only_latency == ["kernel_launch_latency"]
    assert tests_run(["--latency", "--no-memory-latency"]) == ["kernel_launch_latency"]
    assert tests_run(["--no-cuda"]) == []
    # --cpu names a backend this build does not carry: nothing runs, a note says why, the status is non-zero
    rc, ev = ffi.launch(["--cpu"] + FAST)
    assert rc == 1 and [e["t"] for e in ev] == ["note", "done"] and "CPU backend is not built" in ev[0]["message"]
    rc, ev = ffi.launch(["--cpu", "--cuda", "--kernel-launch-latency"] + FAST)
    assert rc == 0 and any(e["t"] == "note" for e in ev) and any(e["t"] == "metric" for e in ev)
    assert tests_run(["--cuda", "--int-compute", "--no-cublas"]) == [
        "integer_compute", "integer_compute_int8_dp", "wmma_int4", "wmma_int8", "wmma_int8_k32", "wmma_int8_sparse"]
    assert tests_run(["--half-precision-compute", "--double-precision-compute", "--mixed-precision-compute",
                      "--bfloat16-compute"]) == ["bfloat16_compute", "double_precision_compute",
                                                 "half_precision_compute", "mixed_precision_compute"]
    assert tests_run(["--bandwidth", "--no-global-memory-bandwidth", "--no-transfer-bandwidth"]) == [
        "image_memory_bandwidth", "local_memory_bandwidth"]
    rc, ev = ffi.launch(["--integer-compute", "--int8-dot-product-compute", "--local-memory-bandwidth",
                         "--image-memory-bandwidth", "--half-precision-compute", *FAST])
    rows = {(e["test"], e["metric"]): e for e in ev if e["t"] == "metric"}
    for key in (("integer_compute", "int"), ("integer_compute_int8_dp", "int8_dp"), ("integer_compute_int8_dp", "int8_dp8"),
                ("half_precision_compute", "half2"), ("local_memory_bandwidth", "float4"),
                ("image_memory_bandwidth", "float4")):
        assert rows[key]["status"] == "ok" and rows[key]["value"] > 0, rows[key]
    assert rows[("integer_compute", "int")]["unit"] == "gops" and rows[("local_memory_bandwidth", "float")]["unit"] == "gbps"
    both = tests_run(["--wmma", "--no-fp-compute"])
    assert "wmma_int8_k32" in both and "wmma_bf16" not in both


def test_busy_and_cancel(ffi, one_device):
    seen = {}
    results = {}

    def on_event(ev):
        if ev["t"] == "test_begin" and "second" not in seen:
            seen["second"] = True
            rc2, ev2 = ffi.launch(["--kernel-launch-latency"])
            results["busy"] = (rc2, ev2)
            ffi.lib.clpeak_request_cancel()

    rc, ev = ffi.launch(["--cuda", "--wmma", *FAST], on_event)
    assert results["busy"] == (-3, [])                        # BUSY, and no done event for the refused call
    assert rc == -2 and ev[-1] == {"t": "done", "status": -2, "cancelled": True}
    assert kinds(ev).count("test_begin") < 5                  # the rest of the plan was dropped
    rc, ev = ffi.launch(["--kernel-launch-latency", *FAST])   # the flag resets on the next launch
    assert rc == 0 and ev[-1]["cancelled"] is False


def test_multi_device_run(ffi, monkeypatch, tmp_path):
    monkeypatch.setenv("CLPK_FAKE_DEVICES", "3")
    js = tmp_path / "run.json"
    rc, ev = ffi.launch(["--cuda", "--wmma", "--global-memory-bandwidth", "--kernel-launch-latency", "--no-int-compute",
                         *FAST, "--json-file", str(js)])
    assert rc == 0
    devs = [e for e in ev if e["t"] == "device"]
    assert [d["device"] for d in devs] == ["FAKE B200 #0", "FAKE B200 #1", "FAKE B200 #2", "FAKE B200 x3 (box aggregate)"]
    assert [d["device_index"] for d in devs] == [0, 1, 2, -1]
    # one open test at a time, scopes properly nested
    depth = 0
    for e in ev:
        if e["t"] == "test_begin":
            assert depth == 0
            depth = 1
        elif e["t"] == "test_end":
            assert depth == 1
            depth = 0
        elif e["t"] == "metric":
            assert depth == 1
    per_dev = {}
    for e in ev:
        if e["t"] == "metric" and e["status"] == "ok":
            per_dev.setdefault(e["device"], {})[(e["test"], e["metric"])] = e["value"]
    agg = per_dev["FAKE B200 x3 (box aggregate)"]
    key = ("wmma_bf16", "wmma_bf16")
    singles = [per_dev[f"FAKE B200 #{i}"][key] for i in range(3)]
    assert 0.5 * sum(singles) < agg[key] <= 3.0 * max(singles) * 1.01
    lat = ("kernel_launch_latency", "roundtrip")
    assert agg[lat] == pytest.approx(sum(per_dev[f"FAKE B200 #{i}"][lat] for i in range(3)) / 3)
    doc = json.loads(js.read_text())
    assert len(doc["devices"]) == 4 and len({e["device"] for e in doc["entries"]}) == 4

    rc, ev = ffi.launch(["--cuda", "--cuda-device", "1", "--kernel-launch-latency", *FAST])
    (d,) = [e for e in ev if e["t"] == "device"]
    assert d["device"] == "FAKE B200" and d["device_index"] == 1          # a single selected GPU keeps its plain name


def test_cli_text_output_and_compare(ffi, one_device, tmp_path):
    base = tmp_path / "base.csv"
    out = subprocess.run([str(ffi.exe), "--cuda", "--kernel-launch-latency", "--wmma", "--no-fp-compute", *FAST,
                          "--csv-file", str(base)], capture_output=True, text=True, check=True).stdout
    assert "Backend: CUDA" in out and "Device 0: FAKE B200" in out
    assert "Kernel launch latency (US)" in out and "roundtrip" in out and "[unsupported]" in out
    head = base.read_text().splitlines()[0]
    assert head.startswith("format_version,backend,platform,device,driver,category,test,metric,unit,status,value,reason")
    out2 = subprocess.run([str(ffi.exe), "--cuda", "--kernel-launch-latency", *FAST, "--compare", str(base), "--describe"],
                          capture_output=True, text=True, check=True).stdout
    assert "(was 5.00, +0.0%)" in out2
    assert "overhead of asking the GPU" in out2                  # --describe prints the test's description
    lst = subprocess.run([str(ffi.exe), "--list-devices"], capture_output=True, text=True, check=True).stdout
    assert "CUDA Device 0: FAKE B200 [sm_100]" in lst
    r = subprocess.run([str(ffi.exe), "--nope"], capture_output=True, text=True)
    assert r.returncode != 0 and "unknown option" in r.stderr


@pytest.mark.skipif(not REF_RESULTS.is_dir(), reason="reference result files not present")
@pytest.mark.parametrize("rel", ["Nvidia/GeForce_RTX_5060.xml", "AMD/Ryzen_Threadripper_PRO_3955WX_16_Cores.xml",
                                 "Apple/M1_Pro.xml"])
def test_reference_result_files_load(ffi, rel):
    """The reference's saved runs are the schema fixtures: they must load, and carry what the GUI reads."""
    src = REF_RESULTS / rel
    doc = json.loads(ffi.take(ffi.lib.clpeak_load_result_file_json(str(src).encode())))
    root = ET.parse(src).getroot()
    n_metrics = len(root.findall(".//metric"))
    assert len(doc["entries"]) == n_metrics
    assert len(doc["devices"]) == len([r for r in root.findall("run") if r.findall("prop")])
    for e, m in zip(doc["entries"], root.findall(".//metric")):
        assert e["metric"] == m.get("name")
        if m.get("status"):
            assert e["status"] == m.get("status") and e["reason"] == m.get("reason") and "value" not in e
        else:
            assert abs(e["value"] - float(m.text)) <= 1e-4 * max(1.0, abs(float(m.text)))
    cats = {e["category"] for e in doc["entries"]}
    assert cats <= {"fp_compute", "int_compute", "crypto", "string", "bandwidth", "latency"}


def test_xml_save_is_byte_stable_through_load(ffi, one_device, tmp_path):
    """saveXml(loadXml(x)) == x for a file this build wrote (writer and loader agree on every field)."""
    a, b = tmp_path / "a.xml", tmp_path / "b.json"
    ffi.launch(["--cuda", "--wmma", "--no-fp-compute", "--kernel-launch-latency", *FAST, "--xml-file", str(a)])
    doc = json.loads(ffi.take(ffi.lib.clpeak_load_result_file_json(str(a).encode())))
    ffi.launch(["--cuda", "--wmma", "--no-fp-compute", "--kernel-launch-latency", *FAST, "--json-file", str(b)])
    doc_b = json.loads(ffi.take(ffi.lib.clpeak_load_result_file_json(str(b).encode())))
    strip = lambda d: [{k: v for k, v in e.items() if k not in ("value", "metric_description")} for e in d["entries"]]
    assert strip(doc) == strip(doc_b)
    assert doc["devices"] == doc_b["devices"]
    assert ffi.lib.clpeak_load_result_file_json(b"/nonexistent/file.xml") is None
    v1 = tmp_path / "old.json"
    v1.write_text('{"format_version":1,"entries":[\n]}\n')
    assert ffi.lib.clpeak_load_result_file_json(str(v1).encode()) is None
