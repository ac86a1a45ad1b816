"""The launcher for the reference's own CUDA kernels (oracle/ref_cuda_runner.cpp) writes a
result file that `clpeak --compare` matches by backend / device / category / test /
metric.  This checks, on the CPU and against the test double of the kernel shim, that
every row the launcher can emit has a row with the same category, test tag, metric
label and unit in this backend's own output -- otherwise the comparison would silently
show nothing for it.  Tags and labels are the reference's: src/cuda/wmma.cpp:29-417,
src/cuda/compute_float.cpp:15-120, src/cuda/compute_int.cpp:18-57,
src/cuda/global_bandwidth.cpp:19, src/cuda/local_bandwidth.cpp:9,
src/cuda/image_bandwidth.cpp:9, src/cuda/kernel_latency.cpp:12."""
import re
from pathlib import Path

import pytest

from tests.host_fake import FakeFfi

ROOT = Path(__file__).resolve().parent.parent
SRC = (ROOT / "oracle" / "ref_cuda_runner.cpp").read_text()

CATEGORY = {"gflops": "fp_compute", "tflops": "fp_compute", "gops": "int_compute", "tops": "int_compute",
            "gbps": "bandwidth", "us": "latency"}


def runner_rows():
    """(test, label, unit, skipped) for every row of the launcher's tables."""
    rows = []
    table = SRC[SRC.index("const ComputeRow kComputeRows[]"):]
    table = table[:table.index("};")]
    for m in re.finditer(r'\{"(\w+)", "(\w+)", "(\w*)", "(\w*)", "(\w+)",[^}]*?(nullptr|kNeeds120|"[^"]+")\}', table, re.S):
        test, label, _module, _kernel, unit, skip = m.groups()
        rows.append((test, label, unit, skip != "nullptr"))
    for test, labels in (("global_memory_bandwidth", ("float", "float2", "float4")),
                         ("local_memory_bandwidth", ("float", "float2", "float4")),
                         ("image_memory_bandwidth", ("float4",))):
        assert f'"{test}"' in SRC
        rows += [(test, lb, "gbps", False) for lb in labels]
    assert '"kernel_launch_latency"' in SRC
    rows.append(("kernel_launch_latency", "roundtrip", "us", False))
    return rows


@pytest.fixture(scope="module")
def backend_metrics():
    import os
    os.environ["CLPK_FAKE_DEVICES"] = "1"
    try:
        rc, ev = FakeFfi().launch(["--cuda", "-i", "1", "-w", "0"])
    finally:
        os.environ.pop("CLPK_FAKE_DEVICES", None)
    assert rc == 0
    return {(m["category"], m["test"], m["metric"]): m for m in ev if m["t"] == "metric"}


def test_table_is_parsed_whole():
    rows = runner_rows()
    assert len(rows) == 27 + 3 + 3 + 1 + 1
    assert sum(1 for r in rows if r[3]) == 6          # five fp4 block-scale rows and int4
    assert len({(r[0], r[1]) for r in rows}) == len(rows)


def test_every_launcher_row_has_a_backend_row(backend_metrics):
    missing = []
    for test, label, unit, _skipped in runner_rows():
        key = (CATEGORY[unit], test, label)
        if key not in backend_metrics:
            missing.append(key)
        else:
            assert backend_metrics[key]["unit"] == unit, key
    assert not missing, f"rows the comparison cannot match: {missing}"


def test_rows_the_reference_skips_here_are_rows_this_backend_runs(backend_metrics):
    """The fp4 / block-scaled rows are the point of the sm_100a backend: they must be `ok` here."""
    for test, label, unit, skipped in runner_rows():
        if skipped and label != "int4":
            assert backend_metrics[(CATEGORY[unit], test, label)]["status"] == "ok", (test, label)
