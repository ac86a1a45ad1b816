"""Drop-in proof: the reference project's own CLI and common library (argument
parser, logger, result writers -- compiled unmodified from where they lie) take
this repository's CudaPeak in their CUDA slot.  Only the backend source
(host/b200_peak.cpp + host/cuda/cuda_peak.h) comes from here; the kernel shim is
the CPU test double, so the binary runs without a GPU."""
import os
import shutil
import subprocess
import xml.etree.ElementTree as ET
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
REF = Path(os.environ.get("CLPEAK_REFERENCE_DIR", "/root/reference"))
OUT = ROOT / "tests" / "_build" / "dropin"

pytestmark = pytest.mark.skipif(not (REF / "src" / "cli" / "main.cpp").exists(), reason="reference tree not present")


@pytest.fixture(scope="module")
def ref_cli_with_b200_backend():
    inc = OUT / "inc"
    (inc / "cuda").mkdir(parents=True, exist_ok=True)
    # only the backend's own header is placed ahead of the reference's include tree
    shutil.copy(ROOT / "clpeak_b200/csrc/host/cuda/cuda_peak.h", inc / "cuda" / "cuda_peak.h")
    (inc / "version.h").write_text('#pragma once\n#define CLPEAK_VERSION_STR "2.0.16"\n')
    exe = OUT / "clpeak_ref_with_b200"
    srcs = [REF / "src/cli/main.cpp", *sorted((REF / "src/common").glob("*.cpp")),
            ROOT / "clpeak_b200/csrc/host/b200_peak.cpp", ROOT / "tests/fake_shim/fake_kernels.cpp"]
    newest = max(p.stat().st_mtime for p in srcs + [ROOT / "clpeak_b200/csrc/host/cuda/cuda_peak.h"])
    if not exe.exists() or exe.stat().st_mtime < newest:
        subprocess.run(["g++", "-std=c++17", "-O1", "-pthread", "-DENABLE_CUDA", "-I", str(inc),
                        "-I", str(REF / "include"), "-I", str(REF / "include/common"), "-I", str(ROOT / "include"),
                        "-o", str(exe), *map(str, srcs), "-ldl"], check=True)
    return exe


def test_backend_compiles_against_reference_headers_only(ref_cli_with_b200_backend):
    deps = subprocess.run(["g++", "-std=c++17", "-M", "-DENABLE_CUDA", "-I", str(OUT / "inc"), "-I", str(REF / "include"),
                           "-I", str(REF / "include/common"), "-I", str(ROOT / "include"),
                           str(ROOT / "clpeak_b200/csrc/host/b200_peak.cpp")], capture_output=True, text=True,
                          check=True).stdout
    assert f"{REF}/include/common/peak.h" in deps and f"{REF}/include/common/logger.h" in deps
    assert "clpeak_api.hpp" not in deps              # none of this repository's contract header was needed


def test_reference_cli_runs_the_b200_backend(ref_cli_with_b200_backend, tmp_path):
    xml = tmp_path / "run.xml"
    env = dict(os.environ, CLPK_FAKE_DEVICES="2")
    out = subprocess.run([str(ref_cli_with_b200_backend), "--cuda", "--kernel-launch-latency", "--wmma",
                          "--no-fp-compute", "-i", "1", "-w", "0", "--xml-file", str(xml)],
                         capture_output=True, text=True, check=True, env=env).stdout
    assert "Backend: CUDA" in out and "Device 0: FAKE B200 #0" in out and "Device 1: FAKE B200 #1" in out
    assert "box aggregate" in out and "int8_k32" in out and "roundtrip" in out
    root = ET.parse(xml).getroot()               # written by the reference's own saveXml
    runs = root.findall("run")
    assert [r.get("device") for r in runs] == ["FAKE B200 #0", "FAKE B200 #1", "FAKE B200 x2 (box aggregate)"]
    assert runs[0].find("./category[@name='latency']/test[@name='kernel_launch_latency']/metric[@name='roundtrip']") is not None
    lst = subprocess.run([str(ref_cli_with_b200_backend), "--list-devices"], capture_output=True, text=True, env=env).stdout
    assert "CUDA Device 1: FAKE B200 [sm_100]" in lst
