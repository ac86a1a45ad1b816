"""The backend's own host references (product code, host_check.hpp) against the CPU oracle."""
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_backend_host_references_agree_with_the_oracle(orc):
    out = ROOT / "tests" / "_build"
    out.mkdir(exist_ok=True)
    exe = out / "cross_check"
    src = ROOT / "tests" / "host_check" / "cross_check.cpp"
    subprocess.run(["g++", "-O1", "-std=c++17", "-ffp-contract=off", "-I", str(ROOT / "include"),
                    "-I", str(ROOT / "clpeak_b200" / "csrc" / "host"), "-I", str(ROOT / "clpeak_b200" / "csrc"),
                    "-o", str(exe), str(src), str(ROOT / "clpeak_b200" / "csrc" / "host" / "core.cpp"),
                    str(ROOT / "oracle" / "_build" / "liboracle.so"),
                    f"-Wl,-rpath,{ROOT / 'oracle' / '_build'}", "-lm", "-pthread"], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-3000:]
    assert r.stdout.count(" ok") >= 27


def test_start_gate_meets_times_out_and_releases_on_leave():
    """The gate the device threads of the multi-GPU driver meet at (before each test and before each
    timed batch): never a deadlock when a thread is missing."""
    out = ROOT / "tests" / "_build"
    out.mkdir(exist_ok=True)
    exe = out / "gate_check"
    subprocess.run(["g++", "-O1", "-std=c++17", "-pthread", "-I", str(ROOT / "clpeak_b200" / "csrc" / "host"),
                    "-o", str(exe), str(ROOT / "tests" / "host_check" / "gate_check.cpp")], check=True)
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout
    assert r.stdout.count(" ok") == 6
