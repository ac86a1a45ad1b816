"""The C-ABI libraries load and export exactly what include/*.h declares.
No compute entry point is called here (there is no GPU on this side)."""
import ctypes as C
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def declared(header: str, macro: str):
    text = (ROOT / "include" / header).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = "\n".join(ln for ln in text.splitlines() if not ln.lstrip().startswith("#"))
    return sorted(set(re.findall(macro + r"[^;(]*?\b(\w+)\s*\(", text)))


def exported(lib: Path):
    out = subprocess.run(["nm", "-D", "--defined-only", str(lib)], capture_output=True, text=True, check=True).stdout
    return sorted(line.split()[-1] for line in out.splitlines() if " T " in line)


def test_kernel_shim_exports_match_header(K):
    names = declared("clpeak_b200_kernels.h", "CLPK_API")
    assert len(names) >= 40
    assert exported(K.path) == names


def test_python_binding_covers_every_declared_symbol():
    from clpeak_b200 import native
    assert sorted(native.KERNEL_API) == declared("clpeak_b200_kernels.h", "CLPK_API")
    assert sorted(native.FFI_API) == declared("clpeak_ffi.h", "CLPEAK_FFI_EXPORT")


def test_ffi_library_exports_exactly_the_six_symbols():
    from clpeak_b200 import build, native
    lib = native.LIB_DIR / "libclpeak_ffi.so"
    if not lib.exists():
        build.build_all()
    assert exported(lib) == declared("clpeak_ffi.h", "CLPEAK_FFI_EXPORT")
    assert exported(lib) == sorted(["clpeak_version", "clpeak_copy_backend_catalog_json", "clpeak_free_string",
                                    "clpeak_launch", "clpeak_request_cancel", "clpeak_load_result_file_json"])
    ffi = native.ffi()
    assert ffi.clpeak_version().decode().startswith("2.")


def test_compute_fails_loudly_without_a_gpu(K):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from clpeak_b200 import native
    n = C.c_int(-1)
    rc = K.raw("clpk_device_count")(C.byref(n))
    assert rc in (native.ERR_NO_DEVICE, native.ERR_CUDA) and n.value == 0
    with pytest.raises(native.ClpkError) as e:
        K.clpk_compute_sp(None, 1.0, 1, None)
    assert e.value.code in (native.ERR_NO_DEVICE, native.ERR_CUDA, native.ERR_UNSUPPORTED)


def test_status_helpers_need_no_gpu(K):
    assert K.raw("clpk_mma_kind_k")(1) == 16
    assert K.raw("clpk_mma_flops_per_instr")(1) == 2.0 * 128 * 256 * 16
    assert K.raw("clpk_mma_flops_per_instr")(9) == 2.0 * 128 * 256 * 128      # sparse: logical K
    assert b"sm_100a" in K.raw("clpk_version")()


def test_tuning_knobs_environment_once_then_setter(tmp_path):
    """The CLPK_* environment variables give a knob its default and are read once per process; clpk_set_tuning
    replaces the value afterwards; a negative value means "not set"; unknown knobs are refused.  Run in a child
    process so that the variables are in place before the library's first use of them."""
    import os
    import sys
    code = """
import ctypes as C, os, sys
sys.path.insert(0, sys.argv[1])
from clpeak_b200 import native as N
K = N.kernels()
v = C.c_int(99)
K.clpk_get_tuning(N.TUNE_GEMM_GROUP, C.byref(v)); assert v.value == 5, v.value          # from the environment
K.clpk_get_tuning(N.TUNE_MMA_PAIR, C.byref(v)); assert v.value == -1                     # not set anywhere
os.environ["CLPK_GEMM_GROUP"] = "9"                                                      # too late: read once
K.clpk_get_tuning(N.TUNE_GEMM_GROUP, C.byref(v)); assert v.value == 5
K.clpk_set_tuning(N.TUNE_GEMM_GROUP, 16)
K.clpk_get_tuning(N.TUNE_GEMM_GROUP, C.byref(v)); assert v.value == 16
K.clpk_set_tuning(N.TUNE_GEMM_GROUP, -3)
K.clpk_get_tuning(N.TUNE_GEMM_GROUP, C.byref(v)); assert v.value == -1
for bad in (-1, 7, 1000):
    try:
        K.clpk_set_tuning(bad, 1)
    except N.ClpkError as e:
        assert e.code == N.ERR_BAD_ARG
    else:
        raise AssertionError("knob %d accepted" % bad)
assert K.raw("clpk_gemm_last_launch_aligned")() == -1                                    # nothing launched yet
print("ok")
"""
    script = tmp_path / "knobs.py"
    script.write_text(code)
    env = dict(os.environ, CLPK_GEMM_GROUP="5")
    env.pop("CLPK_MMA_PAIR", None)
    r = subprocess.run([sys.executable, str(script), str(ROOT)], env=env, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stdout + r.stderr
