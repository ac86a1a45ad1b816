"""Builds the C++ host side against the CPU test double of the kernel shim
(tests/fake_shim/fake_kernels.cpp) so that clpeak_launch and the CLI can run
without a GPU.  Output goes to tests/_build/ (not tracked)."""
import ctypes as C
import json
import os
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
HOST = ROOT / "clpeak_b200" / "csrc" / "host"
OUT = ROOT / "tests" / "_build"


def build():
    OUT.mkdir(exist_ok=True)
    srcs = sorted(p for p in HOST.glob("*.cpp") if p.name != "cli_main.cpp")
    fake = ROOT / "tests" / "fake_shim" / "fake_kernels.cpp"
    deps = srcs + [fake, HOST / "cli_main.cpp"] + list(HOST.glob("*.hpp")) + list(HOST.glob("*/*.h")) + \
        [ROOT / "include" / "clpeak_b200_kernels.h", ROOT / "include" / "clpeak_ffi.h"]
    so, exe = OUT / "libclpeak_ffi_fake.so", OUT / "clpeak_fake"
    newest = max(p.stat().st_mtime for p in deps)
    if so.exists() and exe.exists() and min(so.stat().st_mtime, exe.stat().st_mtime) > newest:
        return so, exe
    flags = ["-O1", "-std=c++17", "-fPIC", "-pthread", "-fvisibility=hidden", "-I", str(ROOT / "include"),
             "-I", str(HOST.parent), "-I", str(HOST)]
    subprocess.run(["g++", *flags, "-shared", "-Wl,--exclude-libs,ALL", "-o", str(so), *map(str, srcs), str(fake)],
                   check=True)
    subprocess.run(["g++", *flags, "-o", str(exe), str(HOST / "cli_main.cpp"),
                    *[str(s) for s in srcs if s.name != "ffi.cpp"], str(fake)], check=True)
    return so, exe


CALLBACK = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class FakeFfi:
    def __init__(self):
        so, self.exe = build()
        self.lib = C.CDLL(str(so))
        self.lib.clpeak_version.restype = C.c_char_p
        self.lib.clpeak_copy_backend_catalog_json.restype = C.c_void_p
        self.lib.clpeak_free_string.argtypes = [C.c_void_p]
        self.lib.clpeak_launch.argtypes = [C.c_int, C.POINTER(C.c_char_p), CALLBACK, C.c_void_p]
        self.lib.clpeak_load_result_file_json.argtypes = [C.c_char_p]
        self.lib.clpeak_load_result_file_json.restype = C.c_void_p

    def take(self, p):
        if not p:
            return None
        s = C.string_at(p).decode()
        self.lib.clpeak_free_string(p)
        return s

    def launch(self, argv, on_event=None):
        events = []

        def cb(_ud, p):
            ev = json.loads(self.take(p))
            events.append(ev)
            if on_event:
                on_event(ev)

        args = [b"clpeak"] + [a.encode() for a in argv]
        arr = (C.c_char_p * len(args))(*args)
        rc = self.lib.clpeak_launch(len(args), arr, CALLBACK(cb), None)
        return rc, events
