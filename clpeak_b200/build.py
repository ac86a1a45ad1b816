"""Builds the native parts of clpeak_b200 in-tree with nvcc / g++.

Outputs (all under clpeak_b200/_lib/, which is not tracked):
  libclpeak_b200_kernels.so  the sm_100a kernels behind the C ABI of
                             include/clpeak_b200_kernels.h
  libclpeak_ffi.so           the host side (options, logger, result store, the
                             B200 backend) behind the clpeak_ffi C ABI of
                             include/clpeak_ffi.h
  clpeak                     the command-line front end

Only sm_100a code is generated.  Run as `python -m clpeak_b200.build`.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
ROOT = PKG.parent
CSRC = PKG / "csrc"
LIB = PKG / "_lib"
OBJ = LIB / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC,-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-pthread", "-Wall", "-Wextra",
             "-Wno-unused-parameter"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found")


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {cmd[0]} ... {cmd[-1]}")


def build_kernels(force: bool = False) -> Path:
    OBJ.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()
    headers = sorted(CSRC.glob("*.h")) + sorted(CSRC.glob("*.cuh")) + [ROOT / "include" / "clpeak_b200_kernels.h"]
    sources = sorted((CSRC / "kernels").glob("*.cu"))
    jobs = []
    objs = []
    for src in sources:
        obj = OBJ / (src.stem + ".o")
        objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append([nvcc, *NVCC_FLAGS, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    so = LIB / "libclpeak_b200_kernels.so"
    if force or jobs or _stale(so, objs):
        _run([nvcc, "-shared", "-o", str(so), *map(str, objs), "-cudart", "static", "-Xlinker", "--exclude-libs,ALL"])
    return so


def build_host(force: bool = False) -> list[Path]:
    host = CSRC / "host"
    sources = sorted(host.glob("*.cpp"))
    if not sources:
        return []
    OBJ.mkdir(parents=True, exist_ok=True)
    cxx = os.environ.get("CXX") or shutil.which("g++") or "g++"
    headers = sorted(host.glob("*.h")) + sorted(host.glob("*.hpp")) + sorted((ROOT / "include").glob("*.h")) + \
        sorted(CSRC.glob("*.h"))
    inc = ["-I", str(ROOT / "include"), "-I", str(CSRC), "-I", str(host)]
    jobs, objs = [], []
    for src in sources:
        obj = OBJ / ("host_" + src.stem + ".o")
        if src.stem != "cli_main":
            objs.append(obj)
        if force or _stale(obj, [src] + headers):
            jobs.append([cxx, *CXX_FLAGS, *inc, "-c", str(src), "-o", str(obj)])
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(_run, jobs))
    outs = []
    ffi = LIB / "libclpeak_ffi.so"
    link_kernels = ["-L", str(LIB), "-lclpeak_b200_kernels", "-Wl,-rpath,$ORIGIN"]
    if force or jobs or _stale(ffi, objs):
        # --exclude-libs keeps a statically linked libstdc++ from leaking its symbols: the
        # library exports the clpeak_* C symbols and nothing else.
        _run([cxx, "-shared", "-pthread", "-Wl,--exclude-libs,ALL", "-o", str(ffi), *map(str, objs), *link_kernels,
              "-ldl"])
    outs.append(ffi)
    cli_obj = OBJ / "host_cli_main.o"
    if cli_obj.exists():
        exe = LIB / "clpeak"
        if force or jobs or _stale(exe, [cli_obj, ffi]):
            # libclpeak_ffi.so exports only its six C symbols (like the reference's), so the CLI
            # links the host objects themselves.
            core = [o for o in objs if o.name != "host_ffi.o"]
            _run([cxx, "-pthread", "-o", str(exe), str(cli_obj), *map(str, core), "-L", str(LIB),
                  "-lclpeak_b200_kernels", "-Wl,-rpath,$ORIGIN", "-ldl"])
        outs.append(exe)
    return outs


def build_all(force: bool = False) -> None:
    build_kernels(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built:", *(p.name for p in sorted(LIB.iterdir()) if p.is_file()))
