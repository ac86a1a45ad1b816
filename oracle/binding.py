"""ctypes binding for the CPU oracle (oracle/_build/liboracle.so).

TEST INFRASTRUCTURE: imported by tests/, the smoke check and the CPU-baseline
legs of bench.py only.  Nothing under clpeak_b200/ imports this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from functools import lru_cache
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB = HERE / "_build" / "liboracle.so"

_u64, _u32, _i, _f, _d, _vp = C.c_uint64, C.c_uint32, C.c_int, C.c_float, C.c_double, C.c_void_p

_API = {
    "orc_rand64": ([_u64, _u64], _u64),
    "orc_uniform01": ([_u64, _u64], _f),
    "orc_uniform_pm1": ([_u64, _u64], _f),
    "orc_uniform_i4": ([_u64, _u64], _i),
    "orc_normal01": ([_u64, _u64], _f),
    "orc_fill_f32": ([_vp, _u64, _u64, _u64, _i, _f, _f], None),
    "orc_fill_i8": ([_vp, _u64, _u64, _u64], None),
    "orc_populate_reference": ([_vp, _u64], None),
    "orc_f32_to_bf16": ([_f], C.c_uint16),
    "orc_f32_to_f16": ([_f], C.c_uint16),
    "orc_f32_to_e4m3": ([_f], C.c_uint8),
    "orc_f32_to_e5m2": ([_f], C.c_uint8),
    "orc_f32_to_e2m1": ([_f], C.c_uint8),
    "orc_f32_to_i8": ([_f], C.c_int8),
    "orc_bf16_to_f32": ([C.c_uint16], _f),
    "orc_f16_to_f32": ([C.c_uint16], _f),
    "orc_e4m3_to_f32": ([C.c_uint8], _f),
    "orc_e5m2_to_f32": ([C.c_uint8], _f),
    "orc_e2m1_to_f32": ([C.c_uint8], _f),
    "orc_ue8m0_to_f32": ([C.c_uint8], _f),
    "orc_ue8m0_for_absmax": ([_f], C.c_uint8),
    "orc_convert_f32": ([_vp, _vp, _u64, _i], None),
    "orc_absmax_f32": ([_vp, _u64], _f),
    "orc_quantize_fp4": ([_vp, _vp, _vp, _u64, _u64, _i, _f], None),
    "orc_fp4_element": ([_vp, _vp, _u64, _i, _u64, _u64], _d),
    "orc_prune_2to4": ([_vp, _vp, _vp, _vp, _u64, _u64], None),
    "orc_global_bandwidth": ([_i, _vp, _vp, _u64], None),
    "orc_xor_words": ([_vp, _u64], _u32),
    "orc_triad": ([_vp, _vp, _vp, _f, _u64], None),
    "orc_stream_pass_mt": ([_i, _vp, _vp, _vp, _u64, _i, _i, C.POINTER(_u32)], _d),
    "orc_compute_sp": ([_vp, _f, _u64], None),
    "orc_mad_chain": ([_vp, _u64, _u64, _u64, _f, _u32], None),
    "orc_compute_chain": ([_i, _vp, _d, _u64], None),
    "orc_local_bandwidth": ([_i, _vp, _u64], None),
    "orc_image_bandwidth": ([_vp, _u64, _u64, _u64, _u64, _u64], None),
    "orc_image_bandwidth_tiled": ([_vp, _u64, _u64, _u32, _u32, _u64], None),
    "orc_chase_cycle": ([_vp, _u64, _u64], None),
    "orc_is_single_cycle": ([_vp, _u64], _i),
    "orc_chase": ([_vp, _u32, _u64, C.POINTER(_u32), C.POINTER(_u32)], None),
    "orc_mma_tile": ([_i, _vp, _vp, _vp, _vp, _vp, _vp], None),
    "orc_mma_tile_i8": ([_vp, _vp, _u32, _vp], None),
    "orc_prune_pairs_2to4": ([_vp, _vp, _vp, _vp, _u64, _u64], None),
    "orc_mma_tile_sp": ([_i, _vp, _vp, _vp, _vp, _vp, _vp, _vp], None),
    "orc_gemm_element": ([_i, _vp, _vp, _vp, _vp, _u64, _u64, _u64, C.POINTER(_d)], _d),
    "orc_dmma_tiles": ([_vp, _vp, _u32, _i, _i, _vp], None),
    "orc_pick_iters": ([_d, C.c_uint, C.c_uint, C.c_uint], C.c_uint),
}


def build() -> Path:
    """Compile oracle.c (gcc, seconds).  Raises if the compiler fails."""
    subprocess.run(["make", "-s", "-C", str(HERE), "oracle"], check=True)
    return LIB


@lru_cache(maxsize=None)
def lib() -> C.CDLL:
    if not LIB.exists() or LIB.stat().st_mtime < (HERE / "oracle.c").stat().st_mtime:
        build()
    l = C.CDLL(str(LIB))
    for name, (argtypes, restype) in _API.items():
        fn = getattr(l, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return l


def ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ---- numpy conveniences ---------------------------------------------------------

def fill_f32(n: int, seed: int, dist: int, mean: float = 0.0, std: float = 1.0, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().orc_fill_f32(ptr(out), first, n, seed, dist, mean, std)
    return out


def fill_i8(n: int, seed: int, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.int8)
    lib().orc_fill_i8(ptr(out), first, n, seed)
    return out


_DT_NP = {1: np.uint16, 2: np.uint16, 3: np.uint8, 4: np.uint8, 5: np.int8, 10: np.uint32, 12: np.float64}


def convert_f32(src: np.ndarray, dtype: int) -> np.ndarray:
    """Plain conversions; dtype 10 (TF32) returns the fp32 words, 11 (E2M1) a flat array of n/2 packed bytes."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    if dtype == 11:
        assert src.size % 2 == 0
        out = np.zeros(src.size // 2, dtype=np.uint8)
        lib().orc_convert_f32(ptr(out), ptr(src), src.size, dtype)
        return out
    out = np.empty(src.shape, dtype=_DT_NP[dtype])
    lib().orc_convert_f32(ptr(out), ptr(src), src.size, dtype)
    return out


def quantize_fp4(src: np.ndarray, dtype: int, tensor_scale: float = 1.0):
    src = np.ascontiguousarray(src, dtype=np.float32)
    rows, cols = src.shape
    blk = {6: 32, 7: 16, 8: 64, 9: 32}[dtype]
    packed = np.empty((rows, cols // 2), dtype=np.uint8)
    scales = np.empty((rows, cols // blk), dtype=np.uint8)
    lib().orc_quantize_fp4(ptr(packed), ptr(scales), ptr(src), rows, cols, dtype, tensor_scale)
    return packed, scales


def global_bandwidth(width: int, src: np.ndarray) -> np.ndarray:
    out = np.empty(src.size // (16 * width), dtype=np.float32)
    lib().orc_global_bandwidth(width, ptr(src), ptr(out), src.size)
    return out


def xor_words(a: np.ndarray) -> int:
    return int(lib().orc_xor_words(ptr(a), a.nbytes))


def triad(b: np.ndarray, c: np.ndarray, s: float) -> np.ndarray:
    a = np.empty_like(b)
    lib().orc_triad(ptr(a), ptr(b), ptr(c), s, b.size)
    return a


def compute_sp(a: float, n_threads: int) -> np.ndarray:
    out = np.empty(n_threads, dtype=np.float32)
    lib().orc_compute_sp(ptr(out), a, n_threads)
    return out


def compute_chain(chain: int, a: float, n_threads: int) -> np.ndarray:
    """chain = CLPK_CHAIN_*; float32 output for 0, 1, 3, 4, float64 for 2, int32 for 5..9."""
    dtype = np.float64 if chain == 2 else (np.int32 if chain >= 5 else np.float32)
    out = np.empty(n_threads, dtype=dtype)
    lib().orc_compute_chain(chain, ptr(out), a, n_threads)
    return out


def local_bandwidth(width: int, n_threads: int) -> np.ndarray:
    out = np.empty(n_threads, dtype=np.float32)
    lib().orc_local_bandwidth(width, ptr(out), n_threads)
    return out


def image_bandwidth(n_threads: int, texels: int, seed: int, first: int = 0, count: int | None = None) -> np.ndarray:
    count = n_threads - first if count is None else count
    out = np.empty(count, dtype=np.float32)
    lib().orc_image_bandwidth(ptr(out), first, count, n_threads, texels, seed)
    return out


def image_bandwidth_tiled(n_threads: int, width: int, height: int, seed: int, first: int = 0,
                          count: int | None = None) -> np.ndarray:
    count = n_threads - first if count is None else count
    out = np.empty(count, dtype=np.float32)
    lib().orc_image_bandwidth_tiled(ptr(out), first, count, width, height, seed)
    return out


def mad_chain(n_items: int, seed: int, y: float, iters: int, first: int = 0) -> np.ndarray:
    out = np.empty(n_items, dtype=np.float32)
    lib().orc_mad_chain(ptr(out), first, n_items, seed, y, iters)
    return out


def chase_cycle(n: int, seed: int) -> np.ndarray:
    out = np.empty(n, dtype=np.uint32)
    lib().orc_chase_cycle(ptr(out), n, seed)
    return out


def chase(nxt: np.ndarray, start: int, hops: int):
    f, x = _u32(0), _u32(0)
    lib().orc_chase(ptr(nxt), start, hops, C.byref(f), C.byref(x))
    return int(f.value), int(x.value)


def mma_tile(kind: int, a: np.ndarray, b: np.ndarray, sfa=None, sfb=None):
    p = np.empty((128, 256), dtype=np.float64)
    s = np.empty((128, 256), dtype=np.float64)
    lib().orc_mma_tile(kind, ptr(a), ptr(b), ptr(sfa) if sfa is not None else None,
                       ptr(sfb) if sfb is not None else None, ptr(p), ptr(s))
    return p, s


def mma_tile_i8(a: np.ndarray, b: np.ndarray, n_mma: int) -> np.ndarray:
    out = np.empty((128, 256), dtype=np.int32)
    lib().orc_mma_tile_i8(ptr(a), ptr(b), n_mma, ptr(out))
    return out


def gemm_element(dtype: int, a: np.ndarray, b: np.ndarray, k: int, i: int, j: int, sfa=None, sfb=None):
    s = _d(0.0)
    v = lib().orc_gemm_element(dtype, ptr(a), ptr(b), ptr(sfa) if sfa is not None else None,
                               ptr(sfb) if sfb is not None else None, k, i, j, C.byref(s))
    return float(v), float(s.value)


def prune_2to4(dense: np.ndarray, pairs: bool = False):
    """(compressed, meta bytes, pruned dense) of a [rows][k] float tile; pairs=True for 4-bit operands."""
    dense = np.ascontiguousarray(dense, dtype=np.float32)
    rows, k = dense.shape
    comp = np.zeros((rows, k // 2), dtype=np.float32)
    meta = np.zeros((rows, k // (16 if pairs else 8)), dtype=np.uint8)
    pruned = np.zeros_like(dense)
    fn = lib().orc_prune_pairs_2to4 if pairs else lib().orc_prune_2to4
    fn(ptr(comp), ptr(meta), ptr(pruned), ptr(dense), rows, k)
    return comp, meta, pruned


def mma_tile_sp(kind: int, a_comp: np.ndarray, meta: np.ndarray, b: np.ndarray, sfa=None, sfb=None):
    p = np.empty((128, 256), dtype=np.float64)
    s = np.empty((128, 256), dtype=np.float64)
    lib().orc_mma_tile_sp(kind, ptr(a_comp), ptr(meta), ptr(b), ptr(sfa) if sfa is not None else None,
                          ptr(sfb) if sfb is not None else None, ptr(p), ptr(s))
    return p, s


def dmma_tiles(a: np.ndarray, b: np.ndarray, n_mma: int, warps: int, chains: int) -> np.ndarray:
    out = np.empty((warps, 8, 8), dtype=np.float64)
    lib().orc_dmma_tiles(ptr(a), ptr(b), n_mma, warps, chains, ptr(out))
    return out
