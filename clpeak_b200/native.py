"""ctypes bindings for the two native libraries.

``kernels()`` loads ``libclpeak_b200_kernels.so`` and declares every symbol of
``include/clpeak_b200_kernels.h``; ``ffi()`` loads ``libclpeak_ffi.so``
(``include/clpeak_ffi.h``).  Loading fails loudly if the library has not been
built -- nothing here substitutes for it.
"""
from __future__ import annotations

import ctypes as C
from functools import lru_cache
from pathlib import Path

LIB_DIR = Path(__file__).resolve().parent / "_lib"

OK, ERR_CUDA, ERR_BAD_ARG, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_NO_DEVICE, ERR_TOO_LARGE = range(7)

DIST_UNIFORM01, DIST_UNIFORM_PM1, DIST_NORMAL = 0, 1, 2
(DT_F32, DT_F16, DT_BF16, DT_E4M3, DT_E5M2, DT_I8, DT_MXF4, DT_NVF4, DT_MXF4_B64, DT_NVF4_B32, DT_TF32,
 DT_E2M1, DT_F64) = range(13)
TUNE_GEMM_NO_ALIGN, TUNE_GEMM_ALIGN_AT, TUNE_GEMM_GROUP, TUNE_MMA_PAIR, TUNE_GEMM_FP4_TILE, TUNE_MMA_LONE_LANE, TUNE_GEMM_NO_PDL = range(7)
STREAM_LDG, STREAM_TMA, STREAM_WIDE = 0, 1, 2
STREAM_VARIANTS = (STREAM_LDG, STREAM_TMA, STREAM_WIDE)
(MMA_F16, MMA_BF16, MMA_E4M3, MMA_E5M2, MMA_I8, MMA_MXF4, MMA_NVF4,
 MMA_E4M3_SP, MMA_MXF4_SP, MMA_NVF4_SP, MMA_I8_SP, MMA_TF32, MMA_F16_F16, MMA_E2M1) = range(14)

(CHAIN_HALF, CHAIN_HALF2, CHAIN_DOUBLE, CHAIN_MIXED, CHAIN_BF16, CHAIN_INT32, CHAIN_INT8_DOT1, CHAIN_INT8_DOT2,
 CHAIN_INT8_DOT4, CHAIN_INT8_DOT8) = range(10)
CHAIN_NAMES = {CHAIN_HALF: "half", CHAIN_HALF2: "half2", CHAIN_DOUBLE: "double", CHAIN_MIXED: "mp", CHAIN_BF16: "bf16",
               CHAIN_INT32: "int", CHAIN_INT8_DOT1: "int8_dp", CHAIN_INT8_DOT2: "int8_dp2", CHAIN_INT8_DOT4: "int8_dp4",
               CHAIN_INT8_DOT8: "int8_dp8"}

MMA_KIND_NAMES = {
    MMA_F16: "fp16", MMA_BF16: "bf16", MMA_E4M3: "fp8_e4m3", MMA_E5M2: "fp8_e5m2", MMA_I8: "int8",
    MMA_MXF4: "mxf4_e2m1", MMA_NVF4: "nvf4_e2m1", MMA_E4M3_SP: "fp8_e4m3_sparse",
    MMA_MXF4_SP: "mxf4_sparse", MMA_NVF4_SP: "nvf4_sparse", MMA_I8_SP: "int8_sparse",
    MMA_TF32: "tf32", MMA_F16_F16: "fp16_f16acc", MMA_E2M1: "fp4_e2m1",
}


class ClpkError(RuntimeError):
    def __init__(self, code: int, detail: str, what: str):
        super().__init__(f"{what} failed with status {code}: {detail}")
        self.code = code
        self.detail = detail


class DeviceInfo(C.Structure):
    _fields_ = [
        ("name", C.c_char * 256),
        ("cc_major", C.c_int), ("cc_minor", C.c_int),
        ("num_sms", C.c_int),
        ("total_mem_bytes", C.c_uint64),
        ("driver_version", C.c_int), ("runtime_version", C.c_int),
        ("sm_clock_khz", C.c_int), ("mem_clock_khz", C.c_int),
        ("mem_bus_bits", C.c_int), ("l2_bytes", C.c_int), ("smem_optin_bytes", C.c_int),
    ]


class MmaPeakArgs(C.Structure):
    _fields_ = [
        ("kind", C.c_int),
        ("d_a", C.c_void_p), ("d_b", C.c_void_p), ("d_sfa", C.c_void_p), ("d_sfb", C.c_void_p),
        ("d_meta", C.c_void_p),
        ("n_mma", C.c_uint32), ("grid", C.c_uint32), ("n_out_tiles", C.c_uint32),
        ("d_out", C.c_void_p), ("d_checksum", C.c_void_p), ("d_status", C.c_void_p),
        ("d_clock", C.c_void_p),
    ]


class GemmArgs(C.Structure):
    _fields_ = [
        ("dtype", C.c_int),
        ("m", C.c_uint32), ("n", C.c_uint32), ("k", C.c_uint32),
        ("d_a", C.c_void_p), ("d_b", C.c_void_p), ("d_c", C.c_void_p),
        ("d_sfa", C.c_void_p), ("d_sfb", C.c_void_p),
        ("alpha", C.c_float),
        ("d_workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("d_status", C.c_void_p),
    ]


_vp, _u64, _u32, _i, _f = C.c_void_p, C.c_uint64, C.c_uint32, C.c_int, C.c_float

# name -> argtypes; every function returns int unless listed in _RESTYPES.
KERNEL_API = {
    "clpk_last_error": [],
    "clpk_version": [],
    "clpk_device_count": [C.POINTER(_i)],
    "clpk_device_info": [_i, C.POINTER(DeviceInfo)],
    "clpk_set_device": [_i],
    "clpk_malloc": [C.POINTER(_vp), C.c_size_t],
    "clpk_free": [_vp],
    "clpk_malloc_host": [C.POINTER(_vp), C.c_size_t],
    "clpk_free_host": [_vp],
    "clpk_memset": [_vp, _i, C.c_size_t, _vp],
    "clpk_memcpy_h2d": [_vp, _vp, C.c_size_t, _vp],
    "clpk_memcpy_d2h": [_vp, _vp, C.c_size_t, _vp],
    "clpk_memcpy_d2d": [_vp, _vp, C.c_size_t, _vp],
    "clpk_stream_create": [C.POINTER(_vp)],
    "clpk_stream_destroy": [_vp],
    "clpk_stream_sync": [_vp],
    "clpk_event_create": [C.POINTER(_vp)],
    "clpk_event_destroy": [_vp],
    "clpk_event_record": [_vp, _vp],
    "clpk_event_sync": [_vp],
    "clpk_event_elapsed_ms": [_vp, _vp, C.POINTER(_f)],
    "clpk_flush_l2": [_vp, C.c_size_t, _vp],
    "clpk_fill_f32": [_vp, _u64, _u64, _i, _f, _f, _vp],
    "clpk_fill_i8": [_vp, _u64, _u64, _vp],
    "clpk_convert_f32": [_vp, _vp, _u64, _i, _vp],
    "clpk_absmax_f32": [_vp, _vp, _u64, _vp],
    "clpk_quantize_fp4": [_vp, _vp, _vp, _u64, _u64, _i, _f, _vp],
    "clpk_global_bandwidth": [_i, _vp, _vp, _u64, _vp],
    "clpk_stream_read_grid": [_i, C.POINTER(_i)],
    "clpk_stream_read": [_i, _vp, _u64, _vp, _vp],
    "clpk_stream_copy": [_i, _vp, _vp, _u64, _vp],
    "clpk_stream_triad": [_i, _vp, _vp, _vp, _f, _u64, _vp],
    "clpk_stream_status": [C.POINTER(_u32), _vp],
    "clpk_stream_checksum_static": [_vp, _u64, _u32, _vp, _vp],
    "clpk_compute_sp": [_vp, _f, _u32, _vp],
    "clpk_mad_chain": [_vp, _u64, _u64, _f, _u32, _vp],
    "clpk_compute_chain": [_i, _vp, C.c_double, _u32, _vp],
    "clpk_compute_chain_info": [_i, C.POINTER(_u32), C.POINTER(_u32)],
    "clpk_local_bandwidth": [_i, _vp, _u32, _vp],
    "clpk_image_create": [C.POINTER(_vp), _u32, _u32, _u64, _vp],
    "clpk_image_bandwidth": [_vp, _vp, _u32, _vp],
    "clpk_image_bandwidth_tiled": [_vp, _vp, _u32, _vp],
    "clpk_image_destroy": [_vp],
    "clpk_pointer_chase": [_vp, _u32, _u64, _vp, _vp],
    "clpk_build_chase_cycle": [_vp, _u64, _u64],
    "clpk_launch_noop": [_vp],
    "clpk_launch_latency": [_u32, _u32, C.POINTER(C.c_double), _vp],
    "clpk_graph_launch_latency": [_u32, _u32, _u32, C.POINTER(C.c_double), _vp],
    "clpk_mma_peak": [C.POINTER(MmaPeakArgs), _vp],
    "clpk_dmma_peak": [_vp, _vp, _u32, _u32, _u32, _vp, _vp, _vp],
    "clpk_mma_kind_k": [_i],
    "clpk_mma_flops_per_instr": [_i],
    "clpk_gemm_workspace_bytes": [_i, _u32, _u32, _u32, C.POINTER(C.c_size_t)],
    "clpk_gemm": [C.POINTER(GemmArgs), _vp],
    "clpk_gemm_pack_scales": [C.POINTER(GemmArgs), _vp],
    "clpk_gemm_last_launch_aligned": [],
    "clpk_gemm_last_clock": [C.POINTER(C.c_ulonglong), C.POINTER(C.c_ulonglong), _vp],
    "clpk_set_tuning": [_i, _i],
    "clpk_get_tuning": [_i, C.POINTER(_i)],
}
_RESTYPES = {
    "clpk_last_error": C.c_char_p,
    "clpk_version": C.c_char_p,
    "clpk_mma_flops_per_instr": C.c_double,
}

FFI_API = {
    "clpeak_version": ([], C.c_char_p),
    "clpeak_copy_backend_catalog_json": ([], C.c_void_p),
    "clpeak_free_string": ([C.c_void_p], None),
    "clpeak_launch": ([C.c_int, C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p], C.c_int),
    "clpeak_request_cancel": ([], None),
    "clpeak_load_result_file_json": ([C.c_char_p], C.c_void_p),
}
EVENT_CALLBACK = C.CFUNCTYPE(None, C.c_void_p, C.c_void_p)


class Kernels:
    """Checked calls into libclpeak_b200_kernels.so."""

    def __init__(self, path: Path):
        if not path.exists():
            raise FileNotFoundError(
                f"{path} is missing: build it with `python -m clpeak_b200.build` (needs nvcc); "
                "there is no fallback implementation")
        self.path = path
        self.lib = C.CDLL(str(path))
        for name, argtypes in KERNEL_API.items():
            fn = getattr(self.lib, name)          # AttributeError if the export is missing
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, C.c_int)

    def last_error(self) -> str:
        return (self.lib.clpk_last_error() or b"").decode()

    def raw(self, name: str):
        return getattr(self.lib, name)

    def call(self, name: str, *args):
        rc = getattr(self.lib, name)(*args)
        if rc != OK:
            raise ClpkError(rc, self.last_error(), name)

    def __getattr__(self, name: str):
        if name.startswith("clpk_"):
            return lambda *a: self.call(name, *a)
        raise AttributeError(name)


@lru_cache(maxsize=None)
def kernels() -> Kernels:
    return Kernels(LIB_DIR / "libclpeak_b200_kernels.so")


@lru_cache(maxsize=None)
def ffi() -> C.CDLL:
    path = LIB_DIR / "libclpeak_ffi.so"
    if not path.exists():
        raise FileNotFoundError(f"{path} is missing: build it with `python -m clpeak_b200.build`")
    lib = C.CDLL(str(path))
    for name, (argtypes, restype) in FFI_API.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = restype
    return lib
