"""The allocation-free checksum entry point against the ordinary streaming read.

clpk_stream_checksum_static exists for callers that cannot allocate device memory
when they need the result (no cudaMalloc allowed at that point: a host that
forbids allocator calls after start-up, a region that must not take cudaMalloc's
implicit synchronisation, a fully handed-out memory pool).  Its scratch is a
fixed array inside the library, shared by every call on the device, so this test
makes two calls in a row -- on different data and sizes -- and checks each,
bit for bit, against clpk_stream_read through the same C ABI.  The file sorts
last on purpose: with `-x` every other test has already run when it starts.
"""
import ctypes as C

import numpy as np
import pytest

from clpeak_b200 import native as N
from tests.gpu_util import dev_empty, stream_ptr, sync, to_np

pytestmark = pytest.mark.gpu


def reference_xor(K, cuda, d_src, n_bytes):
    grid = C.c_int(0)
    K.clpk_stream_read_grid(N.STREAM_LDG, C.byref(grid))
    parts = dev_empty(grid.value, cuda.int32)
    K.clpk_stream_read(N.STREAM_LDG, d_src.data_ptr(), n_bytes, parts.data_ptr(), stream_ptr())
    sync()
    return int(np.bitwise_xor.reduce(to_np(parts).view(np.uint32)))


def test_static_scratch_checksum_matches_stream_read_twice_in_a_row(K, cuda):
    out = dev_empty(1, cuda.int32)                      # the caller's output word
    cases = [((192 << 20) + 4096 + 48, 31, 0), ((64 << 20) + 16, 32, 37), (0, 33, 0)]
    for n_bytes, seed, grid in cases:
        src = dev_empty(max(n_bytes // 4, 4), cuda.float32)
        K.clpk_fill_f32(src.data_ptr(), src.numel(), seed, N.DIST_UNIFORM01, 0.0, 1.0, stream_ptr())
        want = reference_xor(K, cuda, src, n_bytes)
        out.fill_(-1)
        K.clpk_stream_checksum_static(src.data_ptr(), n_bytes, grid, out.data_ptr(), stream_ptr())
        sync()
        got = int(to_np(out).view(np.uint32)[0])
        assert got == want, f"n_bytes={n_bytes} grid={grid}: {got:#x} vs {want:#x}"


def test_static_scratch_capacity_is_enforced(K, cuda):
    src = dev_empty(1024, cuda.float32)
    out = dev_empty(1, cuda.int32)
    with pytest.raises(N.ClpkError) as e:
        K.clpk_stream_checksum_static(src.data_ptr(), 4096, 4097, out.data_ptr(), stream_ptr())
    assert e.value.code == N.ERR_TOO_LARGE and "4096" in e.value.detail
    K.clpk_stream_checksum_static(src.data_ptr(), 4096, 4096, out.data_ptr(), stream_ptr())    # the limit itself is fine
    sync()
