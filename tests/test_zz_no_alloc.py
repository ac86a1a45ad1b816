"""The allocation-free checksum entry point against the ordinary streaming read.

clpk_stream_checksum_static exists for callers that cannot allocate device memory
when they need the result (no cudaMalloc allowed at that point: a host that
forbids allocator calls after start-up, a region that must not take cudaMalloc's
implicit synchronisation, a fully handed-out memory pool).  Its scratch is a
fixed array inside the library, shared by every call on the device, so this test
makes two calls in a row -- on different data and sizes -- and checks each,
bit for bit, against clpk_stream_read through the same C ABI and against the CPU
oracle's XOR of the same words.  It also checks the property the entry point exists
for -- the free device memory does not move across calls -- and that stale partials of
a large grid do not leak into a later call with a small one.  The file sorts
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


def test_static_scratch_checksum_matches_stream_read_twice_in_a_row(K, orc, cuda):
    out = dev_empty(1, cuda.int32)                      # the caller's output word
    cases = [((192 << 20) + 4096 + 48, 31, 0), ((64 << 20) + 16, 32, 37), (0, 33, 0)]
    for n_bytes, seed, grid in cases:
        src = dev_empty(max(n_bytes // 4, 4), cuda.float32)
        K.clpk_fill_f32(src.data_ptr(), src.numel(), seed, N.DIST_UNIFORM01, 0.0, 1.0, stream_ptr())
        want = reference_xor(K, cuda, src, n_bytes)
        host = orc.fill_f32(n_bytes // 4, seed, 0)
        assert want == (orc.xor_words(host) if n_bytes else 0)
        out.fill_(-1)
        K.clpk_stream_checksum_static(src.data_ptr(), n_bytes, grid, out.data_ptr(), stream_ptr())
        sync()
        got = int(to_np(out).view(np.uint32)[0])
        assert got == want, f"n_bytes={n_bytes} grid={grid}: {got:#x} vs {want:#x}"


def test_static_scratch_allocates_nothing_and_ignores_stale_partials(K, orc, cuda):
    """After the first call on the device (which looks the array's address up), further calls leave the
    free-memory figure of the device where it was; a 4096-CTA call followed by a 1-CTA call on other data
    gives that data's checksum, not a mix with the partials the large grid left behind."""
    out = dev_empty(1, cuda.int32)
    big = dev_empty((96 << 20) // 4, cuda.float32)
    small = dev_empty((1 << 20) // 4, cuda.float32)
    K.clpk_fill_f32(big.data_ptr(), big.numel(), 41, N.DIST_UNIFORM01, 0.0, 1.0, stream_ptr())
    K.clpk_fill_f32(small.data_ptr(), small.numel(), 42, N.DIST_UNIFORM01, 0.0, 1.0, stream_ptr())
    K.clpk_stream_checksum_static(small.data_ptr(), small.numel() * 4, 0, out.data_ptr(), stream_ptr())
    sync()
    free_before = cuda.cuda.mem_get_info()[0]
    results = []
    for buf, grid in ((big, 4096), (small, 1), (big, 7), (small, 4096)):
        K.clpk_stream_checksum_static(buf.data_ptr(), buf.numel() * 4, grid, out.data_ptr(), stream_ptr())
        sync()
        results.append(int(to_np(out).view(np.uint32)[0]))
    assert cuda.cuda.mem_get_info()[0] == free_before, "device memory was allocated or freed"
    want_big = orc.xor_words(orc.fill_f32(big.numel(), 41, 0))
    want_small = orc.xor_words(orc.fill_f32(small.numel(), 42, 0))
    assert results == [want_big, want_small, want_big, want_small]


def test_static_scratch_capacity_is_enforced(K, cuda):
    src = dev_empty(1024, cuda.float32)
    out = dev_empty(1, cuda.int32)
    with pytest.raises(N.ClpkError) as e:
        K.clpk_stream_checksum_static(src.data_ptr(), 4096, 4097, out.data_ptr(), stream_ptr())
    assert e.value.code == N.ERR_TOO_LARGE and "4096" in e.value.detail
    K.clpk_stream_checksum_static(src.data_ptr(), 4096, 4096, out.data_ptr(), stream_ptr())    # the limit itself is fine
    sync()
