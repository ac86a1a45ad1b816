"""Parity of the typed shader-core chains, the shared-memory rotation and the texture
read against the CPU oracle: bit-exact (NaN-aware for the floating chains, which run
away to infinity from the reference's start value exactly as the reference's do)."""
import ctypes as C

import numpy as np
import pytest

from clpeak_b200 import native as N
from tests.gpu_util import assert_floats_equal_nan_aware

pytestmark = pytest.mark.gpu

REFERENCE_START = {N.CHAIN_HALF: 1.3, N.CHAIN_HALF2: 1.3, N.CHAIN_DOUBLE: 1.3, N.CHAIN_MIXED: 1.3, N.CHAIN_BF16: 1.3,
                   N.CHAIN_INT32: 3, N.CHAIN_INT8_DOT1: 4, N.CHAIN_INT8_DOT2: 4, N.CHAIN_INT8_DOT4: 4,
                   N.CHAIN_INT8_DOT8: 4}


def run_chain(K, torch, chain, a, grid):
    ops, elem = C.c_uint32(0), C.c_uint32(0)
    K.clpk_compute_chain_info(chain, C.byref(ops), C.byref(elem))
    dtype = {4: torch.int32, 8: torch.int64}[elem.value]
    out = torch.zeros(grid * 256, dtype=dtype, device="cuda")
    K.clpk_compute_chain(chain, out.data_ptr(), float(a), grid, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy(), ops.value


@pytest.mark.parametrize("chain", sorted(REFERENCE_START))
def test_chain_matches_the_oracle_at_the_reference_start(K, orc, cuda, chain):
    got, ops = run_chain(K, cuda, chain, REFERENCE_START[chain], 3)
    want = orc.compute_chain(chain, REFERENCE_START[chain], 3 * 256)
    assert ops == (8192 if chain >= N.CHAIN_INT8_DOT1 else 4096)
    if chain >= N.CHAIN_INT32:
        assert np.array_equal(got, want)
        assert len(np.unique(got[:256])) > 200               # the integer chains do not collapse
    elif chain == N.CHAIN_DOUBLE:
        assert np.array_equal(got.view(np.uint64), want.view(np.uint64))
    else:
        assert_floats_equal_nan_aware(got.view(np.float32), want, f"chain {chain}")
    assert np.array_equal(got[:256], got[256:512])            # c depends on the thread, not the block


@pytest.mark.parametrize("chain", [N.CHAIN_HALF, N.CHAIN_HALF2, N.CHAIN_DOUBLE, N.CHAIN_MIXED, N.CHAIN_BF16])
@pytest.mark.parametrize("a", [0.0, 0.25, -0.75, 1e-3, 300.0, -1.3])
def test_floating_chains_other_starts(K, orc, cuda, chain, a):
    got, _ = run_chain(K, cuda, chain, a, 1)
    want = orc.compute_chain(chain, a, 256)
    if chain == N.CHAIN_DOUBLE:
        g = got.view(np.float64)
        assert np.all((g.view(np.uint64) == want.view(np.uint64)) | (np.isnan(g) & np.isnan(want)))
    else:
        assert_floats_equal_nan_aware(got.view(np.float32), want, f"chain {chain}")


@pytest.mark.parametrize("chain", [N.CHAIN_INT32, N.CHAIN_INT8_DOT1, N.CHAIN_INT8_DOT2, N.CHAIN_INT8_DOT4, N.CHAIN_INT8_DOT8])
@pytest.mark.parametrize("a", [0, 1, 3, 4, 125, 255, -7, 2**31 - 1])
def test_integer_chains_other_starts(K, orc, cuda, chain, a):
    got, _ = run_chain(K, cuda, chain, a, 2)
    assert np.array_equal(got, orc.compute_chain(chain, a, 512))


def test_chain_argument_checks(K, orc, cuda):
    out = cuda.zeros(256, dtype=cuda.int32, device="cuda")
    for bad in (-1, N.CHAIN_INT8_DOT8 + 1):
        with pytest.raises(N.ClpkError):
            K.clpk_compute_chain(bad, out.data_ptr(), 1.0, 1, None)
    with pytest.raises(N.ClpkError):
        K.clpk_compute_chain(N.CHAIN_INT32, None, 1.0, 1, None)
    with pytest.raises(N.ClpkError):
        K.clpk_compute_chain(N.CHAIN_INT32, out.data_ptr(), 1.0, 0, None)


@pytest.mark.parametrize("width", [1, 2, 4])
@pytest.mark.parametrize("grid", [1, 5, 148 * 8])
def test_local_bandwidth_rotation(K, orc, cuda, width, grid):
    out = cuda.zeros(grid * 256, dtype=cuda.float32, device="cuda")
    K.clpk_local_bandwidth(width, out.data_ptr(), grid, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy().view(np.uint32), orc.local_bandwidth(width, grid * 256).view(np.uint32))


def test_local_bandwidth_rejects_other_widths(K, orc, cuda):
    out = cuda.zeros(256, dtype=cuda.float32, device="cuda")
    for w in (0, 3, 8):
        with pytest.raises(N.ClpkError):
            K.clpk_local_bandwidth(w, out.data_ptr(), 1, None)


def make_image(K, w, h, seed, stream):
    img = C.c_void_p(None)
    K.clpk_image_create(C.byref(img), w, h, seed, stream)
    return img


@pytest.mark.parametrize("shape", [(256, 128), (64, 64), (1024, 48), (384, 96), (1000, 512)])
def test_image_bandwidth_small_images_every_thread(K, orc, cuda, shape):
    w, h = shape
    stream = cuda.cuda.current_stream().cuda_stream
    img = make_image(K, w, h, 11, stream)
    try:
        threads = w * h // 16
        out = cuda.zeros(threads, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth(img, out.data_ptr(), threads // 256, stream)
        cuda.cuda.synchronize()
        want = orc.image_bandwidth(threads, w * h, 11)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    finally:
        K.clpk_image_destroy(img)


@pytest.mark.parametrize("shape", [(256, 128), (64, 64), (1024, 64), (8, 32), (4096, 32)])
def test_image_bandwidth_tiled_every_thread(K, orc, cuda, shape):
    """The tiled order (8 x 32 tiles, 16 neighbouring tiles per block): every thread against the oracle,
    and the same multiset of texels as the strided order (each read exactly once) when threads * 16 = texels."""
    w, h = shape
    stream = cuda.cuda.current_stream().cuda_stream
    img = make_image(K, w, h, 11, stream)
    try:
        threads = max(256, w * h // 16)
        out = cuda.zeros(threads, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth_tiled(img, out.data_ptr(), threads // 256, stream)
        cuda.cuda.synchronize()
        want = orc.image_bandwidth_tiled(threads, w, h, 11)
        assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32))
    finally:
        K.clpk_image_destroy(img)


def test_image_bandwidth_tiled_covers_every_texel_once(orc):
    """Host-only property of the mapping: with threads * 16 = width * height the tiled order visits each texel once."""
    w, h = 64, 128
    threads = w * h // 16
    seen = np.zeros((h, w), dtype=np.int32)
    tiles_x = w // 8
    for t in range(threads):
        b, r = divmod(t, 256)
        wp, l = divmod(r, 32)
        for i in range(16):
            tile = (b * 16 + i) % (tiles_x * (h // 32))
            seen[(tile // tiles_x) * 32 + (wp // 2) * 8 + l // 4, (tile % tiles_x) * 8 + (wp % 2) * 4 + l % 4] += 1
    assert (seen == 1).all()


def test_image_bandwidth_tiled_rejects_ragged_images(K, cuda):
    stream = cuda.cuda.current_stream().cuda_stream
    img = make_image(K, 100, 64, 1, stream)
    try:
        out = cuda.zeros(256, dtype=cuda.float32, device="cuda")
        with pytest.raises(N.ClpkError) as e:
            K.clpk_image_bandwidth_tiled(img, out.data_ptr(), 1, stream)
        assert e.value.code == N.ERR_BAD_ARG
    finally:
        K.clpk_image_destroy(img)


def test_image_bandwidth_tiled_full_size_sampled(K, orc, cuda):
    w = h = 4096
    stream = cuda.cuda.current_stream().cuda_stream
    img = make_image(K, w, h, 5, stream)
    try:
        threads = w * h // 16
        out = cuda.zeros(threads, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth_tiled(img, out.data_ptr(), threads // 256, stream)
        cuda.cuda.synchronize()
        got = out.cpu().numpy()
        for first in (0, 123456, threads - 512):
            want = orc.image_bandwidth_tiled(threads, w, h, 5, first=first, count=512)
            assert np.array_equal(got[first:first + 512].view(np.uint32), want.view(np.uint32))
    finally:
        K.clpk_image_destroy(img)


def test_image_bandwidth_wraps_when_threads_exceed_texels(K, orc, cuda):
    stream = cuda.cuda.current_stream().cuda_stream
    img = make_image(K, 64, 32, 3, stream)          # 2048 texels, 1024 threads x 16 fetches = 8 passes
    try:
        out = cuda.zeros(1024, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth(img, out.data_ptr(), 4, stream)
        cuda.cuda.synchronize()
        assert np.array_equal(out.cpu().numpy().view(np.uint32), orc.image_bandwidth(1024, 2048, 3).view(np.uint32))
    finally:
        K.clpk_image_destroy(img)


def test_image_bandwidth_full_size_sampled(K, orc, cuda):
    """The 4096 x 4096 float4 image of the reference (256 MiB, every texel read once)."""
    stream = cuda.cuda.current_stream().cuda_stream
    w = h = 4096
    img = make_image(K, w, h, 5, stream)
    try:
        threads = w * h // 16
        out = cuda.zeros(threads, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth(img, out.data_ptr(), threads // 256, stream)
        cuda.cuda.synchronize()
        got = out.cpu().numpy()
        for first in (0, 123456, threads - 512):
            want = orc.image_bandwidth(threads, w * h, 5, first=first, count=512)
            assert np.array_equal(got[first:first + 512].view(np.uint32), want.view(np.uint32))
        # every texel once: the grand total equals the sum of the whole stream (float64 accumulate, loose)
        assert abs(float(got.astype(np.float64).sum()) / (w * h * 4) - 0.5) < 1e-3
    finally:
        K.clpk_image_destroy(img)
