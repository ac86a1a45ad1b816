"""GPU parity: seeded fills, conversions, bandwidth kernels, chains, pointer
chase -- all bit-exact against the CPU oracle, called through the C ABI."""
import ctypes as C

import numpy as np
import pytest

from clpeak_b200 import native as N
from tests.gpu_util import (assert_bits_equal, assert_floats_equal_nan_aware, dev_empty, dev_from, stream_ptr, sync,
                            to_np)

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dist", [0, 1, 2])
@pytest.mark.parametrize("n", [0, 1, 1000, 1 << 20])
def test_fill_f32_matches_oracle(K, orc, cuda, dist, n):
    d = dev_empty(max(n, 1), cuda.float32)
    K.clpk_fill_f32(d.data_ptr(), n, 7 + dist, dist, 0.25, 0.02, stream_ptr())
    sync()
    want = orc.fill_f32(n, 7 + dist, dist, 0.25, 0.02)
    assert_bits_equal(to_np(d)[:n], want, f"fill dist={dist}")


def test_fill_f32_high_index_window(K, orc, cuda):
    # element indices beyond 2^32 (an 8 GiB fp32 buffer has 2^31 elements; check far past it)
    n = 1 << 16
    seed = 11
    big = dev_empty((1 << 22), cuda.float32)
    K.clpk_fill_f32(big.data_ptr(), big.numel(), seed, 0, 0.0, 1.0, stream_ptr())
    sync()
    first = (1 << 22) - n
    want = orc.fill_f32(n, seed, 0, first=first)
    assert_bits_equal(to_np(big)[first:], want, "fill tail window")


def test_fill_i8(K, orc, cuda):
    n = 100_000
    d = dev_empty(n, cuda.int8)
    K.clpk_fill_i8(d.data_ptr(), n, 2, stream_ptr())
    sync()
    got = to_np(d)
    assert got.min() >= -8 and got.max() <= 7
    assert_bits_equal(got, orc.fill_i8(n, 2), "fill_i8")


@pytest.mark.parametrize("dtype,scale", [(N.DT_F16, 1.0), (N.DT_BF16, 1.0), (N.DT_E4M3, 200.0),
                                         (N.DT_E5M2, 3.0e4), (N.DT_I8, 60.0), (N.DT_TF32, 1.0), (N.DT_E2M1, 3.0)])
def test_convert_matches_oracle(K, orc, cuda, dtype, scale):
    n = 1 << 18
    src = orc.fill_f32(n, 5, 2, 0.0, scale)
    # edge values: zeros, ties, saturation, subnormals of the narrow formats
    edges = np.array([0.0, -0.0, 0.5, 1.5, 2.5, 448.0, 449.0, 464.0, 1e9, -1e9, 2 ** -9, 2 ** -10, 3 * 2 ** -11,
                      57344.0, 61440.0, 65504.0, 65520.0, 127.5, -128.5, 1e-30], dtype=np.float32)
    src[: edges.size] = edges
    src[edges.size: edges.size + 10] = np.array([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 6.0, 7.0, -0.25], dtype=np.float32)
    tdt = {N.DT_F16: cuda.int16, N.DT_BF16: cuda.int16, N.DT_E4M3: cuda.uint8, N.DT_E5M2: cuda.uint8,
           N.DT_I8: cuda.int8, N.DT_TF32: cuda.int32, N.DT_E2M1: cuda.uint8}[dtype]
    d_src = dev_from(src)
    d_dst = dev_empty(n // 2 if dtype == N.DT_E2M1 else n, tdt)
    K.clpk_convert_f32(d_dst.data_ptr(), d_src.data_ptr(), n, dtype, stream_ptr())
    sync()
    assert_bits_equal(to_np(d_dst), orc.convert_f32(src, dtype), f"convert dtype={dtype}")


@pytest.mark.parametrize("dtype", [N.DT_MXF4, N.DT_NVF4])
def test_quantize_fp4_matches_oracle(K, orc, cuda, dtype):
    rows, cols = 384, 256
    src = orc.fill_f32(rows * cols, 3, 2).reshape(rows, cols)
    src[0, :32] = 0.0                      # an all-zero block
    src[1, 5] = 1e6                        # an outlier
    blk = 32 if dtype == N.DT_MXF4 else 16
    d_src = dev_from(src)
    d_absmax = dev_empty(1, cuda.float32)
    K.clpk_absmax_f32(d_absmax.data_ptr(), d_src.data_ptr(), src.size, stream_ptr())
    sync()
    amax = float(to_np(d_absmax)[0])
    assert amax == float(np.abs(src).max())
    ts = np.float32(amax) / np.float32(6.0 * 448.0) if dtype == N.DT_NVF4 else np.float32(1.0)
    d_packed = dev_empty(rows * cols // 2, cuda.uint8)
    d_scales = dev_empty(rows * cols // blk, cuda.uint8)
    K.clpk_quantize_fp4(d_packed.data_ptr(), d_scales.data_ptr(), d_src.data_ptr(), rows, cols, dtype,
                        float(ts), stream_ptr())
    sync()
    packed, scales = orc.quantize_fp4(src, dtype, float(ts))
    assert_bits_equal(to_np(d_scales), scales.ravel(), "fp4 scales")
    assert_bits_equal(to_np(d_packed), packed.ravel(), "fp4 payload")


@pytest.mark.parametrize("width", [1, 2, 4])
@pytest.mark.parametrize("blocks", [1, 3, 64])
def test_global_bandwidth_reference_order(K, orc, cuda, width, blocks):
    n = 256 * 16 * width * blocks
    src = orc.fill_f32(n, 1, 0)
    d_in = dev_from(src)
    d_out = dev_empty(n // (16 * width), cuda.float32)
    K.clpk_global_bandwidth(width, d_in.data_ptr(), d_out.data_ptr(), n, stream_ptr())
    sync()
    assert_bits_equal(to_np(d_out), orc.global_bandwidth(width, src), f"global_bandwidth v{width}")


def test_global_bandwidth_rejects_ragged(K, cuda):
    d = dev_empty(4096, cuda.float32)
    with pytest.raises(N.ClpkError) as e:
        K.clpk_global_bandwidth(4, d.data_ptr(), d.data_ptr(), 4096 + 4, stream_ptr())
    assert e.value.code == N.ERR_BAD_ARG


def _read_xor(K, cuda, variant, d_src, n_bytes):
    grid = C.c_int(0)
    K.clpk_stream_read_grid(variant, C.byref(grid))
    parts = dev_empty(grid.value, cuda.int32)
    K.clpk_stream_read(variant, d_src.data_ptr(), n_bytes, parts.data_ptr(), stream_ptr())
    st = C.c_uint32(0)
    K.clpk_stream_status(C.byref(st), stream_ptr())
    return int(np.bitwise_xor.reduce(to_np(parts).view(np.uint32)))


# sizes in bytes: empty, one vector, ragged tails around the tile sizes, larger than one wave
SIZES = [0, 16, 4096 + 16, 8192, 8192 + 16, 32768, 32768 * 3 + 48, (1 << 24) + 1616, 1 << 27]


@pytest.mark.parametrize("variant", list(N.STREAM_VARIANTS))
@pytest.mark.parametrize("n_bytes", SIZES)
def test_stream_read_xor(K, orc, cuda, variant, n_bytes):
    n = max(n_bytes // 4, 4)
    src = orc.fill_f32(n, 21, 0)
    d_src = dev_from(src)
    got = _read_xor(K, cuda, variant, d_src, n_bytes)
    assert got == orc.xor_words(src[: n_bytes // 4])


@pytest.mark.parametrize("variant", list(N.STREAM_VARIANTS))
@pytest.mark.parametrize("n_bytes", SIZES)
def test_stream_copy(K, orc, cuda, variant, n_bytes):
    n = max(n_bytes // 4, 4)
    src = orc.fill_f32(n + 8, 22, 0)
    d_src = dev_from(src)
    d_dst = cuda.full((n + 8,), -1.0, dtype=cuda.float32, device="cuda")
    K.clpk_stream_copy(variant, d_dst.data_ptr(), d_src.data_ptr(), n_bytes, stream_ptr())
    st = C.c_uint32(0)
    K.clpk_stream_status(C.byref(st), stream_ptr())
    got = to_np(d_dst)
    assert_bits_equal(got[: n_bytes // 4], src[: n_bytes // 4], "copy body")
    assert np.all(got[n_bytes // 4:] == -1.0), "copy wrote past the end"


@pytest.mark.parametrize("variant", list(N.STREAM_VARIANTS))
@pytest.mark.parametrize("n_floats", [0, 4, 8192 + 4, 3 * 8192 + 12, (1 << 22) + 404, 1 << 25])
def test_stream_triad(K, orc, cuda, variant, n_floats):
    n = max(n_floats, 4)
    b = orc.fill_f32(n + 8, 23, 0)
    c = orc.fill_f32(n + 8, 24, 0)
    d_b, d_c = dev_from(b), dev_from(c)
    d_a = cuda.full((n + 8,), -1.0, dtype=cuda.float32, device="cuda")
    K.clpk_stream_triad(variant, d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), 1.5, n_floats, stream_ptr())
    st = C.c_uint32(0)
    K.clpk_stream_status(C.byref(st), stream_ptr())
    got = to_np(d_a)
    assert_bits_equal(got[:n_floats], orc.triad(b[:n_floats].copy(), c[:n_floats].copy(), 1.5), "triad body")
    assert np.all(got[n_floats:] == -1.0)


def test_stream_triad_ldg_ragged_floats(K, orc, cuda):
    n = 1027                                   # not a multiple of 4: LDG variant only
    b = orc.fill_f32(n, 23, 0)
    c = orc.fill_f32(n, 24, 0)
    d_a = dev_empty(n, cuda.float32)
    d_b, d_c = dev_from(b), dev_from(c)
    K.clpk_stream_triad(N.STREAM_LDG, d_a.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), 1.5, n, stream_ptr())
    sync()
    assert_bits_equal(to_np(d_a), orc.triad(b, c, 1.5), "triad ragged")
    with pytest.raises(N.ClpkError):
        K.clpk_stream_triad(N.STREAM_TMA, d_a.data_ptr(), d_a.data_ptr(), d_a.data_ptr(), 1.5, n, stream_ptr())
    # the 256-bit flavour takes any length (its tail is element-wise) but wants 32-byte aligned pointers
    d_a2 = dev_empty(n, cuda.float32)
    K.clpk_stream_triad(N.STREAM_WIDE, d_a2.data_ptr(), d_b.data_ptr(), d_c.data_ptr(), 1.5, n, stream_ptr())
    sync()
    assert_bits_equal(to_np(d_a2), orc.triad(b, c, 1.5), "triad ragged, 256-bit flavour")
    with pytest.raises(N.ClpkError):
        K.clpk_stream_triad(N.STREAM_WIDE, d_a2.data_ptr() + 16, d_b.data_ptr() + 16, d_c.data_ptr() + 16, 1.5, 64, stream_ptr())
    with pytest.raises(N.ClpkError):
        K.clpk_stream_copy(N.STREAM_WIDE, d_a2.data_ptr() + 16, d_b.data_ptr(), 64, stream_ptr())


def test_stream_variants_agree_on_a_large_buffer(K, orc, cuda):
    """512 MiB: the three flavours of each kernel give identical bits (read: identical XOR)."""
    n = (512 << 20) // 4
    b, c = dev_empty(n, cuda.float32), dev_empty(n, cuda.float32)
    K.clpk_fill_f32(b.data_ptr(), n, 31, 0, 0.0, 1.0, stream_ptr())
    K.clpk_fill_f32(c.data_ptr(), n, 32, 0, 0.0, 1.0, stream_ptr())
    xors = {v: _read_xor(K, cuda, v, b, n * 4) for v in N.STREAM_VARIANTS}
    assert len(set(xors.values())) == 1
    outs = []
    for v in N.STREAM_VARIANTS:
        a = dev_empty(n, cuda.float32)
        K.clpk_stream_triad(v, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.5, n, stream_ptr())
        st = C.c_uint32(0)
        K.clpk_stream_status(C.byref(st), stream_ptr())
        outs.append(a)
    assert cuda.equal(outs[0].view(cuda.int32), outs[1].view(cuda.int32)) and cuda.equal(outs[0].view(cuda.int32), outs[2].view(cuda.int32))
    d = dev_empty(n, cuda.float32)
    K.clpk_stream_copy(N.STREAM_WIDE, d.data_ptr(), outs[0].data_ptr(), n * 4, stream_ptr())
    sync()
    assert cuda.equal(d.view(cuda.int32), outs[0].view(cuda.int32))


def test_compute_sp_reference_chain(K, orc, cuda):
    grid = 5
    d = dev_empty(grid * 256, cuda.float32)
    K.clpk_compute_sp(d.data_ptr(), 1.3, grid, stream_ptr())
    sync()
    assert_bits_equal(to_np(d), orc.compute_sp(1.3, grid * 256), "compute_sp")


@pytest.mark.parametrize("iters", [0, 16, 64, 4096])
def test_mad_chain(K, orc, cuda, iters):
    n = 4096
    d = dev_empty(n, cuda.float32)
    K.clpk_mad_chain(d.data_ptr(), n, 0, 0.999, iters, stream_ptr())
    sync()
    got = to_np(d)
    # x roughly doubles per step, so past ~128 steps every lane is +-inf and a
    # work-item whose lanes disagree in sign sums to NaN: compare NaN-aware.
    assert_floats_equal_nan_aware(got, orc.mad_chain(n, 0, 0.999, iters), f"mad_chain iters={iters}")
    if iters <= 64:
        assert np.all(np.isfinite(got))            # the finite-range prefix has real values
        assert_bits_equal(got, orc.mad_chain(n, 0, 0.999, iters), "finite prefix")


def test_mad_chain_full_config_sampled(K, orc, cuda):
    # 2^20 work-items x 4096 iterations; the oracle replays a window of it.
    n = 1 << 20
    d = dev_empty(n, cuda.float32)
    K.clpk_mad_chain(d.data_ptr(), n, 0, 0.999, 4096, stream_ptr())
    sync()
    got = to_np(d)
    for first in (0, 123456, n - 512):
        assert_floats_equal_nan_aware(got[first:first + 512], orc.mad_chain(512, 0, 0.999, 4096, first=first),
                                      "mad window")


@pytest.mark.parametrize("n,hops", [(2, 7), (1000, 5000), (1 << 20, 1 << 16)])
def test_pointer_chase(K, orc, cuda, n, hops):
    nxt = np.empty(n, dtype=np.uint32)
    K.clpk_build_chase_cycle(nxt.ctypes.data, n, 9)
    assert_bits_equal(nxt, orc.chase_cycle(n, 9), "chase cycle construction")
    assert orc.lib().orc_is_single_cycle(nxt.ctypes.data, n) == 1
    d_next = dev_from(nxt.view(np.int32))
    d_res = dev_empty(4, cuda.int32)
    K.clpk_pointer_chase(d_next.data_ptr(), 0, hops, d_res.data_ptr(), stream_ptr())
    sync()
    res = to_np(d_res).view(np.uint32)
    fin, x = orc.chase(nxt, 0, hops)
    assert (int(res[0]), int(res[1])) == (fin, x)
    assert (int(res[2]) | (int(res[3]) << 32)) > 0


def test_launch_latency(K, cuda):
    mean = C.c_double(0.0)
    K.clpk_launch_latency(200, 3, C.byref(mean), stream_ptr())
    assert 0.5 < mean.value < 1000.0


def test_graph_launch_latency_is_below_the_single_launch_round_trip(K, cuda):
    """1000 empty kernels replayed as one CUDA graph: the per-node cost must undercut launch + synchronise of
    one kernel, on the caller's stream and on the call's own (NULL) stream; the stream stays usable afterwards."""
    one, node = C.c_double(0.0), C.c_double(0.0)
    K.clpk_launch_latency(200, 3, C.byref(one), stream_ptr())
    for s in (stream_ptr(), None):
        K.clpk_graph_launch_latency(1000, 20, 2, C.byref(node), s)
        assert 0.05 < node.value < one.value
    x = cuda.zeros(16, device="cuda") + 1                   # the captured stream is back to normal work
    assert float(x.sum()) == 16.0
