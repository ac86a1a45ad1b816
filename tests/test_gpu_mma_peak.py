"""GPU parity for the tcgen05 tensor-core probes: the final accumulator tile of
every CTA against the oracle's exact product tile (int8 bit-exact, floating
kinds within the tolerance stated in tests/mma_util.py)."""
import numpy as np
import pytest

from clpeak_b200 import native as N
from tests import mma_util as M

pytestmark = pytest.mark.gpu

DENSE = [N.MMA_F16, N.MMA_BF16, N.MMA_E4M3, N.MMA_E5M2, N.MMA_I8, N.MMA_TF32, N.MMA_E2M1]
SCALED = [N.MMA_MXF4, N.MMA_NVF4]


@pytest.mark.parametrize("kind", DENSE + SCALED)
@pytest.mark.parametrize("n_mma", [1, 2, 64])
def test_single_cta_tile(K, orc, cuda, kind, n_mma):
    ops = M.make_operands(orc, kind)
    status, tiles, chk = M.run_peak(K, cuda, kind, ops, n_mma, grid=1, n_out_tiles=1)
    assert status == 0
    want, tol = M.expected_tile(orc, kind, ops, n_mma)
    M.check_tile(kind, tiles[0], want, tol)
    assert int(chk[0]) == int(np.bitwise_xor.reduce(tiles[0].view(np.uint32).ravel()))


@pytest.mark.parametrize("kind", DENSE + SCALED)
def test_full_config_all_ctas_agree(K, orc, cuda, kind):
    # full configuration: 2^14 instructions per CTA, grid = 4 x SM count.
    sms = cuda.cuda.get_device_properties(0).multi_processor_count
    grid = 4 * sms
    n_mma = 1 << 14
    ops = M.make_operands(orc, kind)
    status, tiles, chk = M.run_peak(K, cuda, kind, ops, n_mma, grid=grid, n_out_tiles=3)
    assert status == 0
    want, tol = M.expected_tile(orc, kind, ops, n_mma)
    for t in tiles:
        M.check_tile(kind, t, want, tol)
    # every CTA computed the same tile: one checksum value across the grid
    assert np.all(chk == chk[0])
    assert int(chk[0]) == int(np.bitwise_xor.reduce(tiles[0].view(np.uint32).ravel()))


@pytest.mark.parametrize("kind", [N.MMA_BF16, N.MMA_E4M3])
def test_doubling_an_operand_doubles_every_accumulator_bit_for_bit(K, orc, cuda, kind):
    """A truncating binary adder is blind to a common power of two: with A replaced by 2A (exact in the
    operand format) every accumulator of the full 2^14-instruction run must be exactly twice what it was.
    A wrong low-order accumulate that the tolerance of the full run would let through does not survive this."""
    ops = M.make_operands(orc, kind)
    if kind == N.MMA_BF16:
        fa = (ops["a"].astype(np.uint32) << 16).view(np.float32)
    else:
        L = orc.lib()
        fa = np.array([L.orc_e4m3_to_f32(int(v)) for v in ops["a"].ravel()], dtype=np.float32).reshape(ops["a"].shape)
    twice = orc.convert_f32(fa * np.float32(2.0), M.DENSE_DT[kind]).reshape(ops["a"].shape)
    n_mma = 1 << 14
    _, base, _ = M.run_peak(K, cuda, kind, ops, n_mma, grid=2, n_out_tiles=1)
    _, dbl, _ = M.run_peak(K, cuda, kind, dict(ops, a=twice), n_mma, grid=2, n_out_tiles=1)
    b = base[0].view(np.float32)
    assert np.isfinite(b).all() and not np.any((b != 0) & (np.abs(b) < 2.0 ** -100))     # nothing near the subnormals
    assert np.count_nonzero(b) > b.size // 2
    assert np.array_equal(dbl[0].view(np.float32), b * np.float32(2.0))


@pytest.mark.parametrize("n_mma", [1, 2, 3])
def test_fp16_accumulate_tile(K, orc, cuda, n_mma):
    """kind::f16 with a 16-bit accumulator: one half per 32-bit tensor-memory cell, low 16 bits."""
    ops = M.make_operands(orc, N.MMA_F16_F16)
    status, tiles, chk = M.run_peak(K, cuda, N.MMA_F16_F16, ops, n_mma, grid=2, n_out_tiles=2)
    assert status == 0
    want, tol = M.expected_tile(orc, N.MMA_F16_F16, ops, n_mma)
    for t in tiles:
        M.check_tile(N.MMA_F16_F16, t, want, tol)
    assert chk[0] == chk[1]


def test_fp16_accumulate_full_config_runs_and_ctas_agree(K, orc, cuda):
    # 2^14 accumulations saturate a 16-bit accumulator, so only agreement between CTAs is checked here
    sms = cuda.cuda.get_device_properties(0).multi_processor_count
    ops = M.make_operands(orc, N.MMA_F16_F16)
    status, _, chk = M.run_peak(K, cuda, N.MMA_F16_F16, ops, 1 << 14, grid=4 * sms, n_out_tiles=1)
    assert status == 0 and np.all(chk == chk[0])


def test_tf32_ignores_the_low_mantissa_bits(K, orc, cuda):
    # the same tile with noise in the 13 bits below the tf32 mantissa gives the same accumulator
    ops = M.make_operands(orc, N.MMA_TF32)
    _, clean, _ = M.run_peak(K, cuda, N.MMA_TF32, ops, 3, 1, 1)
    noisy = dict(ops)
    noisy["a"] = (ops["a"].view(np.uint32) | np.uint32(0x1555)).view(ops["a"].dtype)
    noisy["b"] = (ops["b"].view(np.uint32) | np.uint32(0x0AAA)).view(ops["b"].dtype)
    _, dirty, _ = M.run_peak(K, cuda, N.MMA_TF32, noisy, 3, 1, 1)
    assert np.array_equal(clean[0], dirty[0])


@pytest.mark.parametrize("kind", DENSE + SCALED)
def test_cta_pairs_and_lone_ctas_compute_the_same_tile(K, orc, cuda, kind):
    """cta_group::2 (two CTAs share B) against cta_group::1: same accumulator bits, tile by tile."""
    ops = M.make_operands(orc, kind)
    out = {}
    try:
        for pair in ("0", "1"):
            K.clpk_set_tuning(N.TUNE_MMA_PAIR, int(pair))
            status, tiles, chk = M.run_peak(K, cuda, kind, ops, 5, grid=4, n_out_tiles=4)
            assert status == 0
            out[pair] = (tiles.copy(), chk.copy())
    finally:
        K.clpk_set_tuning(N.TUNE_MMA_PAIR, -1)
    assert np.array_equal(out["0"][0], out["1"][0]) and np.array_equal(out["0"][1], out["1"][1])
    want, tol = M.expected_tile(orc, kind, ops, 5)
    for t in out["1"][0]:
        M.check_tile(kind, t, want, tol)


def test_linearity_in_instruction_count(K, orc, cuda):
    # int8 is exact, so n instructions give exactly n times one instruction.
    ops = M.make_operands(orc, N.MMA_I8)
    _, t1, _ = M.run_peak(K, cuda, N.MMA_I8, ops, 1, 1, 1)
    _, t7, _ = M.run_peak(K, cuda, N.MMA_I8, ops, 7, 1, 1)
    assert np.array_equal(t7[0], t1[0] * 7)


def test_rejects_bad_arguments(K, cuda):
    import ctypes as C
    args = N.MmaPeakArgs(kind=99)
    with pytest.raises(N.ClpkError) as e:
        K.clpk_mma_peak(C.byref(args), None)
    assert e.value.code == N.ERR_BAD_ARG


def test_probe_reports_cycles_and_time_of_cta_0(K, orc, cuda):
    """d_clock: {SM cycles, nanoseconds} around CTA 0's issue loop.  Two co-resident bf16 CTAs share the tensor pipe,
    so CTA 0's 2^14 instructions take about 2 x 128 cycles each; the quotient cycles / ns is a plausible SM clock."""
    import ctypes as C
    from tests.gpu_util import dev_empty, dev_from, stream_ptr, sync, to_np
    ops = M.make_operands(orc, N.MMA_BF16)
    sms = cuda.cuda.get_device_properties(0).multi_processor_count
    n_mma, grid = 1 << 14, 4 * sms
    d_a, d_b = dev_from(ops["a"].view(np.uint8)), dev_from(ops["b"].view(np.uint8))
    d_chk, d_status = dev_empty(grid, cuda.int32), dev_empty(1, cuda.int32)
    d_clock = cuda.zeros(2, dtype=cuda.int64, device="cuda")
    args = N.MmaPeakArgs(kind=N.MMA_BF16, d_a=d_a.data_ptr(), d_b=d_b.data_ptr(), n_mma=n_mma, grid=grid, n_out_tiles=0,
                         d_checksum=d_chk.data_ptr(), d_status=d_status.data_ptr(), d_clock=d_clock.data_ptr())
    try:
        K.clpk_set_tuning(N.TUNE_MMA_PAIR, 0)
        K.clpk_mma_peak(C.byref(args), stream_ptr())
        sync()
    finally:
        K.clpk_set_tuning(N.TUNE_MMA_PAIR, -1)
    cyc, ns = (int(v) for v in to_np(d_clock))
    assert int(to_np(d_status)[0]) == 0
    assert 500.0 < cyc / ns * 1e3 < 2100.0
    assert 250.0 <= cyc / n_mma <= 275.0, cyc / n_mma
