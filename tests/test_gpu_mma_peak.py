"""GPU parity for the tcgen05 tensor-core probes: the final accumulator tile of
every CTA against the oracle's exact product tile (int8 bit-exact, floating
kinds within the tolerance stated in tests/mma_util.py)."""
import numpy as np
import pytest

from clpeak_b200 import native as N
from tests import mma_util as M

pytestmark = pytest.mark.gpu

DENSE = [N.MMA_F16, N.MMA_BF16, N.MMA_E4M3, N.MMA_E5M2, N.MMA_I8]
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
    # BASELINE config: 2^14 instructions per CTA, grid = 4 x SM count.
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
