"""GPU parity for the 2:4 sparse tcgen05.mma.sp probes (fp8 e4m3 and int8 at logical
K = 64, MXFP4 and NVFP4 at logical K = 128): real per-group selectors produced by
pruning seeded data, accumulator tile checked against the oracle."""
import numpy as np
import pytest

from clpeak_b200 import native as N
from tests import mma_util as M

pytestmark = pytest.mark.gpu
SP = [N.MMA_E4M3_SP, N.MMA_I8_SP, N.MMA_MXF4_SP, N.MMA_NVF4_SP]


@pytest.mark.parametrize("kind", SP)
def test_compressed_operand_decodes_to_the_pruned_tile(orc, kind):
    """The compressed A + selectors must reproduce the pruned dense tile exactly (host-only property)."""
    ops = M.make_operands(orc, kind)
    k = M.KIND_K[kind]
    pruned = ops["pruned"].reshape(128, k)
    kept = (pruned != 0).reshape(128, k // 4, 4).sum(axis=2) if kind in (N.MMA_E4M3_SP, N.MMA_I8_SP) else \
        (np.abs(pruned).reshape(128, k // 8, 4, 2).sum(axis=3) != 0).sum(axis=2)
    assert kept.max() <= 2
    nibbles = np.stack([ops["meta"] & 0xF, ops["meta"] >> 4], axis=2).reshape(128, -1)
    assert np.all((nibbles & 3) < (nibbles >> 2))          # first selector strictly below the second


@pytest.mark.parametrize("kind", SP)
@pytest.mark.parametrize("n_mma", [1, 3, 64])
def test_single_cta_sparse_tile(K, orc, cuda, kind, n_mma):
    ops = M.make_operands(orc, kind)
    status, tiles, chk = M.run_peak(K, cuda, kind, ops, n_mma, grid=1, n_out_tiles=1)
    assert status == 0
    want, tol = M.expected_tile(orc, kind, ops, n_mma)
    M.check_tile(kind, tiles[0], want, tol)
    assert int(chk[0]) == int(np.bitwise_xor.reduce(tiles[0].view(np.uint32).ravel()))


@pytest.mark.parametrize("kind", SP)
def test_sparse_full_config(K, orc, cuda, kind):
    sms = cuda.cuda.get_device_properties(0).multi_processor_count
    ops = M.make_operands(orc, kind)
    status, tiles, chk = M.run_peak(K, cuda, kind, ops, 1 << 14, grid=4 * sms, n_out_tiles=2)
    assert status == 0
    want, tol = M.expected_tile(orc, kind, ops, 1 << 14)
    for t in tiles:
        M.check_tile(kind, t, want, tol)
    assert np.all(chk == chk[0])


@pytest.mark.parametrize("kind", SP)
def test_sparse_cta_pairs_and_lone_ctas_compute_the_same_tile(K, orc, cuda, kind):
    """cta_group::2 (each CTA stages half of B, both the same compressed A and selectors) against
    cta_group::1: the same accumulator bits in every tile."""
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


def test_selectors_matter(K, orc, cuda):
    """Flipping one selector nibble changes exactly one row of the result (int8: exact arithmetic)."""
    ops = M.make_operands(orc, N.MMA_I8_SP)
    _, base, _ = M.run_peak(K, cuda, N.MMA_I8_SP, ops, 1, 1, 1)
    meta = ops["meta"].copy()
    old = meta[17, 3] & 0xF
    new = 0b1110 if old != 0b1110 else 0b0100
    meta[17, 3] = (meta[17, 3] & 0xF0) | new
    _, alt, _ = M.run_peak(K, cuda, N.MMA_I8_SP, dict(ops, meta=meta), 1, 1, 1)
    changed = np.flatnonzero((base[0] != alt[0]).any(axis=1))
    assert changed.tolist() in ([17], [])                    # [] only if the swapped-in B columns happen to cancel
    want = M.expected_tile(orc, N.MMA_I8_SP, dict(ops, meta=meta), 1)[0]
    assert np.array_equal(alt[0], want)


def test_sparse_needs_metadata(K, cuda):
    import ctypes as C
    d = cuda.zeros(8192, dtype=cuda.uint8, device="cuda")
    st = cuda.zeros(1, dtype=cuda.int32, device="cuda")
    args = N.MmaPeakArgs(kind=N.MMA_E4M3_SP, d_a=d.data_ptr(), d_b=d.data_ptr(), d_meta=None, n_mma=1, grid=1,
                         n_out_tiles=0, d_status=st.data_ptr())
    with pytest.raises(N.ClpkError) as e:
        K.clpk_mma_peak(C.byref(args), None)
    assert e.value.code == N.ERR_BAD_ARG
