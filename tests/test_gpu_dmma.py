"""The fp64 tensor probe (mma.sync.m8n8k4.f64, the successor of the reference's wmma_fp64 row,
src/cuda/cuda_kernels/wmma_fp64.cu:15-46) against the CPU oracle.

Operands that are multiples of 2^-8 in [-1,1) make every product and partial sum exact in
fp64, so those cases are bit-exact whatever order the tensor core adds the four products in.
General operands are compared within 64 ulp-of-the-running-sum per instruction: relative
tolerance n_mma * 4 * 2^-52 on sum|a||b| * n_mma."""
import numpy as np
import pytest

from clpeak_b200 import native as N

pytestmark = pytest.mark.gpu

WARPS, CHAINS = 8, 8


def run(K, torch, a, b, n_mma, grid, n_out):
    d_a, d_b = torch.from_numpy(a).cuda(), torch.from_numpy(b).cuda()
    out = torch.zeros(n_out * WARPS * 64, dtype=torch.float64, device="cuda")
    chk = torch.zeros(grid, dtype=torch.int32, device="cuda")
    K.clpk_dmma_peak(d_a.data_ptr(), d_b.data_ptr(), n_mma, grid, n_out, out.data_ptr(), chk.data_ptr(),
                     torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return out.cpu().numpy().reshape(n_out, WARPS, 8, 8), chk.cpu().numpy()


def dyadic(orc, seed):
    x = orc.fill_f32(64, seed, 1).astype(np.float64)
    x = np.floor(x * 256.0) / 256.0
    return np.ascontiguousarray(x[:32]), np.ascontiguousarray(x[32:])


@pytest.mark.parametrize("n_mma", [1, 2, 3, 64, 1 << 13])
def test_dyadic_operands_are_bit_exact(K, orc, cuda, n_mma):
    a, b = dyadic(orc, 2)
    tiles, chk = run(K, cuda, a, b, n_mma, grid=5, n_out=3)
    want = orc.dmma_tiles(a, b, n_mma, WARPS, CHAINS)
    for t in tiles:
        assert np.array_equal(t.view(np.uint64), want.view(np.uint64))
    assert len(set(chk.tolist())) == 1
    # closed form: sum of the start values + chains * n * (A B^T)
    prod = a.reshape(8, 4) @ b.reshape(8, 4).T
    for w in range(WARPS):
        init = sum(w * CHAINS + j for j in range(CHAINS))
        assert np.array_equal(want[w], init + CHAINS * n_mma * prod)


def test_full_grid_agrees_and_differs_between_operands(K, orc, cuda):
    a, b = dyadic(orc, 2)
    tiles, chk = run(K, cuda, a, b, 1 << 13, grid=8 * 148, n_out=1)
    assert len(set(chk.tolist())) == 1
    a2, b2 = dyadic(orc, 3)
    tiles2, chk2 = run(K, cuda, a2, b2, 1 << 13, grid=8 * 148, n_out=1)
    assert chk2[0] != chk[0] and not np.array_equal(tiles, tiles2)


@pytest.mark.parametrize("n_mma", [1, 17, 1000])
def test_general_operands_within_tolerance(K, orc, cuda, n_mma):
    x = orc.fill_f32(64, 9, 1).astype(np.float64) * 1.000000123
    a, b = np.ascontiguousarray(x[:32]), np.ascontiguousarray(x[32:])
    tiles, _ = run(K, cuda, a, b, n_mma, grid=2, n_out=2)
    want = orc.dmma_tiles(a, b, n_mma, WARPS, CHAINS)
    s_abs = np.abs(a.reshape(8, 4)) @ np.abs(b.reshape(8, 4)).T
    tol = n_mma * 4 * 2.0 ** -52 * (CHAINS * n_mma * s_abs + 64 * CHAINS)
    for t in tiles:
        assert np.all(np.abs(t - want) <= tol), float(np.max(np.abs(t - want) / tol))


def test_argument_checks(K, orc, cuda):
    a, b = dyadic(orc, 2)
    d = cuda.from_numpy(a).cuda()
    with pytest.raises(N.ClpkError):
        K.clpk_dmma_peak(None, d.data_ptr(), 1, 1, 0, None, None, None)
    with pytest.raises(N.ClpkError):
        K.clpk_dmma_peak(d.data_ptr(), d.data_ptr(), 0, 1, 0, None, None, None)
    with pytest.raises(N.ClpkError):
        K.clpk_dmma_peak(d.data_ptr(), d.data_ptr(), 1, 1, 2, None, None, None)
