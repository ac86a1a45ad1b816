"""GPU parity for the GEMM: sampled elements of C against the oracle's fp64 dot
product of the same quantised operands."""
import ctypes as C

import numpy as np
import pytest

from clpeak_b200 import native as N
from tests.gpu_util import dev_empty, stream_ptr, sync, to_np

pytestmark = pytest.mark.gpu

NP_DT = {N.DT_BF16: np.uint16, N.DT_F16: np.uint16, N.DT_E4M3: np.uint8}


def make_gemm_operands(K, cuda, dtype, m, n, k, seed=40):
    """A, B ~ N(0, 0.02) generated and quantised on the device (config 5)."""
    tdt = cuda.int16 if NP_DT[dtype] == np.uint16 else cuda.uint8
    out = []
    for rows, sd in ((m, seed), (n, seed + 1)):
        f = dev_empty(rows * k, cuda.float32)
        K.clpk_fill_f32(f.data_ptr(), rows * k, sd, N.DIST_NORMAL, 0.0, 0.02, stream_ptr())
        q = dev_empty(rows * k, tdt)
        K.clpk_convert_f32(q.data_ptr(), f.data_ptr(), rows * k, dtype, stream_ptr())
        out.append(q)
    sync()
    return out


def run_gemm(K, cuda, dtype, m, n, k, d_a, d_b):
    d_c = cuda.full((m * n,), 0x7FC0, dtype=cuda.int16, device="cuda")     # bf16 NaN canary
    d_status = dev_empty(1, cuda.int32)
    args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=d_a.data_ptr(), d_b=d_b.data_ptr(), d_c=d_c.data_ptr(),
                      d_sfa=None, d_sfb=None, alpha=1.0, d_workspace=None, workspace_bytes=0,
                      d_status=d_status.data_ptr())
    K.clpk_gemm(C.byref(args), stream_ptr())
    sync()
    assert int(to_np(d_status)[0]) == 0, "a device-side wait timed out"
    return d_c


def bf16_to_f64(u16: np.ndarray) -> np.ndarray:
    return (u16.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def check_samples(orc, dtype, a, b, c_u16, m, n, k, samples):
    worst = 0.0
    for (i, j) in samples:
        want, s = orc.gemm_element(dtype, a, b, k, int(i), int(j))
        got = float(bf16_to_f64(c_u16[i * n + j: i * n + j + 1])[0])
        # fp32 accumulation over K terms (<= K*2^-24 relative to sum|a||b|, generous
        # for a truncating adder) plus the final rounding to bf16 (2^-9 relative).
        tol = k * 2.0 ** -23 * s + 2.0 ** -8 * abs(want) + 1e-30
        worst = max(worst, abs(got - want) / tol)
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_F16, N.DT_E4M3])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (256, 256, 1024), (512, 768, 256), (1024, 1024, 2048)])
def test_gemm_small_full_check(K, orc, cuda, dtype, m, n, k):
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    d_c = run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    c = to_np(d_c).view(np.uint16)
    assert not np.any(c == 0x7FC0), "some of C was never written"
    rng = np.random.default_rng(1)
    samples = list(zip(rng.integers(0, m, 200), rng.integers(0, n, 200)))
    samples += [(0, 0), (m - 1, n - 1), (127, 128), (128, 127), (255, 255), (m - 1, 0), (0, n - 1)]
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_E4M3])
def test_gemm_4096_sampled(K, orc, cuda, dtype):
    m = n = k = 4096
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    d_c = run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    c = to_np(d_c).view(np.uint16)
    assert not np.any(c == 0x7FC0)
    rng = np.random.default_rng(2)
    samples = list(zip(rng.integers(0, m, 300), rng.integers(0, n, 300)))
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


def test_gemm_rejects_ragged(K, cuda):
    d = dev_empty(16, cuda.int16)
    args = N.GemmArgs(dtype=N.DT_BF16, m=250, n=256, k=128, d_a=d.data_ptr(), d_b=d.data_ptr(), d_c=d.data_ptr(),
                      alpha=1.0, d_status=d.data_ptr())
    with pytest.raises(N.ClpkError) as e:
        K.clpk_gemm(C.byref(args), None)
    assert e.value.code == N.ERR_BAD_ARG
