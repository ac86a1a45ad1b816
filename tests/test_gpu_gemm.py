"""GPU parity for the GEMM: sampled elements of C against the oracle's fp64 dot
product of the same quantised operands."""
import ctypes as C

import numpy as np
import pytest

from clpeak_b200 import native as N
from tests.gpu_util import dev_empty, stream_ptr, sync, to_np

pytestmark = pytest.mark.gpu

NP_DT = {N.DT_BF16: np.uint16, N.DT_F16: np.uint16, N.DT_E4M3: np.uint8, N.DT_E5M2: np.uint8, N.DT_I8: np.int8,
         N.DT_TF32: np.uint32}
WIDE_OUT = (N.DT_TF32, N.DT_I8)          # fp32 / int32 output; everything else writes bf16


def make_gemm_operands(K, cuda, dtype, m, n, k, seed=40):
    """A, B ~ N(0, 0.02) generated and quantised on the device (config 5); int8 draws uniform[-8, 7].
    The E5M2 variant pairs an e5m2 A with an e4m3 B."""
    tdt = {np.uint16: cuda.int16, np.uint8: cuda.uint8, np.int8: cuda.int8, np.uint32: cuda.int32}[NP_DT[dtype]]
    out = []
    for which, (rows, sd) in enumerate(((m, seed), (n, seed + 1))):
        q = dev_empty(rows * k, tdt)
        if dtype == N.DT_I8:
            K.clpk_fill_i8(q.data_ptr(), rows * k, sd, stream_ptr())
        else:
            f = dev_empty(rows * k, cuda.float32)
            K.clpk_fill_f32(f.data_ptr(), rows * k, sd, N.DIST_NORMAL, 0.0, 0.02, stream_ptr())
            conv = N.DT_E4M3 if (dtype == N.DT_E5M2 and which == 1) else dtype
            K.clpk_convert_f32(q.data_ptr(), f.data_ptr(), rows * k, conv, stream_ptr())
        out.append(q)
    sync()
    return out


def run_gemm(K, cuda, dtype, m, n, k, d_a, d_b):
    if dtype in WIDE_OUT:
        d_c = cuda.full((m * n,), 0x7FC00000, dtype=cuda.int32, device="cuda")   # fp32 NaN / unlikely int canary
    else:
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
        if dtype == N.DT_I8:
            assert int(c_u16.view(np.int32)[i * n + j]) == int(want), f"int8 GEMM element ({i},{j}) is not exact"
            continue
        if dtype == N.DT_TF32:
            got = float(c_u16.view(np.float32)[i * n + j])
            worst = max(worst, abs(got - want) / (k * 2.0 ** -23 * s + 1e-30))      # fp32 out: no output rounding term
            continue
        got = float(bf16_to_f64(c_u16[i * n + j: i * n + j + 1])[0])
        # fp32 accumulation over K terms (<= K*2^-24 relative to sum|a||b|, generous
        # for a truncating adder) plus the final rounding to bf16 (2^-9 relative).
        tol = k * 2.0 ** -23 * s + 2.0 ** -8 * abs(want) + 1e-30
        worst = max(worst, abs(got - want) / tol)
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"


def c_view(dtype, d_c):
    c = to_np(d_c)
    if dtype in WIDE_OUT:
        assert not np.any(c.view(np.uint32) == 0x7FC00000), "some of C was never written"
        return c.view(np.uint32)
    assert not np.any(c.view(np.uint16) == 0x7FC0), "some of C was never written"
    return c.view(np.uint16)


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_F16, N.DT_E4M3, N.DT_E5M2, N.DT_TF32, N.DT_I8])
@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (256, 256, 1024), (512, 768, 256), (1024, 1024, 2048)])
def test_gemm_small_full_check(K, orc, cuda, dtype, m, n, k):
    if dtype == N.DT_TF32:
        k = max(k // 4, 32)               # K counts elements; the kernel wants 128 bytes of K per stage
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    d_c = run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    c = c_view(dtype, d_c)
    rng = np.random.default_rng(1)
    samples = list(zip(rng.integers(0, m, 200), rng.integers(0, n, 200)))
    samples += [(0, 0), (m - 1, n - 1), (127, 128), (128, 127), (255, 255), (m - 1, 0), (0, n - 1)]
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_E4M3, N.DT_I8, N.DT_TF32])
def test_gemm_4096_sampled(K, orc, cuda, dtype):
    m = n = k = 4096
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    d_c = run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    c = c_view(dtype, d_c)
    rng = np.random.default_rng(2)
    samples = list(zip(rng.integers(0, m, 300), rng.integers(0, n, 300)))
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_E4M3])
def test_gemm_8192_sampled(K, orc, cuda, dtype):
    """The middle size of the GEMM configuration (M = N = K = 8192): 16 x 32 tiles, several waves."""
    m = n = k = 8192
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    d_c = run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    c = c_view(dtype, d_c)
    rng = np.random.default_rng(3)
    samples = list(zip(rng.integers(0, m, 200), rng.integers(0, n, 200))) + [(0, 0), (m - 1, n - 1), (511, 256), (512, 255)]
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_E4M3, N.DT_TF32, N.DT_I8])
@pytest.mark.parametrize("m,n,k", [(8, 8, 16), (200, 328, 80), (513, 264, 1040), (1000, 1016, 528), (2304, 1800, 144)])
def test_gemm_ragged_shapes_every_element(K, orc, cuda, dtype, m, n, k):
    """Shapes that are not whole tiles: TMA zero-fills what a box reads beyond A and B and clips what a box would
    store beyond C.  int8, bf16 and tf32 compare every element of C, e4m3 a sample with the four corners; the canary
    after C must stay (nothing is written beyond it) and none may remain inside it."""
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    wide = dtype in WIDE_OUT
    pad = 4096
    d_c = cuda.full((m * n + pad,), 0x7FC00000 if wide else 0x7FC0, dtype=cuda.int32 if wide else cuda.int16, device="cuda")
    d_status = dev_empty(1, cuda.int32)
    args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=d_a.data_ptr(), d_b=d_b.data_ptr(), d_c=d_c.data_ptr(), alpha=1.0,
                      d_status=d_status.data_ptr())
    K.clpk_gemm(C.byref(args), stream_ptr())
    sync()
    assert int(to_np(d_status)[0]) == 0
    c_all = to_np(d_c)
    canary = 0x7FC00000 if wide else 0x7FC0
    assert np.all(c_all[m * n:].view(np.uint32 if wide else np.uint16) == canary), "the kernel wrote beyond C"
    c = c_all[:m * n].view(np.uint32 if wide else np.uint16)
    assert not np.any(c == canary), "some of C was never written"
    a = to_np(d_a).view(NP_DT[dtype])
    b = to_np(d_b).view(NP_DT[dtype])
    if dtype == N.DT_I8:
        want = a.reshape(m, k).astype(np.int64) @ b.reshape(n, k).astype(np.int64).T
        assert np.array_equal(c.view(np.int32).reshape(m, n), want.astype(np.int32))
        return
    if dtype in (N.DT_BF16, N.DT_TF32):
        fa = (bf16_to_f64(a) if dtype == N.DT_BF16 else a.view(np.float32).astype(np.float64)).reshape(m, k)
        fb = (bf16_to_f64(b) if dtype == N.DT_BF16 else b.view(np.float32).astype(np.float64)).reshape(n, k)
        want, s = fa @ fb.T, np.abs(fa) @ np.abs(fb).T
        got = (bf16_to_f64(c) if dtype == N.DT_BF16 else c.view(np.float32).astype(np.float64)).reshape(m, n)
        tol = k * 2.0 ** -23 * s + (2.0 ** -8 * np.abs(want) if dtype == N.DT_BF16 else 0.0) + 1e-30
        worst = float(np.max(np.abs(got - want) / tol))
        assert worst <= 1.0, f"worst error over all of C is {worst:.3g}x the stated tolerance"
        return
    rng = np.random.default_rng(11)
    samples = list(zip(rng.integers(0, m, 300), rng.integers(0, n, 300))) + [(0, 0), (m - 1, n - 1), (m - 1, 0), (0, n - 1)]
    check_samples(orc, dtype, a, b, c, m, n, k, samples)


def test_gemm_rejects_misaligned_rows(K, cuda):
    d = dev_empty(4096, cuda.int16)
    for m, n, k in ((256, 256, 100), (256, 250, 128)):           # a row of A or of C that is not a multiple of 16 bytes
        args = N.GemmArgs(dtype=N.DT_BF16, m=m, n=n, k=k, d_a=d.data_ptr(), d_b=d.data_ptr(), d_c=d.data_ptr(),
                          alpha=1.0, d_status=d.data_ptr())
        with pytest.raises(N.ClpkError) as e:
            K.clpk_gemm(C.byref(args), None)
        assert e.value.code == N.ERR_BAD_ARG


# ---- NVFP4 ---------------------------------------------------------------------------------

def make_nvfp4_operand(K, cuda, rows, k, seed, dtype=N.DT_NVF4):
    """N(0, 0.02) values quantised on the device: packed e2m1 with a ue4m3 scale per 16 and an fp32
    tensor scale (NVFP4), or a ue8m0 scale per 32 and no tensor scale (MXFP4)."""
    f = dev_empty(rows * k, cuda.float32)
    K.clpk_fill_f32(f.data_ptr(), rows * k, seed, N.DIST_NORMAL, 0.0, 0.02, stream_ptr())
    am = dev_empty(1, cuda.float32)
    K.clpk_absmax_f32(am.data_ptr(), f.data_ptr(), rows * k, stream_ptr())
    sync()
    ts = float(np.float32(to_np(am)[0]) / np.float32(6.0 * 448.0)) if dtype == N.DT_NVF4 else 1.0
    q = dev_empty(rows * k // 2, cuda.uint8)
    sf = dev_empty(rows * k // (16 if dtype == N.DT_NVF4 else 32), cuda.uint8)
    K.clpk_quantize_fp4(q.data_ptr(), sf.data_ptr(), f.data_ptr(), rows, k, dtype, ts, stream_ptr())
    sync()
    return q, sf, ts, f


def run_nvfp4(K, cuda, m, n, k, dtype=N.DT_NVF4):
    a, sfa, tsa, fa = make_nvfp4_operand(K, cuda, m, k, 40, dtype)
    b, sfb, tsb, fb = make_nvfp4_operand(K, cuda, n, k, 41, dtype)
    c = cuda.full((m * n + 2048,), 0x7FC0, dtype=cuda.int16, device="cuda")     # the tail is a canary: nothing is written beyond C
    need = C.c_size_t(0)
    K.clpk_gemm_workspace_bytes(dtype, m, n, k, C.byref(need))
    pad = lambda rows: (rows + 255) // 256 * 256                # scale blocks cover whole 256-row tiles
    assert need.value == (pad(m) + pad(n)) * (k // (16 if dtype == N.DT_NVF4 else 32))
    ws = dev_empty(need.value, cuda.uint8)
    st = dev_empty(1, cuda.int32)
    alpha = float(np.float32(tsa) * np.float32(tsb))
    args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=a.data_ptr(), d_b=b.data_ptr(), d_c=c.data_ptr(),
                      d_sfa=sfa.data_ptr(), d_sfb=sfb.data_ptr(), alpha=alpha, d_workspace=ws.data_ptr(),
                      workspace_bytes=need.value, d_status=st.data_ptr())
    K.clpk_gemm(C.byref(args), stream_ptr())
    sync()
    assert int(to_np(st)[0]) == 0
    c_all = to_np(c).view(np.uint16)
    assert np.all(c_all[m * n:] == 0x7FC0), "the kernel wrote beyond C"
    return dict(a=to_np(a), b=to_np(b), sfa=to_np(sfa), sfb=to_np(sfb), c=c_all[:m * n], alpha=alpha, fa=fa, fb=fb)


@pytest.mark.parametrize("dtype", [N.DT_NVF4, N.DT_MXF4])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (256, 512, 1024), (768, 256, 512), (2048, 2048, 2048),
                                   (200, 328, 256), (1000, 1016, 512), (264, 8, 768), (1, 136, 256)])
def test_gemm_nvfp4(K, orc, cuda, m, n, k, dtype):
    """Whole tiles and shapes that are not (the scale blocks are packed for whole tiles, with zero factors for the
    rows beyond M and N)."""
    r = run_nvfp4(K, cuda, m, n, k, dtype)
    assert not np.any(r["c"] == 0x7FC0)
    rng = np.random.default_rng(5)
    samples = list(zip(rng.integers(0, m, 120), rng.integers(0, n, 120))) + [(0, 0), (m - 1, n - 1), (min(127, m - 1), min(128, n - 1)), (min(128, m - 1), min(127, n - 1))]
    worst = 0.0
    for (i, j) in samples:
        want, s = orc.gemm_element(dtype, r["a"], r["b"], k, int(i), int(j), r["sfa"], r["sfb"])
        want *= r["alpha"]
        s *= r["alpha"]
        got = float(bf16_to_f64(r["c"][i * n + j: i * n + j + 1])[0])
        tol = k * 2.0 ** -23 * s + 2.0 ** -8 * abs(want) + 1e-30
        worst = max(worst, abs(got - want) / tol)
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"


@pytest.mark.parametrize("dtype", [N.DT_NVF4, N.DT_MXF4])
@pytest.mark.parametrize("m", [4096, 8192])
def test_gemm_fp4_config_sizes_sampled(K, orc, cuda, dtype, m):
    """The block-scaled GEMM at the sizes the GEMM configuration names (4096 and 8192 cubed; 16384 cubed is
    checked by the benchmark itself on the result it times)."""
    r = run_nvfp4(K, cuda, m, m, m, dtype)
    assert not np.any(r["c"] == 0x7FC0)
    rng = np.random.default_rng(6)
    samples = list(zip(rng.integers(0, m, 150), rng.integers(0, m, 150))) + [(0, 0), (m - 1, m - 1), (255, 256), (256, 255)]
    worst = 0.0
    for (i, j) in samples:
        want, s_abs = orc.gemm_element(dtype, r["a"], r["b"], m, int(i), int(j), r["sfa"], r["sfb"])
        want *= r["alpha"]
        s_abs *= r["alpha"]
        got = float(bf16_to_f64(r["c"][i * m + j: i * m + j + 1])[0])
        tol = m * 2.0 ** -23 * s_abs + 2.0 ** -8 * abs(want) + 1e-30
        worst = max(worst, abs(got - want) / tol)
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"


@pytest.mark.parametrize("dtype", [N.DT_NVF4, N.DT_MXF4])
@pytest.mark.parametrize("m,n,k", [(256, 256, 256), (256, 768, 1024), (1024, 512, 2304), (4096, 4096, 4096), (520, 392, 512)])
def test_gemm_fp4_both_tile_shapes_give_the_same_bits(K, orc, cuda, dtype, m, n, k):
    """The 256 x 128 two-accumulator tile (the epilogue of one tile overlaps the main loop of the next) against
    the 256 x 256 single-accumulator tile: every element of C is one cluster's sum over K in the same order
    either way, so the outputs are bit-identical; the wide one is checked against the oracle elsewhere, the
    narrow one here as well."""
    try:
        K.clpk_set_tuning(N.TUNE_GEMM_FP4_TILE, 1)
        wide = run_nvfp4(K, cuda, m, n, k, dtype)
        K.clpk_set_tuning(N.TUNE_GEMM_FP4_TILE, 2)
        narrow = run_nvfp4(K, cuda, m, n, k, dtype)
    finally:
        K.clpk_set_tuning(N.TUNE_GEMM_FP4_TILE, -1)
    assert not np.any(narrow["c"] == 0x7FC0), "some of C was never written"
    rng = np.random.default_rng(8)
    worst = 0.0
    for (i, j) in list(zip(rng.integers(0, m, 60), rng.integers(0, n, 60))) + [(0, 0), (m - 1, n - 1), (255, 127), (128, 128)]:
        want, s_abs = orc.gemm_element(dtype, narrow["a"], narrow["b"], k, int(i), int(j), narrow["sfa"], narrow["sfb"])
        want *= narrow["alpha"]
        s_abs *= narrow["alpha"]
        got = float(bf16_to_f64(narrow["c"][i * n + j: i * n + j + 1])[0])
        worst = max(worst, abs(got - want) / (k * 2.0 ** -23 * s_abs + 2.0 ** -8 * abs(want) + 1e-30))
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"
    assert np.array_equal(wide["c"], narrow["c"])


@pytest.mark.parametrize("dtype", [N.DT_NVF4, N.DT_MXF4])
def test_gemm_nvfp4_tracks_the_unquantised_product(K, orc, cuda, dtype):
    """End-to-end sanity of the whole recipe (quantiser + scales + tensor scale): C correlates with fp32 A.B^T."""
    m = n = 256
    k = 2048
    r = run_nvfp4(K, cuda, m, n, k, dtype)
    ref = (r["fa"].view(m, k) @ r["fb"].view(n, k).T).cpu().numpy().astype(np.float64)
    got = bf16_to_f64(r["c"]).reshape(m, n)
    assert np.corrcoef(ref.ravel(), got.ravel())[0, 1] > 0.98


@pytest.mark.parametrize("dtype", [N.DT_NVF4, N.DT_MXF4])
def test_gemm_fp4_scales_packed_once_give_the_same_bits(K, cuda, dtype):
    """clpk_gemm_pack_scales + clpk_gemm(d_sfa = d_sfb = NULL) is the one-call path split in two."""
    m, n, k = 512, 768, 1024
    r = run_nvfp4(K, cuda, m, n, k, dtype)
    a, sfa, tsa, _ = make_nvfp4_operand(K, cuda, m, k, 40, dtype)
    b, sfb, tsb, _ = make_nvfp4_operand(K, cuda, n, k, 41, dtype)
    need = C.c_size_t(0)
    K.clpk_gemm_workspace_bytes(dtype, m, n, k, C.byref(need))
    ws = dev_empty(need.value, cuda.uint8)
    st = dev_empty(1, cuda.int32)
    c = cuda.full((m * n,), 0x7FC0, dtype=cuda.int16, device="cuda")
    args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=a.data_ptr(), d_b=b.data_ptr(), d_c=c.data_ptr(),
                      d_sfa=sfa.data_ptr(), d_sfb=sfb.data_ptr(), alpha=r["alpha"], d_workspace=ws.data_ptr(),
                      workspace_bytes=need.value, d_status=st.data_ptr())
    K.clpk_gemm_pack_scales(C.byref(args), stream_ptr())
    args.d_sfa = None
    args.d_sfb = None
    for _ in range(2):                              # the packed workspace is not consumed by a call
        c.fill_(0x7FC0)
        K.clpk_gemm(C.byref(args), stream_ptr())
        sync()
        assert int(to_np(st)[0]) == 0
        assert np.array_equal(to_np(c).view(np.uint16), r["c"])
    args.d_sfa = sfa.data_ptr()                     # one scale array without the other is an error
    with pytest.raises(N.ClpkError) as e:
        K.clpk_gemm(C.byref(args), stream_ptr())
    assert e.value.code == N.ERR_BAD_ARG


def test_gemm_nvfp4_argument_checks(K, cuda):
    d = dev_empty(64, cuda.uint8)
    args = N.GemmArgs(dtype=N.DT_NVF4, m=256, n=256, k=128, d_a=d.data_ptr(), d_b=d.data_ptr(), d_c=d.data_ptr(),
                      d_sfa=d.data_ptr(), d_sfb=d.data_ptr(), alpha=1.0, d_workspace=d.data_ptr(), workspace_bytes=64,
                      d_status=d.data_ptr())
    with pytest.raises(N.ClpkError) as e:
        K.clpk_gemm(C.byref(args), None)                 # K must be a multiple of 256
    assert e.value.code == N.ERR_BAD_ARG
    args.k, args.n = 256, 260
    with pytest.raises(N.ClpkError) as e:
        K.clpk_gemm(C.byref(args), None)                 # a row of C (bf16) must be a multiple of 16 bytes
    assert e.value.code == N.ERR_BAD_ARG
    args.n = 256
    with pytest.raises(N.ClpkError) as e:
        K.clpk_gemm(C.byref(args), None)                 # workspace too small
    assert e.value.code == N.ERR_BAD_ARG


# ---- scheduling knobs do not change the numbers ---------------------------------------------

@pytest.mark.parametrize("dtype", [N.DT_BF16, N.DT_I8])
def test_gemm_is_bitwise_the_same_with_and_without_producer_alignment(K, cuda, dtype):
    """The per-wave meeting of the producers and the raster group width only move work in time and
    across SM pairs; every element of C is still one cluster's sum over K in the same order."""
    m, n, k = 8192, 8192, 256                # 512 tiles on 74 clusters: seven waves, so the producers do meet
    d_a, d_b = make_gemm_operands(K, cuda, dtype, m, n, k)
    knobs = (N.TUNE_GEMM_NO_ALIGN, N.TUNE_GEMM_GROUP, N.TUNE_GEMM_ALIGN_AT)
    for knob in knobs:
        K.clpk_set_tuning(knob, -1)
    base = to_np(run_gemm(K, cuda, dtype, m, n, k, d_a, d_b)).copy()
    assert K.raw("clpk_gemm_last_launch_aligned")() == 1          # seven waves: the producers do meet
    try:
        for knob, val in ((N.TUNE_GEMM_NO_ALIGN, 1), (N.TUNE_GEMM_GROUP, 3), (N.TUNE_GEMM_ALIGN_AT, 0)):
            K.clpk_set_tuning(knob, val)
            other = to_np(run_gemm(K, cuda, dtype, m, n, k, d_a, d_b))
            assert K.raw("clpk_gemm_last_launch_aligned")() == (0 if knob == N.TUNE_GEMM_NO_ALIGN else 1)
            assert np.array_equal(base.view(np.uint8), other.view(np.uint8)), (knob, val)
            K.clpk_set_tuning(knob, -1)
    finally:
        for knob in knobs:
            K.clpk_set_tuning(knob, -1)


def test_gemm_many_waves_small_k(K, orc, cuda):
    """Many short tiles: 16 x 32 = 512 tiles of 512 x 256 on 74 clusters (7 waves) with K = 128."""
    m = n = 8192
    k = 128
    d_a, d_b = make_gemm_operands(K, cuda, N.DT_BF16, m, n, k)
    d_c = run_gemm(K, cuda, N.DT_BF16, m, n, k, d_a, d_b)
    a = to_np(d_a).view(np.uint16)
    b = to_np(d_b).view(np.uint16)
    c = c_view(N.DT_BF16, d_c)
    rng = np.random.default_rng(9)
    samples = list(zip(rng.integers(0, m, 400), rng.integers(0, n, 400))) + [(m - 1, n - 1), (0, 0), (511, 255), (512, 256)]
    check_samples(orc, N.DT_BF16, a, b, c, m, n, k, samples)


# ---- fp32 (CUDA cores) and fp64 (DMMA): the rows without a tcgen05 kind --------------------------------

def run_simt_gemm(K, cuda, dtype, m, n, k, alpha=1.0):
    """A, B ~ N(0, 0.02) generated on the device as fp32; the fp64 operands are those floats widened."""
    wide = dtype == N.DT_F64
    tdt = cuda.float64 if wide else cuda.float32
    ops = []
    for rows, seed in ((m, 40), (n, 41)):
        f = dev_empty(rows * k, cuda.float32)
        K.clpk_fill_f32(f.data_ptr(), rows * k, seed, N.DIST_NORMAL, 0.0, 0.02, stream_ptr())
        if wide:
            q = dev_empty(rows * k, cuda.float64)
            K.clpk_convert_f32(q.data_ptr(), f.data_ptr(), rows * k, N.DT_F64, stream_ptr())
            f = q
        ops.append(f)
    pad = 1024                                                 # canary after C: nothing may be written there
    c = cuda.full((m * n + pad,), float("nan"), dtype=tdt, device="cuda")
    st = dev_empty(1, cuda.int32)
    args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=ops[0].data_ptr(), d_b=ops[1].data_ptr(), d_c=c.data_ptr(),
                      d_sfa=None, d_sfb=None, alpha=alpha, d_workspace=None, workspace_bytes=0, d_status=st.data_ptr())
    K.clpk_gemm(C.byref(args), stream_ptr())
    sync()
    assert int(to_np(st)[0]) == 0
    c_all = to_np(c)
    assert np.isnan(c_all[m * n:]).all(), "the kernel wrote beyond C"
    return to_np(ops[0]), to_np(ops[1]), c_all[:m * n]


@pytest.mark.parametrize("dtype", [N.DT_F32, N.DT_F64])
@pytest.mark.parametrize("m,n,k", [(128, 128, 16), (256, 384, 64), (384, 128, 1040), (2048, 2048, 512), (4096, 4096, 4096),
                                   (1, 1, 4), (100, 72, 20), (129, 131, 36), (300, 202, 1044), (64, 257, 16), (1000, 1001, 260)])
def test_simt_gemm_against_the_oracle(K, orc, cuda, dtype, m, n, k):
    """Every element of the small cases, samples of the large one, against the oracle's fp64 dot product; whole
    tiles and shapes that are not (M, N not multiples of the tile, K not of the k block, N odd).
    Tolerance: K sequential roundings of the accumulator, K * u * sum|a||b| with u = 2^-23 (fp32; one extra
    bit over the unit roundoff for the host's own accumulation) or 2^-51 (fp64)."""
    a, b, c = run_simt_gemm(K, cuda, dtype, m, n, k)
    assert not np.isnan(c).any(), "some of C was never written"
    u = 2.0 ** -51 if dtype == N.DT_F64 else 2.0 ** -23
    if m * n <= 256 * 384:
        want = a.reshape(m, k).astype(np.float64) @ b.reshape(n, k).astype(np.float64).T
        s_abs = np.abs(a.reshape(m, k)).astype(np.float64) @ np.abs(b.reshape(n, k)).astype(np.float64).T
        assert np.all(np.abs(c.reshape(m, n).astype(np.float64) - want) <= k * u * s_abs + 1e-300)
    rng = np.random.default_rng(4)
    samples = list(zip(rng.integers(0, m, 150), rng.integers(0, n, 150))) + [(0, 0), (m - 1, n - 1), (min(127, m - 1), 0), (0, min(127, n - 1))]
    worst = 0.0
    for i, j in samples:
        want, s_abs = orc.gemm_element(dtype, a, b, k, int(i), int(j))
        worst = max(worst, abs(float(c[i * n + j]) - want) / (k * u * s_abs + 1e-300))
    assert worst <= 1.0, f"worst sampled error is {worst:.3g}x the stated tolerance"


@pytest.mark.parametrize("dtype", [N.DT_F32, N.DT_F64])
def test_simt_gemm_alpha_and_argument_checks(K, orc, cuda, dtype):
    a, b, c1 = run_simt_gemm(K, cuda, dtype, 128, 256, 64)
    _, _, c2 = run_simt_gemm(K, cuda, dtype, 128, 256, 64, alpha=0.5)
    assert np.array_equal(c2, c1 * 0.5)                        # a power of two scales exactly
    d = dev_empty(64, cuda.float64)
    for m, n, k in ((0, 128, 16), (128, 128, 0), (128, 128, 17), (128, 64, 1)):      # empty, or rows not a multiple of 16 bytes
        args = N.GemmArgs(dtype=dtype, m=m, n=n, k=k, d_a=d.data_ptr(), d_b=d.data_ptr(), d_c=d.data_ptr(), alpha=1.0,
                          d_status=d.data_ptr())
        with pytest.raises(N.ClpkError) as e:
            K.clpk_gemm(C.byref(args), None)
        assert e.value.code == N.ERR_BAD_ARG


def test_gemm_reports_the_clock_it_ran_at(K, cuda):
    """clpk_gemm_last_clock: CTA 0's clock64 / %globaltimer span of the last tensor-core GEMM; the quotient is an SM
    clock, which on a B200 lies between the idle floor and the 1.965 GHz maximum, and the span is close to the
    launch's CUDA-event duration."""
    m = n = k = 4096
    d_a, d_b = make_gemm_operands(K, cuda, N.DT_BF16, m, n, k)
    run_gemm(K, cuda, N.DT_BF16, m, n, k, d_a, d_b)                      # warm
    e0, e1 = cuda.cuda.Event(enable_timing=True), cuda.cuda.Event(enable_timing=True)
    e0.record()
    run_gemm(K, cuda, N.DT_BF16, m, n, k, d_a, d_b)
    e1.record()
    cuda.cuda.synchronize()
    cyc, ns = C.c_ulonglong(0), C.c_ulonglong(0)
    K.clpk_gemm_last_clock(C.byref(cyc), C.byref(ns), stream_ptr())
    mhz = cyc.value / ns.value * 1e3
    assert 500.0 < mhz < 2100.0, mhz
    assert 50e3 < ns.value < e0.elapsed_time(e1) * 1e6                    # the kernel's span lies inside the bracketed call
