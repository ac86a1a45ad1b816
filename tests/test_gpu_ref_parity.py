"""The parity pin: the reference project's OWN CUDA kernels, compiled unchanged for sm_100a
(oracle/Makefile target `refcuda`), are launched on this GPU by oracle/ref_cuda_runner
(`--dump`), and their output buffers are compared bit for bit with the CPU oracle and with
this backend's kernels on the same inputs:

    reference kernel output == oracle == clpk_* output

Rows: src/cuda/cuda_kernels/compute_sp.cu:12-24, compute_hp.cu:24-58, compute_dp.cu:10-22,
compute_mp.cu:21-36, compute_bf16.cu:19-32, compute_int32.cu:15-27, compute_int8_dp.cu:26-122,
global_bandwidth.cu:14-71 (input: the reference's own `populate` stream,
src/common/common.cpp:76-95), local_bandwidth.cu:7-66, image_bandwidth.cu:9-26.
Floating chains that run away to +-inf are compared NaN-aware (a generated NaN's payload is not
part of the contract); everything else is bit-exact.  The tcgen05 rows have no counterpart in
the reference (its tensor kernels use constant fragments and `mma.sync`), so they stay pinned
to the oracle alone."""
import ctypes as C
import subprocess
from pathlib import Path

import numpy as np
import pytest

from clpeak_b200 import native as N

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
RUNNER = ROOT / "oracle" / "_ref" / "ref_cuda_runner"
CUBINS = ROOT / "oracle" / "_ref" / "cuda"


@pytest.fixture(scope="module")
def ref():
    if not RUNNER.exists() or not (CUBINS / "compute_sp.cubin").exists():
        pytest.skip("the reference's kernels have not been compiled (make -C oracle refcuda needs the reference checkout)")

    def dump(row, tmp_path, dtype=np.uint32, blocks=2, arg=None, input_array=None, dim=None):
        out = tmp_path / "ref.bin"
        cmd = [str(RUNNER), str(CUBINS), "--dump", row, str(out), "--blocks", str(blocks)]
        if arg is not None:
            cmd += ["--arg", repr(arg)]
        if input_array is not None:
            inp = tmp_path / "in.bin"
            np.ascontiguousarray(input_array).tofile(inp)
            cmd += ["--input", str(inp)]
        if dim is not None:
            cmd += ["--dim", str(dim[0]), str(dim[1])]
        r = subprocess.run(cmd, capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, f"{' '.join(cmd)}\n{r.stdout}\n{r.stderr}"
        return np.fromfile(out, dtype=dtype)

    return dump


def same_bits_nan_aware(got, want, ftype, what):
    g = np.ascontiguousarray(got).view(ftype)
    w = np.ascontiguousarray(want).view(ftype)
    assert g.shape == w.shape, f"{what}: {g.shape} vs {w.shape}"
    itype = np.uint32 if ftype == np.float32 else np.uint64
    ok = (g.view(itype) == w.view(itype)) | (np.isnan(g) & np.isnan(w))
    assert ok.all(), f"{what}: {np.count_nonzero(~ok)} values differ, first at {np.flatnonzero(~ok)[0]}"


# label of the reference row -> (test tag, CLPK_CHAIN_* or None for compute_sp, start values)
FLOAT_STARTS = [1.3, 0.25, -0.75, -0.5, 1e-3]
INT_STARTS = [3, 4, 125, -7]
CHAINS = [
    ("single_precision_compute/float", None, FLOAT_STARTS),
    ("half_precision_compute/half", N.CHAIN_HALF, FLOAT_STARTS),
    ("half_precision_compute/half2", N.CHAIN_HALF2, FLOAT_STARTS),
    ("double_precision_compute/double", N.CHAIN_DOUBLE, FLOAT_STARTS),
    ("mixed_precision_compute/mp", N.CHAIN_MIXED, FLOAT_STARTS),
    ("bfloat16_compute/bf16", N.CHAIN_BF16, FLOAT_STARTS),
    ("integer_compute/int", N.CHAIN_INT32, INT_STARTS),
    ("integer_compute_int8_dp/int8_dp", N.CHAIN_INT8_DOT1, INT_STARTS),
    ("integer_compute_int8_dp/int8_dp2", N.CHAIN_INT8_DOT2, INT_STARTS),
    ("integer_compute_int8_dp/int8_dp4", N.CHAIN_INT8_DOT4, INT_STARTS),
    ("integer_compute_int8_dp/int8_dp8", N.CHAIN_INT8_DOT8, INT_STARTS),
]


@pytest.mark.parametrize("row,chain,starts", CHAINS, ids=[c[0].split("/")[1] for c in CHAINS])
def test_chain_reference_kernel_equals_oracle_equals_ours(K, orc, cuda, ref, tmp_path, row, chain, starts):
    blocks = 3
    stream = cuda.cuda.current_stream().cuda_stream
    finite_outputs = 0
    for a in starts:
        wide = chain == N.CHAIN_DOUBLE
        theirs = ref(row, tmp_path, dtype=np.uint64 if wide else np.uint32, blocks=blocks, arg=a)
        if chain is None:
            want = orc.compute_sp(a, blocks * 256)
            out = cuda.zeros(blocks * 256, dtype=cuda.float32, device="cuda")
            K.clpk_compute_sp(out.data_ptr(), a, blocks, stream)
        else:
            want = orc.compute_chain(chain, a, blocks * 256)
            out = cuda.zeros(blocks * 256, dtype=cuda.int64 if wide else cuda.int32, device="cuda")
            K.clpk_compute_chain(chain, out.data_ptr(), float(a), blocks, stream)
        cuda.cuda.synchronize()
        ours = out.cpu().numpy()
        what = f"{row} from {a}"
        if chain is not None and chain >= N.CHAIN_INT32:
            assert np.array_equal(theirs.view(np.int32), want), what + ": reference kernel vs oracle"
            assert np.array_equal(ours, want), what + ": this backend vs oracle"
        else:
            ftype = np.float64 if wide else np.float32
            same_bits_nan_aware(theirs, want, ftype, what + ": reference kernel vs oracle")
            same_bits_nan_aware(ours, want, ftype, what + ": this backend vs oracle")
            same_bits_nan_aware(ours, theirs, ftype, what + ": this backend vs reference kernel")
            finite_outputs += int(np.isfinite(want.astype(np.float64)).sum())
    # some start keeps real numbers in the output (thread 0 adds c = 0, so a start below one in magnitude
    # decays instead of running away): the comparison is not inf == inf throughout
    if chain is None or chain < N.CHAIN_INT32:
        assert finite_outputs > 0, f"{row}: every output of every start is non-finite"


@pytest.mark.parametrize("width", [1, 2, 4])
@pytest.mark.parametrize("source", ["populate", "uniform"])
def test_global_bandwidth_reference_kernel_equals_oracle_equals_ours(K, orc, cuda, ref, tmp_path, width, source):
    blocks = 37
    n = blocks * 256 * 16 * width
    if source == "populate":
        src = np.empty(n, dtype=np.float32)
        orc.lib().orc_populate_reference(orc.ptr(src), n)      # the reference's own input stream
    else:
        src = orc.fill_f32(n, 1, 0)
    label = {1: "float", 2: "float2", 4: "float4"}[width]
    theirs = ref(f"global_memory_bandwidth/{label}", tmp_path, blocks=blocks, input_array=src)
    want = orc.global_bandwidth(width, src)
    d_in = cuda.from_numpy(src).cuda()
    d_out = cuda.zeros(blocks * 256, dtype=cuda.float32, device="cuda")
    K.clpk_global_bandwidth(width, d_in.data_ptr(), d_out.data_ptr(), n, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    ours = d_out.cpu().numpy()
    # The reference's stream sets bit 23 of every pattern, so one value in 128 has the exponent 0xFF
    # (infinity or NaN) and many sums are NaN; a generated NaN's payload is not part of the contract.
    same_bits_nan_aware(theirs, want, np.float32, "reference kernel vs oracle")
    same_bits_nan_aware(ours, want, np.float32, "this backend vs oracle")
    same_bits_nan_aware(ours, theirs, np.float32, "this backend vs reference kernel")
    finite = want[np.isfinite(want)]
    assert len(np.unique(finite)) > blocks * (200 if source == "uniform" else 100)
    if source == "uniform":
        assert np.isfinite(want).all()
        assert np.array_equal(theirs, want.view(np.uint32)) and np.array_equal(ours.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("width", [1, 2, 4])
def test_local_bandwidth_reference_kernel_equals_oracle_equals_ours(K, orc, cuda, ref, tmp_path, width):
    blocks = 5
    label = {1: "float", 2: "float2", 4: "float4"}[width]
    theirs = ref(f"local_memory_bandwidth/{label}", tmp_path, blocks=blocks)
    want = orc.local_bandwidth(width, blocks * 256)
    out = cuda.zeros(blocks * 256, dtype=cuda.float32, device="cuda")
    K.clpk_local_bandwidth(width, out.data_ptr(), blocks, cuda.cuda.current_stream().cuda_stream)
    cuda.cuda.synchronize()
    assert np.array_equal(theirs, want.view(np.uint32)), "reference kernel vs oracle"
    assert np.array_equal(out.cpu().numpy().view(np.uint32), want.view(np.uint32)), "this backend vs oracle"


@pytest.mark.parametrize("shape", [(256, 128), (1024, 48), (384, 96)])
def test_image_bandwidth_reference_kernel_equals_oracle_equals_ours(K, orc, cuda, ref, tmp_path, shape):
    w, h = shape
    seed = 11
    texels = w * h
    threads = texels // 16
    image = orc.fill_f32(texels * 4, seed, 0)                    # texel p, channel ch = uniform01(seed, 4p + ch)
    theirs = ref("image_memory_bandwidth/float4", tmp_path, input_array=image, dim=(w, h))
    want = orc.image_bandwidth(threads, texels, seed)
    stream = cuda.cuda.current_stream().cuda_stream
    img = C.c_void_p(None)
    K.clpk_image_create(C.byref(img), w, h, seed, stream)
    try:
        out = cuda.zeros(threads, dtype=cuda.float32, device="cuda")
        K.clpk_image_bandwidth(img, out.data_ptr(), threads // 256, stream)
        cuda.cuda.synchronize()
        ours = out.cpu().numpy()
    finally:
        K.clpk_image_destroy(img)
    assert np.array_equal(theirs, want.view(np.uint32)), "reference kernel vs oracle"
    assert np.array_equal(ours.view(np.uint32), want.view(np.uint32)), "this backend vs oracle"
