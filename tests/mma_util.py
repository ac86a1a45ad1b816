"""Operand construction and checking for the tensor-core tests.

Benchmark configuration: dense kinds draw uniform[-1,1) (ints uniform[-8,7]) from
seed 2; block-scaled kinds draw N(0,1) from seed 3 and quantise per block.
"""
import numpy as np

from clpeak_b200 import native as N

DENSE_DT = {N.MMA_F16: N.DT_F16, N.MMA_BF16: N.DT_BF16, N.MMA_E4M3: N.DT_E4M3, N.MMA_E5M2: N.DT_E5M2,
            N.MMA_TF32: N.DT_TF32, N.MMA_F16_F16: N.DT_F16}
KIND_K = {N.MMA_TF32: 8, N.MMA_F16_F16: 16, N.MMA_E2M1: 32, N.MMA_F16: 16, N.MMA_BF16: 16, N.MMA_E4M3: 32, N.MMA_E5M2: 32, N.MMA_I8: 32, N.MMA_MXF4: 64,
          N.MMA_NVF4: 64, N.MMA_E4M3_SP: 64, N.MMA_I8_SP: 64, N.MMA_MXF4_SP: 128, N.MMA_NVF4_SP: 128}
SPARSE = (N.MMA_E4M3_SP, N.MMA_I8_SP, N.MMA_MXF4_SP, N.MMA_NVF4_SP)


def make_sparse_operands(orc, kind):
    """2:4 sparse kinds: a dense A tile is pruned (top-2 |x| of every 4; 4-bit kinds in pairs:
    top-2 of every 4 pairs), compressed to K/2 and quantised; B stays dense over the logical K."""
    k = KIND_K[kind]
    if kind == N.MMA_I8_SP:
        dense = orc.fill_i8(128 * k, 2).astype(np.float32).reshape(128, k)
        comp, meta, pruned = orc.prune_2to4(dense)
        b = orc.fill_i8(256 * k, 2, first=128 * k).reshape(256, k)
        return dict(a=comp.astype(np.int8), b=b, meta=meta, sfa=None, sfb=None, pruned=pruned, tensor_scale=(1.0, 1.0))
    if kind == N.MMA_E4M3_SP:
        dense = orc.fill_f32(128 * k, 2, 1).reshape(128, k)
        comp, meta, pruned = orc.prune_2to4(dense)
        b = orc.convert_f32(orc.fill_f32(256 * k, 2, 1, first=128 * k), N.DT_E4M3).reshape(256, k)
        return dict(a=orc.convert_f32(comp.ravel(), N.DT_E4M3).reshape(128, k // 2), b=b, meta=meta, sfa=None, sfb=None,
                    pruned=pruned, tensor_scale=(1.0, 1.0))
    dense = orc.fill_f32(128 * k, 3, 2).reshape(128, k)
    comp, meta, pruned = orc.prune_2to4(dense, pairs=True)
    fb = orc.fill_f32(256 * k, 3, 2, first=128 * k).reshape(256, k)
    if kind == N.MMA_NVF4_SP:
        tsa = np.float32(np.abs(comp).max()) / np.float32(6.0 * 448.0)
        tsb = np.float32(np.abs(fb).max()) / np.float32(6.0 * 448.0)
        a, sfa = orc.quantize_fp4(comp, N.DT_NVF4, float(tsa))          # 16 compressed = 32 logical per scale
        b, sfb = orc.quantize_fp4(fb, N.DT_NVF4_B32, float(tsb))
    else:
        tsa = tsb = np.float32(1.0)
        a, sfa = orc.quantize_fp4(comp, N.DT_MXF4)                       # 32 compressed = 64 logical per scale
        b, sfb = orc.quantize_fp4(fb, N.DT_MXF4_B64)
    return dict(a=a, b=b, meta=meta, sfa=sfa, sfb=sfb, pruned=pruned, tensor_scale=(float(tsa), float(tsb)))


def make_operands(orc, kind):
    """Returns dict(a, b, sfa, sfb, tensor_scale) of numpy arrays in the kernel's input encoding."""
    if kind in SPARSE:
        return make_sparse_operands(orc, kind)
    k = KIND_K[kind]
    if kind == N.MMA_I8:
        a = orc.fill_i8(128 * k, 2).reshape(128, k)
        b = orc.fill_i8(256 * k, 2, first=128 * k).reshape(256, k)
        return dict(a=a, b=b, sfa=None, sfb=None, tensor_scale=(1.0, 1.0))
    if kind == N.MMA_E2M1:
        # unscaled 4-bit operands: uniform[-1,1) stretched over e2m1's range (+-6)
        fa = orc.fill_f32(128 * k, 2, 1) * np.float32(6.0)
        fb = orc.fill_f32(256 * k, 2, 1, first=128 * k) * np.float32(6.0)
        return dict(a=orc.convert_f32(fa, N.DT_E2M1).reshape(128, k // 2),
                    b=orc.convert_f32(fb, N.DT_E2M1).reshape(256, k // 2), sfa=None, sfb=None, tensor_scale=(1.0, 1.0))
    if kind in DENSE_DT:
        fa = orc.fill_f32(128 * k, 2, 1)
        fb = orc.fill_f32(256 * k, 2, 1, first=128 * k)
        a = orc.convert_f32(fa, DENSE_DT[kind]).reshape(128, k)
        b = orc.convert_f32(fb, DENSE_DT[kind]).reshape(256, k)
        return dict(a=a, b=b, sfa=None, sfb=None, tensor_scale=(1.0, 1.0))
    dt = N.DT_MXF4 if kind == N.MMA_MXF4 else N.DT_NVF4
    fa = orc.fill_f32(128 * k, 3, 2).reshape(128, k)
    fb = orc.fill_f32(256 * k, 3, 2, first=128 * k).reshape(256, k)
    if dt == N.DT_NVF4:
        tsa = np.float32(np.abs(fa).max()) / np.float32(6.0 * 448.0)
        tsb = np.float32(np.abs(fb).max()) / np.float32(6.0 * 448.0)
    else:
        tsa = tsb = np.float32(1.0)
    a, sfa = orc.quantize_fp4(fa, dt, float(tsa))
    b, sfb = orc.quantize_fp4(fb, dt, float(tsb))
    return dict(a=a, b=b, sfa=sfa, sfb=sfb, tensor_scale=(float(tsa), float(tsb)))


def expected_tile(orc, kind, ops, n_mma):
    """(expected tile, tolerance tile).  int8: exact int32, tolerance None."""
    if kind == N.MMA_I8:
        return orc.mma_tile_i8(ops["a"], ops["b"], n_mma), None
    if kind in SPARSE:
        p, s = orc.mma_tile_sp(kind, ops["a"], ops["meta"], ops["b"], ops["sfa"], ops["sfb"])
        if kind == N.MMA_I8_SP:
            return (p.astype(np.int64) * n_mma).astype(np.int32), None
    else:
        p, s = orc.mma_tile(kind, ops["a"], ops["b"], ops["sfa"], ops["sfb"])
    k = KIND_K[kind]
    if kind == N.MMA_F16_F16:
        # 16-bit accumulator: one rounding to half per instruction at least; the bound is relative to the
        # running magnitude n*S and only meant for a handful of instructions
        return p * n_mma, (n_mma + 1) * 2.0 ** -11 * n_mma * s + 1e-30
    # fp32 accumulation in the tensor core is not IEEE round-to-nearest: the
    # addends are aligned to the running sum and truncated, so the error is one-sided and grows
    # with the square of the instruction count.  Model: each of the n additions into the running
    # sum, and each of the K product additions inside one instruction, loses up to 1.5 units in
    # the last place of a 24-bit running magnitude (1.5 * 2^-23 relative); the running magnitude
    # is at most n*S with S = sum|a||b|.  Measured worst case on B200 at n = 2^14: 0.6 of this
    # bound (bf16/fp16; less for the 8- and 4-bit kinds), i.e. the constant carries a margin of
    # 40 % over what the hardware does and nothing more.  The small-n cases (1, 2, 3, 64) and the
    # exact power-of-two scaling test pin the low-order behaviour.
    rel = 1.5 * (n_mma + k) * 2.0 ** -23
    return p * n_mma, rel * n_mma * s + 1e-30


def run_peak(K, cuda, kind, ops, n_mma, grid, n_out_tiles):
    from tests.gpu_util import dev_empty, dev_from, stream_ptr, sync, to_np
    import ctypes as C
    d_a = dev_from(ops["a"].view(np.uint8))
    d_b = dev_from(ops["b"].view(np.uint8))
    d_sfa = dev_from(ops["sfa"]) if ops["sfa"] is not None else None
    d_sfb = dev_from(ops["sfb"]) if ops["sfb"] is not None else None
    d_meta = dev_from(ops["meta"]) if ops.get("meta") is not None else None
    d_out = dev_empty(max(n_out_tiles, 1) * 128 * 256, cuda.int32)
    d_chk = dev_empty(grid, cuda.int32)
    d_status = dev_empty(1, cuda.int32)
    args = N.MmaPeakArgs(kind=kind, d_a=d_a.data_ptr(), d_b=d_b.data_ptr(),
                         d_sfa=d_sfa.data_ptr() if d_sfa is not None else None,
                         d_sfb=d_sfb.data_ptr() if d_sfb is not None else None,
                         d_meta=d_meta.data_ptr() if d_meta is not None else None, n_mma=n_mma, grid=grid,
                         n_out_tiles=n_out_tiles,
                         d_out=d_out.data_ptr(), d_checksum=d_chk.data_ptr(), d_status=d_status.data_ptr())
    K.clpk_mma_peak(C.byref(args), stream_ptr())
    sync()
    status = int(to_np(d_status)[0])
    tiles = to_np(d_out).reshape(-1, 128, 256)[:n_out_tiles]
    return status, tiles, to_np(d_chk).view(np.uint32)


def check_tile(kind, got_i32, want, tol):
    if kind in (N.MMA_I8, N.MMA_I8_SP):
        assert np.array_equal(got_i32, want), f"int8 tile differs in {(got_i32 != want).sum()} elements"
        return 0.0
    if kind == N.MMA_F16_F16:
        assert not (got_i32.view(np.uint32) >> 16).any(), "fp16 accumulator words carry data in their high halves"
        got = (got_i32.view(np.uint32) & 0xFFFF).astype(np.uint16).view(np.float16).astype(np.float64)
    else:
        got = got_i32.view(np.float32).astype(np.float64)
    err = np.abs(got - want)
    worst = float((err / tol).max())
    assert worst <= 1.0, f"kind {kind}: error is {worst:.3g}x the stated tolerance"
    return worst
