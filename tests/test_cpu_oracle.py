"""The CPU oracle against what the reference project pins for this path:
format constants, the fill it uses, the read-and-sum access order, the chain
shape, the Sattolo construction, pickIters -- and against independent
restatements in numpy / torch where the reference pins nothing."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

GOLD = Path(__file__).resolve().parent / "golden"


def test_format_constants_the_reference_hard_codes(orc):
    L = orc.lib()
    # src/cuda/cuda_blas.cpp:655-660: 0x7F = 1.0 in UE8M0, 0x38 = 1.0 in UE4M3
    assert L.orc_ue8m0_to_f32(0x7F) == 1.0
    assert L.orc_e4m3_to_f32(0x38) == 1.0
    assert L.orc_f32_to_e4m3(1.0) == 0x38
    # src/cuda/cuda_kernels/wmma_nvf4_e2m1.cu:30-33 feeds 0x3c scale bytes ("~1.0"): exactly 1.5
    assert L.orc_e4m3_to_f32(0x3C) == 1.5
    # wmma_mxf4_e2m1.cu:23-24 feeds 0x3f ue8m0 scale bytes: 2^(63-127)
    assert L.orc_ue8m0_to_f32(0x3F) == np.float32(2.0 ** -64)


def test_populate_matches_reference_xorshift(orc):
    # src/common/common.cpp:76-95 restated independently in Python
    st, want = 0xDEADBEEF, []
    for _ in range(64):
        st ^= (st << 13) & 0xFFFFFFFF
        st ^= st >> 17
        st ^= (st << 5) & 0xFFFFFFFF
        want.append((st & 0x7F7FFFFF) | 0x00800000)
    got = np.empty(64, dtype=np.float32)
    orc.lib().orc_populate_reference(orc.ptr(got), 64)
    assert got.view(np.uint32).tolist() == want
    assert np.all(np.isfinite(got))


@pytest.mark.parametrize("dtype,tdt,scale", [(1, torch.float16, 1e-3), (2, torch.bfloat16, 1.0),
                                             (3, torch.float8_e4m3fn, 50.0), (4, torch.float8_e5m2, 5e3)])
def test_codecs_agree_with_torch(orc, dtype, tdt, scale):
    x = (orc.fill_f32(1 << 16, 5, 2) * np.float32(scale)).astype(np.float32)
    x[:8] = [0.0, -0.0, 2 ** -9, 3 * 2 ** -11, 1.5, 2.5, -3.5, 6.0e-8]
    t = torch.from_numpy(x).to(tdt)
    view = torch.int16 if t.element_size() == 2 else torch.uint8
    want = t.view(view).numpy().view(np.uint16 if t.element_size() == 2 else np.uint8)
    assert np.array_equal(orc.convert_f32(x, dtype), want)
    # decode round trip
    L = orc.lib()
    dec = {1: L.orc_f16_to_f32, 2: L.orc_bf16_to_f32, 3: L.orc_e4m3_to_f32, 4: L.orc_e5m2_to_f32}[dtype]
    back = np.array([dec(int(v)) for v in want[:512]], dtype=np.float32)
    assert np.array_equal(back, t.to(torch.float32).numpy()[:512])


def test_e4m3_saturates_and_e2m1_ties_to_even(orc):
    L = orc.lib()
    assert L.orc_f32_to_e4m3(448.0) == 0x7E and L.orc_f32_to_e4m3(1e9) == 0x7E and L.orc_f32_to_e4m3(-1e9) == 0xFE
    assert L.orc_f32_to_e5m2(1e9) == 0x7B
    ties = {0.25: 0.0, 0.75: 1.0, 1.25: 1.0, 1.75: 2.0, 2.5: 2.0, 3.5: 4.0, 5.0: 4.0, 7.0: 6.0, -0.75: -1.0}
    for x, want in ties.items():
        assert L.orc_e2m1_to_f32(L.orc_f32_to_e2m1(x)) == want, x
    for v in (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0):
        assert L.orc_e2m1_to_f32(L.orc_f32_to_e2m1(v)) == v


def test_ue8m0_block_exponent_rule(orc):
    L = orc.lib()
    for amax, want_exp in ((6.0, 0), (5.9, 0), (4.0, 0), (3.9, -1), (1.0, -2), (12.0, 1), (0.3, -4)):
        assert L.orc_ue8m0_for_absmax(amax) == 127 + want_exp, amax
    assert L.orc_ue8m0_for_absmax(0.0) == 127


@pytest.mark.parametrize("dtype", [6, 7])
def test_fp4_quantiser_properties(orc, dtype):
    x = orc.fill_f32(64 * 128, 3, 2).reshape(64, 128)
    ts = float(np.abs(x).max() / (6 * 448)) if dtype == 7 else 1.0
    packed, scales = orc.quantize_fp4(x, dtype, ts)
    blk = 32 if dtype == 6 else 16
    assert packed.shape == (64, 64) and scales.shape == (64, 128 // blk)
    deq = np.array([[orc.lib().orc_fp4_element(orc.ptr(packed), orc.ptr(scales), 128, dtype, r, c) for c in range(128)]
                    for r in range(8)]) * ts
    # per-block relative error of a 4-bit format with a shared scale: a few tens of percent at worst, and
    # the block maximum is reproduced within one e2m1 step
    err = np.abs(deq - x[:8])
    amax = np.abs(x[:8]).reshape(8, -1, blk).max(axis=2).repeat(blk, axis=1)
    assert np.all(err <= 0.30 * amax + 1e-6)
    assert np.corrcoef(deq.ravel(), x[:8].ravel())[0, 1] > 0.98


def test_prune_2to4(orc):
    x = orc.fill_f32(16 * 64, 9, 2).reshape(16, 64)
    x[0, :4] = [1.0, -1.0, 1.0, 0.5]               # ties: the lower indices win
    comp = np.zeros((16, 32), dtype=np.float32)
    meta = np.zeros((16, 8), dtype=np.uint8)
    pruned = np.zeros_like(x)
    orc.lib().orc_prune_2to4(orc.ptr(comp), orc.ptr(meta), orc.ptr(pruned), orc.ptr(x), 16, 64)
    assert (meta[0, 0] & 0xF) == (0 | (1 << 2))
    g = pruned.reshape(16, 16, 4)
    assert np.all((g != 0).sum(axis=2) <= 2)
    # the kept values are the two largest magnitudes of every group
    kept = np.sort(np.abs(g), axis=2)[:, :, 2:]
    best = np.sort(np.abs(x.reshape(16, 16, 4)), axis=2)[:, :, 2:]
    assert np.array_equal(kept, best)
    # compressed + metadata decode back to the pruned dense tile exactly
    rebuilt = np.zeros_like(x)
    for r in range(16):
        for gi in range(16):
            nib = (meta[r, gi // 2] >> (4 * (gi & 1))) & 0xF
            rebuilt[r, gi * 4 + (nib & 3)] = comp[r, gi * 2]
            rebuilt[r, gi * 4 + (nib >> 2)] = comp[r, gi * 2 + 1]
    assert np.array_equal(rebuilt, pruned)


@pytest.mark.parametrize("width", [1, 2, 4])
def test_global_bandwidth_follows_the_reference_thread_order(orc, width):
    # global_bandwidth.cu:14-71 restated with numpy: element offset = block*256*16 + lid + i*256
    blocks = 3
    n = 256 * 16 * width * blocks
    src = orc.fill_f32(n, 1, 0)
    elems = src.reshape(-1, width)
    out = np.zeros(blocks * 256, dtype=np.float32)
    for b in range(blocks):
        for lid in range(256):
            acc = np.zeros(width, dtype=np.float32)
            for i in range(16):
                acc = (acc + elems[b * 256 * 16 + lid + i * 256]).astype(np.float32)
            r = acc[0]
            for l in range(1, width):
                r = np.float32(r + acc[l])
            out[b * 256 + lid] = r
    assert np.array_equal(orc.global_bandwidth(width, src).view(np.uint32), out.view(np.uint32))


def test_triad_is_two_roundings(orc):
    b, c = orc.fill_f32(4096, 23, 0), orc.fill_f32(4096, 24, 0)
    want = (b + (np.float32(1.5) * c).astype(np.float32)).astype(np.float32)
    assert np.array_equal(orc.triad(b, c, 1.5).view(np.uint32), want.view(np.uint32))
    fused = np.array([np.float32(float(bb) + 1.5 * float(cc)) for bb, cc in zip(b, c)], dtype=np.float32)
    assert np.any(fused.view(np.uint32) != want.view(np.uint32))        # an FMA would differ somewhere


def test_compute_sp_chain_shape(orc):
    # compute_sp.cu:12-24: 128 x 16 dependent FMAs of x = x*x + c with c = thread index in the block
    got = orc.compute_sp(0.5, 512)
    import math
    for lane in (0, 1, 255, 256, 300):
        x, c = np.float32(0.5), np.float32(lane % 256)
        for _ in range(2048):
            x = np.float32(math.fma(float(x), float(x), float(c))) if hasattr(math, "fma") else np.float32(np.float64(x) * np.float64(x) + np.float64(c))
            if not np.isfinite(x):
                break
        assert (np.isinf(got[lane]) and np.isinf(x)) or got[lane] == x
    assert got[256] == got[0] or (np.isnan(got[256]) and np.isnan(got[0]))


def test_mad_chain_overflows_as_documented(orc):
    out64 = orc.mad_chain(256, 0, 0.999, 64)
    out4096 = orc.mad_chain(256, 0, 0.999, 4096)
    assert np.all(np.isfinite(out64))
    assert not np.any(np.isfinite(out4096))       # x doubles per step: only infinities and NaNs are left


@pytest.mark.parametrize("n", [2, 3, 64, 1 << 16])
def test_sattolo_cycle_is_one_cycle(orc, n):
    nxt = orc.chase_cycle(n, 9)
    assert sorted(nxt.tolist()) == list(range(n))          # a permutation
    assert np.all(nxt != np.arange(n))                      # no fixed points
    assert orc.lib().orc_is_single_cycle(orc.ptr(nxt), n) == 1
    fin, _ = orc.chase(nxt, 0, n)
    assert fin == 0                                         # n hops return to the start


def test_pick_iters_matches_reference_contract(orc):
    f = orc.lib().orc_pick_iters
    assert f(50.0, 500000, 0, 10000) == 10000
    assert f(1000.0, 500000, 0, 10000) == 500
    assert f(1e9, 500000, 0, 10000) == 1
    assert f(0.1, 500000, 0, 10000) == 10000               # per-iter clamped to 1 us
    assert f(1000.0, 0, 0, 10000) == 5000                   # zero budget -> 5 s
    assert f(1000.0, 500000, 7, 10000) == 7


def test_generator_golden_vectors(orc):
    gold = json.loads((GOLD / "generator_vectors.json").read_text())
    for case in gold["cases"]:
        got = orc.fill_f32(case["n"], case["seed"], case["dist"], case["mean"], case["std"], first=case["first"])
        assert got.view(np.uint32).tolist() == case["bits"], case
    assert orc.fill_i8(32, 2).tolist() == gold["i8_seed2"]
    assert orc.chase_cycle(16, 9).tolist() == gold["cycle16_seed9"]


def test_generator_distributions(orc):
    u = orc.fill_f32(1 << 20, 1, 0)
    assert 0.0 <= u.min() and u.max() < 1.0 and abs(u.mean() - 0.5) < 2e-3
    s = orc.fill_f32(1 << 20, 2, 1)
    assert -1.0 <= s.min() and s.max() < 1.0 and abs(s.mean()) < 4e-3
    g = orc.fill_f32(1 << 20, 3, 2)
    assert abs(g.mean()) < 5e-3 and abs(g.std() - 1.0) < 5e-3
    from scipy import stats
    assert stats.kstest(g[:200000].astype(np.float64), "norm").statistic < 0.01


def test_mma_tile_oracle_against_numpy(orc):
    from tests import mma_util as M
    from clpeak_b200 import native as N
    ops = M.make_operands(orc, N.MMA_BF16)
    p, s = orc.mma_tile(N.MMA_BF16, ops["a"], ops["b"])
    a = (ops["a"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    b = (ops["b"].astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    assert np.allclose(p, a @ b.T, rtol=0, atol=1e-12)
    assert np.allclose(s, np.abs(a) @ np.abs(b).T, rtol=0, atol=1e-12)
    i8 = M.make_operands(orc, N.MMA_I8)
    want = (i8["a"].astype(np.int64) @ i8["b"].astype(np.int64).T) * 5
    assert np.array_equal(orc.mma_tile_i8(i8["a"], i8["b"], 5), want.astype(np.int32))


# ---- typed chains, shared-memory rotation, texture read -------------------------------------

def test_int32_chain_against_python_integers(orc):
    got = orc.compute_chain(5, 3, 256)
    for tid in (0, 1, 2, 97, 255):
        x = 3
        for _ in range(2048):
            x = (x * x + tid) & 0xFFFFFFFF
        assert int(got[tid]) & 0xFFFFFFFF == x


def _dp4a(x, y, a):
    s = a
    for b in range(4):
        xb = (x >> (8 * b)) & 0xFF
        yb = (y >> (8 * b)) & 0xFF
        s += (xb - 256 if xb > 127 else xb) * (yb - 256 if yb > 127 else yb)
    s &= 0xFFFFFFFF
    return s - (1 << 32) if s >= (1 << 31) else s


@pytest.mark.parametrize("row", [0, 1, 2, 3])
def test_int8_dot_chains_against_python_integers(orc, row):
    offsets = [[0], [0, 7], [0, 7, 13, 19], [0, 11, 17, 23, 29, 31, 37, 41]][row]
    chains = 1 << row
    got = orc.compute_chain(6 + row, 4, 256)
    x = 4 | (5 << 8) | (6 << 16) | (7 << 24)          # the reference packs A, A+1, A+2, A+3 with A = 4
    for tid in (0, 3, 200, 255):
        y = [(tid + j) & 0xFFFFFFFF for j in range(chains)]
        acc = [tid + offsets[j] for j in range(chains)]
        for _ in range(64 // chains):
            for j in range(chains):
                for _ in range(16):
                    acc[j] = _dp4a(x, y[j], acc[j])
                    y[j] ^= acc[j] & 0xFFFFFFFF
        total = sum(a & 0xFFFFFFFF for a in acc) & 0xFFFFFFFF
        assert int(got[tid]) & 0xFFFFFFFF == total


def test_floating_chains_run_away_like_the_reference(orc):
    # x = x*x + c from 1.3 overflows every format within a few steps: the stored value is +inf
    for chain in (0, 1, 2, 3, 4):
        out = orc.compute_chain(chain, 1.3, 256)
        assert np.all(np.isinf(out)) and np.all(out > 0)


def test_half_chain_small_start_against_numpy_float16(orc):
    # thread 0 (c = 0) from 0.5: repeated squaring in half, underflows to zero; thread 1 runs away
    got = orc.compute_chain(1, 0.5, 2)
    x = np.float16(0.5)
    for _ in range(1024):
        x = np.float16(np.float64(x) * np.float64(x))
    assert got[0] == np.float32(x) + np.float32(x) == 0.0
    assert np.isinf(got[1])
    # mixed chain, thread 0, a few exact steps: 0.5 -> 2^-2 -> ... stays a power of two until it underflows
    assert orc.compute_chain(3, 0.5, 1)[0] == 0.0


def test_local_bandwidth_closed_form(orc):
    out = orc.local_bandwidth(4, 512)
    assert out[0] == 64 + 65 + 66 + 67 and out[200] == sum(range(8, 12)) and out[256] == sum(range(320, 324))
    assert orc.local_bandwidth(1, 256)[255] == 63.0


def test_image_bandwidth_reads_every_texel_once(orc):
    threads, texels, seed = 64, 1024, 9
    out = orc.image_bandwidth(threads, texels, seed)
    vals = orc.fill_f32(4 * texels, seed, 0)
    assert abs(float(out.astype(np.float64).sum()) - float(vals.astype(np.float64).sum())) < 1e-2
    # thread 5: texels 5, 69, 133, ...; channel-wise sums in order
    s = np.zeros(4, dtype=np.float32)
    for i in range(16):
        px = (5 + i * threads) % texels
        s = (s + vals[4 * px:4 * px + 4]).astype(np.float32)
    assert out[5] == np.float32(np.float32(np.float32(s[0] + s[1]) + s[2]) + s[3])
    assert np.array_equal(orc.image_bandwidth(threads, texels, seed, first=10, count=7), out[10:17])
