"""Small helpers shared by the GPU parity tests (torch is used only to hold
device buffers and to move them to numpy)."""
import ctypes as C

import numpy as np
import torch


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def dev_empty(n, dtype):
    return torch.empty(n, dtype=dtype, device="cuda")


def dev_from(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def to_np(t: torch.Tensor) -> np.ndarray:
    return t.detach().cpu().numpy()


def sync():
    torch.cuda.synchronize()


def u32_view(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a).view(np.uint32)


def assert_bits_equal(got: np.ndarray, want: np.ndarray, what: str):
    g = np.ascontiguousarray(got).view(np.uint8)
    w = np.ascontiguousarray(want).view(np.uint8)
    assert g.shape == w.shape, f"{what}: shape {g.shape} vs {w.shape}"
    if not np.array_equal(g, w):
        bad = np.flatnonzero(g != w)
        raise AssertionError(f"{what}: {bad.size} differing bytes, first at byte {bad[0]}")


def assert_floats_equal_nan_aware(got: np.ndarray, want: np.ndarray, what: str):
    """Bit-exact, except that any NaN matches any NaN: the payload and sign of a
    generated NaN (inf - inf) differ between x86 and the GPU."""
    g = np.ascontiguousarray(got, dtype=np.float32)
    w = np.ascontiguousarray(want, dtype=np.float32)
    assert g.shape == w.shape
    both_nan = np.isnan(g) & np.isnan(w)
    same = (g.view(np.uint32) == w.view(np.uint32)) | both_nan
    if not same.all():
        bad = np.flatnonzero(~same)
        raise AssertionError(f"{what}: {bad.size} differing values, first at {bad[0]}: {g[bad[0]]!r} vs {w[bad[0]]!r}")
