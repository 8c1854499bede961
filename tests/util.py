"""Helpers for the GPU tests: device buffers through the library's own C-ABI helpers."""
import ctypes as C

import numpy as np


class Dev:
    """A device allocation made with bpdq_alloc, filled from / read into numpy."""

    def __init__(self, lib, src=None, nbytes=None, fill=None):
        self.lib = lib
        if src is not None:
            src = np.ascontiguousarray(src)
            nbytes = src.nbytes
        self.nbytes = int(nbytes)
        self.ptr = lib.bpdq_alloc(max(self.nbytes, 16))
        assert self.ptr, "device allocation failed"
        if src is not None and self.nbytes:
            lib.bpdq_h2d(self.ptr, src.ctypes.data, self.nbytes)
        elif fill is not None and self.nbytes:
            host = np.full(self.nbytes, fill, np.uint8)
            lib.bpdq_h2d(self.ptr, host.ctypes.data, self.nbytes)

    def read(self, dtype, count=None):
        dtype = np.dtype(dtype)
        n = self.nbytes // dtype.itemsize if count is None else count
        out = np.empty(n, dtype)
        if n:
            self.lib.bpdq_d2h(out.ctypes.data, self.ptr, n * dtype.itemsize)
        return out

    def free(self):
        if self.ptr:
            self.lib.bpdq_free(self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bits_equal(got, want):
    """0-ULP comparison for finite values; NaN must meet NaN (payload and sign free)."""
    got = np.asarray(got, np.float32)
    want = np.asarray(want, np.float32)
    assert got.shape == want.shape
    nan_g, nan_w = np.isnan(got), np.isnan(want)
    assert np.array_equal(nan_g, nan_w), "NaN positions differ"
    ok = bits(got) == bits(want)
    ok |= nan_g
    if not ok.all():
        idx = np.flatnonzero(~ok.ravel())[:5]
        raise AssertionError(f"{(~ok).sum()} of {ok.size} values differ; first at {idx}: "
                             f"got {got.ravel()[idx]} want {want.ravel()[idx]}")


def normwise(got, want):
    """max|got - want| / max|want| -- the norm-wise relative error used for fp32 sums."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-300))
