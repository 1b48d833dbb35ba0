"""Helpers for the GPU parity tests: device buffers through the C ABI itself."""
import ctypes as C

import numpy as np

from neuralrs_b200 import _lib


class Dev:
    """A device buffer allocated with nrs_alloc and filled from a numpy array."""

    def __init__(self, ctx, arr=None, *, shape=None, dtype=np.float32, zero=False):
        self.ctx = ctx
        self.l = _lib.lib()
        if arr is not None:
            arr = np.ascontiguousarray(arr)
            shape, dtype = arr.shape, arr.dtype
        self.shape, self.dtype = tuple(shape), np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        _lib.check(ctx.h, self.l.nrs_alloc(ctx.h, max(self.nbytes, 1), int(zero), C.byref(p)))
        self.ptr = p
        if arr is not None and self.nbytes:
            _lib.check(ctx.h, self.l.nrs_h2d(ctx.h, self.ptr, C.c_void_p(arr.ctypes.data), self.nbytes))
            ctx.sync()

    def get(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        if self.nbytes:
            _lib.check(self.ctx.h, self.l.nrs_d2h(self.ctx.h, C.c_void_p(out.ctypes.data), self.ptr, self.nbytes))
        return out

    def free(self):
        if self.ptr:
            self.l.nrs_free(self.ctx.h, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


def call(ctx, name, *args):
    l = _lib.lib()
    conv = [a.ptr if isinstance(a, Dev) else a for a in args]
    _lib.check(ctx.h, getattr(l, name)(ctx.h, *conv))
