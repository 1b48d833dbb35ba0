"""The allocation-free column sum (nrs_sum_axis0_static) against nrs_sum_axis0.

Some callers may not allocate device memory while they run (a stream capture in
progress, a real-time loop, a host framework that owns every byte of the GPU),
so this entry point keeps its split partial sums in a fixed array inside the
library.  It must give what the allocating entry point gives, call after call,
whatever the shared array held before.  Collected last on purpose: a failure
here cannot hide the result of any other test in a run that stops at the first
failure.
"""
import numpy as np
import pytest

from neuralrs_b200 import _lib
from .gpu_util import Dev, call

pytestmark = pytest.mark.gpu


def test_static_scratch_column_sum_matches_allocating_entry_point(gpu_ctx):
    rng = np.random.default_rng(2024)
    l = _lib.lib()
    # two calls in a row with different shapes: the second finds the first one's partials in the array
    for rows, cols in [(4096, 512), (3000, 1000), (70, 33), (1, 5)]:
        g = rng.normal(size=(rows, cols)).astype(np.float32)
        dg = Dev(gpu_ctx, g)
        ref, got = Dev(gpu_ctx, shape=(cols,)), Dev(gpu_ctx, shape=(cols,))
        call(gpu_ctx, "nrs_sum_axis0", dg, ref, rows, cols, 0)
        call(gpu_ctx, "nrs_sum_axis0_static", dg, got, rows, cols, 0)
        r = ref.get()
        assert np.abs(got.get() - r).max() <= 1e-5 * max(1.0, np.abs(r).max())
        assert np.abs(r - g.astype(np.float64).sum(0)).max() <= 1e-5 * max(1.0, np.abs(r).max())
        # accumulate mode, second call in a row on the same buffers
        call(gpu_ctx, "nrs_sum_axis0", dg, ref, rows, cols, 1)
        call(gpu_ctx, "nrs_sum_axis0_static", dg, got, rows, cols, 1)
        assert np.abs(got.get() - ref.get()).max() <= 2e-5 * max(1.0, np.abs(r).max())
    # beyond the built-in scratch the call is refused with a clear message, not attempted
    big = Dev(gpu_ctx, shape=(2, 8193))
    out = Dev(gpu_ctx, shape=(8193,))
    st = l.nrs_sum_axis0_static(gpu_ctx.h, big.ptr, out.ptr, 2, 8193, 0)
    assert st == 7
    assert b"exceed the built-in scratch" in l.nrs_last_error(gpu_ctx.h)
