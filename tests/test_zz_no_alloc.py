"""The allocation-free row-sum entry point (nt_sum_rows_noalloc) against the regular nt_sum.

Some users of the library own every byte of device memory themselves (a runtime with its own arena, a
loop that cannot afford cudaMalloc's device-wide synchronisation); for them one entry point keeps its
cross-CTA scratch in a fixed array inside the library.  Collected last on purpose (file name): the
scratch is shared state, so it runs after everything else and is also run on its own in a fresh
process.  Two calls in a row must both be right: the second finds the first one's leftovers.
"""

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _check(nt, n_rows, row_len, seed):
    _C = nt._C
    x = np.random.default_rng(seed).standard_normal((n_rows, row_len)).astype(np.float32)
    t = nt.Tensor.from_numpy(x, "cuda")
    want = nt.Tensor._new_contiguous(_C.sum(t._C_view, [1], nt.float32), (n_rows,)).numpy()
    out = _C.Storage.allocate(n_rows, nt.float32, nt.Device.Cuda)  # the caller's buffer
    # neither a cudaMalloc nor a block of the library's caching arena (a request served from its cache
    # would leave the cudaMalloc count alone: the arena's own request counter is what shows it)
    mallocs, requests = _C.allocator_stats()["n_cuda_malloc"], _C.allocator_requests()
    _C.sum_rows_noalloc(t.storage, n_rows, row_len, out)
    assert _C.allocator_stats()["n_cuda_malloc"] == mallocs and _C.allocator_requests() == requests
    got = nt.Tensor._new_contiguous(out, (n_rows,)).numpy()
    scale = np.abs(x).astype(np.float64).sum(axis=1)
    assert (np.abs(got.astype(np.float64) - want) <= 1e-5 * scale).all(), "differs from nt_sum"
    assert (np.abs(got - x.astype(np.float64).sum(axis=1)) <= 1e-6 * scale).all(), "differs from the fp64 sum"
    return got, want


def test_two_calls_in_a_row_match_the_allocating_entry_point(nt):
    # rows long enough to be split over several CTAs, so the shared scratch (partials + tickets) is used
    a, wa = _check(nt, 8, 1 << 20, 1)
    b, wb = _check(nt, 8, 1 << 20, 2)          # second call: finds the first call's partial sums
    assert not np.array_equal(a, b)
    c, wc = _check(nt, 3, 3_000_001, 3)        # other shape, ragged length, fewer rows than before
    d, _ = _check(nt, 1, 1 << 24, 4)           # a full reduction: 1024 partials, one ticket
    # same split rule in both entry points => same order of additions
    assert np.array_equal(a, wa) and np.array_equal(b, wb) and np.array_equal(c, wc)


def test_short_rows_and_limits(nt):
    _C = nt._C
    _check(nt, 5000, 100, 5)                   # short rows: one warp per row, no scratch at all
    _check(nt, 4096, 8192, 6)                  # one CTA per row, no split
    _check(nt, 256, 40000, 7)                  # the largest row count that may still be split
    big = _C.Storage.allocate(300 * 40000, nt.float32, nt.Device.Cuda)
    out = _C.Storage.allocate(300, nt.float32, nt.Device.Cuda)
    with pytest.raises(ValueError, match="fixed scratch"):
        _C.sum_rows_noalloc(big, 300, 40000, out)    # 300 long rows would be split: more tickets than the array holds
    with pytest.raises(ValueError):
        _C.sum_rows_noalloc(big, 8, 0, out)
