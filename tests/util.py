"""Comparators used by the parity tests."""

import numpy as np


def bits(a: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def assert_bit_exact(got: np.ndarray, want: np.ndarray, what: str = ""):
    """uint32 view equality; NaNs compare equal to NaNs whatever their payload."""
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    same = (bits(got) == bits(want)) | (np.isnan(got) & np.isnan(want))
    if not same.all():
        bad = np.argwhere(~same)
        i = tuple(bad[0])
        raise AssertionError(f"{what}: {len(bad)} of {got.size} elements differ bitwise; first at {i}: "
                             f"got {got[i]!r} want {want[i]!r}")


def ulp_distance(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in units in the last place between float32 arrays (monotone integer mapping)."""
    def key(x):
        i = np.ascontiguousarray(x, dtype=np.float32).view(np.int32).astype(np.int64)
        return np.where(i < 0, -(i & 0x7FFFFFFF), i)
    d = np.abs(key(a) - key(b))
    both_nan = np.isnan(a) & np.isnan(b)
    return np.where(both_nan, 0, d)


def assert_ulp(got: np.ndarray, want: np.ndarray, max_ulp: int, what: str = ""):
    got = np.asarray(got, dtype=np.float32)
    want = np.asarray(want, dtype=np.float32)
    assert got.shape == want.shape, f"{what}: shape {got.shape} != {want.shape}"
    assert not (np.isnan(got) ^ np.isnan(want)).any(), f"{what}: NaN pattern differs"
    d = ulp_distance(got, want)
    worst = int(d.max()) if d.size else 0
    if worst > max_ulp:
        i = np.unravel_index(int(d.argmax()), d.shape)
        raise AssertionError(f"{what}: max ulp distance {worst} > {max_ulp} at {i}: got {got[i]!r} want {want[i]!r} "
                             f"({int((d > max_ulp).sum())} elements over)")
    return worst


def assert_scaled(got: np.ndarray, want: np.ndarray, scale: np.ndarray, rel: float, what: str = ""):
    """|got - want| <= rel * scale elementwise (norm-wise criterion: `scale` is sum|x| of the reduced
    slice for sums, (|A||B|)_ij for matmul, the largest intermediate for a fused backward chain)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    err = np.abs(got - want)
    bound = rel * np.asarray(scale, dtype=np.float64)
    over = err > bound
    if over.any():
        i = np.unravel_index(int((err - bound).argmax()), err.shape)
        raise AssertionError(f"{what}: |diff| {err[i]:.3e} > {rel:g} * scale {np.broadcast_to(scale, err.shape)[i]:.3e} "
                             f"at {i} ({int(over.sum())} elements over)")
    return float((err / np.maximum(np.asarray(scale, dtype=np.float64), 1e-300)).max()) if err.size else 0.0


# ---------------------------------------------------------------------------------------------
# Index-array / mask indexing cases shared by tests/golden/make_golden.py (which records what the
# reference returns for them) and the parity tests.  Each entry is the source of an index tuple for
# a tensor of shape INDEX_SHAPE; evaluate with index_case().
INDEX_SHAPE = (5, 6, 7)
INDEX_GET_CASES = [
    "([4, 0, -1],)",
    "(slice(None), [0, 2, 5])",
    "(slice(None), slice(None), [[0, 1], [6, -2]])",
    "([0, 1], slice(None), [2, 3])",                 # separated index dims: index shape moves to the front
    "([0, 1], [2, 3])",
    "([0, 1], [1, 2], [2, 3])",
    "(slice(1, 4), [0, 2], slice(None, None, 2))",
    "([True, False, True, False, True],)",
    "(slice(None), [False, True, True, False, False, True])",
    "(slice(None), [1, 1, 1])",
    "(2, [0, 5])",
    "(0, slice(None), [1, 2])",                      # the int is consumed first: result (6, 2), unlike numpy
    "(None, [1, 2])",
    "([[0], [1]], [[1, 2, 3]])",                     # broadcast index arrays
    "(Ellipsis, [0, 3])",
    "([1, 3], Ellipsis)",
    "(slice(None, None, -1), [5, 0])",               # negative-stride view under the index array
]
# setitem: cases whose basic selectors are full slices (where the reference writes to the right place)
INDEX_SET_CASES = [
    ("([4, 0, -1],)", "full"),
    ("(slice(None), [0, 2, 5])", "full"),
    ("(slice(None), slice(None), [[0, 1], [6, -2]])", "full"),
    ("([0, 1], slice(None), [2, 3])", "full"),
    ("([0, 1], [2, 3])", "row"),
    ("([True, False, True, False, True],)", "scalar"),
    ("(slice(None), [1, 1, 1])", "full"),            # colliding destinations: the last writer wins
    ("([[0], [1]], [[1, 2, 3]])", "row"),
    ("([3, 3, 0, 3],)", "full"),
]


def index_case(source: str):
    return eval(source, {"__builtins__": {}}, {"slice": slice, "Ellipsis": Ellipsis, "None": None,
                                               "True": True, "False": False})


def index_value(kind: str, shape, rng):
    """The right-hand side of a setitem case: a full-shape array, a broadcast row, or a scalar."""
    if kind == "full":
        return rng.standard_normal(shape).astype(np.float32)
    if kind == "row":
        return rng.standard_normal(shape[-1:]).astype(np.float32)
    return np.float32(rng.standard_normal())
