"""GPU parity of the reductions and of matmul (through the C ABI).

sum/mean: |got - ref| <= 1e-5 * sum|x_i| over the reduced slice (norm-wise form of "rel 1e-5": the
reference's own sequential fp32 sum is 7e-5 away from the exact sum on the 8192^2 case, so an
elementwise-relative 1e-5 against it is not attainable by any accurate parallel sum).
max/min: bit-exact.  matmul: mode 2 bit-exact against the CPU oracle; modes 0 and 1 within
|C - C_ref|_ij <= 1e-4 * (|A||B|)_ij.
"""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import assert_bit_exact, assert_scaled

pytestmark = pytest.mark.gpu


def dev(nt, a, requires_grad=False):
    return nt.Tensor.from_numpy(a, "cuda", requires_grad=requires_grad)


AXES = [(0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2), None]


@pytest.mark.parametrize("axes", AXES)
@pytest.mark.parametrize("name", ["sum", "mean", "max", "min"])
def test_reductions_golden(nt, golden, name, axes):
    x = golden["red/in/x"]
    key = f"red/{name}/{'all' if axes is None else ''.join(map(str, axes))}"
    for keepdim in (False, True):
        t = dev(nt, x, True)
        res = getattr(t, name)(axes, keepdim)
        want = golden[f"{key}/{int(keepdim)}/out"]
        assert res.shape == want.shape
        if name in ("max", "min"):
            assert_bit_exact(res.numpy(), want, name)
        else:
            ax = tuple(range(3)) if axes is None else axes
            scale = np.abs(x).sum(axis=ax, keepdims=keepdim) / (1 if name == "sum" else x.size // want.size)
            assert_scaled(res.numpy(), want, scale, 1e-5, name)
        res.sum().backward()
        assert_bit_exact(t.grad.numpy(), golden[f"{key}/{int(keepdim)}/gx"], f"{name} backward")


def test_reduction_ties_views_and_last_dim(nt, golden):
    tie = golden["red/tie/in"]
    t = dev(nt, tie, True)
    t.max((1,)).sum().backward()
    assert_bit_exact(t.grad.numpy(), golden["red/tie/max_gx"], "tied max: zero gradient on the tied slice")
    t = dev(nt, tie, True)
    t.min((0,)).sum().backward()
    assert_bit_exact(t.grad.numpy(), golden["red/tie/min_gx"], "tied min")
    x = golden["red/in/x"]
    got = dev(nt, x).transpose(0, 2).sum((0,)).numpy()
    assert_scaled(got, golden["red/sum_transposed/out"], np.abs(x).sum(axis=2).T, 1e-5, "transposed view")
    y = golden["red/in/y"]
    for name in ("sum", "mean", "max", "min"):
        t = dev(nt, y, True)
        res = getattr(t, name)(-1)
        want = golden[f"red/y/{name}/out"]
        if name in ("max", "min"):
            assert_bit_exact(res.numpy(), want, name)
        else:
            assert_scaled(res.numpy(), want, np.abs(y).sum(-1) / (1 if name == "sum" else 40), 1e-5, name)
        res.sum().backward()
        assert_bit_exact(t.grad.numpy(), golden[f"red/y/{name}/gx"], f"{name} backward")


SHAPES = [((1000, 1003), [1]), ((1000, 1003), [0]), ((1000, 1003), [0, 1]), ((37, 5, 64), [2]), ((37, 5, 64), [0]),
          ((37, 5, 64), [1]), ((37, 5, 64), [0, 2]), ((3, 70000), [1]), ((70000, 3), [0]), ((64, 1, 16384), [2]),
          ((2, 3, 4, 5, 6), [1, 3]), ((1,), [0]), ((5, 1), [1])]


@pytest.mark.parametrize("shape,axes", SHAPES)
def test_reductions_vs_oracle(nt, port, shape, axes):
    rng = np.random.default_rng(abs(hash((shape, tuple(axes)))) % (2 ** 32))
    x = rng.standard_normal(shape).astype(np.float32)
    t = dev(nt, x)
    for name in ("max", "min"):
        assert_bit_exact(getattr(t, name)(tuple(axes)).numpy(), port.reduce(name, x, axes), f"{name} {shape} {axes}")
    got = t.sum(tuple(axes)).numpy()
    exact = x.astype(np.float64).sum(axis=tuple(axes))
    scale = np.abs(x).astype(np.float64).sum(axis=tuple(axes))
    assert_scaled(got, port.reduce("sum", x, axes), scale, 1e-5, f"sum vs oracle {shape} {axes}")
    assert_scaled(got, exact, scale, 1e-6, f"sum vs fp64 {shape} {axes}")
    # strided input views: sliced with a step, reversed, offset
    if len(shape) == 2 and shape[0] > 8:
        xv = x[::-2, 3:]
        tv = t[::-2, 3:]
        for name in ("max", "min"):
            assert_bit_exact(getattr(tv, name)(tuple(axes)).numpy(), port.reduce(name, xv, axes), f"{name} view")
        assert_scaled(tv.sum(tuple(axes)).numpy(), xv.astype(np.float64).sum(axis=tuple(axes)),
                      np.abs(xv).astype(np.float64).sum(axis=tuple(axes)), 1e-6, "sum view")


def test_argmax_argmin(nt, port):
    rng = np.random.default_rng(3)
    x = rng.integers(-5, 5, (40, 300)).astype(np.float32)  # many ties: the lowest index wins
    t = dev(nt, x)
    for name in ("argmax", "argmin"):
        for axes in ([0], [1], [0, 1]):
            storage = getattr(nt._C, name)(t._C_view, axes)
            got = nt.Tensor._new_contiguous(storage, tuple(s for i, s in enumerate(x.shape) if i not in axes)).numpy()
            assert np.array_equal(got, port.reduce(name, x, axes)), (name, axes)


@pytest.fixture(scope="module")
def big(nt):
    x = np.random.default_rng(20).standard_normal((8192, 8192)).astype(np.float32)
    return x, dev(nt, x)


@pytest.mark.parametrize("axes", [(0,), (1,), None])
def test_reductions_full_size(nt, port, big, axes):
    """[8192, 8192] along dim 0, dim 1 and over the full tensor."""
    x, t = big
    ax = (0, 1) if axes is None else axes
    # seeded input has no tied extrema per slice (the backward's tie quirk is not exercised here)
    mx = x.max(axis=ax, keepdims=True)
    assert ((x == mx).sum(axis=ax) == 1).all()
    scale = np.abs(x).astype(np.float64).sum(axis=ax)
    exact = x.astype(np.float64).sum(axis=ax)
    got = t.sum(axes).numpy()
    err_exact = assert_scaled(got, exact, scale, 1e-6, "sum vs fp64")
    assert_scaled(got, port.reduce("sum", x, list(ax)), scale, 1e-5, "sum vs the reference's sequential fp32 sum")
    print(f"sum axes={axes}: max |err| / sum|x| vs fp64 = {err_exact:.2e}")
    count = x.size // max(got.size, 1)
    assert_scaled(t.mean(axes).numpy(), exact / count, scale / count, 1e-6, "mean")
    assert_bit_exact(t.max(axes).numpy(), x.max(axis=ax), "max")
    assert_bit_exact(t.min(axes).numpy(), x.min(axis=ax), "min")
    # backward: gradient broadcast of ones
    tg = nt.Tensor.from_numpy(x, "cuda", requires_grad=True)
    tg.max(axes).sum().backward()
    assert_bit_exact(tg.grad.numpy(), (x == mx).astype(np.float32), "max backward")
    tg = nt.Tensor.from_numpy(x, "cuda", requires_grad=True)
    tg.mean(axes).sum().backward()
    assert_bit_exact(tg.grad.numpy(), np.full(x.shape, np.float32(1.0) / np.float32(count), np.float32), "mean backward")
    tg = nt.Tensor.from_numpy(x, "cuda", requires_grad=True)
    tg.sum(axes).sum().backward()
    g = tg.grad
    # the gradient of a sum is a stride-0 view over at most one row/column of storage: no N-sized write
    assert g.shape == x.shape and g.storage.size <= max(x.shape) and 0 in g.strides[0]


# ---------------------------------------------------------------------------------------------
MM_CASES = ["2d", "batched", "bcast_batch", "vec_mat", "mat_vec", "vec_vec", "odd"]


@pytest.mark.parametrize("mode", [2, 0, 1, 3])
@pytest.mark.parametrize("case", MM_CASES)
def test_matmul_golden(nt, golden, case, mode):
    nt._C.set_matmul_mode(mode)
    try:
        a, b, g = golden[f"mm/{case}/a"], golden[f"mm/{case}/b"], golden[f"mm/{case}/g"]
        ta, tb = dev(nt, a, True), dev(nt, b, True)
        res = ta @ tb
        (res * dev(nt, g)).sum().backward()
        # shapes included: a 1-D right operand gets its gradient back as (k, 1), as in the reference
        # (autograd/ops_binary.py:253-267)
        assert tb.grad.shape == golden[f"mm/{case}/gb"].shape
        checks = [(res.numpy(), golden[f"mm/{case}/out"]), (ta.grad.numpy(), golden[f"mm/{case}/ga"]),
                  (tb.grad.numpy(), golden[f"mm/{case}/gb"])]
        for got, want in checks:
            if mode == 2 and case != "bcast_batch":
                assert_bit_exact(got, want, case)  # bcast_batch sums the batch gradient in another order
            else:
                assert_scaled(got, want, np.abs(want).max() * 8 + 1e-6, 1e-4, case)
    finally:
        nt._C.set_matmul_mode(1)


def _mm_views(rng, M, K, N):
    a = rng.uniform(-1, 1, (M, K)).astype(np.float32)
    b = rng.uniform(-1, 1, (K, N)).astype(np.float32)
    at = np.ascontiguousarray(a.T)
    bt = np.ascontiguousarray(b.T)
    return [("nn", a, b, lambda t: t, lambda t: t), ("tn", at, b, lambda t: t.T, lambda t: t),
            ("nt", a, bt, lambda t: t, lambda t: t.T), ("tt", at, bt, lambda t: t.T, lambda t: t.T)]


@pytest.mark.parametrize("dims", [(256, 300, 200), (129, 64, 257), (64, 1000, 10), (10, 7, 3), (512, 512, 512)])
def test_matmul_layouts_vs_oracle(nt, port, dims):
    M, K, N = dims
    rng = np.random.default_rng(M * 31 + K * 17 + N)
    for lname, ha, hb, va, vb in _mm_views(rng, M, K, N):
        want = port.matmul(va(ha), vb(hb))
        bound = np.abs(va(ha)).astype(np.float64) @ np.abs(vb(hb)).astype(np.float64)
        for mode in (2, 0, 1, 3):
            nt._C.set_matmul_mode(mode)
            try:
                got = (va(dev(nt, ha)) @ vb(dev(nt, hb))).numpy()
            finally:
                nt._C.set_matmul_mode(1)
            if mode == 2:
                assert_bit_exact(got, want, f"{lname} {dims} mode 2")
            else:
                assert_scaled(got, want, bound, 1e-4, f"{lname} {dims} mode {mode}")
                # and well inside fp32 accuracy against the exact product
                exact = va(ha).astype(np.float64) @ vb(hb).astype(np.float64)
                assert_scaled(got, exact, bound, 2e-6, f"{lname} {dims} mode {mode} vs fp64")


def test_matmul_batched_and_sliced(nt, port):
    rng = np.random.default_rng(9)
    A = rng.uniform(-1, 1, (4, 3, 64, 48)).astype(np.float32)
    B = rng.uniform(-1, 1, (4, 3, 48, 80)).astype(np.float32)
    for mode in (2, 0, 1):
        nt._C.set_matmul_mode(mode)
        try:
            got = (dev(nt, A) @ dev(nt, B)).numpy()
            got_b = (dev(nt, A[0, 0]).expand(4, 3, 64, 48) @ dev(nt, B)).numpy()
            got_s = (dev(nt, A)[:, :, 3:40, 5:37] @ dev(nt, B)[:, :, 8:40, ::2]).numpy()
        finally:
            nt._C.set_matmul_mode(1)
        want = port.matmul(A, B)
        want_b = port.matmul(np.broadcast_to(A[0, 0], A.shape), B)
        want_s = port.matmul(A[:, :, 3:40, 5:37], B[:, :, 8:40, ::2])
        for g, w in ((got, want), (got_b, want_b), (got_s, want_s)):
            if mode == 2:
                assert_bit_exact(g, w, "batched")
            else:
                assert_scaled(g, w, 48.0, 1e-4, "batched")


@pytest.mark.parametrize("shape", [(4096, 4096, 4096), (8192, 1024, 4096)])
def test_matmul_full_size(nt, shape):
    """Forward and both gradients at the benchmark shapes; checked on sampled rows against fp64."""
    M, K, N = shape
    A = np.random.default_rng(30).uniform(-1, 1, (M, K)).astype(np.float32)
    B = np.random.default_rng(31).uniform(-1, 1, (K, N)).astype(np.float32)
    G = np.random.default_rng(32).uniform(-1, 1, (M, N)).astype(np.float32)
    rows = np.random.default_rng(33).choice(M, 48, replace=False)
    cols = np.random.default_rng(34).choice(N, 48, replace=False)
    krows = np.random.default_rng(35).choice(K, 48, replace=False)
    for mode in (1, 3, 0):
        nt._C.set_matmul_mode(mode)
        try:
            ta, tb = dev(nt, A, True), dev(nt, B, True)
            out = ta @ tb
            (out * dev(nt, G)).sum().backward()
            C, gA, gB = out.numpy(), ta.grad.numpy(), tb.grad.numpy()
        finally:
            nt._C.set_matmul_mode(1)
        A64, B64, G64 = A.astype(np.float64), B.astype(np.float64), G.astype(np.float64)
        assert_scaled(C[rows], A64[rows] @ B64, np.abs(A64[rows]) @ np.abs(B64), 1e-4, f"forward mode {mode}")
        assert_scaled(gA[rows], G64[rows] @ B64.T, np.abs(G64[rows]) @ np.abs(B64.T), 1e-4, f"grad A mode {mode}")
        assert_scaled(gB[krows], A64[:, krows].T @ G64, np.abs(A64[:, krows].T) @ np.abs(G64), 1e-4, f"grad B mode {mode}")
        rel = np.abs(C[rows] - A64[rows] @ B64).max() / np.abs(A64[rows] @ B64).max()
        print(f"mode {mode} {shape}: max|C - C64| / max|C64| = {rel:.2e}")
        # the stated tolerance in its plain max-relative reading; the default mode holds fp32 accuracy
        assert rel < (1e-4 if mode == 3 else 3e-6)
    del cols


def test_matmul_batched_full_size(nt):
    A = np.random.default_rng(30).uniform(-1, 1, (32, 512, 512)).astype(np.float32)
    B = np.random.default_rng(31).uniform(-1, 1, (32, 512, 512)).astype(np.float32)
    want = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    for mode in (1, 0):
        nt._C.set_matmul_mode(mode)
        try:
            got = (dev(nt, A) @ dev(nt, B)).numpy()
        finally:
            nt._C.set_matmul_mode(1)
        assert_scaled(got, want, bound, 1e-4, f"batched mode {mode}")


def test_matmul_errors(nt):
    a = dev(nt, np.zeros((3, 4), np.float32))
    b = dev(nt, np.zeros((5, 6), np.float32))
    with pytest.raises(RuntimeError):
        a @ b  # shape rule of MatmulOp
    with pytest.raises(ValueError):
        nt._C.matmul(a._C_view, b._C_view)  # native check: std::invalid_argument -> ValueError
    with pytest.raises(ValueError):
        nt._C.matmul(a._C_view, dev(nt, np.zeros((2, 4, 6), np.float32))._C_view)


@pytest.mark.parametrize("L", [4, 260, 1024, 4100, 8192, 16384, 16388, 1023])
def test_extremum_backward_row_slices_with_ties(nt, port, L):
    """Max/min over the last dim with enough slices for the one-pass kernel (slice kept in registers,
    L <= 16384 and a multiple of 4) and for the two-launch path beyond it; a third of the slices carry a
    tied extremum (zero gradient there, the reference's integer-division quirk); upstream gradient random."""
    rng = np.random.default_rng(L)
    rows = 333
    x = rng.standard_normal((rows, L)).astype(np.float32)
    tied = rng.random(rows) < 0.33
    for r in np.flatnonzero(tied):
        i, j = rng.choice(L, 2, replace=False)
        x[r, i] = x[r, j] = 9.0          # two positions share the maximum
        x[r, (i + 1) % L if (i + 1) % L != j else (i + 2) % L] = -9.0
    g = rng.standard_normal((rows,)).astype(np.float32)
    for name, sign in (("max", 1.0), ("min", -1.0)):
        xs = (x * sign).astype(np.float32)
        t = dev(nt, xs, True)
        red = getattr(t, name)((1,))
        (red * dev(nt, g)).sum().backward()
        m = xs.max(axis=1) if name == "max" else xs.min(axis=1)
        want = O.extremum_backward(port, np.broadcast_to(g[:, None], xs.shape), xs,
                                   np.broadcast_to(m[:, None], xs.shape), [1])
        assert_bit_exact(t.grad.numpy(), want, f"{name} backward, L={L}")
        assert (want[tied] == 0).all() and (np.abs(want[~tied]).sum(axis=1) > 0).all()


@pytest.mark.parametrize("axes", [(0,), (0, 1)])
def test_extremum_backward_leading_dim_and_full_with_ties(nt, port, axes):
    """Max/min backward over the leading dim and over the whole tensor: one optimistic pass writes g * (x == m)
    while counting the matches per slice, a second launch revisits only the tied slices (zero gradient there, the
    reference's integer-division quirk).  A third of the columns carry a tied extremum; for the full reduction
    both the tied and the unique case are run."""
    rng = np.random.default_rng(len(axes) + 40)
    R, C = 3000, 2048
    for tie_everything in ((False, True) if axes == (0, 1) else (False,)):
        x = rng.standard_normal((R, C)).astype(np.float32)
        if axes == (0,):
            tied = rng.random(C) < 0.33
            for c in np.flatnonzero(tied):
                i, j = rng.choice(R, 2, replace=False)
                x[i, c] = x[j, c] = 9.0
        elif tie_everything:
            x[17, 33] = x[2999, 2047] = 9.0
        else:
            x[17, 33] = 9.0
        g_np = rng.standard_normal((C,) if axes == (0,) else ()).astype(np.float32)
        for name, sign in (("max", 1.0), ("min", -1.0)):
            xs = (x * sign).astype(np.float32)
            t = dev(nt, xs, True)
            red = getattr(t, name)(axes)
            (red * dev(nt, g_np)).sum().backward()
            m = getattr(xs, name)(axis=axes)
            want = O.extremum_backward(port, np.broadcast_to(g_np, xs.shape), xs, np.broadcast_to(m, xs.shape), list(axes))
            assert_bit_exact(t.grad.numpy(), want, f"{name} backward over {axes}, tie={tie_everything}")
            if axes == (0,):
                assert (want[:, tied] == 0).all() and (np.abs(want[:, ~tied]).sum(axis=0) > 0).all()
            else:
                assert (np.abs(want).sum() == 0) == tie_everything
