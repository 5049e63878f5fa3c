"""GPU parity on the cases the other files leave out (through the C ABI):

  - pow with exponents other than 2 -- the hand-written products and reciprocals for 3, -1, -2 and the
    double-precision path for the rest -- at 2^24 elements against the CPU oracle (<= 2 ulp), over special
    values against the reference's own outputs, and PowOp's backward for exponents 3, 4, -1;
  - Storage::cast over every dtype pair: the reference's tables (out-of-range and NaN inputs included),
    and 2^22-element inputs, also through strided and reversed views;
  - comparisons and `equals` on strided / reversed Float32, Float64 and Int64 views with NaN and signed zeros;
  - the exact-mode matmul (mode 2) at 2048^3, bit for bit against the oracle's triple loop on sampled rows;
  - min / max over slices holding NaN or zeros of both signs: what this library returns is pinned;
  - matmul with infinite, NaN and near-FLT_MAX operands in every mode;
  - the bounded device-side wait: made to run out on purpose, reported as an error, context still usable.
"""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import assert_bit_exact, assert_scaled, assert_ulp, ulp_distance

pytestmark = pytest.mark.gpu

NP = {"bool": np.bool_, "int32": np.int32, "int64": np.int64, "float32": np.float32, "float64": np.float64}


def dev(nt, a, requires_grad=False):
    return nt.Tensor.from_numpy(a, "cuda", requires_grad=requires_grad)


def nt_dtype(nt, name):
    return {"bool": nt.bool_, "int32": nt.int32, "int64": nt.int64, "float32": nt.float32, "float64": nt.float64}[name]


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("e", [3.0, -2.0, -1.0, 0.5, 3.7, 4.0, 0.0, 1.0, -0.5])
def test_pow_special_values_vs_reference(nt, golden_extra, e):
    x = golden_extra["powx/in/x"]
    got = (dev(nt, x) ** e).numpy()
    assert_ulp(got, golden_extra[f"powx/{e}/out"], 2, f"pow {e}")


@pytest.mark.parametrize("e", [3.0, -2.0, -1.0, 0.5, 3.7])
def test_pow_full_size(nt, port, e):
    n = 1 << 24
    rng = np.random.default_rng(int(abs(e) * 10) + 50)
    if e == int(e):
        x = rng.uniform(-3, 3, n).astype(np.float32)
        x[:4096] = (rng.uniform(0.3, 3.0, 4096) * 1e-19).astype(np.float32)   # 1/x^2 near the top of the range
        x[4096:8192] = rng.uniform(1e12, 1e13, 4096).astype(np.float32)       # x^3 near the top of the range
    else:
        x = rng.uniform(0.1, 10, n).astype(np.float32)
    with np.errstate(all="ignore"):
        want = port.unary("pow", x, e)
    got = (dev(nt, x.reshape(4096, 4096)) ** e).numpy().reshape(-1)
    worst = assert_ulp(got, want, 2, f"pow {e} at 2^24")
    print(f"pow {e}: worst {worst} ulp, {int((ulp_distance(got, want) > 0).sum())} of {n} elements differ")


@pytest.mark.parametrize("e", [3.0, 4.0, -1.0])
def test_pow_backward_full_size(nt, port, e):
    """(g * e) * x ** (e - 1): exponents 3, 4 and -1 land on the product / reciprocal special cases."""
    n = 1 << 24
    rng = np.random.default_rng(int(e) + 70)
    x = rng.uniform(0.2, 3, n).astype(np.float32) * rng.choice([-1.0, 1.0], n).astype(np.float32)
    g = rng.standard_normal(n).astype(np.float32)
    tx = dev(nt, x.reshape(4096, 4096), True)
    ((tx ** e) * dev(nt, g.reshape(4096, 4096))).sum().backward()
    want = O.pow_backward(port, g, x, e)
    assert_ulp(tx.grad.numpy().reshape(-1), want, 2, f"pow {e} backward")


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("src", list(NP))
def test_cast_tables(nt, golden_extra, src):
    a = golden_extra[f"cast/in/{src}"]
    t = dev(nt, a)
    for dst in NP:
        got = t.to(nt_dtype(nt, dst)).numpy()
        want = golden_extra[f"cast/{src}/{dst}"]
        assert got.dtype == want.dtype
        if dst.startswith("float"):
            same = (got.view(f"u{got.itemsize}") == want.view(f"u{want.itemsize}")) | (np.isnan(got) & np.isnan(want))
            assert same.all(), (src, dst, got, want)
        else:
            assert np.array_equal(got, want), (src, dst, got, want)


@pytest.mark.parametrize("src", ["float32", "float64", "int64", "int32"])
def test_cast_large_and_through_views(nt, src):
    rng = np.random.default_rng(81)
    R, C = 2048, 2048
    if src.startswith("float"):
        a = (rng.standard_normal((R, C)) * 10.0 ** rng.integers(-3, 12, (R, C))).astype(NP[src])
        a[rng.integers(0, R, 500), rng.integers(0, C, 500)] = np.nan
        a[rng.integers(0, R, 500), rng.integers(0, C, 500)] = np.inf
    else:
        hi = 2 ** 62 if src == "int64" else 2 ** 31 - 1
        a = rng.integers(-hi, hi, (R, C)).astype(NP[src])
    t = dev(nt, a)
    for dst in NP:
        if dst == src:
            continue
        with np.errstate(all="ignore"):
            want = a.astype(NP[dst])
            want_view = np.ascontiguousarray(a[::-1, 1::3]).astype(NP[dst])
        got = t.to(nt_dtype(nt, dst)).numpy()
        got_view = t[::-1, 1::3].to(nt_dtype(nt, dst)).numpy()   # reversed rows, every third column
        for g_, w_ in ((got, want), (got_view, want_view)):
            if dst.startswith("float"):
                assert ((g_ == w_) | (np.isnan(g_) & np.isnan(w_))).all(), (src, dst)
            else:
                assert np.array_equal(g_, w_), (src, dst)


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kind", ["float32", "float64", "int64"])
def test_comparisons_on_views(nt, golden_extra, kind):
    x, y = golden_extra[f"cmp/in/{kind}/x"], golden_extra[f"cmp/in/{kind}/y"]
    tx, ty = dev(nt, x), dev(nt, y).T
    for key, got in (("eq", tx == ty), ("gt", tx > ty), ("ge", tx >= ty), ("lt", tx < ty), ("le", tx <= ty)):
        assert np.array_equal(got.numpy(), golden_extra[f"cmp/{kind}/{key}"]), (kind, key)
    # larger, through reversed / stepped / broadcast views, against numpy (IEEE comparisons are unambiguous)
    rng = np.random.default_rng(91)
    specials = np.array([np.nan, 0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, 2.5], np.float64)
    if kind == "int64":
        a, b = rng.integers(-4, 5, (513, 1030)).astype(np.int64), rng.integers(-4, 5, (1030, 1026)).astype(np.int64)
    else:
        a, b = rng.choice(specials, (513, 1030)).astype(NP[kind]), rng.choice(specials, (1030, 1026)).astype(NP[kind])
    ta, tb = dev(nt, a), dev(nt, b)
    va, na = ta[::-1, ::2], a[::-1, ::2]                         # (513, 515): reversed rows, stepped columns
    vb, nb = tb.T[::2, 5:520][:513], b.T[::2, 5:520][:513]       # transposed, stepped, offset
    with np.errstate(all="ignore"):
        for name, got, want in (("eq", va == vb, na == nb), ("gt", va > vb, na > nb), ("ge", va >= vb, na >= nb)):
            assert np.array_equal(got.numpy(), want), (kind, name)
        row = tb[3, :515]
        assert np.array_equal((va > row).numpy(), na > b[3, :515]), "row broadcast"
    assert nt._C.equals(va._C_view, va._C_view) == (not np.isnan(na.astype(np.float64)).any())
    assert not nt._C.equals(va._C_view, vb._C_view)


# ---------------------------------------------------------------------------------------------
def test_exact_matmul_2048_cubed_bit_for_bit(nt, port):
    """Mode 2 restates the reference's CPU loop (one rounded multiply, one rounded add, ascending k): every
    output row depends on its own row of A only, so 96 rows of the 2048^3 product pin the whole kernel."""
    rng = np.random.default_rng(30)
    A = rng.uniform(-1, 1, (2048, 2048)).astype(np.float32)
    B = rng.uniform(-1, 1, (2048, 2048)).astype(np.float32)
    nt._C.set_matmul_mode(2)
    try:
        got = (dev(nt, A) @ dev(nt, B)).numpy()
        got_t = (dev(nt, np.ascontiguousarray(A.T)).T @ dev(nt, np.ascontiguousarray(B.T)).T).numpy()
    finally:
        nt._C.set_matmul_mode(1)
    rows = np.concatenate([np.arange(32), rng.choice(np.arange(32, 2048), 64, replace=False)])
    want = port.matmul(A[rows], B)
    assert_bit_exact(got[rows], want, "2048^3, mode 2")
    assert_bit_exact(got_t[rows], want, "2048^3, mode 2, both operands through transposed views")


# ---------------------------------------------------------------------------------------------
def test_extremum_over_nan_and_signed_zero_slices_is_pinned(nt, golden_extra):
    """The reference folds a slice sequentially: a NaN replaces the running extremum and the next element
    replaces the NaN, so its answer for a slice that holds a NaN depends on the element order; of +0 and -0
    the first one wins.  This library reduces in parallel and cannot follow an order.  Pinned here: NaNs
    are skipped -- the extremum of a slice is the extremum of its non-NaN elements (which is also what
    the reference returns whenever no larger element precedes the last NaN), a slice of nothing but NaN
    gives the neutral element (-FLT_MAX for max, FLT_MAX for min); a zero extremum is a zero of either
    sign; an all -inf slice gives the reference's -FLT_MAX for max; slices without NaN are unaffected by
    NaNs elsewhere in the tensor and equal the reference's bit for bit."""
    x = golden_extra["ext/in/x"]
    t = dev(nt, x)
    flt_max = np.float32(3.4028235e38)
    for name, want, neutral in (("max", golden_extra["ext/max"], -flt_max), ("min", golden_extra["ext/min"], flt_max)):
        got = getattr(t, name)(1).numpy()
        for i, row in enumerate(x):
            rest = row[~np.isnan(row)]
            if np.isnan(row).any():
                assert got[i] == (getattr(rest, name)() if rest.size else neutral), (name, i, got[i])
            elif want[i] == 0:
                assert got[i] == 0, (name, i, got[i])
            else:
                assert got[i] == want[i], (name, i, got[i], want[i])
    # large: one NaN and one row of signed zeros and negatives among ordinary rows, row and column kernels
    rng = np.random.default_rng(93)
    big = rng.standard_normal((300, 5000)).astype(np.float32)
    big[7, 1234] = np.nan
    big[9, :] = np.where(rng.integers(0, 2, 5000) == 1, 0.0, -0.0) - np.abs(big[9, :]) * (rng.integers(0, 50, 5000) > 0)
    tb = dev(nt, big)
    with np.errstate(all="ignore"):
        assert np.array_equal(tb.max((1,)).numpy(), np.nanmax(big, axis=1))
        assert np.array_equal(tb.min((1,)).numpy(), np.nanmin(big, axis=1))
        assert np.array_equal(tb.max((0,)).numpy(), np.nanmax(big, axis=0))
        assert np.array_equal(tb.max().numpy(), np.nanmax(big))


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("mode", [2, 0, 1, 3])
def test_matmul_nonfinite_operands(nt, golden_extra, mode):
    """Exact modes reproduce the reference's table (infinities, NaN row, products near FLT_MAX).  The
    3xTF32 modes split x = hi + lo: a NaN operand gives NaN where the reference gives NaN; an infinite
    operand gives a non-finite value (an infinity of the right sign, or NaN where the split's cross terms
    meet inf * 0 or inf - inf) where the reference gives an infinity; finite operands up to FLT_MAX,
    including those whose TF32 rounding would overflow, give the finite product."""
    a, b, want = golden_extra["mmx/a"], golden_extra["mmx/b"], golden_extra["mmx/out"]
    nt._C.set_matmul_mode(mode)
    try:
        got = (dev(nt, a) @ dev(nt, b)).numpy()
    finally:
        nt._C.set_matmul_mode(1)
    finite = np.isfinite(want)
    if mode == 2:
        assert_bit_exact(got, want, "mode 2")
        return
    assert np.array_equal(np.isnan(got[1]), np.isnan(want[1])) and np.isnan(got[1]).all()
    if mode == 0:
        assert np.array_equal(got[~finite & ~np.isnan(want)], want[~finite & ~np.isnan(want)])
    else:
        assert (~np.isfinite(got[~finite])).all()
        inf_rows = got[[0, 2]]
        ok = np.isnan(inf_rows) | (inf_rows == want[[0, 2]])
        assert ok.all(), inf_rows
    bound = np.abs(a[3:].astype(np.float64)) @ np.abs(b.astype(np.float64))
    assert np.isfinite(got[3:]).all()
    assert_scaled(got[3:], want[3:], bound, 1e-4, f"finite rows, mode {mode}")


# ---------------------------------------------------------------------------------------------
def test_bounded_wait_runs_out_and_is_reported(nt):
    """Every spin in device code has a limit; past it the kernel records a code and returns.  The probe
    kernel waits, with the helper and the limit the GEMM pipeline uses, on a barrier nothing arrives on.
    With the limit lowered to 10^5 clocks it must return at once, the next synchronisation must raise
    RuntimeError naming the probe's code, and the context must stay usable (no fault, no hang)."""
    _C = nt._C
    a = dev(nt, np.ones((64, 64), np.float32))
    (a @ a).numpy()                       # the tensor-core path is initialised and healthy
    before = _C.get_wait_limit_clocks()
    assert before == 1 << 31
    with pytest.raises(ValueError):
        _C.set_wait_limit_clocks(10)
    _C.set_wait_limit_clocks(100_000)
    try:
        _C.wait_probe()
        with pytest.raises(RuntimeError, match=r"bounded device-side wait ran out \(code 5"):
            _C.cuda_sync()
        _C.cuda_sync()                    # reported once, then cleared
        _C.wait_probe()
        with pytest.raises(RuntimeError, match="code 5"):
            a.numpy()                     # a download reports it too: values are never read past a time-out
    finally:
        _C.set_wait_limit_clocks(before)
    got = (a @ a).numpy()                 # the context still works
    assert np.array_equal(got, np.full((64, 64), 64.0, np.float32))
    _C.cuda_sync()


def test_small_products_take_the_exact_kernel_by_default(nt):
    """With the library's default threshold a product of at most 2^21 multiply-adds is computed by the exact
    FP32 kernel also in the 3xTF32 modes (same bits as mode 0); the fixture of this test-suite sets the
    threshold to 0 so that every other test drives the tensor-core kernel."""
    _C = nt._C
    rng = np.random.default_rng(11)
    a, b = dev(nt, rng.standard_normal((96, 200)).astype(np.float32)), dev(nt, rng.standard_normal((200, 72)).astype(np.float32))  # 1.4 M multiply-adds
    assert _C.get_matmul_tc_min_macs() == 0
    _C.set_matmul_mode(0)
    exact = (a @ b).numpy()
    _C.set_matmul_mode(1)
    tensor_core = (a @ b).numpy()
    _C.set_matmul_tc_min_macs(1 << 21)
    try:
        routed = (a @ b).numpy()
    finally:
        _C.set_matmul_tc_min_macs(0)
    assert_bit_exact(routed, exact, "default routing of a small product")
    assert np.abs(tensor_core - exact).max() <= 2e-6 * (np.abs(a.numpy()) @ np.abs(b.numpy())).max()


# ---------------------------------------------------------------------------------------------
@pytest.mark.parametrize("shape", [(256, 512, 64), (384, 520, 200), (130, 70, 1000), (1, 300, 257), (513, 1, 96)])
def test_every_operand_major_of_the_tensor_core_kernel(nt, shape):
    """The 3xTF32 kernel reads each operand's planes K-major or MN-major, whichever the operand's own row-major
    order makes it: all four combinations, ragged extents included, give the same bits (the planes hold the
    same values, only their walk differs) and are within 2e-6 (|A||B|) of the fp64 product."""
    M, N, K = shape
    rng = np.random.default_rng(M + N + K)
    A, B = rng.uniform(-1, 1, (M, K)).astype(np.float32), rng.uniform(-1, 1, (K, N)).astype(np.float32)
    ref = A.astype(np.float64) @ B.astype(np.float64)
    bound = np.abs(A).astype(np.float64) @ np.abs(B).astype(np.float64)
    tA, tB = dev(nt, A), dev(nt, B)
    tAt, tBt = dev(nt, np.ascontiguousarray(A.T)), dev(nt, np.ascontiguousarray(B.T))
    outs = [(a @ b).numpy() for a, b in ((tA, tB), (tA, tBt.T), (tAt.T, tB), (tAt.T, tBt.T))]
    for got in outs:
        assert_scaled(got, ref, bound, 2e-6, f"{shape}")
        assert_bit_exact(got, outs[0], "same bits whatever the operand order")


def test_operand_plane_cache_follows_every_write(nt):
    """Cached operand planes are dropped by anything that writes the storage they came from: an in-place op,
    a setitem (copy_view), an upload, an SGD update, a graph replay; and they are found again when nothing
    was written (the second product of an unchanged operand launches no split)."""
    _C = nt._C
    rng = np.random.default_rng(17)
    x_np = rng.standard_normal((300, 200)).astype(np.float32)
    w_np = rng.standard_normal((200, 260)).astype(np.float32)
    x, w = dev(nt, x_np), dev(nt, w_np)

    def check(what):
        got = (x @ w).numpy()
        ref = x.numpy().astype(np.float64) @ w.numpy().astype(np.float64)
        bound = np.abs(x.numpy()).astype(np.float64) @ np.abs(w.numpy()).astype(np.float64)
        assert_scaled(got, ref, bound, 2e-6, what)

    check("first use")
    s0, h0 = _C.matmul_split_stats()
    check("second use")
    s1, h1 = _C.matmul_split_stats()
    assert s1 == s0 and h1 == h0 + 2, "an unchanged operand is not split again"
    with nt.no_grad():
        x += 1.5
    check("after an in-place add")
    x[5:9, ::2] = dev(nt, np.full((4, 100), 7.0, np.float32))
    check("after a setitem")
    fresh = rng.standard_normal((300, 200)).astype(np.float32)
    x.storage.upload(fresh.ctypes.data, fresh.nbytes)
    check("after an upload into the same storage")
    g = dev(nt, rng.standard_normal((200, 260)).astype(np.float32))
    s2, _ = _C.matmul_split_stats()
    _C.sgd_update(w._C_view, g._C_view, 0.5, 1.0)
    s3, h3 = _C.matmul_split_stats()
    assert s3 == s2 + 1, "the update re-splits the weight's planes behind itself"
    check("after an SGD update")
    assert _C.matmul_split_stats()[1] == h3 + 2, "and the next product finds both operands ready"
    # a graph replay rewrites storages behind the host's counters: eager calls must not trust old planes
    y = dev(nt, np.zeros((300, 200), np.float32))
    graph = _C.Graph()
    with graph.capture():
        with nt.no_grad():
            x += 1.0
    graph.replay()
    graph.replay()
    check("after graph replays that modified an operand")
    graph.close()
    _C.set_matmul_operand_planes(True, False)
    try:
        s4, h4 = _C.matmul_split_stats()
        check("cache off")
        assert _C.matmul_split_stats() == (s4 + 2, h4)
    finally:
        _C.set_matmul_operand_planes(True, True)
    _C.set_matmul_operand_planes(False, False)
    try:
        check("transposing split (natural planes off)")
    finally:
        _C.set_matmul_operand_planes(True, True)


def test_a_training_step_splits_each_tensor_once(nt):
    """Linear -> Tanh -> Linear -> Tanh -> Linear with 3xTF32 products: 8 products per step (3 forward, 3 weight
    gradients, 2 input gradients) over 3 inputs, 3 weights and 3 output gradients: with natural-layout cached
    planes that is 5 operand splits per step instead of 16, and the SGD update writes the weights' planes itself."""
    import nanotorch_b200.nn as nn

    _C = nt._C
    nt.manual_seed(0)
    model = nn.Sequential(nn.Linear(256, 384), nn.Tanh(), nn.Linear(384, 384), nn.Tanh(), nn.Linear(384, 128)).to("cuda")
    X = dev(nt, np.random.default_rng(1).standard_normal((512, 256)).astype(np.float32))
    Y = dev(nt, np.random.default_rng(2).standard_normal((512, 128)).astype(np.float32))
    opt = nn.GradientDescent(model.parameters(), lr=1e-2)

    def step():
        loss = nt.mean((model(X) - Y) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        return loss

    step()
    s0, h0 = _C.matmul_split_stats()
    step()
    s1, h1 = _C.matmul_split_stats()
    # X is unchanged (hit), the 2 hidden activations and 3 gradients are new (5 splits), the weights' planes were
    # written by the previous update (hits) and are written again by this one, inside the update kernel (no split)
    assert s1 - s0 == 5, s1 - s0
    assert h1 - h0 == 16 - 5, h1 - h0


def test_producers_write_their_own_planes(nt):
    """tanh and tanh_backward on a large dense matrix also write the result's TF32 planes: same result bits as
    the plain kernels, the following products launch no split for that operand, and the products are right."""
    _C = nt._C
    rng = np.random.default_rng(23)
    z_np = rng.standard_normal((1024, 1024)).astype(np.float32)
    w_np = (rng.standard_normal((1024, 512)) * 0.05).astype(np.float32)
    g_np = rng.standard_normal((1024, 1024)).astype(np.float32)
    z, w, g = dev(nt, z_np), dev(nt, w_np), dev(nt, g_np)
    _C.set_producer_planes(False)
    h_plain = nt.tanh(z)
    d_plain = nt.Tensor._new_contiguous(_C.tanh_backward(g._C_view, h_plain._C_view), (1024, 1024))
    _C.set_producer_planes(True)
    (dev(nt, z_np[:64]) @ w).numpy()                     # w's planes exist from here on
    s0, h0 = _C.matmul_split_stats()
    h = nt.tanh(z)
    d = nt.Tensor._new_contiguous(_C.tanh_backward(g._C_view, h._C_view), (1024, 1024))
    assert_bit_exact(h.numpy(), h_plain.numpy(), "tanh")
    assert_bit_exact(d.numpy(), d_plain.numpy(), "tanh backward")
    y1 = (h @ w).numpy()            # K-major use of h's planes
    y2 = (h.T @ d).numpy()          # MN-major use of h's and d's planes
    s1, h1 = _C.matmul_split_stats()
    assert s1 == s0 and h1 == h0 + 4, (s1 - s0, h1 - h0)
    hn, dn = h.numpy().astype(np.float64), d.numpy().astype(np.float64)
    assert_scaled(y1, hn @ w_np.astype(np.float64), np.abs(hn) @ np.abs(w_np.astype(np.float64)), 2e-6, "h @ w")
    assert_scaled(y2, hn.T @ dn, np.abs(hn.T) @ np.abs(dn), 2e-6, "h^T @ d")


@pytest.mark.parametrize("op", ["mul", "div"])
def test_binary_backward_both_gradients_in_one_pass(nt, port, op):
    """x1*x2 and x1/x2 at 4096^2: both gradients come from one launch over g, x1, x2.  mul: bit-exact against the
    oracle's chain; div: dx1 = g/x2 bit-exact, dx2 = ((-x1)/x2^2)*g within 2^-22 of the largest intermediate
    (x2*x2 stands in for powf(x2, 2), at most 1 ulp apart).  A non-dense operand takes the composed kernels."""
    rng = np.random.default_rng(31)
    n = 4096
    x1 = rng.uniform(-1, 1, (n, n)).astype(np.float32)
    x2 = rng.uniform(0.5, 2, (n, n)).astype(np.float32)
    g = rng.standard_normal((n, n)).astype(np.float32)
    t1, t2 = dev(nt, x1, True), dev(nt, x2, True)
    res = t1 * t2 if op == "mul" else t1 / t2
    (res * dev(nt, g)).sum().backward()
    if op == "mul":
        assert_bit_exact(t1.grad.numpy(), port.binary("multiply", x2, g), "dx1")
        assert_bit_exact(t2.grad.numpy(), port.binary("multiply", x1, g), "dx2")
    else:
        assert_bit_exact(t1.grad.numpy(), port.binary("divide", g, x2), "dx1")
        want = O.div_backward_x2(port, g, x1, x2)
        assert_scaled(t2.grad.numpy(), want, np.abs(want) + 1e-30, 2.0 ** -21, "dx2")
    both = getattr(nt._C, f"{op}_backward")(dev(nt, g)._C_view, t1._C_view, t2.T._C_view)
    assert both is None, "a transposed operand is not a dense run: the composed kernels take it"


TILE_PIPELINE_SHAPES = [(1100, 1004), (4096, 4096), (64, 16384), (16384, 64), (3, 520, 772), (1028, 1500)]


@pytest.mark.parametrize("shape", TILE_PIPELINE_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_transposed_operands_through_the_tile_pipeline(nt, shape):
    """Large fp32 elementwise ops with a transposed operand (TMA-fed persistent kernel): edge tiles in both
    dims, a leading dim, sliced operands whose row stride is not their width, one and two transposed
    operands, unary and binary.  Bit-equal to numpy for the exact ops, and to the register-staged tile
    kernel (pipeline off) for all of them."""
    _C = nt._C
    rng = np.random.default_rng(sum(shape))
    *lead, nI, nJ = shape
    a_np = rng.standard_normal(shape).astype(np.float32)
    bt_np = rng.standard_normal((*lead, nJ, nI)).astype(np.float32)       # holds b transposed
    ct_np = rng.standard_normal((*lead, nJ, nI + 8)).astype(np.float32)   # wider: sliced below
    a, bt, ct = dev(nt, a_np), dev(nt, bt_np), dev(nt, ct_np)
    d0, d1 = len(shape) - 2, len(shape) - 1
    b = nt.transpose(bt, d0, d1)
    c = nt.transpose(ct[..., 4:nI + 4], d0, d1)                                # 16-byte aligned offset, stride nI + 8
    b_ref, c_ref = np.swapaxes(bt_np, -1, -2), np.swapaxes(ct_np[..., 4:nI + 4], -1, -2)

    def run():
        return {
            "a+b.T": (a + b).numpy(),
            "b.T-a": (b - a).numpy(),
            "b.T*c.T": (b * c).numpy(),
            "a/c.T": (a / c).numpy(),
            "exp(b.T)": nt.exp(b).numpy(),
            "relu(c.T)": nt.relu(c).numpy(),
        }

    on = run()
    _C.set_transposed_tile_pipeline(False)
    try:
        off = run()
    finally:
        _C.set_transposed_tile_pipeline(True)
    assert_bit_exact(on["a+b.T"], a_np + b_ref, "a + b.T")
    assert_bit_exact(on["b.T-a"], b_ref - a_np, "b.T - a")
    assert_bit_exact(on["b.T*c.T"], b_ref * c_ref, "b.T * c.T")
    assert_bit_exact(on["a/c.T"], a_np / c_ref, "a / c.T")
    assert_bit_exact(on["relu(c.T)"], np.maximum(c_ref, 0), "relu(c.T)")
    for k in on:
        assert_bit_exact(on[k], off[k], k + ": pipeline against the register-staged kernel")


@pytest.mark.parametrize("shape", [(512, 4096, 1024), (128, 16384, 256), (1000, 3000, 1100), (256, 8192, 512)],
                         ids=lambda s: "x".join(map(str, s)))
def test_split_k_products(nt, shape):
    """Products with so few output tiles that most SMs would idle are cut along k (up to 8 parts per tile,
    summed in part order by whichever CTA finishes last).  Against fp64 with the norm-wise bound of the
    unsplit kernel; the same bits on every run; bias in the epilogue equal to the composed form; and close
    to the unsplit result (the partial sums are rounded once more)."""
    _C = nt._C
    M, K, N = shape
    rng = np.random.default_rng(M + N)
    a_np = rng.standard_normal((M, K)).astype(np.float32)
    b_np = rng.standard_normal((K, N)).astype(np.float32)
    bias_np = rng.standard_normal((N,)).astype(np.float32)
    a, b, bias = dev(nt, a_np), dev(nt, b_np), dev(nt, bias_np)
    ref = a_np.astype(np.float64) @ b_np.astype(np.float64)
    bound = np.abs(a_np).astype(np.float64) @ np.abs(b_np).astype(np.float64)
    with nt.no_grad():
        first = (a @ b).numpy()
        again = (a @ b).numpy()
        assert_scaled(first, ref, bound, 2e-6, "split-K product")
        assert_bit_exact(first, again, "two runs of the same split-K product")
        # a.T stored: the MN-major operand paths through the same schedule
        at = dev(nt, np.ascontiguousarray(a_np.T))
        assert_bit_exact((at.T @ b).numpy(), first, "A read MN-major")
        fused = nt.Tensor._new_view(_C.linear(a._C_view, b._C_view, bias._C_view), (M, N), None, None).numpy()
        assert_bit_exact(fused, first + bias_np, "bias in the epilogue of a split product")
        _C.set_matmul_schedule(1, 8)
        try:
            unsplit = (a @ b).numpy()
        finally:
            _C.set_matmul_schedule(8, 8)
    assert_scaled(unsplit, ref, bound, 2e-6, "unsplit product")
    assert np.max(np.abs(first - unsplit) / bound) < 1e-6


@pytest.mark.parametrize("mode", [1, 0])
@pytest.mark.parametrize("shape", [(2048, 1024, 1536), (300, 200, 260), (4096, 512, 4096)], ids=lambda s: "x".join(map(str, s)))
def test_matmul_pair_is_two_products(nt, shape, mode):
    """Both gradients of a product in one call (the second tensor-core launch overlapping the first one's last
    wave as its programmatic dependent): the bits of two separate products, also with the overlap switched off,
    and a kernel queued behind the pair sees both results complete."""
    _C = nt._C
    M, K, N = shape
    rng = np.random.default_rng(M + K)
    g, x, w = (dev(nt, rng.standard_normal(s).astype(np.float32)) for s in ((M, N), (M, K), (K, N)))
    _C.set_matmul_mode(mode)
    try:
        with nt.no_grad():
            gx_ref = (g @ w.T).numpy()
            gw_ref = (x.T @ g).numpy()
            for overlap in (True, False, True):
                _C.set_matmul_pair_overlap(overlap)
                sx, sw = _C.matmul_pair(g._C_view, w.T._C_view, x.T._C_view, g._C_view)
                gx, gw = nt.Tensor._new_contiguous(sx, (M, K)), nt.Tensor._new_contiguous(sw, (K, N))
                total = (gx.sum() + gw.sum()).numpy()       # queued right behind the pair
                assert_bit_exact(gx.numpy(), gx_ref, f"g @ w.T from the pair (overlap {overlap})")
                assert_bit_exact(gw.numpy(), gw_ref, f"x.T @ g from the pair (overlap {overlap})")
                assert_bit_exact(total, (nt.Tensor.from_numpy(gx_ref, "cuda").sum() + nt.Tensor.from_numpy(gw_ref, "cuda").sum()).numpy(),
                                 "a reduction queued behind the pair")
    finally:
        _C.set_matmul_pair_overlap(False)
        _C.set_matmul_mode(1)


@pytest.mark.parametrize("shape", [(1000, 1028), (5, 200, 64), (4096, 4096), (7, 4)], ids=lambda s: "x".join(map(str, s)))
def test_row_broadcast_kernel(nt, shape):
    """A dense operand against one broadcast row (the dedicated contiguous kernel): both argument orders of the
    non-commutative ops, leading dims that collapse into the rows, the in-place forms -- bit-equal to numpy."""
    rng = np.random.default_rng(sum(shape))
    a_np = rng.uniform(0.5, 2.0, shape).astype(np.float32)
    r_np = rng.uniform(0.5, 2.0, shape[-1:]).astype(np.float32)
    a, r = dev(nt, a_np), dev(nt, r_np)
    assert_bit_exact((a + r).numpy(), a_np + r_np, "a + row")
    assert_bit_exact((r - a).numpy(), r_np - a_np, "row - a")
    assert_bit_exact((a - r).numpy(), a_np - r_np, "a - row")
    assert_bit_exact((a * r).numpy(), a_np * r_np, "a * row")
    assert_bit_exact((r / a).numpy(), r_np / a_np, "row / a")
    assert_bit_exact((a / r).numpy(), a_np / r_np, "a / row")
    with nt.no_grad():
        b = dev(nt, a_np.copy())
        b -= r
        assert_bit_exact(b.numpy(), a_np - r_np, "a -= row")
        b = dev(nt, a_np.copy())
        b /= r
        assert_bit_exact(b.numpy(), a_np / r_np, "a /= row")
    # a unary op on the expanded row itself
    rows = int(np.prod(shape[:-1]))
    assert_bit_exact((r.expand(rows, shape[-1]) ** 2).numpy(), np.broadcast_to(r_np * r_np, (rows, shape[-1])), "row**2 expanded")
    assert_bit_exact(nt.relu(-r.expand(rows, shape[-1])).numpy(), np.broadcast_to(np.maximum(-r_np, 0), (rows, shape[-1])), "relu(-row) expanded")
    # a sliced row (offset by 4 elements: still 16-byte aligned) and one that is not aligned (falls back)
    wide = dev(nt, np.concatenate([np.zeros(4, np.float32), r_np, np.zeros(3, np.float32)]))
    assert_bit_exact((a + wide[4:4 + shape[-1]]).numpy(), a_np + r_np, "a + aligned slice of a longer row")
    wide1 = dev(nt, np.concatenate([np.zeros(1, np.float32), r_np]))
    assert_bit_exact((a + wide1[1:]).numpy(), a_np + r_np, "a + misaligned row")
