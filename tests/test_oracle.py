"""The C restatement (oracle/nt_oracle.c) and the op-level chains (oracle/oracle.py) must reproduce,
bit for bit, what the reference itself produced for the same inputs (tests/golden/reference_cpu.npz),
and -- where the reference's native module has been built -- agree with it on random views."""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import assert_bit_exact


def test_rng_stream_matches_reference(golden, port):
    # the reference's own known answer (tests/test_factories.py:239-242): seed 42 -> 0.75515550..., 0.63903135...
    u = port.uniform(42, 16)
    assert abs(u[0] - 0.7551555037498474) < 1e-6 and abs(u[1] - 0.6390313506126404) < 1e-6
    assert_bit_exact(u, golden["rng/seed42"], "seed 42")
    assert_bit_exact(port.uniform(0, 16), golden["rng/seed0"], "seed 0")


BIN = {"add": "add", "sub": "subtract", "mul": "multiply", "div": "divide"}


@pytest.mark.parametrize("op", list(BIN))
@pytest.mark.parametrize("layout", ["contig", "bcast", "transposed"])
def test_binary_forward_and_backward(golden, port, op, layout):
    g = golden
    a, G = g["ew/in/a"], g["ew/in/G"]
    y = {"contig": g["ew/in/d"] if op == "div" else g["ew/in/b"],
         "bcast": g["ew/in/dv"] if op == "div" else g["ew/in/v"],
         "transposed": g["ew/in/dt"] if op == "div" else g["ew/in/bt"]}[layout]
    yv = y.T if layout == "transposed" else np.broadcast_to(y, a.shape)
    assert_bit_exact(port.binary(BIN[op], a, yv), g[f"ew/{op}/{layout}/out"], "forward")
    # backward chains (autograd/ops_binary.py:49-50, 95-100, 145-150, 197-202); upstream = G
    if op == "add":
        gx, gy_full = G, G
    elif op == "sub":
        gx, gy_full = G, port.binary("multiply", np.broadcast_to(np.float32(-1), G.shape), G)
    elif op == "mul":
        gx, gy_full = port.binary("multiply", yv, G), port.binary("multiply", a, G)
    else:
        gx, gy_full = port.binary("divide", G, yv), O.div_backward_x2(port, G, a, yv)
    assert_bit_exact(gx, g[f"ew/{op}/{layout}/gx"], "grad x1")
    if layout == "bcast":
        gy = port.reduce("sum", gy_full, [0])
    elif layout == "transposed":
        gy = gy_full.T
    else:
        gy = gy_full
    assert_bit_exact(np.ascontiguousarray(gy), g[f"ew/{op}/{layout}/gy"], "grad x2")


UNARY = {
    "exp": ("n", "exp", 0.0, lambda o, G, x, y: O.exp_backward(o, G, y)),
    "neg": ("n", "neg", 0.0, lambda o, G, x, y: o.binary("multiply", np.broadcast_to(np.float32(-1), G.shape), G)),
    "relu": ("n", "relu", 0.0, lambda o, G, x, y: O.relu_backward(o, G, y)),
    "tanh": ("n", "tanh", 0.0, lambda o, G, x, y: O.tanh_backward(o, G, y)),
    "sigmoid": ("n", "sigmoid", 0.0, lambda o, G, x, y: O.sigmoid_backward(o, G, y)),
    "log": ("p", "log", 0.0, lambda o, G, x, y: O.log_backward(o, G, x)),
    "sqrt": ("p", "sqrt", 0.0, lambda o, G, x, y: O.sqrt_backward(o, G, y)),
    "pow2": ("a", "pow", 2.0, lambda o, G, x, y: O.pow_backward(o, G, x, 2.0)),
    "pow3.7": ("p", "pow", 3.7, lambda o, G, x, y: O.pow_backward(o, G, x, 3.7)),
    "powm1": ("p", "pow", -1.0, lambda o, G, x, y: O.pow_backward(o, G, x, -1.0)),
}


@pytest.mark.parametrize("name", list(UNARY))
def test_unary_forward_and_backward(golden, port, name):
    src, prim, e, bwd = UNARY[name]
    x, G = golden[f"ew/in/{src}"], golden["ew/in/G"]
    y = port.unary(prim, x, e)
    assert_bit_exact(y, golden[f"ew/{name}/out"], "forward")
    assert_bit_exact(bwd(port, G, x, y), golden[f"ew/{name}/gx"], "backward")


def test_special_values(golden, port):
    x = golden["ew/special/in"]
    with np.errstate(all="ignore"):
        for name, prim, e in [("exp", "exp", 0), ("relu", "relu", 0), ("tanh", "tanh", 0), ("sigmoid", "sigmoid", 0),
                              ("neg", "neg", 0), ("pow2", "pow", 2.0)]:
            assert_bit_exact(port.unary(prim, x, e), golden[f"ew/special/{name}"], name)


AXES = [(0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2), None]


@pytest.mark.parametrize("axes", AXES)
@pytest.mark.parametrize("name", ["sum", "mean", "max", "min"])
def test_reductions(golden, port, name, axes):
    x = golden["red/in/x"]
    ax = list(range(x.ndim)) if axes is None else list(axes)
    key = f"red/{name}/{'all' if axes is None else ''.join(map(str, axes))}"
    got = O.mean_forward(port, x, ax) if name == "mean" else port.reduce(name, x, ax)
    for keepdim in (0, 1):
        want = golden[f"{key}/{keepdim}/out"]
        assert_bit_exact(got.reshape(want.shape), want, f"{name} keepdim={keepdim}")
    # backward with upstream ones
    kept = tuple(1 if d in ax else x.shape[d] for d in range(x.ndim))
    ones = np.broadcast_to(np.float32(1.0), x.shape)
    if name == "sum":
        gx = ones
    elif name == "mean":
        count = x.size // max(got.size, 1)
        gx = port.binary("divide", ones, np.broadcast_to(np.float32(count), x.shape))
    else:
        gx = O.extremum_backward(port, ones, x, np.broadcast_to(got.reshape(kept), x.shape), ax)
    assert_bit_exact(np.ascontiguousarray(gx), golden[f"{key}/0/gx"], f"{name} backward")


def test_reduction_views_ties_and_last_dim(golden, port):
    x = golden["red/in/x"]
    assert_bit_exact(port.reduce("sum", x.transpose(2, 1, 0), [0]), golden["red/sum_transposed/out"], "transposed")
    tie = golden["red/tie/in"]
    ones = np.ones_like(tie)
    m = port.reduce("max", tie, [1]).reshape(2, 1)
    assert_bit_exact(O.extremum_backward(port, ones, tie, np.broadcast_to(m, tie.shape), [1]), golden["red/tie/max_gx"])
    m = port.reduce("min", tie, [0]).reshape(1, 4)
    assert_bit_exact(O.extremum_backward(port, ones, tie, np.broadcast_to(m, tie.shape), [0]), golden["red/tie/min_gx"])
    y = golden["red/in/y"]
    for name in ("sum", "max", "min"):
        assert_bit_exact(port.reduce(name, y, [2]), golden[f"red/y/{name}/out"], name)
    assert_bit_exact(O.mean_forward(port, y, [2]), golden["red/y/mean/out"], "mean")


@pytest.mark.parametrize("case", ["2d", "batched", "bcast_batch", "vec_mat", "mat_vec", "vec_vec", "odd"])
def test_matmul(golden, port, case):
    a, b, g = golden[f"mm/{case}/a"], golden[f"mm/{case}/b"], golden[f"mm/{case}/g"]
    want = golden[f"mm/{case}/out"]
    # shape rules of MatmulOp (autograd/ops_binary.py:318-343): 1-D operands gain a unit dim, batches broadcast
    a2 = a.reshape(1, -1) if a.ndim == 1 else a
    b2 = b.reshape(-1, 1) if b.ndim == 1 else b
    batch = np.broadcast_shapes(a2.shape[:-2], b2.shape[:-2])
    ae = np.broadcast_to(a2, batch + a2.shape[-2:])
    be = np.broadcast_to(b2, batch + b2.shape[-2:])
    out = port.matmul(ae, be)
    assert_bit_exact(out.reshape(want.shape), want, "forward")
    ge = g.reshape(out.shape)
    ga = port.matmul(ge, np.swapaxes(be, -1, -2))
    gb = port.matmul(np.swapaxes(ae, -1, -2), ge)
    lead_b = list(range(gb.ndim - b2.ndim))
    if lead_b:
        gb = port.reduce("sum", gb, lead_b)
    assert_bit_exact(ga.reshape(a.shape), golden[f"mm/{case}/ga"], "grad a")
    # the reference hands a 1-D right operand its gradient with shape (k, 1) (it reshapes to the
    # rebound 2-D operand, autograd/ops_binary.py:255-257, 266); values are compared flat
    assert_bit_exact(gb.reshape(-1), golden[f"mm/{case}/gb"].reshape(-1), "grad b")


def test_matmul_transposed_views(golden, port):
    assert_bit_exact(port.matmul(golden["mm/tt/a"].T, golden["mm/tt/b"].T), golden["mm/tt/out"])


def _seeded_params(port, dims, seed=0):
    stream = port.uniform(seed, sum(dims[i] * dims[i + 1] for i in range(len(dims) - 1)))
    params, pos = [], 0
    for i in range(len(dims) - 1):
        n = dims[i] * dims[i + 1]
        params.append((O.kaiming(port, stream[pos:pos + n], dims[i], dims[i + 1]), np.zeros(dims[i + 1], np.float32)))
        pos += n
    return params


def test_mlp_configuration_1(golden, port):
    """784 -> 256 -> 10, ReLU, batch 256, seed 0: the reference's loss curve, bit for bit (25 steps here)."""
    params = _seeded_params(port, [784, 256, 10])
    assert_bit_exact(params[0][0][0, :8], golden["mlp1/W1_head"], "kaiming init")
    X = np.random.default_rng(1).standard_normal((256, 784)).astype(np.float32)
    Y = np.random.default_rng(2).standard_normal((256, 10)).astype(np.float32)
    losses = [O.mlp_step(port, params, X, Y, 0.01, "relu", compute_input_grad=False) for _ in range(25)]
    assert_bit_exact(np.array(losses, np.float32), golden["mlp1/losses"][:25], "loss curve")


def test_mlp_tanh_small(golden, port):
    params = _seeded_params(port, [24, 32, 32, 32, 16])
    X, Y = golden["mlp5s/X"], golden["mlp5s/Y"]
    losses = [O.mlp_step(port, params, X, Y, 1e-3, "tanh") for _ in range(5)]
    assert_bit_exact(np.array(losses, np.float32), golden["mlp5s/losses"], "loss curve")
    for i, (W, b) in enumerate(params):
        assert_bit_exact(W, golden[f"mlp5s/final/{2 * i}"], f"W{i}")
        assert_bit_exact(b, golden[f"mlp5s/final/{2 * i + 1}"], f"b{i}")


@pytest.mark.skipif(not O.ref_available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_port_matches_reference_native_module(port):
    ref = O.RefOracle()
    rng = np.random.default_rng(7)
    a = rng.standard_normal((9, 14)).astype(np.float32)
    b = rng.uniform(0.5, 2, (14, 9)).astype(np.float32)
    views = [(a, b.T), (a[::-1, ::2], b.T[:, ::-2][::-1]), (a, np.broadcast_to(b[0, :1], a.shape))]
    for x, y in views:
        for name in list(O.BINARY) + list(O.COMPARE):
            got, want = port.binary(name, x, y), ref.binary(name, x, y)
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), name
    for name in O.UNARY:
        src = np.abs(a) + 0.1 if name in ("log", "sqrt", "pow") else a
        for e in ([2.0, -1.0, 0.5, 3.7] if name == "pow" else [0.0]):
            assert_bit_exact(port.unary(name, src, e), ref.unary(name, src, e), name)
    t = rng.standard_normal((3, 4, 5)).astype(np.float32)
    for v in (t, t.transpose(2, 0, 1), t[:, ::-1, ::2]):
        for axes in ([0], [2], [0, 2], [2, 0], [0, 1, 2]):
            for name in O.REDUCE:
                assert np.array_equal(port.reduce(name, v, axes), ref.reduce(name, v, axes)), (name, axes)
    A = rng.standard_normal((2, 3, 5, 4)).astype(np.float32)
    B = rng.standard_normal((2, 3, 4, 6)).astype(np.float32)
    assert_bit_exact(port.matmul(A, B), ref.matmul(A, B), "matmul")
    assert_bit_exact(port.matmul(A.swapaxes(-1, -2)[..., :4, :4], B[..., :4]), ref.matmul(A.swapaxes(-1, -2)[..., :4, :4], B[..., :4]))
    assert_bit_exact(port.uniform(123, 100), ref.uniform(123, 100), "uniform")


# ---------------------------------------------------------------------------------------------
# second fixture file (tests/golden/reference_cpu_extra.npz, same generator)
POW_EXPONENTS = [3.0, -2.0, -1.0, 0.5, 3.7, 4.0, 0.0, 1.0, 2.0, -0.5]


@pytest.mark.parametrize("e", POW_EXPONENTS)
def test_pow_other_exponents(golden_extra, port, e):
    """x ** e and PowOp's backward over negatives, zeros, infinities, NaN and denormals."""
    x, G = golden_extra["powx/in/x"], golden_extra["powx/in/G"]
    with np.errstate(all="ignore"):
        assert_bit_exact(port.unary("pow", x, e), golden_extra[f"powx/{e}/out"], f"pow {e}")
        assert_bit_exact(O.pow_backward(port, G, x, e), golden_extra[f"powx/{e}/gx"], f"pow {e} backward")


def test_compare_with_nan_and_signed_zeros(golden_extra, port):
    x, y = golden_extra["cmp/in/float32/x"], golden_extra["cmp/in/float32/y"]
    for name, key in (("pw_equal", "eq"), ("pw_greater", "gt"), ("pw_greater_eq", "ge")):
        assert np.array_equal(port.binary(name, x, y.T), golden_extra[f"cmp/float32/{key}"]), name
    # the reference's < and <= are the swapped forms of > and >= (src/nanotorch/ops.py)
    assert np.array_equal(port.binary("pw_greater", np.ascontiguousarray(y.T), x), golden_extra["cmp/float32/lt"])
    assert np.array_equal(port.binary("pw_greater_eq", np.ascontiguousarray(y.T), x), golden_extra["cmp/float32/le"])
    # IEEE comparisons are unambiguous: numpy gives the same tables for every dtype
    for kind in ("float32", "float64", "int64"):
        a, b = golden_extra[f"cmp/in/{kind}/x"], golden_extra[f"cmp/in/{kind}/y"].T
        with np.errstate(all="ignore"):
            for key, fn in (("eq", np.equal), ("gt", np.greater), ("ge", np.greater_equal), ("lt", np.less), ("le", np.less_equal)):
                assert np.array_equal(fn(a, b), golden_extra[f"cmp/{kind}/{key}"]), (kind, key)


def test_extremum_over_nan_and_signed_zero_slices(golden_extra, port):
    """The reference's sequential combiner on slices holding NaN (a NaN replaces the running value, the
    next element replaces the NaN) and both zeros (the first one wins)."""
    x = golden_extra["ext/in/x"]
    assert_bit_exact(port.reduce("max", x, [1]), golden_extra["ext/max"], "max")
    assert_bit_exact(port.reduce("min", x, [1]), golden_extra["ext/min"], "min")


def test_matmul_nonfinite_operands(golden_extra, port):
    with np.errstate(all="ignore"):
        assert_bit_exact(port.matmul(golden_extra["mmx/a"], golden_extra["mmx/b"]), golden_extra["mmx/out"], "matmul")


def test_cast_tables_are_the_host_conversions(golden_extra):
    """Storage::cast is a host loop of static_casts in the reference (src/cpp/storage.cpp:47-65), also for
    Cuda storages.  The C conversions of this machine give the same tables, out-of-range and NaN inputs
    included (the conversion instruction's "integer indefinite" result)."""
    for src in ("float32", "float64", "int64", "int32", "bool"):
        a = golden_extra[f"cast/in/{src}"]
        for dst in ("bool", "int32", "int64", "float32", "float64"):
            with np.errstate(all="ignore"):
                want = a.astype(dst)
            got = golden_extra[f"cast/{src}/{dst}"]
            if dst.startswith("float"):
                assert_bit_exact(got.astype(np.float32), want.astype(np.float32), f"{src}->{dst}")
            else:
                assert np.array_equal(got, want), (src, dst, got, want)
