"""GPU parity of the pointwise kernels (through the C ABI) against the reference's outputs
(golden fixtures) and against the CPU oracle on seeded inputs, up to the benchmark sizes.

Tolerances: bit-exact for add, sub, mul, truediv, neg, relu (and tanh, which restates the host
libm's algorithm); <= 2 ulp for exp, log, sqrt, pow, sigmoid.  Fused backward kernels: bit-exact
where the chain only has exactly-rounded steps, otherwise |diff| <= 2^-22 * (largest intermediate).
"""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import assert_bit_exact, assert_scaled, assert_ulp

pytestmark = pytest.mark.gpu

BIN = {"add": "add", "sub": "subtract", "mul": "multiply", "div": "divide"}
EPS = 2.0 ** -22  # two ulp of a value in [1, 2)


def dev(nt, a, requires_grad=False):
    return nt.Tensor.from_numpy(a, "cuda", requires_grad=requires_grad)


def apply_binary(op, x, y):
    return {"add": lambda: x + y, "sub": lambda: x - y, "mul": lambda: x * y, "div": lambda: x / y}[op]()


@pytest.mark.parametrize("op", list(BIN))
@pytest.mark.parametrize("layout", ["contig", "bcast", "transposed"])
def test_binary_golden(nt, golden, op, layout):
    g = golden
    a, G = g["ew/in/a"], g["ew/in/G"]
    y = {"contig": g["ew/in/d"] if op == "div" else g["ew/in/b"],
         "bcast": g["ew/in/dv"] if op == "div" else g["ew/in/v"],
         "transposed": g["ew/in/dt"] if op == "div" else g["ew/in/bt"]}[layout]
    tx, ty = dev(nt, a, True), dev(nt, y, True)
    res = apply_binary(op, tx, ty.T if layout == "transposed" else ty)
    (res * dev(nt, G)).sum().backward()
    assert_bit_exact(res.numpy(), g[f"ew/{op}/{layout}/out"], "forward")
    assert_bit_exact(tx.grad.numpy(), g[f"ew/{op}/{layout}/gx"], "grad x1")
    want = g[f"ew/{op}/{layout}/gy"]
    got = ty.grad.numpy()
    if op == "div" or layout == "bcast":
        # div: x2*x2 stands in for powf(x2, 2) (<= 1 ulp apart); bcast: the column sum runs in a
        # different order than the reference's sequential loop
        scale = np.abs(want) + (np.abs(G).sum(axis=0) if layout == "bcast" else 0) * (4 if op == "div" else 1)
        assert_scaled(got, want, np.broadcast_to(scale, want.shape) + 1e-30, 1e-5 if layout == "bcast" else EPS, "grad x2")
    else:
        assert_bit_exact(got, want, "grad x2")


UNARY_FWD_TOL = {"exp": 2, "neg": 0, "relu": 0, "tanh": 2, "sigmoid": 2, "log": 2, "sqrt": 0, "pow2": 2, "pow3.7": 2,
                 "powm1": 2}


def apply_unary(nt, name, x):
    return {"exp": lambda: x.exp(), "neg": lambda: -x, "relu": lambda: nt.relu(x), "tanh": lambda: nt.tanh(x),
            "sigmoid": lambda: nt.sigmoid(x), "log": lambda: x.log(), "sqrt": lambda: nt.sqrt(x),
            "pow2": lambda: x ** 2.0, "pow3.7": lambda: x ** 3.7, "powm1": lambda: x ** -1.0}[name]()


SRC = {"exp": "n", "neg": "n", "relu": "n", "tanh": "n", "sigmoid": "n", "log": "p", "sqrt": "p", "pow2": "a",
       "pow3.7": "p", "powm1": "p"}


@pytest.mark.parametrize("name", list(UNARY_FWD_TOL))
def test_unary_golden(nt, golden, name):
    x, G = golden[f"ew/in/{SRC[name]}"], golden["ew/in/G"]
    tx = dev(nt, x, True)
    res = apply_unary(nt, name, tx)
    (res * dev(nt, G)).sum().backward()
    want = golden[f"ew/{name}/out"]
    if UNARY_FWD_TOL[name] == 0:
        assert_bit_exact(res.numpy(), want, "forward")
    else:
        assert_ulp(res.numpy(), want, UNARY_FWD_TOL[name], "forward")
    gw = golden[f"ew/{name}/gx"]
    if name in ("neg", "relu"):
        assert_bit_exact(tx.grad.numpy(), gw, "backward")
    else:
        # largest intermediate of the chain: |g| * max(1, |f'|-ish); 4 ulp of that
        scale = np.abs(G) * np.maximum(1.0, np.abs(gw / np.where(G == 0, 1, G))) + 1e-30
        assert_scaled(tx.grad.numpy(), gw, scale, 4 * EPS, "backward")


def test_special_values(nt, golden):
    x = dev(nt, golden["ew/special/in"])
    for name, tol in [("exp", 2), ("relu", 0), ("tanh", 2), ("sigmoid", 2), ("neg", 0), ("pow2", 0)]:
        got = apply_unary(nt, name, x).numpy()
        want = golden[f"ew/special/{name}"]
        if tol == 0:
            assert_bit_exact(got, want, name)
        else:
            assert_ulp(got, want, tol, name)


def _views(rng, R, C):
    """(name, a_view, b_view) pairs over the layouts the kernels special-case."""
    a = rng.uniform(-1, 1, (R, C)).astype(np.float32)
    b = rng.uniform(0.5, 2, (R, C)).astype(np.float32)
    bt = rng.uniform(0.5, 2, (C, R)).astype(np.float32)
    v = rng.uniform(0.5, 2, (C,)).astype(np.float32)
    col = rng.uniform(0.5, 2, (R, 1)).astype(np.float32)
    wide = rng.uniform(0.5, 2, (R, 2 * C + 3)).astype(np.float32)
    return a, [("contig", lambda t: t, b), ("row_bcast", lambda t: t, v), ("col_bcast", lambda t: t, col),
               ("transposed", lambda t: t.T, bt), ("strided_cols", lambda t: t[:, 1:2 * C + 1:2], wide),
               ("offset_slice", lambda t: t[:, 3:C + 3], wide), ("reversed", lambda t: t[::-1, ::-1], b)]


@pytest.mark.parametrize("shape", [(257, 130), (64, 4096), (1023, 1027), (1, 5), (300, 1)])
def test_binary_views_vs_oracle(nt, port, shape):
    rng = np.random.default_rng(shape[0] * 7919 + shape[1])
    R, C = shape
    a, cases = _views(rng, R, C)
    ta = dev(nt, a)
    for lname, view, src in cases:
        tb = view(dev(nt, src))
        nb = np.broadcast_to(view(src), a.shape)
        for op in BIN:
            got = apply_binary(op, ta, tb).numpy()
            assert_bit_exact(got, port.binary(BIN[op], a, nb), f"{op}/{lname}/{shape}")


def test_inplace_and_copy_views(nt, port):
    rng = np.random.default_rng(5)
    base = rng.standard_normal((70, 130)).astype(np.float32)
    other = rng.uniform(0.5, 2, (130,)).astype(np.float32)
    for name, fn in [("add", lambda t, o: t.__iadd__(o)), ("sub", lambda t, o: t.__isub__(o)),
                     ("mul", lambda t, o: t.__imul__(o)), ("div", lambda t, o: t.__itruediv__(o))]:
        want = base.copy()
        port.inplace(name, want[:, ::-1], other)
        t = dev(nt, base)
        v0 = t.version
        fn(t[:, ::-1], dev(nt, other))
        assert_bit_exact(t.numpy(), want, name)
        assert t.version == v0 + 1
    t = dev(nt, base)
    t[3:9, ::2] = dev(nt, other[:65])
    want = base.copy()
    want[3:9, ::2] = other[:65]
    assert_bit_exact(t.numpy(), want, "setitem")
    assert_bit_exact(dev(nt, base).T.reshape(130 * 70).numpy(), base.T.reshape(-1), "reshape of transposed view")
    assert_bit_exact(dev(nt, other).expand(70, 130).clone().numpy(), np.broadcast_to(other, (70, 130)), "materialised broadcast")


def test_dtype_generic_paths(nt):
    i = np.arange(-6, 6, dtype=np.int64).reshape(3, 4)
    j = np.full((3, 4), 3, dtype=np.int64)
    ti, tj = dev(nt, i), dev(nt, j)
    assert np.array_equal((ti + tj).numpy(), i + j) and np.array_equal((ti * tj).numpy(), i * j)
    assert np.array_equal((ti / tj).numpy(), (i / j).astype(np.int64) if False else np.trunc(i / j).astype(np.int64))
    assert np.array_equal((ti ** 3).numpy(), i ** 3)
    assert np.array_equal((ti > tj).numpy(), i > j) and (ti > tj).dtype == nt.bool_
    assert np.array_equal(nt.relu(ti).numpy(), np.maximum(i, 0))
    d = np.linspace(-2, 2, 12).reshape(3, 4)
    td = dev(nt, d)
    np.testing.assert_allclose(td.exp().numpy(), np.exp(d), rtol=1e-15)
    np.testing.assert_allclose(nt.tanh(td).numpy(), np.tanh(d), rtol=1e-15)
    b = dev(nt, np.array([True, False, True]))
    c = dev(nt, np.array([True, True, False]))
    assert np.array_equal((b + c).numpy(), [True, True, True]) and np.array_equal((b * c).numpy(), [True, False, False])
    assert np.array_equal(td.to(nt.int32).numpy(), d.astype(np.int32))
    assert np.array_equal(ti.to(nt.bool_).numpy(), i != 0)
    assert (ti.sum().numpy() == i.sum()) and ti.sum().dtype == nt.int64
    assert np.array_equal(dev(nt, i.astype(np.int32)).max(1).numpy(), i.max(1).astype(np.int32))
    with pytest.raises(ValueError):
        b / c  # Bool has no division kernel (DispatchArithmetic)
    with pytest.raises(RuntimeError):
        nt._C.add(ti._C_view, td._C_view)  # dtype mismatch is checked natively


# ---------------------------------------------------------------------------------------------
# benchmark sizes: every op of the elementwise sweep on [4096, 4096] against the CPU oracle
N = 4096


@pytest.fixture(scope="module")
def big(nt):
    r = np.random.default_rng
    host = {"a": r(10).uniform(-1, 1, (N, N)).astype(np.float32), "b": r(11).uniform(-1, 1, (N, N)).astype(np.float32),
            "d": r(12).uniform(0.5, 2, (N, N)).astype(np.float32), "v": r(13).uniform(-1, 1, (N,)).astype(np.float32),
            "n": r(14).standard_normal((N, N)).astype(np.float32), "p": r(15).uniform(0.1, 10, (N, N)).astype(np.float32),
            "G": r(16).standard_normal((N, N)).astype(np.float32), "dv": r(17).uniform(0.5, 2, (N,)).astype(np.float32)}
    return host, {k: dev(nt, v) for k, v in host.items()}


@pytest.mark.parametrize("op", list(BIN))
def test_binary_full_size(nt, port, big, op):
    h, d = big
    y, yv = ("d", "dv") if op == "div" else ("b", "v")
    assert_bit_exact(apply_binary(op, d["a"], d[y]).numpy(), port.binary(BIN[op], h["a"], h[y]), "contiguous")
    assert_bit_exact(apply_binary(op, d["a"], d[yv]).numpy(), port.binary(BIN[op], h["a"], np.broadcast_to(h[yv], (N, N))), "broadcast")
    assert_bit_exact(apply_binary(op, d["a"], d[y].T).numpy(), port.binary(BIN[op], h["a"], h[y].T), "transposed")


@pytest.mark.parametrize("name,src,prim,e,tol", [("exp", "n", "exp", 0, 2), ("neg", "n", "neg", 0, 0),
                                                 ("relu", "n", "relu", 0, 0), ("tanh", "n", "tanh", 0, 2),
                                                 ("sigmoid", "n", "sigmoid", 0, 2), ("log", "p", "log", 0, 2),
                                                 ("sqrt", "p", "sqrt", 0, 0), ("pow2", "a", "pow", 2.0, 2)])
def test_unary_full_size(nt, port, big, name, src, prim, e, tol):
    h, d = big
    got = apply_unary(nt, name, d[src]).numpy()
    want = port.unary(prim, h[src], e)
    if tol == 0:
        assert_bit_exact(got, want, name)
    else:
        worst = assert_ulp(got, want, tol, name)
        print(f"{name}: max ulp distance to the CPU oracle {worst}, mismatching fraction {(got != want).mean():.2e}")


def test_tanh_bit_exact_mode(nt, port, big, golden):
    """Mode 1 restates the host libm's tanhf operation for operation: identical bits to the CPU oracle,
    on the seeded [4096, 4096] input, on the special values and on a strided view."""
    h, d = big
    nt._C.set_tanh_mode(nt._C.TANH_BIT_EXACT_LIBM)
    try:
        assert_bit_exact(nt.tanh(d["n"]).numpy(), port.unary("tanh", h["n"]), "4096^2")
        assert_bit_exact(nt.tanh(d["n"].T[::3, 5:]).numpy(), port.unary("tanh", h["n"].T[::3, 5:]), "strided view")
        assert_bit_exact(nt.tanh(dev(nt, golden["ew/special/in"])).numpy(), golden["ew/special/tanh"], "special values")
        wide = np.random.default_rng(3).uniform(-25, 25, (1 << 20,)).astype(np.float32)
        assert_bit_exact(nt.tanh(dev(nt, wide)).numpy(), port.unary("tanh", wide), "U(-25, 25)")
    finally:
        nt._C.set_tanh_mode(nt._C.TANH_CORRECTLY_ROUNDED)
    # default mode: the correctly rounded value (float64 tanh rounded once)
    got = nt.tanh(d["n"]).numpy()
    assert_bit_exact(got, np.tanh(h["n"].astype(np.float64)).astype(np.float32), "correctly rounded")


@pytest.mark.parametrize("name", ["relu", "tanh", "sigmoid", "exp", "log", "sqrt", "pow2"])
def test_fused_backward_full_size(nt, port, big, name):
    h, d = big
    src = {"relu": "n", "tanh": "n", "sigmoid": "n", "exp": "n", "log": "p", "sqrt": "p", "pow2": "a"}[name]
    x = nt.Tensor.from_numpy(h[src], "cuda", requires_grad=True)
    y = apply_unary(nt, name, x)
    (y * d["G"]).sum().backward()
    got = x.grad.numpy()
    yh = y.numpy()
    G = h["G"]
    chain = {"relu": lambda: O.relu_backward(port, G, yh), "tanh": lambda: O.tanh_backward(port, G, yh),
             "sigmoid": lambda: O.sigmoid_backward(port, G, yh), "exp": lambda: O.exp_backward(port, G, yh),
             "log": lambda: O.log_backward(port, G, h[src]), "sqrt": lambda: O.sqrt_backward(port, G, yh),
             "pow2": lambda: O.pow_backward(port, G, h[src], 2.0)}[name]()
    if name in ("relu", "exp", "sigmoid", "pow2"):
        assert_bit_exact(got, chain, name)  # only exactly-rounded steps in the chain
    else:
        scale = np.abs(G) * np.maximum(1.0, np.abs(chain / np.where(G == 0, 1, G))) + 1e-30
        assert_scaled(got, chain, scale, 2 * EPS, name)


def test_default_tanh_and_sigmoid_equal_their_host_evaluation(nt, tmp_path):
    """The default tanh and the sigmoid are proven on the HOST (tests/test_tanh_restatement.py: every
    float argument within 2 ulp of the libm-based reference).  That proof carries over to the GPU only if
    the device evaluates the same headers to the same bits: compile nanotorch_b200/csrc/cr_math.h and sigmoid_f32.h with gcc
    and compare with the kernels' output bit for bit on 2^24 N(0,1) values, a sweep of U(-100, 100), the
    small-argument region and the special values."""
    import ctypes
    import subprocess
    from pathlib import Path

    csrc = Path(nt.__file__).resolve().parent / "csrc"
    src = tmp_path / "cr_host.c"
    src.write_text('#include "cr_math.h"\n#include "sigmoid_f32.h"\n'
                   "void eval(const float *x, float *t, float *s, long n) {\n"
                   "  for (long i = 0; i < n; ++i) { t[i] = nt_tanh_fast_f32(x[i]); s[i] = nt_sigmoid_f32(x[i]); }\n}\n")
    lib_path = tmp_path / "libcr_host.so"
    subprocess.run(["gcc", "-O2", "-shared", "-fPIC", "-fno-fast-math", "-ffp-contract=off", f"-I{csrc}",
                    "-o", str(lib_path), str(src), "-lm"], check=True)
    host = ctypes.CDLL(str(lib_path))
    rng = np.random.default_rng(99)
    x = np.concatenate([
        rng.standard_normal(1 << 24).astype(np.float32),
        rng.uniform(-100, 100, 1 << 20).astype(np.float32),
        (rng.standard_normal(1 << 18) * 2.0 ** rng.integers(-40, 0, 1 << 18)).astype(np.float32),
        np.array([0.0, -0.0, np.inf, -np.inf, 1e-45, -1e-45, 0.015625, -0.015625, 88.7, -88.7228394, -88.72283,
                  -104.0, 20.0, 40.0, 41.0, 3e38, -3e38], np.float32)])
    t = np.empty_like(x)
    s = np.empty_like(x)
    host.eval(x.ctypes.data_as(ctypes.c_void_p), t.ctypes.data_as(ctypes.c_void_p), s.ctypes.data_as(ctypes.c_void_p),
              ctypes.c_long(x.size))
    d = dev(nt, x)
    assert nt._C.get_tanh_mode() == nt._C.TANH_CORRECTLY_ROUNDED
    assert_bit_exact(nt.tanh(d).numpy(), t, "tanh, device vs host evaluation of cr_math.h")
    assert_bit_exact(nt.sigmoid(d).numpy(), s, "sigmoid, device vs host evaluation of sigmoid_f32.h")
