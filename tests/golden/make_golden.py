"""Generates tests/golden/*.npz by running the REFERENCE itself (its Python package on its own
native module, CPU path) on seeded inputs.  Run where the reference checkout and oracle/_ref exist:

    make -C oracle ref                      # builds oracle/_ref/_C*.so from the reference sources
    python tests/golden/make_golden.py --ref <reference checkout>

The reference package is imported from a scratch directory that only holds symlinks to the
reference's .py files plus the built native module; nothing is copied into this repository except
the numeric inputs/outputs written to the .npz files.  The fixtures pin oracle/nt_oracle.c and
oracle/oracle.py (tests/test_oracle.py) and are the known answers of the GPU parity tests.
"""

from __future__ import annotations

import argparse
import os
import sys
import tempfile
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent


def import_reference(ref: Path):
    so = next((REPO / "oracle" / "_ref").glob("_C*.so"))
    scratch = Path(tempfile.mkdtemp(prefix="ntref_"))
    pkg = scratch / "nanotorch"
    src = ref / "src" / "nanotorch"
    for path in src.rglob("*.py"):
        dst = pkg / path.relative_to(src)
        dst.parent.mkdir(parents=True, exist_ok=True)
        os.symlink(path, dst)
    os.symlink(so, pkg / so.name)
    sys.path.insert(0, str(scratch))
    import nanotorch as nt  # noqa: E402

    return nt


def T(nt, a: np.ndarray, requires_grad: bool = False):
    t = nt.Tensor(a.tolist(), dtype=nt.float32)
    if a.ndim == 0:
        t = nt.Tensor(float(a), dtype=nt.float32)
    if requires_grad:
        t.enable_grad()
    return t


def A(t) -> np.ndarray:
    """reference tensor -> numpy float32/bool/int64 array"""
    data = t.tolist()
    kind = {"Bool": np.bool_, "Int32": np.int32, "Int64": np.int64, "Float32": np.float32, "Float64": np.float64}
    return np.array(data, dtype=kind[t.dtype.name]).reshape(t.shape)


def elementwise_cases(nt, out: dict):
    rng = np.random.default_rng(100)
    R, C = 33, 18
    a = rng.uniform(-1, 1, (R, C)).astype(np.float32)
    b = rng.uniform(-1, 1, (R, C)).astype(np.float32)
    d = rng.uniform(0.5, 2, (R, C)).astype(np.float32)
    v = rng.uniform(-1, 1, (C,)).astype(np.float32)
    dv = rng.uniform(0.5, 2, (C,)).astype(np.float32)
    bt = rng.uniform(-1, 1, (C, R)).astype(np.float32)
    dt = rng.uniform(0.5, 2, (C, R)).astype(np.float32)
    n = rng.standard_normal((R, C)).astype(np.float32)
    p = rng.uniform(0.1, 10, (R, C)).astype(np.float32)
    G = rng.standard_normal((R, C)).astype(np.float32)
    for k, val in dict(a=a, b=b, d=d, v=v, dv=dv, bt=bt, dt=dt, n=n, p=p, G=G).items():
        out[f"ew/in/{k}"] = val

    ops = {"add": lambda x, y: x + y, "sub": lambda x, y: x - y, "mul": lambda x, y: x * y,
           "div": lambda x, y: x / y}
    for name, fn in ops.items():
        for layout in ("contig", "bcast", "transposed"):
            x = T(nt, a, True)
            if layout == "contig":
                y = T(nt, d if name == "div" else b, True)
                yy = y
            elif layout == "bcast":
                y = T(nt, dv if name == "div" else v, True)
                yy = y
            else:
                y = T(nt, dt if name == "div" else bt, True)
                yy = y.T
            res = fn(x, yy)
            (res * T(nt, G)).sum().backward()
            out[f"ew/{name}/{layout}/out"] = A(res)
            out[f"ew/{name}/{layout}/gx"] = A(x.grad)
            out[f"ew/{name}/{layout}/gy"] = A(y.grad)

    unary = {"exp": (n, lambda x: x.exp()), "neg": (n, lambda x: -x), "relu": (n, lambda x: nt.relu(x)),
             "tanh": (n, lambda x: nt.tanh(x)), "sigmoid": (n, lambda x: nt.sigmoid(x)),
             "log": (p, lambda x: x.log()), "sqrt": (p, lambda x: nt.sqrt(x)),
             "pow2": (a, lambda x: x ** 2.0), "pow3.7": (p, lambda x: x ** 3.7), "powm1": (p, lambda x: x ** -1.0)}
    for name, (src, fn) in unary.items():
        x = T(nt, src, True)
        res = fn(x)
        (res * T(nt, G)).sum().backward()
        out[f"ew/{name}/out"] = A(res)
        out[f"ew/{name}/gx"] = A(x.grad)
    # special values
    sp = np.array([0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-40, -1e-40, 88.7, -104.0, 20.0, -20.0, 0.3,
                   1e-30, 3.0e38], dtype=np.float32)
    out["ew/special/in"] = sp
    x = T(nt, sp)
    with np.errstate(all="ignore"):
        for name, fn in {"exp": lambda t: t.exp(), "relu": nt.relu, "tanh": nt.tanh, "sigmoid": nt.sigmoid,
                         "neg": lambda t: -t, "pow2": lambda t: t ** 2.0}.items():
            out[f"ew/special/{name}"] = A(fn(x))


def reduction_cases(nt, out: dict):
    rng = np.random.default_rng(200)
    x = rng.standard_normal((5, 6, 7)).astype(np.float32)
    out["red/in/x"] = x
    for axes in [(0,), (1,), (2,), (0, 2), (1, 2), (0, 1, 2), None]:
        for keepdim in (False, True):
            for name in ("sum", "mean", "max", "min"):
                t = T(nt, x, True)
                res = getattr(t, name)(axes, keepdim)
                key = f"red/{name}/{'all' if axes is None else ''.join(map(str, axes))}/{int(keepdim)}"
                out[key + "/out"] = A(res)
                res.sum().backward()
                out[key + "/gx"] = A(t.grad)
    # transposed view reduced along what was the contiguous dim
    t = T(nt, x, True)
    res = t.transpose(0, 2).sum((0,))
    out["red/sum_transposed/out"] = A(res)
    # ties: the integer-division quirk zeroes the whole gradient of a tied slice
    tie = np.array([[1.0, 3.0, 3.0, 2.0], [4.0, 0.0, -1.0, 2.0]], dtype=np.float32)
    out["red/tie/in"] = tie
    t = T(nt, tie, True)
    t.max((1,)).sum().backward()
    out["red/tie/max_gx"] = A(t.grad)
    t = T(nt, tie, True)
    t.min((0,)).sum().backward()
    out["red/tie/min_gx"] = A(t.grad)
    y = rng.standard_normal((4, 1, 40)).astype(np.float32)
    out["red/in/y"] = y
    for name in ("sum", "mean", "max", "min"):
        t = T(nt, y, True)
        res = getattr(t, name)(-1)
        out[f"red/y/{name}/out"] = A(res)
        res.sum().backward()
        out[f"red/y/{name}/gx"] = A(t.grad)


def matmul_cases(nt, out: dict):
    rng = np.random.default_rng(300)
    shapes = {"2d": ((5, 7), (7, 3)), "batched": ((2, 3, 5, 4), (2, 3, 4, 6)), "bcast_batch": ((3, 5, 4), (4, 6)),
              "vec_mat": ((7,), (7, 3)), "mat_vec": ((5, 7), (7,)), "vec_vec": ((7,), (7,)),
              "odd": ((37, 19), (19, 10))}
    for name, (sa, sb) in shapes.items():
        a = rng.uniform(-1, 1, sa).astype(np.float32)
        b = rng.uniform(-1, 1, sb).astype(np.float32)
        ta, tb = T(nt, a, True), T(nt, b, True)
        res = ta @ tb
        g = rng.uniform(-1, 1, res.shape).astype(np.float32)
        (res * T(nt, g)).sum().backward()
        out[f"mm/{name}/a"], out[f"mm/{name}/b"], out[f"mm/{name}/g"] = a, b, g
        out[f"mm/{name}/out"], out[f"mm/{name}/ga"], out[f"mm/{name}/gb"] = A(res), A(ta.grad), A(tb.grad)
    # transposed operand views
    a = rng.uniform(-1, 1, (7, 5)).astype(np.float32)
    b = rng.uniform(-1, 1, (3, 7)).astype(np.float32)
    out["mm/tt/a"], out["mm/tt/b"] = a, b
    out["mm/tt/out"] = A(T(nt, a).T @ T(nt, b).T)


def mlp_cases(nt, out: dict):
    import nanotorch.nn as nn
    from nanotorch.nn.optimizers import GradientDescent

    # configuration 1: 784 -> 256 -> 10, ReLU, batch 256, seed 0, lr 0.01, 100 steps on one batch
    nt.manual_seed(0)
    model = nn.Sequential(nn.Linear(784, 256), nn.ReLU(), nn.Linear(256, 10))
    X = np.random.default_rng(1).standard_normal((256, 784)).astype(np.float32)
    Y = np.random.default_rng(2).standard_normal((256, 10)).astype(np.float32)
    tX, tY = T(nt, X), T(nt, Y)
    opt = GradientDescent(model.parameters(), lr=0.01)
    out["mlp1/W1_head"] = A(model.parameters()[0])[0, :8]
    losses = []
    for _ in range(100):
        loss = nt.mean((model(tX) - tY) ** 2)
        opt.zero_grad()
        loss.backward()
        opt.step()
        losses.append(loss.item())
    out["mlp1/losses"] = np.array(losses, dtype=np.float32)
    out["mlp1/W2_final"] = A(model.parameters()[2])
    out["mlp1/b1_final"] = A(model.parameters()[1])

    # a small tanh network in the shape of configuration 5 (Linear/Tanh x3, Linear)
    nt.manual_seed(0)
    dims = [24, 32, 32, 32, 16]
    layers = []
    for i in range(4):
        layers.append(nn.Linear(dims[i], dims[i + 1]))
        if i < 3:
            layers.append(nn.Tanh())
    model = nn.Sequential(*layers)
    X = np.random.default_rng(40).standard_normal((64, 24)).astype(np.float32)
    Y = np.random.default_rng(41).standard_normal((64, 16)).astype(np.float32)
    out["mlp5s/X"], out["mlp5s/Y"] = X, Y
    tX, tY = T(nt, X), T(nt, Y)
    opt = GradientDescent(model.parameters(), lr=1e-3)
    losses = []
    for step in range(5):
        loss = nt.mean((model(tX) - tY) ** 2)
        opt.zero_grad()
        loss.backward()
        if step == 0:
            for i, p in enumerate(model.parameters()):
                out[f"mlp5s/grad0/{i}"] = A(p.grad)
        opt.step()
        losses.append(loss.item())
    out["mlp5s/losses"] = np.array(losses, dtype=np.float32)
    for i, p in enumerate(model.parameters()):
        out[f"mlp5s/final/{i}"] = A(p)


def index_cases(nt, out: dict):
    """Index-array / mask getitem and setitem through the reference's Tensor (CPU path)."""
    sys.path.insert(0, str(REPO / "tests"))
    from util import INDEX_GET_CASES, INDEX_SET_CASES, INDEX_SHAPE, index_case, index_value

    rng = np.random.default_rng(500)
    x = rng.standard_normal(INDEX_SHAPE).astype(np.float32)
    out["idx/in/x"] = x
    for k, source in enumerate(INDEX_GET_CASES):
        out[f"idx/get/{k}"] = A(T(nt, x)[index_case(source)])
    xi = rng.integers(-50, 50, INDEX_SHAPE).astype(np.int64)
    out["idx/in/xi"] = xi
    ti = nt.Tensor(xi.tolist(), dtype=nt.int64)
    out["idx/get_int64"] = A(ti[index_case(INDEX_GET_CASES[2])])
    for k, (source, kind) in enumerate(INDEX_SET_CASES):
        t = T(nt, x)
        index = index_case(source)
        value = index_value(kind, t[index].shape, rng)
        out[f"idx/set/{k}/value"] = np.asarray(value, dtype=np.float32)
        t[index] = T(nt, np.asarray(value, dtype=np.float32))
        out[f"idx/set/{k}/out"] = A(t)


def rng_cases(nt, out: dict):
    nt.manual_seed(42)
    out["rng/seed42"] = A(nt.rand(16))
    nt.manual_seed(0)
    out["rng/seed0"] = A(nt.rand(16))


def _typed(nt, a: np.ndarray):
    dt = {"bool": nt.bool_, "int32": nt.int32, "int64": nt.int64, "float32": nt.float32, "float64": nt.float64}[a.dtype.name]
    return nt.Tensor(a.tolist(), dtype=dt)


CAST_INPUTS = {
    "float32": np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 0.5, -0.5, 1.9, -1.9, 2147483520.0, 2147483648.0,
                         -2147483648.0, -2147483904.0, 3e9, -3e9, 1e10, 9.2e18, 9.3e18, -9.3e18, 1e20, 1e-45, 16777217.0,
                         255.0, 256.0, -1.0, 1.0], np.float32),
    "float64": np.array([np.nan, np.inf, -np.inf, 0.0, -0.0, 0.5, -0.5, 1.9, -1.9, 2147483647.0, 2147483647.5, 2147483648.0,
                         -2147483648.0, -2147483648.9, -2147483649.0, 3e9, 9.2e18, 9.3e18, -9.3e18, 1e300, 1e-320, 3.5e38,
                         16777217.0, 0.1, -1.0, 1.0], np.float64),
    "int64": np.array([0, 1, -1, 2**31 - 1, 2**31, -(2**31), -(2**31) - 1, 2**40 + 3, 2**24 + 1, 2**53 + 1, 2**63 - 1,
                       -(2**63), 255, 256, 123456789012], np.int64),
    "int32": np.array([0, 1, -1, 2**31 - 1, -(2**31), 2**24 + 1, 255, 256, 16777217], np.int32),
    "bool": np.array([True, False, True], np.bool_),
}


def extra_cases(nt, out: dict):
    """Cases the first fixture file does not hold: Storage::cast over every dtype pair with out-of-range,
    NaN and rounding inputs; comparisons with NaN and signed zeros in Float32/Float64/Int64; pow with
    other exponents than 2 (forward and PowOp backward); min/max over slices holding NaN or both zeros;
    matmul with non-finite and huge operands."""
    for src, a in CAST_INPUTS.items():
        out[f"cast/in/{src}"] = a
        for dst in ("bool", "int32", "int64", "float32", "float64"):
            t = _typed(nt, a).to({"bool": nt.bool_, "int32": nt.int32, "int64": nt.int64, "float32": nt.float32,
                                  "float64": nt.float64}[dst])
            out[f"cast/{src}/{dst}"] = A(t)
    # comparisons
    rng = np.random.default_rng(600)
    specials = np.array([np.nan, 0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, 1e-45], np.float64)
    for kind in ("float32", "float64", "int64"):
        if kind == "int64":
            x = rng.integers(-3, 4, (9, 8)).astype(np.int64)
            y = rng.integers(-3, 4, (8, 9)).astype(np.int64)
        else:
            x = rng.choice(specials, (9, 8)).astype(kind)
            y = rng.choice(specials, (8, 9)).astype(kind)
        out[f"cmp/in/{kind}/x"], out[f"cmp/in/{kind}/y"] = x, y
        tx, ty = _typed(nt, x), _typed(nt, y).T          # second operand through a transposed view
        out[f"cmp/{kind}/eq"], out[f"cmp/{kind}/gt"], out[f"cmp/{kind}/ge"] = A(tx == ty), A(tx > ty), A(tx >= ty)
        out[f"cmp/{kind}/lt"], out[f"cmp/{kind}/le"] = A(tx < ty), A(tx <= ty)
    # pow
    base = np.concatenate([rng.uniform(-3, 3, 400), rng.uniform(0.01, 20, 180),
                           [0.0, -0.0, 1.0, -1.0, np.inf, -np.inf, np.nan, 1e-45, -1e-45, 1e-20, 1e20, -1e20, 2.0, 0.5]]).astype(np.float32)
    G = rng.standard_normal(base.shape).astype(np.float32)
    out["powx/in/x"], out["powx/in/G"] = base, G
    for e in (3.0, -2.0, -1.0, 0.5, 3.7, 4.0, 0.0, 1.0, 2.0, -0.5):
        x = T(nt, base, True)
        y = x ** e
        out[f"powx/{e}/out"] = A(y)
        (y * T(nt, G)).sum().backward()
        out[f"powx/{e}/gx"] = A(x.grad)
    # min / max over slices with NaN and signed zeros (the sequential combiner is order dependent there)
    ext = np.array([[1.0, np.nan, 3.0, 2.0], [3.0, np.nan, 1.0, 2.0], [1.0, 2.0, 3.0, np.nan], [np.nan, 1.0, 2.0, 3.0],
                    [0.0, -0.0, -1.0, -2.0], [-0.0, 0.0, -1.0, -2.0], [0.0, -0.0, 1.0, 2.0], [-0.0, 0.0, 1.0, 2.0],
                    [np.nan, np.nan, np.nan, np.nan], [-np.inf, -np.inf, -np.inf, -np.inf]], np.float32)
    out["ext/in/x"] = ext
    out["ext/max"], out["ext/min"] = A(T(nt, ext).max(1)), A(T(nt, ext).min(1))
    # matmul with non-finite and huge operands
    a = rng.uniform(-1, 1, (6, 8)).astype(np.float32)
    b = rng.uniform(-1, 1, (8, 5)).astype(np.float32)
    a[0, 2], a[1, 3], a[2, 4] = np.inf, np.nan, -np.inf
    a[3, :] = 3.0e38 / 8            # finite, products near FLT_MAX
    a[4, 1] = 3.4e38                # rounds to infinity in TF32
    b[:, 4] = 0.25
    b[1, 2] = 0.0
    out["mmx/a"], out["mmx/b"] = a, b
    out["mmx/out"] = A(T(nt, a) @ T(nt, b))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("NT_REFERENCE", str(REPO.parent / "reference")),
                    help="path of the reference checkout (or set NT_REFERENCE)")
    args = ap.parse_args()
    nt = import_reference(Path(args.ref))
    out: dict[str, np.ndarray] = {}
    with np.errstate(all="ignore"):
        rng_cases(nt, out)
        elementwise_cases(nt, out)
        reduction_cases(nt, out)
        matmul_cases(nt, out)
        mlp_cases(nt, out)
        index_cases(nt, out)
    np.savez_compressed(HERE / "reference_cpu.npz", **out)
    size = (HERE / "reference_cpu.npz").stat().st_size
    print(f"wrote {len(out)} arrays, {size / 1024:.0f} KiB")
    extra: dict[str, np.ndarray] = {}
    with np.errstate(all="ignore"):
        extra_cases(nt, extra)
    np.savez_compressed(HERE / "reference_cpu_extra.npz", **extra)
    print(f"wrote {len(extra)} arrays, {(HERE / 'reference_cpu_extra.npz').stat().st_size / 1024:.0f} KiB")


if __name__ == "__main__":
    main()
