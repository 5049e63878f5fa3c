"""Numpy-level access to the two checkers.  TEST INFRASTRUCTURE ONLY.

``PortOracle``  the C restatement in oracle/nt_oracle.c (built into oracle/libnt_oracle.so).
``RefOracle``   the reference's own native module, compiled from the reference checkout into
                oracle/_ref/ by oracle/Makefile and loaded as a bare extension module (its CPU
                path; nothing of the reference's Python package is needed or copied).

Both expose the same primitives on numpy float32 arrays -- arbitrary views allowed: broadcast
(stride 0), transposed, sliced, negative strides -- so that the op-level chains below (the exact
primitive sequences of the reference's Python ``backward`` methods and of one MLP training step)
can be replayed on either.  Only tests/, the smoke check and the benchmark's cpu_baseline /
--impl reference legs may import this module; the product never does.
"""

from __future__ import annotations

import ctypes as C
import importlib.util
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
PORT_LIB = HERE / "libnt_oracle.so"
REF_DIR = HERE / "_ref"

MAX_DIMS = 8


class _View(C.Structure):
    _fields_ = [("ndim", C.c_int32), ("shape", C.c_int64 * MAX_DIMS), ("strides", C.c_int64 * MAX_DIMS),
                ("offset", C.c_int64)]


class _IndexArray(C.Structure):
    _fields_ = [("data", C.c_void_p), ("view", _View)]


def build_port(force: bool = False) -> Path:
    """Compile oracle/nt_oracle.c (gcc, seconds)."""
    src = HERE / "nt_oracle.c"
    if force or not PORT_LIB.exists() or PORT_LIB.stat().st_mtime < src.stat().st_mtime:
        subprocess.run(["gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fno-fast-math", "-ffp-contract=off",
                        "-o", str(PORT_LIB), str(src), "-lm"], check=True)
    return PORT_LIB


def _base_and_view(a: np.ndarray, dtype=np.float32):
    """(flat array owning the memory, element strides, element offset) of any numpy view of `dtype`."""
    assert a.dtype == dtype
    root = a
    while isinstance(root.base, np.ndarray):
        root = root.base
    if not root.flags["C_CONTIGUOUS"] or root.dtype != dtype:
        a = np.ascontiguousarray(a)
        root = a
    flat = root.reshape(-1)
    item = a.itemsize
    offset = (a.__array_interface__["data"][0] - flat.__array_interface__["data"][0]) // item if a.size else 0
    strides = tuple(s // item for s in a.strides)
    return flat, strides, int(offset)


BINARY = {"add": 0, "subtract": 1, "multiply": 2, "divide": 3}
COMPARE = {"pw_equal": 4, "pw_greater": 5, "pw_greater_eq": 6}
INPLACE = {"add": 0, "sub": 1, "mul": 2, "div": 3, "copy": 7}
UNARY = {"exp": 0, "log": 1, "neg": 2, "relu": 3, "sqrt": 4, "tanh": 5, "sigmoid": 6, "pow": 7}
REDUCE = {"sum": 0, "max": 1, "min": 2, "argmax": 3, "argmin": 4}


class PortOracle:
    """oracle/nt_oracle.c through ctypes."""

    kind = "port"

    def __init__(self):
        self.lib = C.CDLL(str(build_port()))

    @staticmethod
    def _cv(a: np.ndarray):
        flat, strides, offset = _base_and_view(a)
        v = _View()
        v.ndim = a.ndim
        for i in range(a.ndim):
            v.shape[i] = a.shape[i]
            v.strides[i] = strides[i]
        v.offset = offset
        return flat, v

    def binary(self, name: str, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        a, b = np.broadcast_arrays(a, b) if a.shape != b.shape else (a, b)
        fa, va = self._cv(a)
        fb, vb = self._cv(b)
        if name in BINARY:
            out = np.empty(a.shape, np.float32)
            rc = self.lib.nto_binary_f32(BINARY[name], fa.ctypes.data_as(C.c_void_p), C.byref(va),
                                         fb.ctypes.data_as(C.c_void_p), C.byref(vb), out.ctypes.data_as(C.c_void_p))
        else:
            out = np.empty(a.shape, np.bool_)
            rc = self.lib.nto_compare_f32(COMPARE[name], fa.ctypes.data_as(C.c_void_p), C.byref(va),
                                          fb.ctypes.data_as(C.c_void_p), C.byref(vb), out.ctypes.data_as(C.c_void_p))
        assert rc == 0
        return out

    def unary(self, name: str, x: np.ndarray, exponent: float = 0.0) -> np.ndarray:
        fx, vx = self._cv(x)
        out = np.empty(x.shape, np.float32)
        rc = self.lib.nto_unary_f32(UNARY[name], fx.ctypes.data_as(C.c_void_p), C.byref(vx),
                                    out.ctypes.data_as(C.c_void_p), C.c_double(exponent))
        assert rc == 0
        return out

    def reduce(self, name: str, x: np.ndarray, axes) -> np.ndarray:
        axes = [a % x.ndim for a in axes]
        fx, vx = self._cv(x)
        keep_shape = tuple(s for i, s in enumerate(x.shape) if i not in axes)
        n_keep = int(np.prod(keep_shape, dtype=np.int64))
        vals = np.empty(n_keep, np.float32)
        idx = np.empty(n_keep, np.int64)
        arr = (C.c_int64 * len(axes))(*axes)
        rc = self.lib.nto_reduce_f32(REDUCE[name], fx.ctypes.data_as(C.c_void_p), C.byref(vx), arr, len(axes),
                                     vals.ctypes.data_as(C.c_void_p), idx.ctypes.data_as(C.c_void_p))
        assert rc == 0
        return (idx if name.startswith("arg") else vals).reshape(keep_shape)

    def matmul(self, a: np.ndarray, b: np.ndarray) -> np.ndarray:
        fa, va = self._cv(a)
        fb, vb = self._cv(b)
        out = np.empty(a.shape[:-1] + (b.shape[-1],), np.float32)
        rc = self.lib.nto_matmul_f32(fa.ctypes.data_as(C.c_void_p), C.byref(va), fb.ctypes.data_as(C.c_void_p),
                                     C.byref(vb), out.ctypes.data_as(C.c_void_p))
        assert rc == 0
        return out

    def inplace(self, name: str, out: np.ndarray, other: np.ndarray) -> None:
        other = np.broadcast_to(other, out.shape)
        fo, vo = self._cv(out)
        fx, vx = self._cv(other)
        rc = self.lib.nto_inplace_f32(INPLACE[name], fo.ctypes.data_as(C.c_void_p), C.byref(vo),
                                      fx.ctypes.data_as(C.c_void_p), C.byref(vx))
        assert rc == 0

    def clone(self, x: np.ndarray) -> np.ndarray:
        fx, vx = self._cv(x)
        out = np.empty(x.shape, np.float32)
        self.lib.nto_clone_f32(fx.ctypes.data_as(C.c_void_p), C.byref(vx), out.ctypes.data_as(C.c_void_p))
        return out

    # index-array gather/scatter on arrays of any supported dtype; `plan` is a FancyPlan (below)
    def _index_args(self, plan):
        arrays = (_IndexArray * max(len(plan.fancy_dims_data), 1))()
        keep = []
        for i, ind in enumerate(plan.fancy_dims_data):
            flat, strides, offset = _base_and_view(ind, np.int64)
            keep.append(flat)
            arrays[i].data = flat.ctypes.data
            arrays[i].view.ndim = ind.ndim
            for d in range(ind.ndim):
                arrays[i].view.shape[d] = ind.shape[d]
                arrays[i].view.strides[d] = strides[d]
            arrays[i].view.offset = offset
        dims = (C.c_int64 * 8)(*plan.fancy_dims_in_src)
        is_fancy = (C.c_uint8 * 8)(*[int(f) for f in plan.out_axis_is_fancy])
        target = (C.c_int64 * 8)(*plan.out_axis_target)
        return arrays, keep, dims, is_fancy, target

    @staticmethod
    def _cv_any(a: np.ndarray):
        flat, strides, offset = _base_and_view(a, a.dtype)
        v = _View()
        v.ndim = a.ndim
        for i in range(a.ndim):
            v.shape[i] = a.shape[i]
            v.strides[i] = strides[i]
        v.offset = offset
        return flat, v

    def gather_from_axes(self, x: np.ndarray, plan) -> np.ndarray:
        fx, vx = self._cv_any(x)
        out = np.empty(plan.new_shape, x.dtype)
        _, vo = self._cv_any(out)
        arrays, keep, dims, is_fancy, target = self._index_args(plan)
        self.lib.nto_gather_from_axes(C.c_int(x.itemsize), fx.ctypes.data_as(C.c_void_p), C.byref(vx),
                                      out.ctypes.data_as(C.c_void_p), C.byref(vo), dims,
                                      C.c_int(len(plan.fancy_dims_in_src)), arrays, is_fancy, target)
        return out

    def scatter_to_axes(self, src: np.ndarray, out: np.ndarray, plan) -> None:
        """Writes through `out` (any writable view) in place."""
        assert src.dtype == out.dtype and src.shape == tuple(plan.new_shape)
        fs, vs = self._cv_any(src)
        fo, vo = self._cv_any(out)
        assert np.shares_memory(fo, out), "scatter target must be a view of a C-contiguous array"
        arrays, keep, dims, is_fancy, target = self._index_args(plan)
        self.lib.nto_scatter_to_axes(C.c_int(src.itemsize), fs.ctypes.data_as(C.c_void_p), C.byref(vs),
                                     fo.ctypes.data_as(C.c_void_p), C.byref(vo), dims,
                                     C.c_int(len(plan.fancy_dims_in_src)), arrays, is_fancy, target)

    def philox(self, ctr, key) -> list[int]:
        out = (C.c_uint32 * 4)()
        self.lib.nto_philox4x32_10((C.c_uint32 * 4)(*ctr), (C.c_uint32 * 2)(*key), out)
        return list(out)

    def philox_uniform(self, seed: int, offset: int, n: int, dtype=np.float32) -> np.ndarray:
        out = np.empty(n, dtype)
        fn = self.lib.nto_philox_uniform_f32 if dtype == np.float32 else self.lib.nto_philox_uniform_f64
        fn(C.c_uint64(seed), C.c_uint64(offset), out.ctypes.data_as(C.c_void_p), C.c_int64(n))
        return out

    def uniform(self, seed: int, n: int) -> np.ndarray:
        self.lib.nto_rng_sizeof.restype = C.c_int64
        state = C.create_string_buffer(self.lib.nto_rng_sizeof())
        self.lib.nto_rng_seed(state, C.c_uint64(seed))
        out = np.empty(n, np.float32)
        self.lib.nto_uniform_f32(state, out.ctypes.data_as(C.c_void_p), C.c_int64(n))
        return out


def ref_available() -> bool:
    return any(REF_DIR.glob("_C*.so"))


def load_ref_module():
    """Import oracle/_ref/_C*.so as a bare module named `_C` (the reference's PYBIND11_MODULE name)."""
    so = next(REF_DIR.glob("_C*.so"))
    if "_nt_ref_C" in sys.modules:
        return sys.modules["_nt_ref_C"]
    spec = importlib.util.spec_from_file_location("_C", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules["_nt_ref_C"] = mod
    return mod


class RefOracle:
    """The reference's native module on its CPU path (src/cpp/_C.cpp:12-24)."""

    kind = "reference"

    def __init__(self):
        self.m = load_ref_module()
        self.F32 = self.m.Dtype.Float32
        self.CPU = self.m.Device.Cpu

    def _tv(self, a: np.ndarray):
        flat, strides, offset = _base_and_view(a)
        s = self.m.Storage.allocate(max(flat.size, 1), self.F32, self.CPU)
        if flat.size:
            np.asarray(memoryview(s))[: flat.size] = flat
        return self.m.TensorView(s, list(a.shape), list(strides), offset), s

    @staticmethod
    def _out(storage, shape, dtype=np.float32):
        return np.array(np.asarray(memoryview(storage)), dtype=dtype, copy=True).reshape(shape)

    def binary(self, name, a, b):
        a, b = np.broadcast_arrays(a, b) if a.shape != b.shape else (a, b)
        (va, _), (vb, _) = self._tv(a), self._tv(b)
        out = getattr(self.m, name)(va, vb)
        return self._out(out, a.shape, np.bool_ if name in COMPARE else np.float32)

    def unary(self, name, x, exponent: float = 0.0):
        vx, _ = self._tv(x)
        out = self.m.pow(vx, float(exponent)) if name == "pow" else getattr(self.m, name)(vx)
        return self._out(out, x.shape)

    def reduce(self, name, x, axes):
        axes = [a % x.ndim for a in axes]
        vx, _ = self._tv(x)
        keep_shape = tuple(s for i, s in enumerate(x.shape) if i not in axes)
        if name == "sum":
            out = self.m.sum(vx, axes, self.F32)
        else:
            out = getattr(self.m, name)(vx, axes)
        return self._out(out, keep_shape, np.int64 if name.startswith("arg") else np.float32)

    def matmul(self, a, b):
        (va, _), (vb, _) = self._tv(a), self._tv(b)
        return self._out(self.m.matmul(va, vb), a.shape[:-1] + (b.shape[-1],))

    def inplace(self, name, out, other):
        other = np.broadcast_to(other, out.shape)
        vo, so = self._tv(out)
        vx, _ = self._tv(other)
        getattr(self.m, name + "_inplace")(vo, vx)
        flat, _, _ = _base_and_view(out)
        flat[:] = np.asarray(memoryview(so))[: flat.size]

    def clone(self, x):
        vx, _ = self._tv(x)
        return self._out(self.m.clone_contiguous_view_from(vx), x.shape)

    def _tv_any(self, a: np.ndarray):
        dt = {np.dtype(np.bool_): self.m.Dtype.Bool, np.dtype(np.int32): self.m.Dtype.Int32,
              np.dtype(np.int64): self.m.Dtype.Int64, np.dtype(np.float32): self.F32,
              np.dtype(np.float64): self.m.Dtype.Float64}[a.dtype]
        flat, strides, offset = _base_and_view(a, a.dtype)
        s = self.m.Storage.allocate(max(flat.size, 1), dt, self.CPU)
        if flat.size:
            np.asarray(memoryview(s))[: flat.size] = flat
        return self.m.TensorView(s, list(a.shape), list(strides), offset), s, flat

    def gather_from_axes(self, x, plan):
        vx, _, _ = self._tv_any(x)
        out = self.m.gather_from_axes(
            x=vx, new_shape=list(plan.new_shape), fancy_dims_in_src=list(plan.fancy_dims_in_src),
            fancy_dims_data=[self._tv_any(i)[0] for i in plan.fancy_dims_data],
            out_axis_is_fancy=list(plan.out_axis_is_fancy), out_axis_target=list(plan.out_axis_target))
        return self._out(out, plan.new_shape, x.dtype)

    def scatter_to_axes(self, src, out, plan):
        vs, _, _ = self._tv_any(src)
        vo, so, flat = self._tv_any(out)
        self.m.scatter_to_axes(
            src=vs, out=vo, fancy_dims_in_src=list(plan.fancy_dims_in_src),
            fancy_dims_data=[self._tv_any(i)[0] for i in plan.fancy_dims_data],
            out_axis_is_fancy=list(plan.out_axis_is_fancy), out_axis_target=list(plan.out_axis_target))
        flat[:] = np.asarray(memoryview(so))[: flat.size]

    def uniform(self, seed, n):
        self.m.manual_seed(seed)
        return self._out(self.m.uniform(n, self.F32, self.CPU), (n,))


# =============================================================================================
# Op-level chains: the primitive sequences of the reference's Python layer, one rounded kernel per
# step.  `o` is either oracle.  Scalars are 0-d fp32 arrays expanded with stride 0, as the
# reference's `Tensor(scalar).to(float32).expand(...)` makes them.
def _s(value, like: np.ndarray) -> np.ndarray:
    return np.broadcast_to(np.float32(value), like.shape)


def relu_backward(o, g, y):      # autograd/ops_unary.py:287-289   g * float(y > 0)
    mask = o.binary("pw_greater", y, _s(0.0, y)).astype(np.float32)
    return o.binary("multiply", g, mask)


def tanh_backward(o, g, t):      # autograd/ops_unary.py:180-182   g * (1 - t**2)
    return o.binary("multiply", g, o.binary("subtract", _s(1.0, t), o.unary("pow", t, 2.0)))


def sigmoid_backward(o, g, s):   # autograd/ops_unary.py:218-220   (g * s) * (1 - s)
    return o.binary("multiply", o.binary("multiply", g, s), o.binary("subtract", _s(1.0, s), s))


def exp_backward(o, g, e):       # autograd/ops_unary.py:69-70
    return o.binary("multiply", g, e)


def log_backward(o, g, x):       # autograd/ops_unary.py:105-106   g * x**-1
    return o.binary("multiply", g, o.unary("pow", x, -1.0))


def sqrt_backward(o, g, r):      # autograd/ops_unary.py:142-144   (g * 0.5) * r**-1
    return o.binary("multiply", o.binary("multiply", g, _s(0.5, g)), o.unary("pow", r, -1.0))


def pow_backward(o, g, x, e):    # autograd/ops_unary.py:264-266   (g * e) * x**(e - 1)
    em1 = float(np.float32(e) - np.float32(1.0))
    return o.binary("multiply", o.binary("multiply", g, _s(e, g)), o.unary("pow", x, em1))


def div_backward_x2(o, g, x1, x2):  # autograd/ops_binary.py:197-202   ((-x1) / x2**2) * g
    return o.binary("multiply", o.binary("divide", o.unary("neg", x1), o.unary("pow", x2, 2.0)), g)


def mean_forward(o, x, axes):    # autograd/ops_reduction.py:112-127   sum / float(count)
    total = o.reduce("sum", x, axes)
    count = x.size // max(total.size, 1)
    return o.binary("divide", total, _s(float(count), total))


def extremum_backward(o, g_full, x, m_full, axes):  # autograd/ops_reduction.py:201-212
    mask = o.binary("pw_equal", x, m_full)
    count = mask.sum(axis=tuple(axes), keepdims=True)            # Int64 sum of a Bool mask: exact
    unique = (1 // count).astype(np.bool_)                       # INTEGER division, then Bool
    maskf = np.logical_and(mask, np.broadcast_to(unique, mask.shape)).astype(np.float32)
    return o.binary("multiply", g_full, maskf)


def sgd_update(o, p, g, lr):     # nn/optimizers.py:45-51   p -= g * lr
    o.inplace("sub", p, o.binary("multiply", g, _s(lr, g)))


def kaiming(o, seed_stream: np.ndarray, fan_in: int, fan_out: int) -> np.ndarray:
    """2 * U * z - z (nn/module.py:118-125) on `fan_in*fan_out` draws of the seeded stream."""
    z = float(np.sqrt(6 / fan_in))
    u = seed_stream.reshape(fan_in, fan_out)
    return o.binary("subtract", o.binary("multiply", o.binary("multiply", _s(2.0, u), u), _s(z, u)), _s(z, u))


def mlp_step(o, params, X, Y, lr, activation: str, compute_input_grad: bool = False):
    """One SGD step of Sequential(Linear, act, ..., Linear) with loss mean((pred - Y)**2).

    `params` = [(W, b), ...] float32 arrays, updated in place.  Replays the reference's call order
    (src/nanotorch/nn/module.py:64-76, scripts/train_mlp_basic.py:49-53, core.py:836-872).
    Returns the loss as a Python float.
    """
    acts, zs = [X], []
    h = X
    for li, (W, b) in enumerate(params):
        z = o.binary("add", o.matmul(h, W), np.broadcast_to(b, (h.shape[0], b.shape[0])))
        zs.append(z)
        if li < len(params) - 1:
            h = o.unary(activation, z)
        else:
            h = z
        acts.append(h)
    pred = acts[-1]
    diff = o.binary("subtract", pred, Y)
    sq = o.unary("pow", diff, 2.0)
    loss = mean_forward(o, sq, list(range(sq.ndim)))
    # backward: mean -> pow -> sub
    g = o.binary("divide", _s(1.0, sq), _s(float(sq.size), sq))
    g = pow_backward(o, g, diff, 2.0)
    grads = []
    for li in reversed(range(len(params))):
        W, b = params[li]
        h_in = acts[li]
        gb = o.reduce("sum", g, [0])
        gW = o.matmul(h_in.T, g)
        grads.append((gW, gb))
        if li > 0 or compute_input_grad:
            gh = o.matmul(g, W.T)
            if li > 0:
                g = relu_backward(o, gh, acts[li]) if activation == "relu" else tanh_backward(o, gh, acts[li])
    grads.reverse()
    for (W, b), (gW, gb) in zip(params, grads):
        sgd_update(o, W, gW, lr)
        sgd_update(o, b, gb, lr)
    return float(loss.reshape(-1)[0])


# =============================================================================================
# Index-array / mask indexing as the reference's Python layer plans it.
class FancyPlan:
    """new_shape, fancy_dims_in_src, fancy_dims_data (broadcast int64 arrays), out_axis_is_fancy,
    out_axis_target -- the fields of the reference's _FancyAxes (src/nanotorch/core.py:666-675)."""


def fancy_plan(shape, index) -> FancyPlan:
    """src/nanotorch/core.py:677-772.  `index` has one entry per dim of `shape` (shorter = trailing
    dims basic): None for a basic dim, else a list / bool mask / integer array for that dim."""
    fancy_dims, basic_axes, basic_shape, raw = [], [], [], []
    for dim, extent in enumerate(shape):
        sel = index[dim] if dim < len(index) else None
        if sel is None:
            basic_axes.append(dim)
            basic_shape.append(extent)
            continue
        arr = np.asarray(sel)
        if arr.dtype == np.bool_:                              # :720-728
            if arr.ndim > 1:
                raise NotImplementedError("nD boolean masks not here (yet).")
            if arr.shape[0] != extent:
                raise IndexError(f"Wrong boolean index shape: {arr.shape[0]} (expected {extent}).")
            arr = np.flatnonzero(arr)
        else:                                                  # :712-718: wrap, then range check
            arr = arr.astype(np.int64)
            arr = np.where(arr < 0, arr + extent, arr)
            bad = arr[(arr < 0) | (arr >= extent)]
            if bad.size:
                raise IndexError(f"Invalid index {int(bad.reshape(-1)[0])} in axis of len {extent}.")
        fancy_dims.append(dim)
        raw.append(arr.astype(np.int64))
    ind_shape = np.broadcast_shapes(*(a.shape for a in raw))
    plan = FancyPlan()
    plan.fancy_dims_in_src = fancy_dims
    plan.fancy_dims_data = [np.broadcast_to(a, ind_shape) for a in raw]   # expand = stride 0, :734
    nidx = len(ind_shape)
    scattered = any(b - a != 1 for a, b in zip(fancy_dims, fancy_dims[1:]))  # :739-745
    plan.out_axis_is_fancy, plan.out_axis_target = [], []
    if scattered:
        plan.new_shape = tuple(ind_shape) + tuple(basic_shape)
        for i in range(len(plan.new_shape)):
            plan.out_axis_is_fancy.append(i < nidx)
            plan.out_axis_target.append(i if i < nidx else basic_axes[i - nidx])
    else:
        a0 = fancy_dims[0]
        plan.new_shape = tuple(basic_shape[:a0]) + tuple(ind_shape) + tuple(basic_shape[a0:])
        for i in range(len(plan.new_shape)):
            inside = a0 <= i < a0 + nidx
            plan.out_axis_is_fancy.append(inside)
            plan.out_axis_target.append(i - a0 if inside else basic_axes[i if i < a0 else i - nidx])
    return plan


def _split_index(index, ndim):
    """(numpy basic index with full slices at the index-array positions, residual per view dim)."""
    if not isinstance(index, tuple):
        index = (index,)
    if any(sel is Ellipsis for sel in index):                  # expand_ellipsis, _indexing.py:29-51
        n_real = sum(1 for sel in index if sel is not None and sel is not Ellipsis)
        at = next(i for i, sel in enumerate(index) if sel is Ellipsis)
        index = index[:at] + (slice(None),) * (ndim - n_real) + index[at + 1:]
    basic, residual = [], []
    for sel in index:
        if sel is None:
            basic.append(None)
            residual.append(None)
        elif isinstance(sel, (int, np.integer)) and not isinstance(sel, (bool, np.bool_)):
            basic.append(int(sel))
        elif isinstance(sel, slice):
            basic.append(sel)
            residual.append(None)
        else:
            basic.append(slice(None))
            residual.append(sel)
    return tuple(basic), residual


def getitem(o, x: np.ndarray, index) -> np.ndarray:
    """Tensor.__getitem__ with at least one index-array selector (src/nanotorch/core.py:172-203)."""
    basic, residual = _split_index(index, x.ndim)
    view = x[basic]
    return o.gather_from_axes(view, fancy_plan(view.shape, residual))


def setitem(o, x: np.ndarray, index, value: np.ndarray) -> None:
    """Tensor.__setitem__ with index arrays (src/nanotorch/core.py:205-254), writing through the
    basic-indexed view (what the reference does whenever its basic selectors are full slices)."""
    basic, residual = _split_index(index, x.ndim)
    view = x[basic]
    plan = fancy_plan(view.shape, residual)
    o.scatter_to_axes(np.broadcast_to(np.asarray(value, dtype=x.dtype), plan.new_shape), view, plan)
