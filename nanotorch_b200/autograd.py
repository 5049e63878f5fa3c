"""Differentiable ops over the ``_C`` kernels, and the backward pass.

Same op classes, ``apply``/``forward``/``backward``/``save_for_backward``/``flops``/``mem_bytes``
protocol and results as the reference's ``nanotorch.autograd`` (src/nanotorch/autograd/*.py).
Differences, none of which changes a value:
  - ``backward`` receives ``self.needs_input_grad`` and skips gradients nobody asked for (the
    reference computes all of them, src/nanotorch/core.py:864-867);
  - for Float32 tensors on Cuda each backward is ONE fused kernel that performs the reference's
    chain of primitive kernels with the same per-step rounding (include/nt_b200.h); any other
    dtype takes the reference's composition of primitives;
  - Python scalars become device scalars by a fill kernel instead of a host->device copy, and
    PowOp never reads its exponent back from the device.
"""

from __future__ import annotations

import math
from typing import Any

from . import _C
from ._C import Device, Dtype
from .tensor import Shape, Tensor, broadcast_shapes, promote_dtypes, sizeof

_grad_enabled = True


def is_grad_enabled() -> bool:
    return _grad_enabled


class no_grad:
    """Context manager disabling graph recording (src/nanotorch/autograd/grad_mode.py:11-21)."""

    def __enter__(self):
        global _grad_enabled
        self._prev = _grad_enabled
        _grad_enabled = False

    def __exit__(self, exc_type, exc, tb):
        global _grad_enabled
        _grad_enabled = self._prev


def totensor(x, *, anchor: Tensor) -> Tensor:
    """Python scalars / lists become tensors on the anchor's device."""
    if isinstance(x, Tensor):
        return x
    if isinstance(x, (bool, int, float)) and anchor.device == Device.Cuda:
        dt = Dtype.Bool if isinstance(x, bool) else Dtype.Int64 if isinstance(x, int) else Dtype.Float32
        t = Tensor._scalar(x, dt, anchor.device)
        t._pyvalue = x
        return t
    return Tensor(x, device=anchor.device)


def _cast_operand(x: Tensor, dtype: Dtype) -> Tensor:
    """x.to(dtype); a scalar that still knows its Python value is re-filled at the target dtype."""
    if x.dtype == dtype:
        return x
    if x._pyvalue is not None and x.shape == () and x.device == Device.Cuda:
        return Tensor._scalar(x._pyvalue, dtype, x.device)
    return x.to(dtype)


def _fused(*tensors: Tensor) -> bool:
    return all(t.dtype == Dtype.Float32 and t.device == Device.Cuda for t in tensors)


def unbroadcast(x: Tensor, shape: Shape) -> Tensor:
    """Sum away broadcast axes so that the gradient has `shape` (autograd/ops_utils.py:7-17)."""
    lead = tuple(range(x.ndim - len(shape)))
    if lead:
        x = x.sum(axis=lead)
    trail = tuple(ax for ax in range(len(shape)) if x.shape[ax] != 1 and shape[ax] == 1)
    if trail:
        x = x.sum(axis=trail, keepdim=True)
    return x


def normalize_axes(axis, x: Tensor) -> Shape:
    """int | tuple | None -> tuple of non-negative, distinct axes (autograd/ops_utils.py:20-32)."""
    if isinstance(axis, int):
        axis = (axis,)
    if axis is None or len(axis) == 0:
        axis = tuple(range(x.ndim))
    if any(not isinstance(a, int) for a in axis):
        raise TypeError(f"Invalid axis: {axis}")
    axis = tuple(a + x.ndim if a < 0 else a for a in axis)
    if len(set(axis)) != len(axis):
        raise ValueError(f"Redundant axes: {axis}")
    if any(a < 0 or a >= x.ndim for a in axis):
        raise IndexError(f"Invalid axis: {axis}")
    return axis


class Function:
    """Base class of the differentiable ops (src/nanotorch/autograd/function.py:11-93)."""

    def __init__(self):
        self._inputs: Any = None
        self._inputs_kw: Any = None
        self._saved: tuple[tuple[Tensor, int], ...] | None = None
        self.needs_input_grad: tuple[bool, ...] = ()

    def __repr__(self) -> str:
        return f"[{type(self).__name__}]"

    @property
    def inputs(self):
        if self._inputs is None:
            raise RuntimeError("No inputs saved during apply().")
        return self._inputs

    @property
    def saved_tensors(self) -> tuple[Tensor, ...]:
        if self._saved is None:
            raise RuntimeError("No tensor was saved during forward.")
        for t, v in self._saved:
            if t.version != v:
                raise RuntimeError("One of the tensors needed for grad computation was modified inplace.")
        return tuple(t for t, _ in self._saved)

    def save_for_backward(self, *tensors: Tensor) -> None:
        if is_grad_enabled():
            self._saved = tuple((t, t.version) for t in tensors)

    @classmethod
    def apply(cls, *args, **kwargs) -> Tensor:
        self = cls()
        self._inputs = args
        self._inputs_kw = kwargs
        out = self.forward(*args, **kwargs)
        if is_grad_enabled():
            if any(out is a for a in list(args) + list(kwargs.values())):
                out = out._alias()
            self.needs_input_grad = tuple(isinstance(a, Tensor) and a.requires_grad for a in args)
            if any(self.needs_input_grad):
                out.attach_grad_fn(self)
        return out

    def forward(self, *inputs):
        raise NotImplementedError

    def backward(self, grad_out: Tensor):
        raise NotImplementedError

    @classmethod
    def flops(cls, *args, **kwargs) -> int:
        return 0

    @classmethod
    def mem_bytes(cls, *args, **kwargs) -> int:
        return 0


def _need(fn: Function, i: int) -> bool:
    return i >= len(fn.needs_input_grad) or fn.needs_input_grad[i]


# =============================================================================================
# binary
def _binary(x1: Tensor, x2: Tensor, op, op_inplace, out: Tensor | None) -> Tensor:
    """Promotion + broadcast-by-expand + `out=` handling (autograd/ops_binary.py:283-315)."""
    if out is not None:
        if out.is_leaf and out.requires_grad and is_grad_enabled():
            raise RuntimeError("A leaf variable that requires grad is being used in an in-place op.")
        dtype, shape = out.dtype, out.shape
    else:
        dtype = promote_dtypes(x1.dtype, x2.dtype)
        shape = broadcast_shapes(x1.shape, x2.shape)
    inplace = out is x1
    x1 = _cast_operand(x1, dtype).expand(*shape)
    x2 = _cast_operand(x2, dtype).expand(*shape)
    if out is None:
        return Tensor._new_contiguous(op(x1._C_view, x2._C_view), shape)
    if inplace:
        op_inplace(x1._C_view, x2._C_view)
        return x1
    result = Tensor._new_contiguous(op(x1._C_view, x2._C_view), shape)
    _C.copy_inplace(out._C_view, result._C_view)
    return result


class _BinaryOp(Function):
    @classmethod
    def flops(cls, x1, x2, _=None) -> int:
        return math.prod(broadcast_shapes(x1.shape, x2.shape))

    @classmethod
    def mem_bytes(cls, x1, x2, _=None) -> int:
        return 3 * math.prod(broadcast_shapes(x1.shape, x2.shape)) * sizeof(promote_dtypes(x1.dtype, x2.dtype))


def _negated(g: Tensor) -> Tensor:
    """-1 * g (bitwise the same as negation for every non-NaN float)."""
    if _fused(g):
        return Tensor._new_contiguous(_C.neg(g._C_view), g.shape)
    return -1 * g


class AddOp(_BinaryOp):
    def forward(self, x1, x2, out=None):
        self._shapes = (x1.shape, x2.shape)
        return _binary(x1, x2, _C.add, _C.add_inplace, out)

    def backward(self, g):
        return tuple(unbroadcast(g, s) if _need(self, i) else None for i, s in enumerate(self._shapes))


class SubOp(_BinaryOp):
    def forward(self, x1, x2, out=None):
        self._shapes = (x1.shape, x2.shape)
        return _binary(x1, x2, _C.subtract, _C.sub_inplace, out)

    def backward(self, g):
        s1, s2 = self._shapes
        return (unbroadcast(g, s1) if _need(self, 0) else None,
                unbroadcast(_negated(g), s2) if _need(self, 1) else None)


class MulOp(_BinaryOp):
    def forward(self, x1, x2, out=None):
        self.save_for_backward(x1, x2)
        return _binary(x1, x2, _C.multiply, _C.mul_inplace, out)

    def backward(self, g):
        x1, x2 = self.saved_tensors
        if _need(self, 0) and _need(self, 1) and _fused(g, x1, x2) and g.shape == x1.shape == x2.shape:
            both = _C.mul_backward(g._C_view, x1._C_view, x2._C_view)   # one pass when all three are dense
            if both is not None:
                return Tensor._new_contiguous(both[0], g.shape), Tensor._new_contiguous(both[1], g.shape)
        return (unbroadcast(x2 * g, x1.shape) if _need(self, 0) else None,
                unbroadcast(x1 * g, x2.shape) if _need(self, 1) else None)


class TrueDivOp(_BinaryOp):
    def forward(self, x1, x2, out=None):
        self.save_for_backward(x1, x2)
        return _binary(x1, x2, _C.divide, _C.div_inplace, out)

    def backward(self, g):
        x1, x2 = self.saved_tensors
        if _need(self, 0) and _need(self, 1) and _fused(g, x1, x2) and g.shape == x1.shape == x2.shape:
            both = _C.div_backward(g._C_view, x1._C_view, x2._C_view)
            if both is not None:
                return Tensor._new_contiguous(both[0], g.shape), Tensor._new_contiguous(both[1], g.shape)
        g1 = g2 = None
        if _need(self, 0):
            g1 = unbroadcast(g / x2, x1.shape)
        if _need(self, 1):
            if _fused(g, x1, x2):
                e1, e2 = x1.expand(*g.shape), x2.expand(*g.shape)
                full = Tensor._new_contiguous(_C.div_backward_x2(g._C_view, e1._C_view, e2._C_view), g.shape)
            else:
                full = -x1 / x2**2 * g
            g2 = unbroadcast(full, x2.shape)
        return g1, g2


def _matmul_shapes(s1: Shape, s2: Shape) -> tuple[Shape, Shape, Shape]:
    """1-D / 2-D / batched shape rules of matmul (autograd/ops_binary.py:318-343)."""
    if len(s1) == 0 or len(s2) == 0:
        raise RuntimeError("Scalar value encountered in matmul.")
    squeeze = []
    if len(s1) == 1:
        s1 = (1, *s1)
        squeeze.append(-2)
    if len(s2) == 1:
        s2 = (*s2, 1)
        squeeze.append(-1)
    if s1[-1] != s2[-2]:
        raise RuntimeError(f"Cannot multiply {s1} @ {s2}")
    batch = broadcast_shapes(s1[:-2], s2[:-2])
    raw = list(batch) + [s1[-2], s2[-1]]
    drop = {a + len(raw) for a in squeeze}
    return tuple(batch) + tuple(s1[-2:]), tuple(batch) + tuple(s2[-2:]), tuple(d for i, d in enumerate(raw) if i not in drop)


class MatmulOp(Function):
    def forward(self, x1, x2):
        self.save_for_backward(x1, x2)
        self._shape1, self._shape2, shape_out = _matmul_shapes(x1.shape, x2.shape)
        dtype = promote_dtypes(x1.dtype, x2.dtype)
        a = x1.to(dtype).expand(*self._shape1)
        b = x2
        if b.ndim == 1 and self._shape2[-2:] == (b.shape[0], 1):
            b = b.reshape(b.shape[0], 1)
        b = b.to(dtype).expand(*self._shape2)
        return Tensor._new_contiguous(_C.matmul(a._C_view, b._C_view), shape_out)

    def backward(self, g):
        x1, x2 = self.saved_tensors
        a = x1.expand(*self._shape1)
        b = x2
        if b.ndim == 1 and self._shape2[-2:] == (b.shape[0], 1):
            b = b.reshape(b.shape[0], 1)
        b_orig = b
        b = b.expand(*self._shape2)
        g = g.reshape(*broadcast_shapes(self._shape1[:-2], self._shape2[:-2]), self._shape1[-2], self._shape2[-1])
        g1 = g2 = None
        if (_need(self, 0) and _need(self, 1) and x1.ndim == 2 and x2.ndim == 2 and g.ndim == 2
                and x1.dtype == x2.dtype == g.dtype == Dtype.Float32 and x1.device == x2.device == Device.Cuda):
            # both gradients in one call: the second product starts on the SMs the first one's last wave leaves idle
            s1, s2 = _C.matmul_pair(g._C_view, x2.transpose(-2, -1)._C_view, x1.transpose(-2, -1)._C_view, g._C_view)
            return Tensor._new_contiguous(s1, x1.shape), Tensor._new_contiguous(s2, x2.shape)
        if _need(self, 0):
            g1 = unbroadcast(g @ b.transpose(-2, -1), x1.shape).reshape(*x1.shape)
        if _need(self, 1):
            # a 1-D right operand was rebound to its (k, 1) form above, and its gradient keeps that shape,
            # exactly as the reference returns it (autograd/ops_binary.py:253-267)
            g2 = unbroadcast(a.transpose(-2, -1) @ g, b_orig.shape).reshape(*b_orig.shape)
        return g1, g2

    @classmethod
    def flops(cls, x1, x2) -> int:
        s1, s2, _ = _matmul_shapes(x1.shape, x2.shape)
        return 2 * math.prod(s1[:-2]) * s1[-2] * s2[-1] * s1[-1]

    @classmethod
    def mem_bytes(cls, x1, x2) -> int:
        s1, s2, _ = _matmul_shapes(x1.shape, x2.shape)
        B, M, N, K = math.prod(s1[:-2]), s1[-2], s2[-1], s1[-1]
        return B * (M * K + K * N + M * N) * sizeof(promote_dtypes(x1.dtype, x2.dtype))


class LinearOp(Function):
    """x @ W + b for a 2-D fp32 x on the device, as one call: the bias add runs in the GEMM epilogue.

    Not a class of the reference (its Linear.forward composes MatmulOp and AddOp,
    src/nanotorch/nn/module.py:64-76); forward bits and all three gradients are those of the composed
    form: dX = g @ W^T, dW = x^T @ g (MatmulOp.backward), db = column sums of g (AddOp.backward's
    unbroadcast)."""

    @staticmethod
    def applicable(x, W, b) -> bool:
        return (x.ndim == 2 and W.ndim == 2 and b.ndim == 1 and b.shape[0] == W.shape[1]
                and x.dtype == W.dtype == b.dtype == Dtype.Float32
                and x.device == W.device == b.device == Device.Cuda and x.numel > 0 and W.numel > 0)

    def forward(self, x, W, b):
        self.save_for_backward(x, W)
        self._bias_shape = b.shape
        return Tensor._new_contiguous(_C.linear(x._C_view, W._C_view, b._C_view), (x.shape[0], W.shape[1]))

    def backward(self, g):
        x, W = self.saved_tensors
        if _need(self, 0) and _need(self, 1) and g.dtype == Dtype.Float32 and g.ndim == 2:
            # both products in one call: the second starts on the SMs the first one's last wave leaves idle
            sx, sW = _C.matmul_pair(g._C_view, W.transpose(-2, -1)._C_view, x.transpose(-2, -1)._C_view, g._C_view)
            gx, gW = Tensor._new_contiguous(sx, x.shape), Tensor._new_contiguous(sW, W.shape)
        else:
            gx = g @ W.transpose(-2, -1) if _need(self, 0) else None
            gW = x.transpose(-2, -1) @ g if _need(self, 1) else None
        gb = unbroadcast(g, self._bias_shape) if _need(self, 2) else None
        return gx, gW, gb

    @classmethod
    def flops(cls, x, W, b) -> int:
        return 2 * x.shape[0] * W.shape[1] * x.shape[1] + x.shape[0] * W.shape[1]

    @classmethod
    def mem_bytes(cls, x, W, b) -> int:
        return (x.numel + W.numel + b.numel + x.shape[0] * W.shape[1]) * 4


# =============================================================================================
# unary
class _UnaryOp(Function):
    @classmethod
    def flops(cls, x, *_) -> int:
        return x.numel

    @classmethod
    def mem_bytes(cls, x, *_) -> int:
        return 2 * x.numel * sizeof(x.dtype)


def _float_unary(fn: Function, x: Tensor, kernel, save_output: bool) -> Tensor:
    if x.is_empty:
        return x
    x = x.to(promote_dtypes(x.dtype, Dtype.Float32))
    y = Tensor._new_contiguous(kernel(x._C_view), x.shape)
    fn.save_for_backward(y if save_output else x)
    return y


def _bwd2(kernel, g: Tensor, saved: Tensor) -> Tensor:
    return Tensor._new_contiguous(kernel(g._C_view, saved._C_view), g.shape)


class NegOp(_UnaryOp):
    def forward(self, x):
        self._shape = x.shape
        return Tensor._new_contiguous(_C.neg(x._C_view), x.shape)

    def backward(self, g):
        return (unbroadcast(_negated(g), self._shape),)


class ExpOp(_UnaryOp):
    def forward(self, x):
        return _float_unary(self, x, _C.exp, save_output=True)

    def backward(self, g):
        (e,) = self.saved_tensors
        if _fused(g, e) and g.shape == e.shape:
            return (_bwd2(_C.exp_backward, g, e),)
        return (g * e,)


class LogOp(_UnaryOp):
    def forward(self, x):
        return _float_unary(self, x, _C.log, save_output=False)

    def backward(self, g):
        (x,) = self.saved_tensors
        if _fused(g, x) and g.shape == x.shape:
            return (_bwd2(_C.log_backward, g, x),)
        return (g * x**-1,)


class SqrtOp(_UnaryOp):
    def forward(self, x):
        return _float_unary(self, x, _C.sqrt, save_output=True)

    def backward(self, g):
        (r,) = self.saved_tensors
        if _fused(g, r) and g.shape == r.shape:
            return (_bwd2(_C.sqrt_backward, g, r),)
        return (g * 0.5 * r**-1,)


class TanhOp(_UnaryOp):
    def forward(self, x):
        return _float_unary(self, x, _C.tanh, save_output=True)

    def backward(self, g):
        (t,) = self.saved_tensors
        if _fused(g, t) and g.shape == t.shape:
            return (_bwd2(_C.tanh_backward, g, t),)
        return (g * (1 - t**2),)


class SigmoidOp(_UnaryOp):
    def forward(self, x):
        return _float_unary(self, x, _C.sigmoid, save_output=True)

    def backward(self, g):
        (s,) = self.saved_tensors
        if _fused(g, s) and g.shape == s.shape:
            return (_bwd2(_C.sigmoid_backward, g, s),)
        return (g * s * (1 - s),)


class ReluOp(_UnaryOp):
    def forward(self, x):
        y = Tensor._new_contiguous(_C.relu(x._C_view), x.shape)
        self.save_for_backward(y)
        return y

    def backward(self, g):
        (y,) = self.saved_tensors
        if _fused(g, y) and g.shape == y.shape:
            return (_bwd2(_C.relu_backward, g, y),)
        return (g * (y > totensor(0, anchor=y)),)


def _scalar_value(t: Tensor) -> float:
    if t._pyvalue is not None:
        return float(t._pyvalue)
    if t.numel != 1:
        raise RuntimeError(f"Cannot convert {t} to a scalar.")
    return float(t.cpu().item())  # device read-back only for exponents that were built as tensors


class PowOp(_UnaryOp):
    def forward(self, x, exponent):
        if x.is_empty:
            return x
        if not isinstance(exponent, Tensor):
            exponent = totensor(exponent, anchor=x)
        dtype = promote_dtypes(x.dtype, exponent.dtype)
        e = _scalar_value(exponent)
        if e < 0 and dtype <= Dtype.Int64:
            raise RuntimeError("Cannot use negative exponent with integer tensor.")
        self.save_for_backward(x, exponent)
        self._e = e
        return Tensor._new_contiguous(_C.pow(x.to(dtype)._C_view, e), x.shape)

    def backward(self, g):
        x, exponent = self.saved_tensors
        if _fused(g, x) and g.shape == x.shape and exponent.dtype <= Dtype.Float32:
            return (Tensor._new_contiguous(_C.pow_backward(g._C_view, x._C_view, self._e), g.shape),)
        return (g * exponent * x ** (exponent - 1),)


# =============================================================================================
# reductions
def _reduced_shapes(x: Tensor, axes: Shape, keepdim: bool) -> Shape:
    if keepdim:
        return tuple(1 if i in axes else s for i, s in enumerate(x.shape))
    return tuple(s for i, s in enumerate(x.shape) if i not in axes)


def _expand_back(g: Tensor, orig: Shape, axes: Shape) -> Tensor:
    """grad of a reduction as a stride-0 view of the original shape: no kernel, no bytes."""
    kept = tuple(1 if d in axes else orig[d] for d in range(len(orig)))
    return g.reshape(*kept).expand(*orig)


class _ReductionOp(Function):
    @classmethod
    def flops(cls, x, *a, **k) -> int:
        return x.numel

    @classmethod
    def mem_bytes(cls, x, *a, **k) -> int:
        return x.numel * sizeof(x.dtype)


class SumOp(_ReductionOp):
    def forward(self, x, axis=None, keepdim=False, dtype=None):
        self._axis = normalize_axes(axis, x)
        if dtype is None:
            dtype = max(x.dtype, Dtype.Int64)
        new_shape = _reduced_shapes(x, self._axis, keepdim)
        self._orig_shape = x.shape
        if x.is_empty:
            return Tensor._new_contiguous(_C.zeros(math.prod(new_shape), dtype, x.device), new_shape)
        return Tensor._new_contiguous(_C.sum(x._C_view, self._axis, dtype), new_shape)

    def backward(self, g):
        if not self._orig_shape:
            return (g,)
        return (_expand_back(g, self._orig_shape, self._axis),)


class MeanOp(_ReductionOp):
    def forward(self, x, axis=None, keepdim=False, dtype=None):
        if dtype is None:
            dtype = x.dtype
        if dtype < Dtype.Float32:
            raise TypeError("Cannot take mean of integer tensor, cast to fp.")
        self._axis = normalize_axes(axis, x)
        self._orig_shape = x.shape
        if _fused(x) and dtype == Dtype.Float32 and not x.is_empty:
            # sum and the true division by the count in one launch (same bits as the two steps below);
            # the count is exact in fp32 up to 2^24 elements per slice, beyond that the composed form runs
            new_shape = _reduced_shapes(x, self._axis, keepdim)
            denom = x.numel // max(1, math.prod(new_shape))
            if denom <= (1 << 24):
                fused = _C.mean_f32(x._C_view, self._axis, denom)
                if fused is not None:
                    self._denom = denom
                    return Tensor._new_contiguous(fused, new_shape)
        total = x.sum(axis=self._axis, keepdim=keepdim, dtype=dtype)
        self._denom = x.numel // total.numel
        return total / self._denom  # true division by the count, not a multiply by its reciprocal

    def backward(self, g):
        if not self._orig_shape:
            return (g,)
        # The reference divides the expanded gradient element by element (autograd/ops_reduction.py:129-137);
        # dividing the kept elements once and expanding the quotient (a stride-0 view, like Sum's
        # gradient) yields the same bits without a division and a write per input element.
        return (_expand_back(g / self._denom, self._orig_shape, self._axis),)


class _ExtremumOp(_ReductionOp):
    _kernel = None

    def forward(self, x, axis=None, keepdim=False):
        self._axis = normalize_axes(axis, x)
        new_shape = _reduced_shapes(x, self._axis, keepdim)
        self._orig_shape = x.shape
        if x.is_empty:
            if math.prod(new_shape) != 0:
                raise IndexError("argmin() expects reduction dim to be specified for numel=0.")
            return Tensor._new_contiguous(_C.zeros(0, x.dtype, x.device), new_shape)
        m = Tensor._new_contiguous(type(self)._kernel(x._C_view, self._axis), new_shape)
        self.save_for_backward(x, m)
        return m

    def backward(self, g):
        if not self._orig_shape:
            return (g,)
        x, m = self.saved_tensors
        m_full = _expand_back(m, self._orig_shape, self._axis)
        g_full = _expand_back(g, self._orig_shape, self._axis)
        if _fused(g, x, m):
            out = _C.extremum_backward(g_full._C_view, x._C_view, m_full._C_view, self._axis)
            return (Tensor._new_contiguous(out, self._orig_shape),)
        # The reference's mask arithmetic: Bool mask times the INTEGER quotient 1 // count, which is
        # 1 where the extremum is unique and 0 on every tied slice (autograd/ops_reduction.py:209-212).
        mask = x == m_full
        mask *= 1 / mask.sum(axis=self._axis, keepdim=True)
        return (g_full * mask,)


class MaxOp(_ExtremumOp):
    _kernel = staticmethod(_C.max)


class MinOp(_ExtremumOp):
    _kernel = staticmethod(_C.min)


# =============================================================================================
# view ops (no kernels unless a non-contiguous tensor is reshaped)
class ReshapeOp(Function):
    def forward(self, x, *dims):
        if math.prod(dims) != x.numel:
            raise ValueError(f"Can't reshape {x.shape} into {dims}.")
        self._shape = x.shape
        if dims == x.shape:
            return x
        x = x._to_contiguous()
        return Tensor._new_view(x.storage, tuple(dims), None, x._offset)

    def backward(self, g):
        return (g.reshape(*self._shape),)


class ExpandOp(Function):
    def forward(self, x, *dims):
        if len(dims) < x.ndim:
            raise ValueError(f"Cannot broadcast {x.shape} to {dims}.")
        self._orig_shape = x.shape
        if dims == x.shape:
            return x
        pad = len(dims) - x.ndim
        strides = [0] * pad + list(x._strides)
        for i in range(x.ndim):
            src, tgt = x.shape[i], dims[pad + i]
            if src == tgt:
                continue
            if src != 1:
                raise ValueError(f"Cannot broadcast {x.shape} to {dims} (mismatch).")
            strides[pad + i] = 0
        return Tensor._new_view(x.storage, tuple(dims), tuple(strides), x._offset)

    def backward(self, g):
        return (unbroadcast(g, self._orig_shape),)


class TOp(Function):
    def forward(self, x):
        if x.ndim < 2:
            return x
        return Tensor._new_view(x.storage, tuple(reversed(x.shape)), tuple(reversed(x._strides)), x._offset)

    def backward(self, g):
        return (g.T,)


class TransposeOp(Function):
    def forward(self, x, dim0, dim1):
        self._dims = (dim0, dim1)
        if x.ndim < 2 or dim0 == dim1:
            return x
        shape, strides = list(x.shape), list(x._strides)
        shape[dim0], shape[dim1] = shape[dim1], shape[dim0]
        strides[dim0], strides[dim1] = strides[dim1], strides[dim0]
        return Tensor._new_view(x.storage, tuple(shape), tuple(strides), x._offset)

    def backward(self, g):
        return (g.transpose(*self._dims),)


ALL_OPS_ = [AddOp, ExpOp, ExpandOp, LogOp, MatmulOp, MeanOp, MulOp, NegOp, PowOp, ReluOp, ReshapeOp, SigmoidOp,
            SqrtOp, SubOp, SumOp, TOp, TanhOp, TransposeOp, TrueDivOp, MinOp, MaxOp]


# =============================================================================================
# backward pass
# id(leaf tensor) -> callable(leaf): called ONCE per backward pass, right after the last contribution to
# that leaf's gradient has been added (a leaf used several times in the graph gets one call, with the
# summed gradient).  The data-parallel trainer starts the parameter's all-reduce from it while the
# rest of backward continues.
leaf_grad_hooks: dict[int, Any] = {}


def run_backward(root: Tensor) -> None:
    """Reverse-topological sweep from `root`, whose ``_grad`` holds the seed.

    Same contract as the reference's ``_backpropagate_grad`` (src/nanotorch/core.py:836-872): a node
    runs once every consumer has reported, leaf gradients accumulate, intermediate gradients are
    dropped as soon as they have been consumed.
    """
    order: list[Tensor] = []
    seen: set[int] = set()
    stack: list[tuple[Tensor, bool]] = [(root, False)]
    while stack:
        node, expanded = stack.pop()
        if expanded:
            order.append(node)
            continue
        if id(node) in seen or node.grad_fn is None:
            continue
        seen.add(id(node))
        stack.append((node, True))
        for inp in node.grad_fn.inputs:
            if isinstance(inp, Tensor) and inp.requires_grad and inp.grad_fn is not None and id(inp) not in seen:
                stack.append((inp, False))
    # contributions each hooked leaf is still to receive in this pass
    pending: dict[int, int] = {}
    if leaf_grad_hooks:
        for node in order:
            for a in node.grad_fn.inputs:
                if isinstance(a, Tensor) and a.requires_grad and a.grad_fn is None and id(a) in leaf_grad_hooks:
                    pending[id(a)] = pending.get(id(a), 0) + 1
    with no_grad():  # gradients are values, not graph nodes
        for node in reversed(order):
            fn = node.grad_fn
            if node._grad is None:
                raise RuntimeError("f_x.grad is None.")
            tensor_inputs = [a for a in fn.inputs if isinstance(a, Tensor)]
            grads = fn.backward(node._grad)
            for x, gx in zip(tensor_inputs, grads):
                if not x.requires_grad:
                    continue
                if gx is not None:
                    x._grad = gx if x._grad is None else x._grad + gx
                left = pending.get(id(x))
                if left is not None and x.grad_fn is None:
                    pending[id(x)] = left - 1
                    if left == 1 and x._grad is not None:
                        leaf_grad_hooks[id(x)](x)
            node._grad = None
