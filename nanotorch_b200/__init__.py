"""nanotorch op-kernel hot path on B200: Tensor/autograd API over hand-written sm_100a kernels.

Mirrors the public surface of the reference package for this path (src/nanotorch/__init__.py):
``Tensor``, dtypes, ``no_grad``, functional ops, factories, ``manual_seed``; operators are bound
onto ``Tensor`` here exactly as the reference binds them at import (src/nanotorch/__init__.py:124-177).
"""

from . import _C
from ._C import Device, Dtype
from .autograd import (ALL_OPS_, AddOp, ExpandOp, ExpOp, Function, LogOp, MatmulOp, MaxOp, MeanOp, MinOp, MulOp,
                       NegOp, PowOp, ReluOp, ReshapeOp, SigmoidOp, SqrtOp, SubOp, SumOp, TanhOp, TOp, TransposeOp,
                       TrueDivOp, no_grad, totensor)
from .tensor import Tensor, TensorLike, broadcast_shapes, promote_dtypes, sizeof
from . import cuda  # noqa: E402  (nt.cuda.is_available(), nt.cuda.sync(), as in the reference)

bool_ = Dtype.Bool
int32 = Dtype.Int32
int64 = Dtype.Int64
float32 = Dtype.Float32
float64 = Dtype.Float64


def is_available() -> bool:
    """True when a CUDA device is usable (src/nanotorch/cuda.py:12-14)."""
    return _C.is_cuda_available()


def sync() -> None:
    """Wait for every kernel enqueued so far (src/nanotorch/cuda.py:17-19)."""
    _C.cuda_sync()


def manual_seed(seed: int) -> None:
    """Seed the host generator behind ``rand`` (src/nanotorch/__init__.py:112-115)."""
    _C.manual_seed(seed)


# ---- operator binding
def _t(other, self):
    return totensor(other, anchor=self)


Tensor.__add__ = lambda self, other: AddOp.apply(self, _t(other, self))
Tensor.__radd__ = lambda self, other: AddOp.apply(self, _t(other, self))
Tensor.__iadd__ = lambda self, other: AddOp.apply(self, _t(other, self), out=self)
Tensor.__mul__ = lambda self, other: MulOp.apply(self, _t(other, self))
Tensor.__rmul__ = lambda self, other: MulOp.apply(self, _t(other, self))
Tensor.__imul__ = lambda self, other: MulOp.apply(self, _t(other, self), out=self)
Tensor.__sub__ = lambda self, other: SubOp.apply(self, _t(other, self))
Tensor.__rsub__ = lambda self, other: SubOp.apply(_t(other, self), self)
Tensor.__isub__ = lambda self, other: SubOp.apply(self, _t(other, self), out=self)
Tensor.__truediv__ = lambda self, other: TrueDivOp.apply(self, _t(other, self))
Tensor.__rtruediv__ = lambda self, other: TrueDivOp.apply(_t(other, self), self)
Tensor.__itruediv__ = lambda self, other: TrueDivOp.apply(self, _t(other, self), out=self)
Tensor.__neg__ = lambda self: NegOp.apply(self)
Tensor.__matmul__ = lambda self, other: MatmulOp.apply(self, _t(other, self))
Tensor.__pow__ = lambda self, exponent: PowOp.apply(self, _t(exponent, self))
Tensor.__rpow__ = lambda self, base: PowOp.apply(_t(base, self), self)


def _compare(kernel):
    def op(x1: Tensor, x2: Tensor) -> Tensor:
        dtype = promote_dtypes(x1.dtype, x2.dtype)
        shape = broadcast_shapes(x1.shape, x2.shape)
        a = x1.to(dtype).expand(*shape)
        b = x2.to(dtype).expand(*shape)
        return Tensor._new_contiguous(kernel(a._C_view, b._C_view), shape)

    return op


equal_op_ = _compare(_C.pw_equal)
greater_op_ = _compare(_C.pw_greater)
greater_eq_op_ = _compare(_C.pw_greater_eq)
Tensor.__eq__ = lambda self, other: equal_op_(self, _t(other, self))
Tensor.__gt__ = lambda self, other: greater_op_(self, _t(other, self))
Tensor.__ge__ = lambda self, other: greater_eq_op_(self, _t(other, self))
Tensor.__lt__ = lambda self, other: _t(other, self) > self
Tensor.__le__ = lambda self, other: _t(other, self) >= self
Tensor.exp = lambda self: ExpOp.apply(self)
Tensor.log = lambda self: LogOp.apply(self)
Tensor.sqrt = lambda self: SqrtOp.apply(self)
Tensor.tanh = lambda self: TanhOp.apply(self)
Tensor.sigmoid = lambda self: SigmoidOp.apply(self)
Tensor.relu = lambda self: ReluOp.apply(self)
Tensor.pow = lambda self, exponent: PowOp.apply(self, exponent)
Tensor.sum = lambda self, axis=None, keepdim=False, dtype=None: SumOp.apply(self, axis, keepdim, dtype)
Tensor.mean = lambda self, axis=None, keepdim=False, dtype=None: MeanOp.apply(self, axis, keepdim, dtype)
Tensor.max = lambda self, axis=None, keepdim=False: MaxOp.apply(self, axis, keepdim)
Tensor.min = lambda self, axis=None, keepdim=False: MinOp.apply(self, axis, keepdim)
Tensor.reshape = lambda self, *dims: ReshapeOp.apply(self, *dims)
Tensor.expand = lambda self, *dims: ExpandOp.apply(self, *dims)
Tensor.transpose = lambda self, dim0, dim1: TransposeOp.apply(self, dim0, dim1)


# ---- functional forms (src/nanotorch/ops.py)
# The reference's forms are the Python operators (`x + y`, src/nanotorch/ops.py:42-60), so a scalar may
# stand on either side; `out=` is an addition that forwards to the op's in-place form.
def add(x1, x2, out=None): return x1 + x2 if out is None else AddOp.apply(x1, _t(x2, x1), out=out)
def subtract(x1, x2, out=None): return x1 - x2 if out is None else SubOp.apply(x1, _t(x2, x1), out=out)
def multiply(x1, x2, out=None): return x1 * x2 if out is None else MulOp.apply(x1, _t(x2, x1), out=out)
def divide(x1, x2, out=None): return x1 / x2 if out is None else TrueDivOp.apply(x1, _t(x2, x1), out=out)
def matmul(x1, x2): return x1 @ x2
def negate(x): return -x
def exp(x): return ExpOp.apply(x)
def log(x): return LogOp.apply(x)
def sqrt(x): return SqrtOp.apply(x)
def tanh(x): return TanhOp.apply(x)
def sigmoid(x): return SigmoidOp.apply(x)
def relu(x): return ReluOp.apply(x)
def pow(x, exponent): return PowOp.apply(x, _t(exponent, x))  # noqa: A001
def sum(x, axis=None, keepdim=False, dtype=None): return SumOp.apply(x, axis, keepdim, dtype)  # noqa: A001
def mean(x, axis=None, keepdim=False, dtype=None): return MeanOp.apply(x, axis, keepdim, dtype)
def reshape(x, *dims): return ReshapeOp.apply(x, *dims)
def transpose(x, dim0, dim1): return TransposeOp.apply(x, dim0, dim1)
def flatten(x): return x.flatten()
def clone(x): return x.clone()
def equals(x1, x2): return x1.equals(x2)
def eq(x, y): return x == y
def gt(x, y): return x > y
def geq(x, y): return x >= y
def lt(x, y): return x < y
def leq(x, y): return x <= y


def _arg_extremum(name, kernel, x, axis, keepdim):
    """src/nanotorch/ops.py:155-232: index of the extremum along one axis (int) or all axes (None)."""
    import math
    if isinstance(axis, int) and not isinstance(axis, bool):
        full_axis = (axis,)
    elif axis is None:
        full_axis = tuple(range(x.ndim))
    else:
        raise ValueError(f"Axis must be int or None, found {type(axis)}")
    if keepdim:
        new_shape = tuple(1 if i in full_axis else s for i, s in enumerate(x.shape))
    else:
        new_shape = tuple(s for i, s in enumerate(x.shape) if i not in full_axis)
    if x.is_empty:
        if math.prod(new_shape) != 0:
            raise IndexError(f"{name}() expects reduction dim to be specified for numel=0.")
        return Tensor._new_contiguous(_C.zeros(math.prod(new_shape), x.dtype, x.device), new_shape)
    return Tensor._new_contiguous(kernel(x._C_view, full_axis), new_shape)


def argmin(x, axis=None, keepdim=False): return _arg_extremum("argmin", _C.argmin, x, axis, keepdim)
def argmax(x, axis=None, keepdim=False): return _arg_extremum("argmax", _C.argmax, x, axis, keepdim)



def compute_on_device(t: Tensor, fn):
    """``fn(t)`` for a factory whose recipe is a few ops on a freshly generated tensor (randint, the
    Kaiming initialisation).  There are no Cpu kernels in this library: a Cpu tensor is moved to the
    device, the ops run there, and the result comes back -- same values as the reference computes on
    the host, no host arithmetic.  Without a device the ops are issued where the tensor is."""
    if t.device == Device.Cpu and _C.is_cuda_available():
        return fn(t.to(Device.Cuda)).to(Device.Cpu)
    return fn(t)


# ---- factories (src/nanotorch/factories.py)
def _shape_args(shape) -> tuple:
    if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
        shape = tuple(shape[0])
    return tuple(int(s) for s in shape)


def _new(storage, shape, requires_grad):
    t = Tensor._new_contiguous(storage, shape)
    if requires_grad:
        t.enable_grad()
    return t


def zeros(*shape, dtype=Dtype.Float32, requires_grad=False, device=Device.Cpu):
    import math
    shape = _shape_args(shape)
    from .tensor import std_device
    return _new(_C.zeros(math.prod(shape), dtype, std_device(device)), shape, requires_grad)


def ones(*shape, dtype=Dtype.Float32, requires_grad=False, device=Device.Cpu):
    import math
    shape = _shape_args(shape)
    from .tensor import std_device
    return _new(_C.ones(math.prod(shape), dtype, std_device(device)), shape, requires_grad)


def full(*shape, value, dtype=Dtype.Float32, requires_grad=False, device=Device.Cpu):
    """A tensor filled with ``value`` (src/nanotorch/factories.py:83-112): ``full(2, 3, value=1.5)``."""
    import math
    from .tensor import std_device
    shape = _shape_args(shape)
    return _new(_C.full(math.prod(shape), value, dtype, std_device(device)), shape, requires_grad)


def eye(n, dtype=Dtype.Float32, requires_grad=False, device=Device.Cpu):
    """The (n, n) identity (src/nanotorch/factories.py:115-142); written by a kernel on the device."""
    from .tensor import std_device
    return _new(_C.eye(n, dtype, std_device(device)), (n, n), requires_grad)


def arange(n, start=0, step=1, dtype=Dtype.Int64, requires_grad=False, device=Device.Cpu):
    """``x[i] = start + i * step`` for ``i < n`` (src/nanotorch/factories.py:145-176)."""
    from .tensor import std_device
    return _new(_C.arange(n, start, step, dtype, std_device(device)), (n,), requires_grad)


def rand(*shape, dtype=Dtype.Float32, requires_grad=False, device=Device.Cpu):
    """Uniform [0, 1) from the seeded host mt19937_64 stream (src/cpp/factory.cu:73-83)."""
    import math
    shape = _shape_args(shape)
    from .tensor import std_device
    if dtype <= Dtype.Int64:
        raise ValueError("rand() cannot output non-float values.")
    return _new(_C.uniform(math.prod(shape), dtype, std_device(device)), shape, requires_grad)


def randint(low, high, shape=None, dtype=Dtype.Int64, requires_grad=False, device=Device.Cpu):
    """Random integers in [low, high): ``rand * (high - low) + low`` truncated through Int64, the
    reference's own recipe (src/nanotorch/factories.py:212-252)."""
    import math
    from .tensor import std_device
    if dtype == Dtype.Bool:
        raise ValueError("randint() cannot output bool values.")
    dims = () if shape is None else tuple(shape)
    base = _new(_C.uniform(math.prod(dims) if dims else 1, Dtype.Float32, std_device(device)), dims, False)
    base = compute_on_device(base, lambda t: (t * (high - low) + low).to(Dtype.Int64).to(dtype))
    if requires_grad:
        base.enable_grad()
    return base


def tensor(data, **kw):
    return Tensor(data, **kw)
