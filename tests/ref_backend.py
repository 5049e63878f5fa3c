"""TEST INFRASTRUCTURE: the reference's own native module (oracle/_ref, its CPU path) dressed as
``nanotorch_b200._C``.

Putting this module into ``sys.modules["nanotorch_b200._C"]`` before ``nanotorch_b200`` is imported
makes the whole host layer of this package -- Tensor, the autograd op classes, nn, the index plans --
run on top of the reference's CPU kernels instead of libnt_b200.so.  Only the primitives of the
reference's ``_C`` surface exist here (src/nanotorch/_C.pyi): the fused entry points of this library
(``*_backward``, ``sgd_update``, ``linear``) are deliberately absent, so the host layer has to take the
composed paths it keeps for non-device tensors -- the same call sequences the reference's Python layer
issues.  With that, the reference's complete CPU test-suite can be run against this package's Python
layer (tests/test_reference_suite_host.py), and the golden training curves must come out bit for bit.

Never imported by the product."""

from __future__ import annotations

import ctypes
import enum

import numpy as np

from oracle.oracle import load_ref_module

_R = load_ref_module()


class Dtype(enum.IntEnum):
    Bool = 0
    Int32 = 1
    Int64 = 2
    Float32 = 3
    Float64 = 4

    def __str__(self) -> str:
        return f"Dtype.{self.name}"

    def __bool__(self) -> bool:
        # a pybind11 enum value is always truthy; the reference's Python layer relies on it
        # (`auto_dtype or Dtype.Float32`, src/nanotorch/core.py:620), and Bool has the value 0
        return True


class Device(enum.Enum):
    Cpu = 0
    Cuda = 1


def _rd(d: Dtype):
    if not isinstance(d, Dtype):
        raise TypeError(f"expected a Dtype, got {type(d).__name__}")
    return getattr(_R.Dtype, d.name)


def _rdev(d: Device):
    if not isinstance(d, Device):
        raise TypeError(f"expected a Device, got {type(d).__name__}")
    return getattr(_R.Device, d.name)


class Storage:
    __slots__ = ("_s",)

    def __init__(self, *_a, **_k):
        raise TypeError("Storage: use Storage.allocate or Storage.from_iterable")

    @classmethod
    def _wrap(cls, ref_storage) -> "Storage":
        self = object.__new__(cls)
        self._s = ref_storage
        return self

    @staticmethod
    def allocate(n: int, dtype: Dtype, device: Device) -> "Storage":
        return Storage._wrap(_R.Storage.allocate(n, _rd(dtype), _rdev(device)))

    @staticmethod
    def from_iterable(values, dtype: Dtype, device: Device) -> "Storage":
        return Storage._wrap(_R.Storage.from_iterable(list(values), _rd(dtype), _rdev(device)))

    size = property(lambda self: self._s.size)
    itemsize = property(lambda self: self._s.itemsize)
    dtype = property(lambda self: Dtype[self._s.dtype.name])
    device = property(lambda self: Device[self._s.device.name])
    version = property(lambda self: self._s.version)

    def clone(self) -> "Storage":
        return Storage._wrap(self._s.clone())

    def to(self, device: Device) -> "Storage":
        return self if device == self.device else Storage._wrap(self._s.to(_rdev(device)))

    def cast(self, dtype: Dtype) -> "Storage":
        return self if dtype == self.dtype else Storage._wrap(_R.cast(self._s, _rd(dtype)))

    def __buffer__(self, flags: int) -> memoryview:
        return memoryview(self._s)

    def _address(self) -> int:
        return np.asarray(memoryview(self._s)).ctypes.data if self.size else 0

    def upload(self, host_ptr: int, nbytes: int) -> None:
        if nbytes:
            ctypes.memmove(self._address(), host_ptr, nbytes)

    def download(self, host_ptr: int, nbytes: int) -> None:
        if nbytes:
            ctypes.memmove(host_ptr, self._address(), nbytes)


class TensorView:
    __slots__ = ("storage", "shape", "strides", "offset")

    def __init__(self, storage: Storage = None, shape=(), strides=(), offset: int = 0) -> None:
        self.storage, self.shape, self.strides, self.offset = storage, tuple(shape), tuple(strides), int(offset)


def _rv(v: TensorView):
    if not isinstance(v, TensorView):
        raise TypeError(f"expected a TensorView, got {type(v).__name__}")
    return _R.TensorView(v.storage._s, list(v.shape), list(v.strides), v.offset)


def _wrap(ref_storage) -> Storage:
    return Storage._wrap(ref_storage)


def _binary(name):
    fn = getattr(_R, name)
    return lambda x1, x2: _wrap(fn(_rv(x1), _rv(x2)))


def _unary(name):
    fn = getattr(_R, name)
    return lambda x: _wrap(fn(_rv(x)))


def _inplace(name):
    fn = getattr(_R, name)

    def op(out, other):
        fn(_rv(out), _rv(other))

    return op


add, subtract, multiply, divide = (_binary(n) for n in ("add", "subtract", "multiply", "divide"))
pw_equal, pw_greater, pw_greater_eq = (_binary(n) for n in ("pw_equal", "pw_greater", "pw_greater_eq"))
exp, log, sqrt, tanh, sigmoid, neg, relu = (_unary(n) for n in ("exp", "log", "sqrt", "tanh", "sigmoid", "neg", "relu"))
add_inplace, sub_inplace, mul_inplace, div_inplace, copy_inplace = (
    _inplace(n) for n in ("add_inplace", "sub_inplace", "mul_inplace", "div_inplace", "copy_inplace"))
matmul = _binary("matmul")


def equals(x1, x2) -> bool:
    return bool(_R.equals(_rv(x1), _rv(x2)))


def pow(x, exponent):  # noqa: A001
    return _wrap(_R.pow(_rv(x), exponent))


def sum(x, axis, dtype):  # noqa: A001
    return _wrap(_R.sum(_rv(x), [int(a) for a in axis], _rd(dtype)))


def _reduction(name):
    fn = getattr(_R, name)
    return lambda x, axis: _wrap(fn(_rv(x), [int(a) for a in axis]))


max, min, argmax, argmin = (_reduction(n) for n in ("max", "min", "argmax", "argmin"))  # noqa: A001


def cast(s: Storage, dtype: Dtype) -> Storage:
    return s.cast(dtype)


def to(s: Storage, device: Device) -> Storage:
    return s.to(device)


def copy_view(*, src, out):
    _R.copy_view(src=_rv(src), out=_rv(out))
    return out.storage


def clone_contiguous_view_from(src):
    return _wrap(_R.clone_contiguous_view_from(_rv(src)))


def gather_from_axes(*, x, new_shape, fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy, out_axis_target,
                     checked: bool = False):
    return _wrap(_R.gather_from_axes(
        x=_rv(x), new_shape=list(new_shape), fancy_dims_in_src=list(fancy_dims_in_src),
        fancy_dims_data=[_rv(v) for v in fancy_dims_data], out_axis_is_fancy=[bool(f) for f in out_axis_is_fancy],
        out_axis_target=list(out_axis_target)))


def scatter_to_axes(*, src, out, fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy, out_axis_target,
                    checked: bool = False, unique: bool = False):
    _R.scatter_to_axes(
        src=_rv(src), out=_rv(out), fancy_dims_in_src=list(fancy_dims_in_src),
        fancy_dims_data=[_rv(v) for v in fancy_dims_data], out_axis_is_fancy=[bool(f) for f in out_axis_is_fancy],
        out_axis_target=list(out_axis_target))


def zeros(n, dtype, device):
    return _wrap(_R.zeros(n, _rd(dtype), _rdev(device)))


def ones(n, dtype, device):
    return _wrap(_R.ones(n, _rd(dtype), _rdev(device)))


def full(n, value, dtype, device):
    return _wrap(_R.full(n, value, _rd(dtype), _rdev(device)))


def eye(n, dtype, device):
    return _wrap(_R.eye(n, _rd(dtype), _rdev(device)))


def arange(n, start, step, dtype, device):
    return _wrap(_R.arange(n, start, step, _rd(dtype), _rdev(device)))


def uniform(n, dtype, device):
    return _wrap(_R.uniform(n, _rd(dtype), _rdev(device)))


def manual_seed(seed: int) -> None:
    _R.manual_seed(seed)


def is_cuda_available() -> bool:
    return False  # the point of this backend is the Cpu path


def cuda_sync() -> None:
    pass
