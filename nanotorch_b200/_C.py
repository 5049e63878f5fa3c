"""`_C`: the native-module surface of nanotorch, bound to libnt_b200.so through its C ABI.

Same names, argument meaning and exception classes as the reference's pybind11 module
(src/cpp/_C.cpp:12-24, typed in src/nanotorch/_C.pyi:1-136): ``Dtype``, ``Device``, ``Storage``,
``TensorView`` and the free functions that take views and return a fresh ``Storage``.  The extra
entry points of include/nt_b200.h (fused backward kernels, SGD update, data-parallel exchange,
matmul mode) are exposed under the same module.

There is no fallback: if the shared library is missing the import fails, and every compute call
on a machine without a GPU raises RuntimeError.
"""

from __future__ import annotations

import ctypes as C
import enum
from pathlib import Path
from typing import Sequence

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libnt_b200.so"
if not _LIB_PATH.exists():
    raise ImportError(
        f"{_LIB_PATH} is missing: build it with `python nanotorch_b200/build.py` "
        "(there is no CPU or PyTorch fallback for the op kernels)."
    )
_lib = C.CDLL(str(_LIB_PATH))

NT_MAX_DIMS = 8


class Dtype(enum.IntEnum):
    """Data storage types; the order is the promotion order (src/cpp/dtype.h:21)."""

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
    """Data storage devices (src/cpp/allocator.h:10)."""

    Cpu = 0
    Cuda = 1


_ITEMSIZE = {Dtype.Bool: 1, Dtype.Int32: 4, Dtype.Int64: 8, Dtype.Float32: 4, Dtype.Float64: 8}
_CTYPE = {
    Dtype.Bool: C.c_bool,
    Dtype.Int32: C.c_int32,
    Dtype.Int64: C.c_int64,
    Dtype.Float32: C.c_float,
    Dtype.Float64: C.c_double,
}


_FORMAT = {Dtype.Bool: "?", Dtype.Int32: "i", Dtype.Int64: "q", Dtype.Float32: "f", Dtype.Float64: "d"}


class _View(C.Structure):
    _fields_ = [
        ("storage", C.c_void_p),
        ("ndim", C.c_int32),
        ("shape", C.c_int64 * NT_MAX_DIMS),
        ("strides", C.c_int64 * NT_MAX_DIMS),
        ("offset", C.c_int64),
    ]


class _Scalar(C.Structure):
    _fields_ = [("kind", C.c_int32), ("i", C.c_int64), ("d", C.c_double)]


_lib.nt_last_error.restype = C.c_char_p
_lib.nt_storage_size.restype = C.c_int64
_lib.nt_storage_itemsize.restype = C.c_int64
_lib.nt_storage_version.restype = C.c_uint64
_lib.nt_storage_data.restype = C.c_void_p
_lib.nt_stream.restype = C.c_void_p
for _name in (
    "nt_storage_size", "nt_storage_itemsize", "nt_storage_dtype", "nt_storage_device",
    "nt_storage_version", "nt_storage_data", "nt_storage_retain", "nt_storage_release",
):
    getattr(_lib, _name).argtypes = [C.c_void_p]

_ERRORS = {1: RuntimeError, 2: ValueError, 3: TypeError, 4: IndexError}


def _check(status: int) -> None:
    if status != 0:
        msg = _lib.nt_last_error()
        raise _ERRORS.get(status, RuntimeError)(msg.decode() if msg else "unknown native error")


def _dtype(d) -> Dtype:
    if not isinstance(d, Dtype):
        raise TypeError(f"expected a Dtype, got {type(d).__name__}")
    return d


def _device(d) -> Device:
    if not isinstance(d, Device):
        raise TypeError(f"expected a Device, got {type(d).__name__}")
    return d


def _scalar(v) -> _Scalar:
    # bool before int: bool is an int subclass (src/cpp/storage.h:72-80)
    if isinstance(v, bool):
        return _Scalar(0, int(v), float(v))
    if isinstance(v, int):
        return _Scalar(1, v, float(v))
    if isinstance(v, float):
        return _Scalar(2, 0, v)
    raise TypeError("Unknown scalar type.")


class Storage:
    """Pointer to a 1D contiguous, typed memory segment (src/cpp/storage.h:34-66)."""

    __slots__ = ("_h", "_dtype", "_device", "_size", "__weakref__")

    def __init__(self, *_a, **_k):
        raise TypeError("Storage: use Storage.allocate or Storage.from_iterable")

    @classmethod
    def _wrap(cls, handle: int) -> "Storage":
        self = object.__new__(cls)
        self._h = handle
        self._dtype = Dtype(_lib.nt_storage_dtype(handle))
        self._device = Device(_lib.nt_storage_device(handle))
        self._size = _lib.nt_storage_size(handle)
        return self

    def __del__(self):
        h = getattr(self, "_h", None)
        if h and _lib is not None:
            try:
                _lib.nt_storage_release(h)
            except Exception:  # interpreter shutdown
                pass
            self._h = None

    @staticmethod
    def allocate(n: int, dtype: Dtype, device: Device) -> "Storage":
        out = C.c_void_p()
        _check(_lib.nt_storage_allocate(C.c_int64(n), int(_dtype(dtype)), _device(device).value, C.byref(out)))
        return Storage._wrap(out.value)

    @staticmethod
    def from_iterable(values: Sequence, dtype: Dtype, device: Device) -> "Storage":
        dtype = _dtype(dtype)
        device = _device(device)
        n = len(values)
        host = Storage.allocate(n, dtype, Device.Cpu)
        if n:
            ctype = _CTYPE[dtype]
            arr = (ctype * n).from_address(_lib.nt_storage_data(host._h))
            if dtype in (Dtype.Int32, Dtype.Int64):
                for i, v in enumerate(values):
                    if isinstance(v, float):
                        raise TypeError("Unable to cast Python float to an integer storage element")
                    arr[i] = v
            elif dtype == Dtype.Bool:
                for i, v in enumerate(values):
                    arr[i] = bool(v)
            else:
                for i, v in enumerate(values):
                    arr[i] = v
        return host if device == Device.Cpu else host.to(device)

    @property
    def size(self) -> int:
        return self._size

    @property
    def itemsize(self) -> int:
        return _ITEMSIZE[self._dtype]

    @property
    def dtype(self) -> Dtype:
        return self._dtype

    @property
    def device(self) -> Device:
        return self._device

    @property
    def version(self) -> int:
        return _lib.nt_storage_version(self._h)

    @property
    def data_ptr(self) -> int:
        return _lib.nt_storage_data(self._h) or 0

    def clone(self) -> "Storage":
        out = C.c_void_p()
        _check(_lib.nt_storage_clone(C.c_void_p(self._h), C.byref(out)))
        return Storage._wrap(out.value)

    def to(self, device: Device) -> "Storage":
        device = _device(device)
        if device == self._device:
            return self
        out = C.c_void_p()
        _check(_lib.nt_storage_to(C.c_void_p(self._h), device.value, C.byref(out)))
        return Storage._wrap(out.value)

    def cast(self, dtype: Dtype) -> "Storage":
        dtype = _dtype(dtype)
        if dtype == self._dtype:
            return self
        out = C.c_void_p()
        _check(_lib.nt_storage_cast(C.c_void_p(self._h), int(dtype), C.byref(out)))
        return Storage._wrap(out.value)

    # Buffer protocol, 1-D, writable (src/cpp/storage.cpp:67-70, 82-95).  As in the reference the
    # exported pointer of a Cuda storage is a device pointer: its length is meaningful, its
    # contents are not readable from the host.
    def __buffer__(self, flags: int) -> memoryview:
        n = self._size
        ctype = _CTYPE[self._dtype]
        fmt = _FORMAT[self._dtype]
        if n == 0:
            return memoryview((ctype * 0)()).cast("B").cast(fmt)
        arr = (ctype * n).from_address(_lib.nt_storage_data(self._h))
        arr._owner = self  # keep the storage alive while the view is
        return memoryview(arr).cast("B").cast(fmt)

    # fast paths used by the tensor layer and the tests (numpy arrays, bytes)
    def upload(self, host_ptr: int, nbytes: int) -> None:
        _check(_lib.nt_storage_upload(C.c_void_p(self._h), C.c_void_p(host_ptr), C.c_int64(nbytes)))

    def download(self, host_ptr: int, nbytes: int) -> None:
        _check(_lib.nt_storage_download(C.c_void_p(self._h), C.c_void_p(host_ptr), C.c_int64(nbytes)))


class TensorView:
    """Strided tensor view handed to the kernels (src/cpp/tensor_view.cuh:10-15, 93-102)."""

    __slots__ = ("_storage", "_shape", "_strides", "_offset", "_c")

    def __init__(self, storage: Storage = None, shape=(), strides=(), offset: int = 0) -> None:
        self._storage = storage
        self._shape = tuple(shape)
        self._strides = tuple(strides)
        self._offset = int(offset)
        self._c = None

    def _struct(self) -> _View:
        c = self._c
        if c is None:
            nd = len(self._shape)
            if len(self._strides) != nd:
                raise RuntimeError("TensorView: shape and strides differ in length.")
            if nd > NT_MAX_DIMS:
                raise RuntimeError("TensorView: more than 8 dimensions are not supported on device.")
            if not isinstance(self._storage, Storage):
                raise TypeError("TensorView: storage must be a Storage.")
            c = _View()
            c.storage = self._storage._h
            c.ndim = nd
            for i in range(nd):
                c.shape[i] = self._shape[i]
                c.strides[i] = self._strides[i]
            c.offset = self._offset
            self._c = c
        return c

    def _set(self, name, value):
        object.__setattr__(self, name, value)
        object.__setattr__(self, "_c", None)

    storage = property(lambda s: s._storage, lambda s, v: s._set("_storage", v))
    shape = property(lambda s: list(s._shape), lambda s, v: s._set("_shape", tuple(v)))
    strides = property(lambda s: list(s._strides), lambda s, v: s._set("_strides", tuple(v)))
    offset = property(lambda s: s._offset, lambda s, v: s._set("_offset", int(v)))


def _vref(v: TensorView):
    if not isinstance(v, TensorView):
        raise TypeError(f"expected a TensorView, got {type(v).__name__}")
    return C.byref(v._struct())


def _ret_storage(fn, *args) -> Storage:
    out = C.c_void_p()
    _check(fn(*args, C.byref(out)))
    return Storage._wrap(out.value)


def _binary(name):
    fn = getattr(_lib, "nt_" + name)

    def op(x1: TensorView, x2: TensorView) -> Storage:
        return _ret_storage(fn, _vref(x1), _vref(x2))

    op.__name__ = name
    return op


def _unary(name):
    fn = getattr(_lib, "nt_" + name)

    def op(x: TensorView) -> Storage:
        return _ret_storage(fn, _vref(x))

    op.__name__ = name
    return op


def _inplace(name):
    fn = getattr(_lib, "nt_" + name)

    def op(x1: TensorView, x2: TensorView) -> None:
        _check(fn(_vref(x1), _vref(x2)))

    op.__name__ = name
    return op


# ---- pointwise (src/cpp/ops/binary_ops.cu:178-196, unary_ops.cu:109-128)
add = _binary("add")
subtract = _binary("subtract")
multiply = _binary("multiply")
divide = _binary("divide")
pw_equal = _binary("pw_equal")
pw_greater = _binary("pw_greater")
pw_greater_eq = _binary("pw_greater_eq")
matmul = _binary("matmul")
exp = _unary("exp")
log = _unary("log")
sqrt = _unary("sqrt")
tanh = _unary("tanh")
sigmoid = _unary("sigmoid")
neg = _unary("neg")
relu = _unary("relu")


def equals(x1: TensorView, x2: TensorView) -> bool:
    out = C.c_int(0)
    _check(_lib.nt_equals(_vref(x1), _vref(x2), C.byref(out)))
    return bool(out.value)


def pow(x: TensorView, power) -> Storage:  # noqa: A001 - the reference's name
    s = _scalar(power)
    return _ret_storage(_lib.nt_pow, _vref(x), C.byref(s))


# ---- reductions (src/cpp/ops/reduction_ops.cu:263-276)
def _axes(axis: Sequence[int]):
    ax = [int(a) for a in axis]
    return (C.c_int64 * len(ax))(*ax), len(ax)


def sum(x: TensorView, axis: Sequence[int], dtype: Dtype) -> Storage:  # noqa: A001
    arr, n = _axes(axis)
    return _ret_storage(_lib.nt_sum, _vref(x), arr, C.c_int32(n), int(_dtype(dtype)))


def mean_f32(x: TensorView, axis: Sequence[int], count: int) -> "Storage | None":
    """Float32 sum divided by `count` in the launch that finishes the sum (the bits of sum followed by
    divide); None when the view takes none of the single-launch reduction kernels."""
    arr, n = _axes(axis)
    out = C.c_void_p()
    _check(_lib.nt_mean_f32(_vref(x), arr, C.c_int32(n), C.c_float(float(count)), C.byref(out)))
    return Storage._wrap(out.value) if out.value else None


def _reduction(name):
    fn = getattr(_lib, "nt_" + name)

    def op(x: TensorView, axis: Sequence[int]) -> Storage:
        arr, n = _axes(axis)
        return _ret_storage(fn, _vref(x), arr, C.c_int32(n))

    op.__name__ = name
    return op


max = _reduction("max")  # noqa: A001
min = _reduction("min")  # noqa: A001
argmax = _reduction("argmax")
argmin = _reduction("argmin")

def matmul_pair(a1: TensorView, b1: TensorView, a2: TensorView, b2: TensorView) -> tuple[Storage, Storage]:
    """(a1 @ b1, a2 @ b2): two independent products, the second overlapping the first's last wave of tiles
    (addition to the reference's surface; the bits of two `matmul` calls)."""
    o1, o2 = C.c_void_p(), C.c_void_p()
    _check(_lib.nt_matmul_pair(_vref(a1), _vref(b1), _vref(a2), _vref(b2), C.byref(o1), C.byref(o2)))
    return Storage._wrap(o1.value), Storage._wrap(o2.value)


def set_matmul_pair_overlap(on: bool = True) -> None:
    """Launch the second product of `matmul_pair` as the programmatic dependent of the first (off by default)."""
    _check(_lib.nt_set_matmul_pair_overlap(int(bool(on))))


def linear(x: TensorView, w: TensorView, bias: TensorView) -> Storage:
    """x @ w + bias with the bias add fused into the GEMM epilogue (addition to the reference's surface)."""
    return _ret_storage(_lib.nt_linear, _vref(x), _vref(w), _vref(bias))


# ---- in-place (src/cpp/ops/inplace_ops.cu:81-92)
add_inplace = _inplace("add_inplace")
sub_inplace = _inplace("sub_inplace")
mul_inplace = _inplace("mul_inplace")
div_inplace = _inplace("div_inplace")
copy_inplace = _inplace("copy_inplace")


# ---- core ops (src/cpp/storage.cpp:96-102, ops/copy_ops.cu:219-233)
def cast(s: Storage, dtype: Dtype) -> Storage:
    return s.cast(dtype)


def to(s: Storage, device: Device) -> Storage:
    return s.to(device)


def copy_view(*, src: TensorView, out: TensorView) -> Storage:
    _check(_lib.nt_copy_view(_vref(src), _vref(out)))
    return out.storage


def clone_contiguous_view_from(src: TensorView) -> Storage:
    return _ret_storage(_lib.nt_clone_contiguous_view_from, _vref(src))


# Index-array gather/scatter.  Keyword names are the reference's (src/cpp/ops/copy_ops.cu:219-233);
# the reference runs them on CPU storages only, here they are device kernels.  `checked` / `unique`
# are additions: the caller already validated the indices on the host / vouches that no two source
# positions address one destination (see include/nt_b200.h).
INDEX_CHECKED = 1
INDEX_UNIQUE = 2


def _index_plan(fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy, out_axis_target):
    nf, na = len(fancy_dims_in_src), len(out_axis_is_fancy)
    if len(fancy_dims_data) != nf or len(out_axis_target) != na:
        raise ValueError("index plan: list lengths differ.")
    if nf > NT_MAX_DIMS or na > NT_MAX_DIMS:
        raise RuntimeError("index plan: more than 8 dimensions are not supported on device.")
    dims = (C.c_int64 * (nf or 1))(*fancy_dims_in_src)
    views = (_View * (nf or 1))()
    for i, v in enumerate(fancy_dims_data):
        views[i] = v._struct()
    is_fancy = (C.c_uint8 * (na or 1))(*[1 if f else 0 for f in out_axis_is_fancy])
    target = (C.c_int64 * (na or 1))(*out_axis_target)
    return dims, nf, views, is_fancy, target


def scatter_to_axes(*, src: TensorView, out: TensorView, fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy,
                    out_axis_target, checked: bool = False, unique: bool = False) -> None:
    if len(out_axis_is_fancy) != len(src.shape):
        raise ValueError("scatter_to_axes: one axis entry per dimension of src.")
    dims, nf, views, is_fancy, target = _index_plan(fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy,
                                                    out_axis_target)
    flags = (INDEX_CHECKED if checked else 0) | (INDEX_UNIQUE if unique else 0)
    _check(_lib.nt_scatter_to_axes(_vref(src), _vref(out), dims, C.c_int32(nf), views, is_fancy, target,
                                   C.c_uint32(flags)))


def gather_from_axes(*, x: TensorView, new_shape, fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy,
                     out_axis_target, checked: bool = False) -> Storage:
    if len(out_axis_is_fancy) != len(new_shape):
        raise ValueError("gather_from_axes: one axis entry per dimension of new_shape.")
    dims, nf, views, is_fancy, target = _index_plan(fancy_dims_in_src, fancy_dims_data, out_axis_is_fancy,
                                                    out_axis_target)
    shape = (C.c_int64 * (len(new_shape) or 1))(*new_shape)
    return _ret_storage(_lib.nt_gather_from_axes, _vref(x), shape, C.c_int32(len(new_shape)), dims, C.c_int32(nf),
                        views, is_fancy, target, C.c_uint32(INDEX_CHECKED if checked else 0))


# ---- factories (src/cpp/factory.cu:85-99)
def _factory(fn, *args) -> Storage:
    out = C.c_void_p()
    _check(fn(*args, C.byref(out)))
    return Storage._wrap(out.value)


def zeros(n: int, dtype: Dtype, device: Device) -> Storage:
    return _factory(_lib.nt_zeros, C.c_int64(n), int(_dtype(dtype)), _device(device).value)


def ones(n: int, dtype: Dtype, device: Device) -> Storage:
    return _factory(_lib.nt_ones, C.c_int64(n), int(_dtype(dtype)), _device(device).value)


def full(n: int, value, dtype: Dtype, device: Device) -> Storage:
    s = _scalar(value)
    return _factory(_lib.nt_full, C.c_int64(n), C.byref(s), int(_dtype(dtype)), _device(device).value)


def eye(n: int, dtype: Dtype, device: Device) -> Storage:
    return _factory(_lib.nt_eye, C.c_int64(n), int(_dtype(dtype)), _device(device).value)


def arange(n: int, start: int, step: int, dtype: Dtype, device: Device) -> Storage:
    return _factory(_lib.nt_arange, C.c_int64(n), C.c_int64(start), C.c_int64(step), int(_dtype(dtype)),
                    _device(device).value)


def manual_seed(seed: int) -> None:
    _check(_lib.nt_manual_seed(C.c_uint64(seed)))


def uniform(n: int, dtype: Dtype, device: Device) -> Storage:
    return _factory(_lib.nt_uniform, C.c_int64(n), int(_dtype(dtype)), _device(device).value)


# ---- CUDA (src/cpp/cuda.cpp:3-7)
def is_cuda_available() -> bool:
    return bool(_lib.nt_is_cuda_available())


def cuda_sync() -> None:
    _check(_lib.nt_cuda_sync())


# =============================================================================================
# Extensions beyond the reference's surface (include/nt_b200.h)
def set_device(ordinal: int) -> None:
    _check(_lib.nt_set_device(int(ordinal)))


def device_count() -> int:
    out = C.c_int(0)
    _check(_lib.nt_device_count(C.byref(out)))
    return out.value


def stream_handle() -> int:
    return _lib.nt_stream() or 0


def launch_count() -> int:
    out = C.c_uint64(0)
    _check(_lib.nt_launch_count(C.byref(out)))
    return out.value


def allocator_stats() -> dict:
    a, b, c = C.c_uint64(0), C.c_uint64(0), C.c_uint64(0)
    _check(_lib.nt_allocator_stats(C.byref(a), C.byref(b), C.byref(c)))
    return {"bytes_reserved": a.value, "bytes_in_use": b.value, "n_cuda_malloc": c.value}


def allocator_trim() -> None:
    _check(_lib.nt_allocator_trim())


def allocator_requests() -> int:
    """Requests made to the device arena since load (served from its cache or by cudaMalloc)."""
    n = C.c_uint64(0)
    _check(_lib.nt_allocator_requests(C.byref(n)))
    return n.value


_lib.nt_get_wait_limit_clocks.restype = C.c_int64


def set_wait_limit_clocks(clocks: int) -> None:
    """Limit, in SM clocks, of every bounded spin in device code (default 2**31)."""
    _check(_lib.nt_set_wait_limit_clocks(C.c_int64(int(clocks))))


def get_wait_limit_clocks() -> int:
    return _lib.nt_get_wait_limit_clocks()


def wait_probe() -> None:
    """Launch the one-thread kernel that waits (bounded) on a barrier nothing arrives on."""
    _check(_lib.nt_wait_probe())


TANH_CORRECTLY_ROUNDED = 0
TANH_BIT_EXACT_LIBM = 1


def set_tanh_mode(mode: int) -> None:
    _check(_lib.nt_set_tanh_mode(int(mode)))


def get_tanh_mode() -> int:
    return _lib.nt_get_tanh_mode()


RNG_HOST_MT19937_64 = 0   # the reference's seeded host stream (default)
RNG_DEVICE_PHILOX = 1     # Philox4x32-10 generated on the device


def set_rng_mode(mode: int) -> None:
    _check(_lib.nt_set_rng_mode(int(mode)))


def get_rng_mode() -> int:
    return _lib.nt_get_rng_mode()


MATMUL_EXACT_FP32 = 0
MATMUL_3XTF32 = 1
MATMUL_FP32_UNFUSED = 2
MATMUL_3XTF32_SINGLE_CHAIN = 3


def set_matmul_mode(mode: int) -> None:
    _check(_lib.nt_set_matmul_mode(int(mode)))


_lib.nt_get_matmul_tc_min_macs.restype = C.c_int64


def set_matmul_tc_min_macs(macs: int) -> None:
    """Products of at most this many multiply-adds take the exact FP32 kernel in modes 1 and 3 (default 2**21)."""
    _check(_lib.nt_set_matmul_tc_min_macs(C.c_int64(int(macs))))


def get_matmul_tc_min_macs() -> int:
    return _lib.nt_get_matmul_tc_min_macs()


def set_matmul_operand_planes(natural: bool = True, cached: bool = True) -> None:
    """Mode-1 operand planes: `natural` keeps the source's row-major order (no transposing split, the kernel
    reads either major); `cached` remembers them per storage and view until the storage is written again."""
    _check(_lib.nt_set_matmul_operand_planes(int(bool(natural)), int(bool(cached))))


def set_producer_planes(on: bool = True) -> None:
    """tanh / tanh_backward write the TF32 planes of a large dense 2-D result themselves (see the header)."""
    _check(_lib.nt_set_producer_planes(int(bool(on))))


def set_matmul_schedule(max_splits: int = 8, panel: int = 8) -> None:
    """Split-K limit and tile-panel width of the mode-1 tensor-core kernel (see the header)."""
    _check(_lib.nt_set_matmul_schedule(int(max_splits), int(panel)))


def set_transposed_tile_pipeline(on: bool = True) -> None:
    """Large fp32 elementwise ops with a transposed operand: TMA-fed persistent kernel (default) or the
    register-staged tile kernel (see the header)."""
    _check(_lib.nt_set_transposed_tile_pipeline(int(bool(on))))


def matmul_split_stats() -> tuple[int, int]:
    """(operand-split launches, operand-plane cache hits) since load."""
    a, b = C.c_uint64(0), C.c_uint64(0)
    _check(_lib.nt_matmul_split_stats(C.byref(a), C.byref(b)))
    return a.value, b.value


def get_matmul_mode() -> int:
    return _lib.nt_get_matmul_mode()


relu_backward = _binary("relu_backward")
tanh_backward = _binary("tanh_backward")
sigmoid_backward = _binary("sigmoid_backward")
exp_backward = _binary("exp_backward")
log_backward = _binary("log_backward")
sqrt_backward = _binary("sqrt_backward")


def pow_backward(g: TensorView, x: TensorView, exponent: float) -> Storage:
    return _ret_storage(_lib.nt_pow_backward, _vref(g), _vref(x), C.c_float(exponent))


def div_backward_x2(g: TensorView, x1: TensorView, x2: TensorView) -> Storage:
    return _ret_storage(_lib.nt_div_backward_x2, _vref(g), _vref(x1), _vref(x2))


def extremum_backward(g_expanded: TensorView, x: TensorView, m_expanded: TensorView, axis: Sequence[int]) -> Storage:
    arr, n = _axes(axis)
    return _ret_storage(_lib.nt_extremum_backward, _vref(g_expanded), _vref(x), _vref(m_expanded), arr, C.c_int32(n))


def _backward_both(fn):
    def op(g: TensorView, x1: TensorView, x2: TensorView):
        a, b = C.c_void_p(), C.c_void_p()
        _check(fn(_vref(g), _vref(x1), _vref(x2), C.byref(a), C.byref(b)))
        return (Storage._wrap(a.value), Storage._wrap(b.value)) if a.value else None
    return op


mul_backward = _backward_both(_lib.nt_mul_backward)   # (x2*g, x1*g) in one pass, or None
div_backward = _backward_both(_lib.nt_div_backward)   # (g/x2, ((-x1)/x2**2)*g) in one pass, or None


def sgd_update(param: TensorView, grad: TensorView, lr: float, grad_scale: float = 1.0) -> None:
    _check(_lib.nt_sgd_update(_vref(param), _vref(grad), C.c_float(lr), C.c_float(grad_scale)))


def sum_rows_noalloc(src: Storage, n_rows: int, row_len: int, out: Storage) -> None:
    """out[r] = sum of row r of the dense fp32 [n_rows, row_len] matrix at the start of `src`, through
    the entry point that never allocates: both storages are the caller's, the kernel's scratch is a
    fixed array inside the library (see nt_sum_rows_noalloc in include/nt_b200.h for the limits)."""
    for s, need in ((src, n_rows * row_len), (out, n_rows)):
        if s.device != Device.Cuda or s.dtype != Dtype.Float32 or s.size < need:
            raise ValueError("sum_rows_noalloc: Float32 Cuda storages of at least n_rows*row_len and n_rows elements")
    _check(_lib.nt_sum_rows_noalloc(C.c_void_p(src.data_ptr), C.c_int64(n_rows), C.c_int64(row_len),
                                    C.c_void_p(out.data_ptr)))


COMM_ID_BYTES = 128


def comm_unique_id() -> bytes:
    buf = (C.c_uint8 * COMM_ID_BYTES)()
    _check(_lib.nt_comm_unique_id(buf))
    return bytes(buf)


def comm_init(rank: int, world: int, unique_id: bytes) -> None:
    if len(unique_id) != COMM_ID_BYTES:
        raise ValueError("comm_init: unique id must be 128 bytes")
    buf = (C.c_uint8 * COMM_ID_BYTES).from_buffer_copy(unique_id)
    _check(_lib.nt_comm_init(int(rank), int(world), buf))


def comm_init_timeout(rank: int, world: int, unique_id: bytes, timeout_ms: int) -> None:
    """comm_init with an explicit limit on the rendezvous: RuntimeError if a rank has not joined in time."""
    if len(unique_id) != COMM_ID_BYTES:
        raise ValueError("comm_init: unique id must be 128 bytes")
    buf = (C.c_uint8 * COMM_ID_BYTES).from_buffer_copy(unique_id)
    _check(_lib.nt_comm_init_timeout(int(rank), int(world), buf, C.c_int64(int(timeout_ms))))


def comm_group_begin() -> None:
    """Open a bucket: orders the communication stream after the compute stream; the all-reduces issued
    until comm_group_end go out as one NCCL launch."""
    _check(_lib.nt_comm_group_begin())


def comm_group_end() -> None:
    _check(_lib.nt_comm_group_end())


def comm_sgd_update(param: "TensorView", grad: "TensorView", lr: float, grad_scale: float = 1.0) -> None:
    """sgd_update enqueued on the communication stream, behind the collectives issued so far."""
    _check(_lib.nt_comm_sgd_update(_vref(param), _vref(grad), C.c_float(lr), C.c_float(grad_scale)))


def comm_sync(timeout_ms: int) -> None:
    """Host-side wait for the communication stream with a time limit; aborts the communicator past it."""
    _check(_lib.nt_comm_sync(C.c_int64(int(timeout_ms))))


def comm_abort() -> None:
    _check(_lib.nt_comm_abort())


def comm_allreduce_sum(s: Storage) -> None:
    _check(_lib.nt_comm_allreduce_sum(C.c_void_p(s._h)))


def comm_wait() -> None:
    _check(_lib.nt_comm_wait())


def comm_destroy() -> None:
    _check(_lib.nt_comm_destroy())


class Event:
    """CUDA event on the library's compute stream."""

    def __init__(self):
        h = C.c_void_p()
        _check(_lib.nt_event_create(C.byref(h)))
        self._h = h.value

    def record(self) -> "Event":
        _check(_lib.nt_event_record(C.c_void_p(self._h)))
        return self

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float(0)
        _check(_lib.nt_event_elapsed_ms(C.c_void_p(self._h), C.c_void_p(stop._h), C.byref(ms)))
        return ms.value

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _lib.nt_event_destroy(C.c_void_p(h))
            except Exception:
                pass
            self._h = None


class Graph:
    """A captured sequence of launches: `with g.capture(): ...` records whatever the block enqueues
    (kernels, NCCL collectives, stream joins), `g.replay()` re-issues it as one CUDA-graph launch.
    Tensors created inside the block keep their device addresses, so results are read from the same
    tensors after every replay."""

    def __init__(self):
        self._id = 0

    def capture(self):
        return _GraphCapture(self)

    def replay(self) -> None:
        _check(_lib.nt_graph_launch(self._id))

    def close(self) -> None:
        if self._id:
            _check(_lib.nt_graph_destroy(self._id))
            self._id = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _GraphCapture:
    def __init__(self, graph: Graph):
        self._g = graph

    def __enter__(self):
        gid = C.c_int(0)
        _check(_lib.nt_graph_begin_capture(C.byref(gid)))
        self._g._id = gid.value
        return self._g

    def __exit__(self, exc_type, exc, tb):
        status = _lib.nt_graph_end_capture(self._g._id)
        if exc_type is None:
            _check(status)
        return False


def matmul_profile_enable(on: bool) -> None:
    _check(_lib.nt_matmul_profile_enable(1 if on else 0))


def matmul_profile_read() -> tuple[float, int]:
    total, n = C.c_double(0), C.c_int64(0)
    _check(_lib.nt_matmul_profile_read(C.byref(total), C.byref(n)))
    return total.value, n.value


def upload_async(s: Storage, host_ptr: int, nbytes: int) -> None:
    _check(_lib.nt_storage_upload_async(C.c_void_p(s._h), C.c_void_p(host_ptr), C.c_int64(nbytes)))


def upload_fence() -> None:
    _check(_lib.nt_upload_fence())


def host_register(ptr: int, nbytes: int) -> None:
    _check(_lib.nt_host_register(C.c_void_p(ptr), C.c_int64(nbytes)))


def host_unregister(ptr: int) -> None:
    _check(_lib.nt_host_unregister(C.c_void_p(ptr)))


def exported_symbols() -> list[str]:
    """Every symbol declared in include/nt_b200.h that this library must export."""
    import re

    header = Path(__file__).resolve().parent.parent / "include" / "nt_b200.h"
    text = header.read_text()
    return sorted(set(re.findall(r"\b(nt_[a-z0-9_]+)\s*\(", text)))
