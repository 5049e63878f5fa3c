"""Tensor: a (storage, shape, strides, offset) view with autograd bookkeeping.

Host-side mirror of the reference's ``nanotorch.Tensor`` for the op-kernel hot path
(src/nanotorch/core.py:47-139, 255-334, 489-563): same view model (strides and offset in elements,
stride 0 = broadcast, views never copy), same attribute and method names, same error classes.
Everything numeric happens in ``_C`` (libnt_b200.so); this file only does bookkeeping.

Not mirrored: fancy (index-array / mask) indexing, which is a CPU-only host feature of the
reference (src/nanotorch/core.py:666-830) and not on the kernel path.
"""

from __future__ import annotations

import math
from typing import Any, Sequence

from . import _C
from ._C import Device, Dtype

Shape = tuple[int, ...]


def sizeof(dtype: Dtype) -> int:
    """Bytes per element of a dtype."""
    return {Dtype.Bool: 1, Dtype.Int32: 4, Dtype.Int64: 8, Dtype.Float32: 4, Dtype.Float64: 8}[dtype]


def promote_dtypes(*dtypes: Dtype) -> Dtype:
    """Highest dtype in enum order (src/nanotorch/_data_type.py:33-37); Float32 for no input."""
    return max(dtypes) if dtypes else Dtype.Float32


def std_device(device: Device | str) -> Device:
    if isinstance(device, Device):
        return device
    if device == "cpu":
        return Device.Cpu
    if device == "cuda":
        return Device.Cuda
    raise ValueError(f"Unknown device {device}.")


def contiguous_strides(shape: Shape) -> Shape:
    strides, acc = [], 1
    for extent in reversed(shape):
        strides.append(acc)
        acc *= extent
    return tuple(reversed(strides))


def broadcast_shapes(*shapes: Shape) -> Shape:
    """Right-aligned broadcast; RuntimeError on mismatch (src/nanotorch/_indexing.py:8-26)."""
    if not shapes:
        return ()
    nd = max(len(s) for s in shapes)
    out = [1] * nd
    for s in shapes:
        padded = (1,) * (nd - len(s)) + tuple(s)
        for i, extent in enumerate(padded):
            if out[i] == 1:
                out[i] = extent
            elif extent != 1 and extent != out[i]:
                raise RuntimeError(f"Cannot broadcast shapes {list(s)} and {out}.")
    return tuple(out)


def _dtype_of_scalar(v) -> Dtype:
    if isinstance(v, bool):
        return Dtype.Bool
    if isinstance(v, int):
        return Dtype.Int64
    if isinstance(v, float):
        return Dtype.Float32
    raise TypeError(f"Unsupported Tensor value type: {type(v)}")


def _flatten_nested(data, max_depth: int = 32):
    """Nested lists -> (shape, flat values, inferred dtype); ValueError on ragged input."""
    shape: list[int] = []
    flat: list = []
    auto = None
    leaf_depth = None

    def walk(node, depth):
        nonlocal auto, leaf_depth
        if depth > max_depth:
            raise ValueError(f"Maximum tensor depth reached: {max_depth}")
        if isinstance(node, (bool, int, float)):
            if leaf_depth is None:
                leaf_depth = depth
            elif leaf_depth != depth:
                raise ValueError("Leaf found at non-terminal level.")
            dt = _dtype_of_scalar(node)
            if auto is None or dt > auto:
                auto = dt
            flat.append(node)
        elif isinstance(node, list):
            if depth >= len(shape):
                shape.append(len(node))
            elif shape[depth] != len(node):
                raise ValueError(f"Unhomogeneous tensor shape detected ({shape[depth]} != {len(node)})")
            for child in node:
                walk(child, depth + 1)
        else:
            raise TypeError(f"Unsupported tensor element type: {type(node)}")

    walk(data, 0)
    return tuple(shape), flat, (auto if auto is not None else Dtype.Float32)


class Tensor:
    """Typed n-dimensional array with autograd; see the module docstring."""

    __slots__ = ("_storage", "_shape", "_strides", "_offset", "_requires_grad", "_grad", "_grad_fn", "_pyvalue")

    def __init__(self, data, *, dtype: Dtype | None = None, requires_grad: bool = False,
                 device: Device | str = Device.Cpu):
        if hasattr(data, "__array__") and hasattr(data, "tolist"):
            data = data.tolist()
        device = std_device(device)
        shape, flat, auto = _flatten_nested(data)
        final = dtype if dtype is not None else auto
        if final == Dtype.Bool:
            flat = [bool(v) for v in flat]
        elif auto >= Dtype.Float32 and final <= Dtype.Int64:
            flat = [int(v) for v in flat]
        self._storage = _C.Storage.from_iterable(flat, final, device)
        self._shape = shape
        self._strides = contiguous_strides(shape)
        self._offset = 0
        if final <= Dtype.Int64 and requires_grad:
            raise RuntimeError("Cannot enable grad on a non-float tensor.")
        self._requires_grad = requires_grad
        self._grad = None
        self._grad_fn = None
        self._pyvalue = data if (shape == () and dtype is None) else None

    # ------------------------------------------------------------------ constructors
    @classmethod
    def _new_view(cls, storage: _C.Storage, shape: Shape, strides: Shape | None, offset: int | None) -> "Tensor":
        shape = tuple(shape)
        strides = contiguous_strides(shape) if strides is None else tuple(strides)
        offset = 0 if offset is None else offset
        if math.prod(shape) > 0:
            lo = offset + sum((s - 1) * st for s, st in zip(shape, strides) if st < 0)
            hi = offset + sum((s - 1) * st for s, st in zip(shape, strides) if st > 0)
            if lo < 0 or hi >= storage.size:
                raise IndexError(f"View max index {hi} exceeds storage capacity {storage.size}.")
        t = object.__new__(cls)
        t._storage = storage
        t._shape = shape
        t._strides = strides
        t._offset = offset
        t._requires_grad = False
        t._grad = None
        t._grad_fn = None
        t._pyvalue = None
        return t

    @classmethod
    def _new_contiguous(cls, storage: _C.Storage, shape: Shape) -> "Tensor":
        return cls._new_view(storage, shape, None, None)

    @classmethod
    def _scalar(cls, value, dtype: Dtype, device: Device) -> "Tensor":
        """0-d tensor written by a device fill: no host->device copy, no synchronisation."""
        t = cls._new_contiguous(_C.full(1, value, dtype, device), ())
        return t

    @classmethod
    def from_numpy(cls, array, device: Device | str = Device.Cuda, requires_grad: bool = False) -> "Tensor":
        """Bulk load through one host->device copy (C-contiguous numpy array of a supported dtype)."""
        import numpy as np

        kinds = {np.dtype(np.bool_): Dtype.Bool, np.dtype(np.int32): Dtype.Int32, np.dtype(np.int64): Dtype.Int64,
                 np.dtype(np.float32): Dtype.Float32, np.dtype(np.float64): Dtype.Float64}
        array = np.ascontiguousarray(array)
        if array.dtype not in kinds:
            raise TypeError(f"Unsupported numpy dtype {array.dtype}")
        device = std_device(device)
        storage = _C.Storage.allocate(array.size, kinds[array.dtype], device)
        if array.size:
            storage.upload(array.ctypes.data, array.nbytes)
        t = cls._new_contiguous(storage, tuple(array.shape))
        if requires_grad:
            t.enable_grad()
        return t

    def numpy(self):
        """Host copy as a numpy array (one device->host copy; synchronises)."""
        import numpy as np

        kinds = {Dtype.Bool: np.bool_, Dtype.Int32: np.int32, Dtype.Int64: np.int64, Dtype.Float32: np.float32,
                 Dtype.Float64: np.float64}
        src = self
        if not src._is_contiguous(full_span=True):
            if src.device == Device.Cuda:
                src = src._to_contiguous(force=True)
            else:
                flat = np.empty(self._storage.size, dtype=kinds[self.dtype])
                if flat.size:
                    self._storage.download(flat.ctypes.data, flat.nbytes)
                return np.lib.stride_tricks.as_strided(
                    flat[self._offset:], shape=self._shape,
                    strides=tuple(s * flat.itemsize for s in self._strides)).copy()
        out = np.empty(src._shape, dtype=kinds[src.dtype])
        if out.size:
            src._storage.download(out.ctypes.data, out.nbytes)
        return out

    # ------------------------------------------------------------------ metadata
    dtype = property(lambda self: self._storage.dtype)
    shape = property(lambda self: self._shape)
    ndim = property(lambda self: len(self._shape))
    numel = property(lambda self: math.prod(self._shape))
    is_empty = property(lambda self: math.prod(self._shape) == 0)
    storage = property(lambda self: self._storage)
    strides = property(lambda self: (self._strides, self._offset))
    device = property(lambda self: self._storage.device)
    version = property(lambda self: self._storage.version)

    def __len__(self) -> int:
        return self._shape[0] if self._shape else 0

    def __repr__(self) -> str:
        return f"nt.Tensor(shape={self.shape}, {self.numel} x <{self.dtype.name}>, d: {self.device.name})"

    @property
    def T(self) -> "Tensor":
        from .autograd import TOp

        return TOp.apply(self)

    @property
    def _C_view(self) -> _C.TensorView:
        return _C.TensorView(self._storage, self._shape, self._strides, self._offset)

    # ------------------------------------------------------------------ moves and copies
    def to(self, target: Dtype | Device | str) -> "Tensor":
        """Cast to a dtype or move to a device; returns self when nothing changes."""
        src = self
        if isinstance(target, Dtype):
            if target == self.dtype:
                return self
            if not src._is_contiguous(full_span=True):
                src = src._to_contiguous(force=True)
            new = _C.cast(src._storage, target)
        else:
            device = std_device(target)
            if device == self.device:
                return self
            if not src._is_contiguous(full_span=True):
                src = src._to_contiguous(force=True)
            new = _C.to(src._storage, device)
        out = Tensor._new_view(new, src._shape, src._strides, src._offset)
        if self.requires_grad and self.grad_fn is None:
            out.enable_grad()
        return out

    def cpu(self) -> "Tensor":
        return self.to(Device.Cpu)

    def cuda(self) -> "Tensor":
        return self.to(Device.Cuda)

    def clone(self) -> "Tensor":
        if self._is_contiguous(full_span=True):
            return Tensor._new_contiguous(self._storage.clone(), self._shape)
        return self._to_contiguous(force=True)

    def flatten(self) -> "Tensor":
        return self.reshape(self.numel)

    def squeeze(self, *axes: int) -> "Tensor":
        if not axes:
            axes = tuple(range(self.ndim))
        axes = tuple(a if a >= 0 else a + self.ndim for a in axes)
        keep = [s for i, s in enumerate(self._shape) if not (i in axes and s == 1)]
        return self.reshape(*keep)

    def equals(self, other: "Tensor") -> bool:
        if self.shape != other.shape:
            return False
        if self.is_empty and other.is_empty:
            return True
        dt = promote_dtypes(self.dtype, other.dtype)
        return _C.equals(self.to(dt)._C_view, other.to(dt)._C_view)

    def tolist(self):
        if self.device != Device.Cpu:
            raise RuntimeError("Tensor on device, call .cpu() first.")
        mem = memoryview(self._storage)
        is_bool = self.dtype == Dtype.Bool

        def build(depth: int, offset: int):
            if depth == len(self._shape):
                return bool(mem[offset]) if is_bool else mem[offset]
            return [build(depth + 1, offset + i * self._strides[depth]) for i in range(self._shape[depth])]

        return build(0, self._offset)

    def item(self):
        if self.numel != 1:
            raise RuntimeError(f"Cannot convert {self} to a scalar.")
        if self.device != Device.Cpu:
            raise RuntimeError("Tensor on device, call .cpu() first.")
        return memoryview(self._storage)[self._offset]

    def _is_contiguous(self, full_span: bool = False) -> bool:
        dense = self._strides == contiguous_strides(self._shape)
        if not full_span:
            return dense
        return dense and self._offset == 0 and self.numel == self._storage.size

    def _to_contiguous(self, force: bool = False) -> "Tensor":
        if not force and self._is_contiguous():
            return self
        if self.device == Device.Cpu:
            raise RuntimeError("clone_contiguous_view_from: requires Cuda (this library has no CPU compute path).")
        return Tensor._new_contiguous(_C.clone_contiguous_view_from(self._C_view), self._shape)

    def _alias(self) -> "Tensor":
        return Tensor._new_view(self._storage, self._shape, self._strides, self._offset)

    # ------------------------------------------------------------------ basic indexing (views)
    def _basic_index(self, index) -> "Tensor":
        if not isinstance(index, tuple):
            index = (index,)
        if self.ndim == 0:
            raise IndexError("Cannot index a scalar value.")
        if sum(1 for i in index if i is Ellipsis) > 1:
            raise IndexError("Multiple ellipses detected.")
        n_real = sum(1 for i in index if i is not None and i is not Ellipsis)
        if n_real > self.ndim:
            raise IndexError(f"Too many indices ({len(index)}) for {self.ndim}D array.")
        expanded: list = []
        for i in index:
            if i is Ellipsis:
                expanded.extend([slice(None)] * (self.ndim - n_real))
            else:
                expanded.append(i)
        shape, strides, offset, dim = [], [], self._offset, 0
        for sel in expanded:
            if sel is None:
                shape.append(1)
                strides.append(0)
                continue
            extent, stride = self._shape[dim], self._strides[dim]
            if isinstance(sel, bool) or not isinstance(sel, (int, slice)):
                raise NotImplementedError("Only int / slice / None / Ellipsis indexing is supported on device.")
            if isinstance(sel, int):
                if sel < 0:
                    sel += extent
                if not 0 <= sel < extent:
                    raise IndexError(f"Cannot index at position {sel} in {extent} elements.")
                offset += sel * stride
            else:
                start, stop, step = sel.indices(extent)
                shape.append(len(range(start, stop, step)))
                strides.append(stride * step)
                offset += start * stride
            dim += 1
        shape.extend(self._shape[dim:])
        strides.extend(self._strides[dim:])
        return Tensor._new_view(self._storage, tuple(shape), tuple(strides), offset)

    def __getitem__(self, index) -> "Tensor":
        return self._basic_index(index)

    def __setitem__(self, index, value) -> None:
        target = self._basic_index(index)
        if not isinstance(value, Tensor):
            value = Tensor(value, dtype=self.dtype, device=self.device)
        elif value.dtype != self.dtype:
            value = value.to(self.dtype)
        try:
            value = value.expand(*target.shape)
        except ValueError as e:
            raise IndexError(str(e)) from e
        if value._storage is self._storage:
            value = value._to_contiguous(force=True)
        _C.copy_view(src=value._C_view, out=target._C_view)

    # ------------------------------------------------------------------ autograd
    @property
    def requires_grad(self) -> bool:
        return self._requires_grad or self._grad_fn is not None

    @property
    def is_leaf(self) -> bool:
        return self._grad_fn is None

    @property
    def grad(self) -> "Tensor | None":
        return self._grad

    @property
    def grad_fn(self):
        return self._grad_fn

    def attach_grad_fn(self, grad_fn) -> None:
        self._grad_fn = grad_fn

    def zero_grad(self) -> None:
        self._grad = None

    def enable_grad(self) -> None:
        if self.dtype <= Dtype.Int64:
            raise RuntimeError("Cannot enable grad on a non-float tensor.")
        self._requires_grad = True

    def backward(self) -> None:
        """Backpropagate from a one-element tensor through the recorded graph."""
        if not self.requires_grad:
            raise RuntimeError(
                "Cannot call .backward() on a tensor that does not require grad and does not have a grad_fn.")
        if self.numel != 1:
            raise RuntimeError(f"Cannot call .backward() on a non-scalar tensor of shape {self.shape}")
        seed = Tensor._new_contiguous(_C.full(1, 1.0, self.dtype, self.device), ())
        if self.shape != ():
            seed = seed.reshape(*self.shape)
        self._grad = seed
        if not self.is_leaf:
            from .autograd import run_backward

            run_backward(self)

    __hash__ = None  # elementwise __eq__
