"""Tensor: a (storage, shape, strides, offset) view with autograd bookkeeping.

Host-side mirror of the reference's ``nanotorch.Tensor`` for the op-kernel hot path
(src/nanotorch/core.py:47-139, 255-334, 489-563): same view model (strides and offset in elements,
stride 0 = broadcast, views never copy), same attribute and method names, same error classes.
Everything numeric happens in ``_C`` (libnt_b200.so); this file only does bookkeeping.

Index-array and mask indexing (src/nanotorch/core.py:172-254, 666-772) follows the reference's plan
(the numpy rule for where the index dimensions land) and runs as device gather/scatter kernels; the
reference copies element by element on the host.
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
        """The reference's format (src/nanotorch/core.py:141-164): values for 0-d, 1-D (first and last three
        beyond 7 elements) and 2-D tensors (first and last two rows beyond 5), a summary line otherwise.
        Only the printed elements are copied from the device, not the whole tensor as the reference does."""
        def compact(row: "Tensor") -> str:
            n = row.shape[0]
            if n < 8:
                return str(row.cpu().tolist())
            head, tail = row[:3].cpu().tolist(), row[n - 3:].cpu().tolist()
            return "[" + ", ".join(str(v) for v in head) + ", ..., " + ", ".join(str(v) for v in tail) + "]"

        if self.ndim == 0:
            return f"nt.Tensor({self.cpu().tolist()})"
        if self.ndim == 1:
            return f"nt.Tensor({compact(self)})"
        if self.ndim == 2:
            rows = list(range(len(self))) if len(self) <= 5 else [0, 1, None, -2, -1]
            lines = ["..." if i is None else compact(self[i]) for i in rows]
            return "nt.Tensor(" + ("\n" + " " * 10).join(lines) + ")"
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
        return Tensor._new_contiguous(_C.clone_contiguous_view_from(self._C_view), self._shape)

    def _alias(self) -> "Tensor":
        return Tensor._new_view(self._storage, self._shape, self._strides, self._offset)

    # ------------------------------------------------------------------ indexing
    def _basic_index(self, index) -> "tuple[Tensor, tuple | None]":
        """int / slice / None / Ellipsis selectors as a view of the same storage
        (src/nanotorch/core.py:775-827).  Index-array and mask selectors keep their dimension in the
        view and come back in the second result, aligned with the view's dims (None elsewhere);
        the second result is None when the whole index was basic."""
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
        shape, strides, residual, offset, dim = [], [], [], self._offset, 0
        for sel in expanded:
            if sel is None:
                shape.append(1)
                strides.append(0)
                residual.append(None)
                continue
            extent, stride = self._shape[dim], self._strides[dim]
            if isinstance(sel, int):
                if sel < 0:
                    sel += extent
                if not 0 <= sel < extent:
                    raise IndexError(f"Cannot index at position {sel} in {extent} elements.")
                offset += sel * stride
            elif isinstance(sel, slice):
                start, stop, step = sel.indices(extent)
                shape.append(len(range(start, stop, step)))
                strides.append(stride * step)
                residual.append(None)
                offset += start * stride
            else:  # index array or mask: resolved by _fancy_plan
                shape.append(extent)
                strides.append(stride)
                residual.append(sel)
            dim += 1
        shape.extend(self._shape[dim:])
        strides.extend(self._strides[dim:])
        residual.extend([None] * (self.ndim - dim))
        view = Tensor._new_view(self._storage, tuple(shape), tuple(strides), offset)
        return view, (tuple(residual) if any(r is not None for r in residual) else None)

    def __getitem__(self, index) -> "Tensor":
        view, residual = self._basic_index(index)
        if residual is None:
            return view
        plan = _fancy_plan(view._shape, residual, self.device)
        storage = _C.gather_from_axes(
            x=view._C_view, new_shape=plan.new_shape, fancy_dims_in_src=plan.fancy_dims_in_src,
            fancy_dims_data=[t._C_view for t in plan.fancy_dims_data], out_axis_is_fancy=plan.out_axis_is_fancy,
            out_axis_target=plan.out_axis_target, checked=plan.checked)
        return Tensor._new_contiguous(storage, plan.new_shape)

    def __setitem__(self, index, value) -> None:
        target, residual = self._basic_index(index)
        if not isinstance(value, Tensor):
            value = Tensor(value, dtype=self.dtype, device=self.device)
        elif value.dtype != self.dtype:
            value = value.to(self.dtype)
        plan = None if residual is None else _fancy_plan(target._shape, residual, self.device)
        try:
            value = value.expand(*(target.shape if plan is None else plan.new_shape))
        except ValueError as e:
            raise IndexError(str(e)) from e
        if value._storage is self._storage:
            value = value._to_contiguous(force=True)
        if plan is None:
            _C.copy_view(src=value._C_view, out=target._C_view)
            return
        # The reference hands the *unsliced* tensor to scatter_to_axes (src/nanotorch/core.py:246-248),
        # which is only right when every basic selector is a full slice; the sliced view is used here,
        # which coincides with it in that case.
        _C.scatter_to_axes(
            src=value._C_view, out=target._C_view, fancy_dims_in_src=plan.fancy_dims_in_src,
            fancy_dims_data=[t._C_view for t in plan.fancy_dims_data], out_axis_is_fancy=plan.out_axis_is_fancy,
            out_axis_target=plan.out_axis_target, checked=plan.checked, unique=plan.unique)

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
        """Enables gradient tracking after construction.  Unlike the constructor this does not look at
        the dtype, as in the reference (src/nanotorch/core.py:536-538; its tests call
        ``arange(60, requires_grad=True)`` on an Int64 range)."""
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


# what the operators accept on either side (src/nanotorch/core.py: TensorLike)
TensorLike = Tensor | float | int | bool | list


# ---------------------------------------------------------------------------------------------
# Index-array / mask indexing plan (the reference's _FancyAxes, src/nanotorch/core.py:666-772)
class _FancyPlan:
    __slots__ = ("new_shape", "fancy_dims_in_src", "fancy_dims_data", "out_axis_is_fancy", "out_axis_target",
                 "checked", "unique")


def _host_index_array(sel, extent: int, dim: int):
    """A host selector (nested list, or a Cpu tensor) as a wrapped, range-checked int64 numpy array."""
    import numpy as np

    if isinstance(sel, Tensor):
        arr = sel.numpy()
    else:
        if not isinstance(sel, Sequence) or isinstance(sel, (str, bytes)):
            raise IndexError(f"Unexpected selector type {type(sel)}")
        try:
            probe = Tensor(sel)  # the reference's own inference of shape and dtype for nested lists
        except Exception as e:
            raise IndexError(f"Could not interpret index {dim} as a Tensor: {e}")
        arr = probe.numpy()
    if arr.dtype == np.bool_:
        if arr.ndim > 1:
            raise NotImplementedError("nD boolean masks not here (yet).")
        if arr.shape[0] != extent:
            raise IndexError(f"Wrong boolean index shape: {arr.shape[0]} (expected {extent}).")
        return np.flatnonzero(arr).astype(np.int64)
    flat = arr.reshape(-1)
    wrapped = np.where(flat < 0, flat + extent, flat)
    bad = np.flatnonzero((wrapped < 0) | (wrapped >= extent))
    if bad.size:
        raise IndexError(f"Invalid index {wrapped[bad[0]].item()} in axis of len {extent}.")
    return wrapped.astype(np.int64).reshape(arr.shape)


def _fancy_plan(shape: Shape, residual: tuple, device: Device) -> _FancyPlan:
    """Where the index dimensions land in the result and which result axis walks which source dim.

    ``residual[d]`` is the index-array / mask selector of dim ``d`` of the (already basic-indexed)
    view of shape ``shape``, or None.  Adjacent indexed dims are replaced in place by the broadcast
    index shape; indexed dims separated by a basic dim move the index shape to the front (the numpy
    rule the reference follows, src/nanotorch/core.py:737-763).
    Host selectors are wrapped and range-checked here (``checked``) and tested for distinct
    destinations (``unique``); Cuda index tensors are checked by the library.
    """
    import numpy as np

    fancy_dims, basic_axes, raw, host_arrays = [], [], [], []
    for dim in range(len(shape)):
        sel = residual[dim] if dim < len(residual) else None
        if sel is None:
            basic_axes.append(dim)
            continue
        fancy_dims.append(dim)
        if isinstance(sel, Tensor) and sel.device == Device.Cuda and sel.dtype != Dtype.Bool:
            if sel.dtype > Dtype.Int64:
                raise IndexError(f"Index tensors must be integer or Bool, got {sel.dtype.name}.")
            raw.append(sel.to(Dtype.Int64))
            host_arrays.append(None)
        else:
            if isinstance(sel, Tensor) and sel.device == Device.Cuda:
                sel = sel.cpu()  # a mask's extent is data dependent: read it back
            arr = _host_index_array(sel, shape[dim], dim)
            host_arrays.append(arr)
            raw.append(Tensor.from_numpy(arr, device))
    ind_shape = broadcast_shapes(*(t.shape for t in raw))  # RuntimeError when they do not broadcast, as in the reference
    plan = _FancyPlan()
    plan.fancy_dims_in_src = fancy_dims
    plan.fancy_dims_data = [t.expand(*ind_shape) for t in raw]
    plan.checked = all(a is not None for a in host_arrays)
    plan.unique = False
    if plan.checked:
        cols = [np.broadcast_to(a, ind_shape).reshape(-1) for a in host_arrays]
        if len(cols) == 1:
            plan.unique = np.unique(cols[0]).size == cols[0].size
        else:
            plan.unique = np.unique(np.stack(cols, axis=1), axis=0).shape[0] == cols[0].size
    basic_shape = [shape[d] for d in basic_axes]
    nidx = len(ind_shape)
    adjacent = all(b - a == 1 for a, b in zip(fancy_dims, fancy_dims[1:]))
    if adjacent:
        first = fancy_dims[0]  # == number of basic dims in front of the indexed block
        plan.new_shape = tuple(basic_shape[:first]) + tuple(ind_shape) + tuple(basic_shape[first:])
        plan.out_axis_is_fancy = [first <= i < first + nidx for i in range(len(plan.new_shape))]
        plan.out_axis_target = [
            (i - first) if first <= i < first + nidx else basic_axes[i if i < first else i - nidx]
            for i in range(len(plan.new_shape))]
    else:
        plan.new_shape = tuple(ind_shape) + tuple(basic_shape)
        plan.out_axis_is_fancy = [i < nidx for i in range(len(plan.new_shape))]
        plan.out_axis_target = [i if i < nidx else basic_axes[i - nidx] for i in range(len(plan.new_shape))]
    if len(plan.new_shape) > 8:
        raise RuntimeError("Indexing result has more than 8 dimensions.")
    return plan
