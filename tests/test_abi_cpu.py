"""CPU-side checks of the C-ABI library: it loads, exports every symbol declared in include/nt_b200.h,
keeps the reference's error classes, and its host-side pieces (storages, factories, RNG stream) work
without a GPU.  No compute entry point is exercised here: without a device they must fail loudly."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

REPO = Path(__file__).resolve().parent.parent


def test_library_exports_every_declared_symbol(nt):
    header = (REPO / "include" / "nt_b200.h").read_text()
    declared = sorted(set(re.findall(r"\b(nt_[a-z0-9_]+)\s*\(", header)))
    assert len(declared) > 70
    lib = ctypes.CDLL(str(REPO / "nanotorch_b200" / "lib" / "libnt_b200.so"))
    missing = [name for name in declared if not hasattr(lib, name)]
    assert missing == []


def test_header_has_no_torch_types():
    header = (REPO / "include" / "nt_b200.h").read_text()
    assert "at::" not in header and "torch::" not in header and "#include <torch" not in header


def test_storage_host_side(nt):
    _C = nt._C
    s = _C.Storage.from_iterable([1.5, 2.5, -3.0], _C.Dtype.Float32, _C.Device.Cpu)
    assert (s.size, s.itemsize, s.dtype, s.device, s.version) == (3, 4, _C.Dtype.Float32, _C.Device.Cpu, 0)
    mem = memoryview(s)
    assert list(mem) == [1.5, 2.5, -3.0]
    mem[1] = 7.0  # writable buffer protocol
    assert list(memoryview(s.clone())) == [1.5, 7.0, -3.0]
    assert list(memoryview(s.cast(_C.Dtype.Int64))) == [1, 7, -3]
    assert list(memoryview(s.cast(_C.Dtype.Bool))) == [True, True, True]
    assert s.cast(_C.Dtype.Float32) is s and s.to(_C.Device.Cpu) is s
    z = _C.Storage.allocate(0, _C.Dtype.Int32, _C.Device.Cpu)
    assert z.size == 0 and len(memoryview(z)) == 0
    with pytest.raises(TypeError):
        _C.Storage.from_iterable([1.5], _C.Dtype.Int64, _C.Device.Cpu)


def test_factories_and_rng_stream(nt):
    _C = nt._C
    cpu = _C.Device.Cpu
    assert list(memoryview(_C.zeros(3, _C.Dtype.Int32, cpu))) == [0, 0, 0]
    assert list(memoryview(_C.ones(2, _C.Dtype.Float64, cpu))) == [1.0, 1.0]
    assert list(memoryview(_C.full(2, 2.5, _C.Dtype.Float32, cpu))) == [2.5, 2.5]
    assert list(memoryview(_C.full(2, True, _C.Dtype.Int64, cpu))) == [1, 1]
    assert list(memoryview(_C.eye(2, _C.Dtype.Int32, cpu))) == [1, 0, 0, 1]
    assert list(memoryview(_C.arange(4, 3, -2, _C.Dtype.Int64, cpu))) == [3, 1, -1, -3]
    # the reference's own known answer (tests/test_factories.py:239-242)
    _C.manual_seed(42)
    u = list(memoryview(_C.uniform(2, _C.Dtype.Float32, cpu)))
    assert abs(u[0] - 0.7551555037498474) < 1e-6 and abs(u[1] - 0.6390313506126404) < 1e-6
    with pytest.raises(ValueError):
        _C.uniform(2, _C.Dtype.Int32, cpu)  # float dtypes only (DispatchFloat)
    with pytest.raises(TypeError):
        _C.full(2, "x", _C.Dtype.Float32, cpu)


def test_rng_matches_oracle_stream(nt, golden, port):
    _C = nt._C
    _C.manual_seed(0)
    u = np.array(memoryview(_C.uniform(16, _C.Dtype.Float32, _C.Device.Cpu)), dtype=np.float32)
    assert np.array_equal(u, golden["rng/seed0"]) and np.array_equal(u, port.uniform(0, 16))


def _view(nt, values, shape, strides=None, offset=0, dtype=None):
    _C = nt._C
    dtype = dtype or _C.Dtype.Float32
    s = _C.Storage.from_iterable(values, dtype, _C.Device.Cpu)
    if strides is None:
        strides, acc = [], 1
        for e in reversed(shape):
            strides.insert(0, acc)
            acc *= e
    return _C.TensorView(s, shape, strides, offset)


def test_error_classes_match_the_reference(nt):
    """RuntimeError / ValueError / TypeError exactly where pybind11 raises them for the reference
    (std::runtime_error / std::invalid_argument / py::type_error)."""
    _C = nt._C
    a = _view(nt, [1.0] * 6, (2, 3))
    b = _view(nt, [1.0] * 6, (3, 2))
    with pytest.raises(RuntimeError, match="same shape"):
        _C.add(a, b)
    with pytest.raises(RuntimeError, match="same dtype"):
        _C.add(a, _view(nt, [1] * 6, (2, 3), dtype=_C.Dtype.Int64))
    with pytest.raises(RuntimeError, match="same shape"):
        _C.add_inplace(a, b)
    with pytest.raises(ValueError, match="different ndim"):
        _C.matmul(a, _view(nt, [1.0] * 6, (6,)))
    with pytest.raises(ValueError, match=">=2d"):
        _C.matmul(_view(nt, [1.0] * 6, (6,)), _view(nt, [1.0] * 6, (6,)))
    with pytest.raises(ValueError, match="Invalid matmul shape"):
        _C.matmul(a, _view(nt, [1.0] * 6, (2, 3)))
    with pytest.raises(RuntimeError, match="exceeds its storage"):
        _C.neg(_view(nt, [1.0] * 6, (2, 4)))
    with pytest.raises(RuntimeError, match="more than 8 dim"):
        _C.neg(_view(nt, [1.0], (1,) * 9))
    with pytest.raises(TypeError):
        _C.add(a, "not a view")
    with pytest.raises(TypeError):
        _C.pow(a, "2")


def test_compute_fails_loudly_without_a_gpu(nt):
    """There is no CPU fallback behind the ABI: a CPU storage handed to an op is an error."""
    _C = nt._C
    a = _view(nt, [1.0] * 6, (2, 3))
    for call in (lambda: _C.add(a, a), lambda: _C.exp(a), lambda: _C.sum(a, [0], _C.Dtype.Float32),
                 lambda: _C.matmul(a, _view(nt, [1.0] * 6, (3, 2))), lambda: _C.add_inplace(a, a),
                 lambda: _C.clone_contiguous_view_from(a), lambda: _C.relu_backward(a, a),
                 lambda: _C.sgd_update(a, a, 0.1)):
        with pytest.raises(RuntimeError, match="requires Cuda"):
            call()
    if not _C.is_cuda_available():
        with pytest.raises(RuntimeError, match="CUDA device required"):
            _C.Storage.allocate(4, _C.Dtype.Float32, _C.Device.Cuda)


def test_matmul_mode_switch(nt):
    _C = nt._C
    assert _C.get_matmul_mode() == 1
    _C.set_matmul_mode(0)
    assert _C.get_matmul_mode() == 0
    _C.set_matmul_mode(3)
    assert _C.get_matmul_mode() == 3
    _C.set_matmul_mode(1)
    with pytest.raises(ValueError):
        _C.set_matmul_mode(7)
