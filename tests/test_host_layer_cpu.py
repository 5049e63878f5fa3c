"""Host logic of the Tensor/autograd mirror, no kernels: view bookkeeping, shape rules, error behaviour
(the cases the reference's own tests pin in tests/test_ops/test_tensor_core*.py)."""

import pytest

from nanotorch_b200.autograd import _matmul_shapes, normalize_axes
from nanotorch_b200.dp import shard_bounds
from nanotorch_b200.tensor import broadcast_shapes, contiguous_strides


def test_construction_and_dtype_inference(nt):
    t = nt.Tensor([[1, 2, 3], [4, 5, 6]])
    assert t.shape == (2, 3) and t.dtype == nt.int64 and t.strides == ((3, 1), 0) and t.numel == 6 and len(t) == 2
    assert nt.Tensor([1, 2.5]).dtype == nt.float32 and nt.Tensor([True, False]).dtype == nt.bool_
    assert nt.Tensor(3.5).shape == () and nt.Tensor(3.5).item() == 3.5
    assert nt.Tensor([1.7, -2.2], dtype=nt.int64).tolist() == [1, -2]
    assert nt.Tensor([]).shape == (0,) and nt.Tensor([]).is_empty
    with pytest.raises(ValueError):
        nt.Tensor([[1, 2], [3]])
    with pytest.raises(ValueError):
        nt.Tensor([1, [2]])
    with pytest.raises(TypeError):
        nt.Tensor(["a"])
    with pytest.raises(RuntimeError):
        nt.Tensor([1, 2], requires_grad=True)
    with pytest.raises(ValueError):
        nt.Tensor([1.0], device="tpu")


def test_views_share_storage_and_never_copy(nt):
    t = nt.Tensor([[1.0, 2.0, 3.0], [4.0, 5.0, 6.0]])
    tt = t.T
    assert tt.storage is t.storage and tt.shape == (3, 2) and tt.strides == ((1, 3), 0)
    assert tt.tolist() == [[1.0, 4.0], [2.0, 5.0], [3.0, 6.0]]
    assert t.transpose(0, 1).tolist() == tt.tolist() and t.transpose(1, 1).storage is t.storage
    e = nt.Tensor([1.0, 2.0, 3.0]).expand(2, 3)
    assert e.strides == ((0, 1), 0) and e.tolist() == [[1.0, 2.0, 3.0]] * 2
    assert t.reshape(3, 2).storage is t.storage and t.reshape(2, 3).storage is t.storage
    assert t.reshape(6).tolist() == [1.0, 2.0, 3.0, 4.0, 5.0, 6.0]
    s = t[:, ::-1]
    assert s.strides == ((3, -1), 2) and s.tolist() == [[3.0, 2.0, 1.0], [6.0, 5.0, 4.0]]
    assert t[1].tolist() == [4.0, 5.0, 6.0] and t[-1, -1].item() == 6.0
    assert t[None, 1, ..., None].shape == (1, 3, 1) and t[..., 0].tolist() == [1.0, 4.0]
    assert t[0:1, 1:].shape == (1, 2)
    with pytest.raises(IndexError):
        t[2]
    with pytest.raises(IndexError):
        t[0, 0, 0]
    with pytest.raises(ValueError):
        t.reshape(4, 2)
    with pytest.raises(ValueError):
        nt.Tensor([1.0, 2.0]).expand(3)
    with pytest.raises(IndexError):
        nt.Tensor._new_view(t.storage, (2, 4), None, None)  # view past the end of its storage


def test_shape_rules():
    assert broadcast_shapes((5, 7), (7,)) == (5, 7) and broadcast_shapes((2, 1, 3), (4, 1)) == (2, 4, 3)
    assert broadcast_shapes() == () and broadcast_shapes((), (3,)) == (3,)
    with pytest.raises(RuntimeError):
        broadcast_shapes((2, 3), (4,))
    assert contiguous_strides((2, 3, 4)) == (12, 4, 1) and contiguous_strides(()) == ()
    assert _matmul_shapes((5, 7), (7, 3)) == ((5, 7), (7, 3), (5, 3))
    assert _matmul_shapes((7,), (7, 3)) == ((1, 7), (7, 3), (3,))
    assert _matmul_shapes((5, 7), (7,)) == ((5, 7), (7, 1), (5,))
    assert _matmul_shapes((7,), (7,)) == ((1, 7), (7, 1), ())
    assert _matmul_shapes((3, 5, 4), (4, 6)) == ((3, 5, 4), (3, 4, 6), (3, 5, 6))
    assert _matmul_shapes((2, 1, 5, 4), (3, 4, 6)) == ((2, 3, 5, 4), (2, 3, 4, 6), (2, 3, 5, 6))
    with pytest.raises(RuntimeError):
        _matmul_shapes((5, 7), (6, 3))
    with pytest.raises(RuntimeError):
        _matmul_shapes((), (3,))


def test_axis_normalisation(nt):
    x = nt.Tensor([[[0.0] * 4] * 3] * 2)
    assert normalize_axes(None, x) == (0, 1, 2) and normalize_axes((), x) == (0, 1, 2)
    assert normalize_axes(-1, x) == (2,) and normalize_axes((0, -1), x) == (0, 2)
    with pytest.raises(ValueError):
        normalize_axes((0, 0), x)
    with pytest.raises(IndexError):
        normalize_axes(3, x)
    with pytest.raises(TypeError):
        normalize_axes((0.5,), x)


def test_autograd_bookkeeping_errors(nt):
    t = nt.Tensor([1.0, 2.0])
    with pytest.raises(RuntimeError):
        t.backward()  # does not require grad
    t.enable_grad()
    with pytest.raises(RuntimeError):
        t.backward()  # not a scalar
    assert t.requires_grad and t.is_leaf and t.grad is None
    with pytest.raises(RuntimeError):
        nt.Tensor([1, 2], requires_grad=True)     # the constructor checks the dtype ...
    i = nt.Tensor([1, 2])
    i.enable_grad()                               # ... enable_grad does not (src/nanotorch/core.py:536-538)
    assert i.requires_grad and nt.arange(4, requires_grad=True).requires_grad
    with pytest.raises(TypeError):
        nt.Tensor([1, 2]).to(nt.Device.Cuda if False else nt.int64).mean()  # mean of an integer tensor


def test_shard_bounds_partition_the_batch():
    for n, world in [(16384, 1), (16384, 8), (10, 4), (7, 8)]:
        pieces = [shard_bounds(n, r, world) for r in range(world)]
        assert pieces[0][0] == 0 and pieces[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(pieces, pieces[1:]))
        sizes = [hi - lo for lo, hi in pieces]
        assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(8, 2, 2)


def test_linear_one_call_path_is_device_only(nt):
    """LinearOp (bias fused into the GEMM) is chosen for 2-D fp32 device tensors only; everything else
    takes the composed matmul + add of the reference."""
    from nanotorch_b200.autograd import LinearOp

    x = nt.Tensor([[1.0, 2.0, 3.0, 4.0]])
    W = nt.Tensor([[0.5] * 3] * 4)
    b = nt.Tensor([0.0, 1.0, 2.0])
    assert not LinearOp.applicable(x, W, b)              # Cpu storages
    with pytest.raises(RuntimeError, match="requires Cuda"):
        (x @ W) + b


def test_factories_and_functional_names_of_the_reference(nt):
    """Signatures of src/nanotorch/factories.py and ops.py (Cpu storages: no kernel involved)."""
    assert nt.full(2, 3, value=1.5).tolist() == [[1.5] * 3] * 2 and nt.full(2, value=7, dtype=nt.int64).tolist() == [7, 7]
    assert nt.eye(3).tolist() == [[1.0, 0.0, 0.0], [0.0, 1.0, 0.0], [0.0, 0.0, 1.0]] and nt.eye(2, dtype=nt.bool_).dtype == nt.bool_
    assert nt.arange(4, 1, 2).tolist() == [1, 3, 5, 7] and nt.arange(3).dtype == nt.int64
    assert nt.arange(3, dtype=nt.float32).tolist() == [0.0, 1.0, 2.0] and nt.arange(0).shape == (0,)
    assert nt.zeros(2, 2).shape == (2, 2) and nt.ones(3, dtype=nt.int32).tolist() == [1, 1, 1]
    nt.manual_seed(42)
    u = nt.rand(2)
    assert abs(u.tolist()[0] - 0.7551555037498474) < 1e-6      # the reference's own known answer for seed 42
    with pytest.raises(ValueError):
        nt.rand(2, dtype=nt.int64)
    with pytest.raises(ValueError):
        nt.randint(0, 5, (3,), dtype=nt.bool_)
    with pytest.raises(ValueError):
        nt.argmax(nt.Tensor([1.0, 2.0]), axis=(0,))
    with pytest.raises(IndexError):
        nt.argmin(nt.zeros(0, 3), axis=0)
    assert nt.argmax(nt.zeros(0, 3), axis=1).shape == (0,)
    for name in ("eq", "gt", "geq", "lt", "leq", "argmax", "argmin", "randint", "TensorLike"):
        assert hasattr(nt, name)


def test_repr_has_the_references_format(nt):
    """src/nanotorch/core.py:141-164 -- checked against the reference's own output when this was written."""
    assert repr(nt.Tensor(3.5)) == "nt.Tensor(3.5)"
    assert repr(nt.Tensor(list(range(7)))) == "nt.Tensor([0, 1, 2, 3, 4, 5, 6])"
    assert repr(nt.Tensor(list(range(20)))) == "nt.Tensor([0, 1, 2, ..., 17, 18, 19])"
    assert repr(nt.Tensor([[1.0, 2.0], [3.0, 4.0]])) == "nt.Tensor([1.0, 2.0]\n          [3.0, 4.0])"
    six = nt.Tensor([[10 * r + c for c in range(10)] for r in range(6)])
    assert repr(six) == ("nt.Tensor([0, 1, 2, ..., 7, 8, 9]\n          [10, 11, 12, ..., 17, 18, 19]\n          ...\n"
                         "          [40, 41, 42, ..., 47, 48, 49]\n          [50, 51, 52, ..., 57, 58, 59])")
    assert repr(nt.zeros(2, 2, 2)) == "nt.Tensor(shape=(2, 2, 2), 8 x <Float32>, d: Cpu)"
    assert repr(six.T[1:3]) == "nt.Tensor([1, 11, 21, 31, 41, 51]\n          [2, 12, 22, 32, 42, 52])"   # through a view
