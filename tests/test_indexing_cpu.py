"""Index-array / mask indexing without a GPU: the oracle's restatement of gather_from_axes /
scatter_to_axes and of the reference's index plan against the reference's own results
(tests/golden/reference_cpu.npz, idx/*), and the product's host-side plan against the oracle's."""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import INDEX_GET_CASES, INDEX_SET_CASES, INDEX_SHAPE, index_case


def _oracles():
    yield O.PortOracle()
    if O.ref_available():
        yield O.RefOracle()


@pytest.mark.parametrize("k", range(len(INDEX_GET_CASES)))
def test_oracle_getitem_matches_reference(golden, k):
    x = golden["idx/in/x"]
    want = golden[f"idx/get/{k}"]
    for o in _oracles():
        got = O.getitem(o, x, index_case(INDEX_GET_CASES[k]))
        assert got.shape == want.shape and np.array_equal(got.view(np.uint32), want.view(np.uint32)), (o.kind, k)


def test_oracle_getitem_int64(golden, port):
    got = O.getitem(port, golden["idx/in/xi"], index_case(INDEX_GET_CASES[2]))
    assert got.dtype == np.int64 and np.array_equal(got, golden["idx/get_int64"])


@pytest.mark.parametrize("k", range(len(INDEX_SET_CASES)))
def test_oracle_setitem_matches_reference(golden, k):
    source, _ = INDEX_SET_CASES[k]
    for o in _oracles():
        x = golden["idx/in/x"].copy()
        O.setitem(o, x, index_case(source), golden[f"idx/set/{k}/value"])
        assert np.array_equal(x.view(np.uint32), golden[f"idx/set/{k}/out"].view(np.uint32)), (o.kind, k)


def test_oracle_agrees_with_numpy_where_the_rules_coincide(port):
    # every case except the int-before-slice one (numpy counts the int as an index array there)
    rng = np.random.default_rng(7)
    x = rng.standard_normal(INDEX_SHAPE).astype(np.float32)
    for k, source in enumerate(INDEX_GET_CASES):
        if source.startswith("(0, slice(None)"):
            continue
        index = index_case(source)
        assert np.array_equal(O.getitem(port, x, index), x[index]), source


def test_oracle_index_errors(port):
    x = np.zeros(INDEX_SHAPE, np.float32)
    with pytest.raises(IndexError, match="Invalid index 5 in axis of len 5"):
        O.getitem(port, x, ([0, 5],))
    with pytest.raises(IndexError, match="Invalid index -2 in axis of len 5"):
        O.getitem(port, x, ([-7],))
    with pytest.raises(IndexError, match="Wrong boolean index shape: 3"):
        O.getitem(port, x, ([True, False, True],))


@pytest.mark.parametrize("k", range(len(INDEX_GET_CASES)))
def test_host_plan_matches_the_oracle_plan(nt, golden, k):
    """nanotorch_b200.tensor._fancy_plan (CPU tensors as index holders, no kernel involved)."""
    from nanotorch_b200.tensor import _fancy_plan

    index = index_case(INDEX_GET_CASES[k])
    t = nt.Tensor(np.zeros(INDEX_SHAPE, np.float32).tolist())
    view, residual = t._basic_index(index)
    assert residual is not None
    plan = _fancy_plan(view.shape, residual, nt.Device.Cpu)
    basic, res = O._split_index(index, len(INDEX_SHAPE))
    want = O.fancy_plan(np.zeros(INDEX_SHAPE, np.float32)[basic].shape, res)
    assert tuple(plan.new_shape) == tuple(want.new_shape) == golden[f"idx/get/{k}"].shape
    assert list(plan.fancy_dims_in_src) == list(want.fancy_dims_in_src)
    assert [bool(f) for f in plan.out_axis_is_fancy] == [bool(f) for f in want.out_axis_is_fancy]
    assert list(plan.out_axis_target) == list(want.out_axis_target)
    for mine, theirs in zip(plan.fancy_dims_data, want.fancy_dims_data):
        assert mine.shape == theirs.shape and mine.dtype == nt.int64
        assert np.array_equal(np.array(mine.tolist()), theirs)
    assert plan.checked


def test_host_plan_uniqueness_and_errors(nt):
    from nanotorch_b200.tensor import _fancy_plan

    t = nt.Tensor(np.zeros(INDEX_SHAPE, np.float32).tolist())

    def plan_of(index):
        view, residual = t._basic_index(index)
        return _fancy_plan(view.shape, residual, nt.Device.Cpu)

    assert plan_of(([4, 0, -2],)).unique
    assert not plan_of(([4, 0, -1],)).unique              # -1 wraps onto 4
    assert not plan_of(([0, -5],)).unique                 # -5 wraps onto 0
    assert plan_of(([0, 0], [1, 2])).unique               # distinct (row, column) pairs
    assert not plan_of(([0, 0], [1, 1])).unique
    assert plan_of(([True, False, True, False, True],)).unique
    with pytest.raises(IndexError, match="Invalid index 5 in axis of len 5"):
        plan_of(([0, 5],))
    with pytest.raises(IndexError, match="Invalid index -2 in axis of len 5"):
        plan_of(([-7],))
    with pytest.raises(IndexError, match="Wrong boolean index shape: 3"):
        plan_of(([True, False, True],))
    with pytest.raises(NotImplementedError):
        plan_of(([[True, False], [False, True]],))
    with pytest.raises(RuntimeError):
        plan_of(([0, 1, 2], [0, 1]))                      # index arrays that do not broadcast (RuntimeError in the reference too)
    with pytest.raises(IndexError):
        t[0, 0, 0, [0]]                                   # too many indices
    empty = plan_of(([],))                                # an empty index list selects nothing
    assert empty.new_shape == (0, 6, 7) and empty.fancy_dims_data[0].dtype == nt.int64
    assert plan_of((slice(None), [[]])).new_shape == (5, 1, 0, 7)
    # a basic index still returns a view of the same storage
    assert t[1:3, None, 2].storage is t.storage and t[1:3, None, 2].shape == (2, 1, 7)


def test_device_kernels_are_required(nt):
    t = nt.Tensor(np.zeros((4, 3), np.float32).tolist())  # Cpu storage
    with pytest.raises(RuntimeError, match="requires Cuda"):
        t[[0, 1]]
    with pytest.raises(RuntimeError, match="requires Cuda"):
        t[[0, 1]] = 1.0
