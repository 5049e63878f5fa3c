"""GPU parity of index-array / mask gather and scatter (nt_gather_from_axes / nt_scatter_to_axes
through the C ABI): bit-exact against what the reference returned for the same index expressions
(golden fixtures), against the CPU oracle on larger seeded inputs in every element width, and --
at a benchmark-sized gather -- through properties that need no oracle (permutation round trip)."""

import numpy as np
import pytest

from oracle import oracle as O
from tests.util import INDEX_GET_CASES, INDEX_SET_CASES, assert_bit_exact, index_case

pytestmark = pytest.mark.gpu


def dev(nt, a):
    return nt.Tensor.from_numpy(a, "cuda")


@pytest.mark.parametrize("k", range(len(INDEX_GET_CASES)))
def test_getitem_golden(nt, golden, k):
    got = dev(nt, golden["idx/in/x"])[index_case(INDEX_GET_CASES[k])]
    assert_bit_exact(got.numpy(), golden[f"idx/get/{k}"], INDEX_GET_CASES[k])


@pytest.mark.parametrize("k", range(len(INDEX_SET_CASES)))
def test_setitem_golden(nt, golden, k):
    source, _ = INDEX_SET_CASES[k]
    t = dev(nt, golden["idx/in/x"])
    v0 = t.version
    t[index_case(source)] = dev(nt, golden[f"idx/set/{k}/value"])
    assert_bit_exact(t.numpy(), golden[f"idx/set/{k}/out"], source)
    assert t.version == v0  # scatter leaves Storage::version alone, as in the reference


def test_getitem_int64_and_bool(nt, golden):
    index = index_case(INDEX_GET_CASES[2])
    got = dev(nt, golden["idx/in/xi"])[index]
    assert got.dtype == nt.int64 and np.array_equal(got.numpy(), golden["idx/get_int64"])
    mask = golden["idx/in/xi"] > 0
    assert np.array_equal(dev(nt, mask)[index].numpy(), mask[index])
    d = golden["idx/in/x"].astype(np.float64)
    assert np.array_equal(dev(nt, d)[index].numpy(), d[index])
    i32 = golden["idx/in/xi"].astype(np.int32)
    assert np.array_equal(dev(nt, i32)[index].numpy(), i32[index])


def test_row_gather_and_scatter_vector_path(nt, port):
    """x[idx] with wide rows: 16-byte work items; odd widths and offset views: element path."""
    rng = np.random.default_rng(11)
    for rows, width in [(1000, 256), (257, 130), (64, 5), (300, 1024)]:
        x = rng.standard_normal((rows, width)).astype(np.float32)
        idx = rng.integers(-rows, rows, 777).astype(np.int64)
        assert_bit_exact(dev(nt, x)[idx.tolist()].numpy(), O.getitem(port, x, (idx.tolist(),)), f"rows {rows}x{width}")
        # column gather (index array on the unit-stride dim) and a sliced, misaligned source view
        cols = rng.integers(0, width, 33).tolist()
        assert_bit_exact(dev(nt, x)[:, cols].numpy(), x[:, cols], "columns")
        assert_bit_exact(dev(nt, x)[1:, 1:][idx[idx >= 0][:50].clip(0, rows - 2).tolist()].numpy(),
                         x[1:, 1:][idx[idx >= 0][:50].clip(0, rows - 2).tolist()], "offset view")
        assert_bit_exact(dev(nt, x).T[cols].numpy(), x.T[cols], "transposed source")
        # scatter: unique rows (single pass) and colliding rows (ordering pass), against the oracle
        perm = rng.permutation(rows)[: rows // 2].astype(np.int64)
        v = rng.standard_normal((perm.size, width)).astype(np.float32)
        t = dev(nt, x)
        t[perm.tolist()] = dev(nt, v)
        want = x.copy()
        O.setitem(port, want, (perm.tolist(),), v)
        assert_bit_exact(t.numpy(), want, "scatter unique rows")
        dup = rng.integers(0, 8, 500).astype(np.int64)
        v = rng.standard_normal((dup.size, width)).astype(np.float32)
        t = dev(nt, x)
        t[dup.tolist()] = dev(nt, v)
        want = x.copy()
        O.setitem(port, want, (dup.tolist(),), v)
        assert_bit_exact(t.numpy(), want, "scatter colliding rows: the last writer wins")


def test_device_index_tensors(nt, port):
    """Index arrays that already live on the device: wrapped and range-checked by the library."""
    rng = np.random.default_rng(12)
    x = rng.standard_normal((40, 9, 16)).astype(np.float32)
    i0 = rng.integers(-40, 40, (6, 1)).astype(np.int64)
    i2 = rng.integers(-16, 16, (1, 5)).astype(np.int32)
    got = dev(nt, x)[dev(nt, i0), :, dev(nt, i2)]
    assert_bit_exact(got.numpy(), O.getitem(port, x, (i0, slice(None), i2.astype(np.int64))), "two device index arrays")
    assert got.shape == (6, 5, 9)
    t = dev(nt, x)
    v = rng.standard_normal((6, 5, 9)).astype(np.float32)
    t[dev(nt, i0), :, dev(nt, i2)] = dev(nt, v)   # collisions possible: ordering pass
    want = x.copy()
    O.setitem(port, want, (i0, slice(None), i2.astype(np.int64)), v)
    assert_bit_exact(t.numpy(), want, "scatter through device index arrays")
    mask = rng.random(40) > 0.5
    assert_bit_exact(dev(nt, x)[dev(nt, mask)].numpy(), x[mask], "device mask")
    before = dev(nt, x)
    with pytest.raises(IndexError, match="Invalid index 40 in axis of len 40"):
        before[dev(nt, np.array([0, 40], np.int64))]
    with pytest.raises(IndexError, match="Invalid index -1 in axis of len 40"):
        before[dev(nt, np.array([3, -41], np.int64))] = 1.0
    assert_bit_exact(before.numpy(), x, "a rejected scatter writes nothing")
    with pytest.raises(IndexError, match="Invalid index 7 in axis of len 5"):
        dev(nt, np.zeros((5, 2), np.float32))[[7]]


def test_colliding_scatter_through_views_and_broadcast_indices(nt):
    """The ordering pass keys its owner table by the destination index tuple and compares source positions over
    the index-array dims only: colliding rows into a reversed, strided destination view; index arrays that
    broadcast against each other with a basic dim in between; a large colliding row scatter on the 16-byte path.
    numpy assigns duplicates in source order, as the reference's sequential loop does."""
    rng = np.random.default_rng(21)
    x = rng.standard_normal((64, 48)).astype(np.float32)
    dup = rng.integers(-10, 10, 300).astype(np.int64)
    v = rng.standard_normal((300, 24)).astype(np.float32)
    t = dev(nt, x)
    t[::-1, ::2][dup.tolist()] = dev(nt, v)
    want = x.copy()
    want[::-1, ::2][dup] = v
    assert_bit_exact(t.numpy(), want, "colliding rows into a reversed, strided view")

    y = rng.standard_normal((12, 7, 10)).astype(np.float32)
    i0 = rng.integers(0, 3, (40, 1)).astype(np.int64)       # many collisions
    i2 = rng.integers(0, 2, (1, 30)).astype(np.int64)
    v = rng.standard_normal((40, 30, 7)).astype(np.float32)
    t = dev(nt, y)
    t[dev(nt, i0), :, dev(nt, i2)] = dev(nt, v)
    want = y.copy()
    want[i0, :, i2] = v
    assert_bit_exact(t.numpy(), want, "two broadcasting index arrays around a basic dim")

    big = rng.standard_normal((2048, 1024)).astype(np.float32)
    idx = rng.integers(0, 64, 4096).astype(np.int64)
    v = rng.standard_normal((4096, 1024)).astype(np.float32)
    t = dev(nt, big)
    t[dev(nt, idx)] = dev(nt, v)
    want = big.copy()
    want[idx] = v
    assert_bit_exact(t.numpy(), want, "4096 rows into 64 destinations")


def test_raw_entry_points_check_their_plan(nt):
    _C = nt._C
    x = dev(nt, np.zeros((4, 6), np.float32))
    idx = dev(nt, np.array([0, 1], np.int64))
    common = dict(fancy_dims_in_src=[0], fancy_dims_data=[idx._C_view])
    with pytest.raises(ValueError):   # result extent does not match the index array
        _C.gather_from_axes(x=x._C_view, new_shape=[3, 6], out_axis_is_fancy=[True, False], out_axis_target=[0, 1], **common)
    with pytest.raises(ValueError):   # a basic axis pointing at the indexed dim
        _C.gather_from_axes(x=x._C_view, new_shape=[2, 4], out_axis_is_fancy=[True, False], out_axis_target=[0, 0], **common)
    with pytest.raises(ValueError):   # index arrays must be Int64
        _C.gather_from_axes(x=x._C_view, new_shape=[2, 6], fancy_dims_in_src=[0],
                            fancy_dims_data=[dev(nt, np.array([0, 1], np.int32))._C_view],
                            out_axis_is_fancy=[True, False], out_axis_target=[0, 1])
    with pytest.raises(RuntimeError):  # dtype mismatch between src and out
        _C.scatter_to_axes(src=dev(nt, np.zeros((2, 6), np.float64))._C_view, out=x._C_view,
                           out_axis_is_fancy=[True, False], out_axis_target=[0, 1], **common)
    empty = _C.gather_from_axes(x=x._C_view, new_shape=[0, 6], fancy_dims_in_src=[0],
                                fancy_dims_data=[dev(nt, np.zeros((0,), np.int64))._C_view],
                                out_axis_is_fancy=[True, False], out_axis_target=[0, 1])
    assert empty.size == 0


def test_full_size_row_permutation_round_trip(nt):
    """[8192, 8192] fp32 (256 MiB): gather by a permutation, scatter back through the same permutation
    -> the original, bit for bit; gather by the inverse permutation undoes the gather."""
    rng = np.random.default_rng(13)
    n = 8192
    x = rng.standard_normal((n, n)).astype(np.float32)
    perm = rng.permutation(n).astype(np.int64)
    inv = np.empty_like(perm)
    inv[perm] = np.arange(n)
    tx = dev(nt, x)
    tp, ti = dev(nt, perm), dev(nt, inv)
    g = tx[tp]
    assert tx.equals(g[ti])
    back = dev(nt, np.zeros((n, n), np.float32))
    back[tp] = g
    assert tx.equals(back)
    rows = rng.integers(0, n, 16)
    assert_bit_exact(g[rows.tolist()].numpy(), x[perm[rows]], "sampled rows against numpy")
