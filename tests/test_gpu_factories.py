"""Factories written by kernels (eye, arange, the optional Philox generator) through the C ABI:
exact against numpy / the oracle; the default generator still reproduces the reference's seeded
host stream (golden fixtures)."""

import numpy as np
import pytest

from tests.util import assert_bit_exact

pytestmark = pytest.mark.gpu

NP = {"bool_": np.bool_, "int32": np.int32, "int64": np.int64, "float32": np.float32, "float64": np.float64}


def _np(nt, storage, shape):
    return nt.Tensor._new_contiguous(storage, shape).numpy()


@pytest.mark.parametrize("dtype", list(NP))
def test_eye_and_arange_on_device(nt, dtype):
    dt = getattr(nt, dtype)
    for n in (0, 1, 7, 300):
        got = _np(nt, nt._C.eye(n, dt, nt.Device.Cuda), (n, n))
        assert got.dtype == NP[dtype] and np.array_equal(got, np.eye(n).astype(NP[dtype]))
    for n, start, step in ((0, 0, 1), (10, 0, 1), (1000, -500, 3), (17, 5, -2), (5, 2 ** 40, 2 ** 33)):
        got = _np(nt, nt._C.arange(n, start, step, dt, nt.Device.Cuda), (n,))
        want = (start + np.arange(n, dtype=np.int64) * step)
        want = (want != 0) if dtype == "bool_" else want.astype(NP[dtype])
        assert np.array_equal(got, want), (dtype, n, start, step)


def test_default_generator_is_the_reference_stream(nt, golden):
    assert nt._C.get_rng_mode() == nt._C.RNG_HOST_MT19937_64
    nt.manual_seed(42)
    assert_bit_exact(_np(nt, nt._C.uniform(16, nt.float32, nt.Device.Cuda), (16,)), golden["rng/seed42"], "seed 42")


def test_device_generator_matches_its_checker(nt, port):
    _C = nt._C
    _C.set_rng_mode(_C.RNG_DEVICE_PHILOX)
    try:
        nt.manual_seed(1234567890123)
        a = _np(nt, _C.uniform(1001, nt.float32, nt.Device.Cuda), (1001,))      # 251 blocks, ragged tail
        b = _np(nt, _C.uniform(6, nt.float32, nt.Device.Cuda), (6,))            # continues at block 251
        c = _np(nt, _C.uniform(33, nt.float64, nt.Device.Cuda), (33,))          # 2 per block from block 253
        assert_bit_exact(a, port.philox_uniform(1234567890123, 0, 1001), "first call")
        assert_bit_exact(b, port.philox_uniform(1234567890123, 251, 6), "second call continues the stream")
        assert np.array_equal(c, port.philox_uniform(1234567890123, 253, 33, np.float64))
        nt.manual_seed(1234567890123)
        assert_bit_exact(_np(nt, _C.uniform(1001, nt.float32, nt.Device.Cuda), (1001,)), a, "reseeding restarts the stream")
        big = _np(nt, _C.uniform(1 << 24, nt.float32, nt.Device.Cuda), (1 << 24,))
        assert big.min() >= 0.0 and big.max() < 1.0
        assert abs(big.astype(np.float64).mean() - 0.5) < 5e-4 and abs(big.astype(np.float64).var() - 1 / 12) < 5e-4
        assert_bit_exact(big[:4096], port.philox_uniform(1234567890123, 251, 4096), "head of the large draw")
        # parameter initialisation without a host loop or a host-to-device copy
        import nanotorch_b200.nn as nn

        layer = nn.Linear(512, 256, device="cuda")
        w = layer.parameters()[0].numpy()
        bound = np.sqrt(6.0 / 512)
        assert w.shape == (512, 256) and np.abs(w).max() <= bound and w.std() > 0.5 * bound / np.sqrt(3)
        with pytest.raises(ValueError):
            _C.set_rng_mode(7)
    finally:
        _C.set_rng_mode(_C.RNG_HOST_MT19937_64)


def test_functional_forms_on_device(nt):
    """nt.argmax/argmin/eq/gt/geq/lt/leq, randint, eye, arange through the public functions
    (src/nanotorch/ops.py:63-85, 155-232; factories.py:115-252)."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((37, 130)).astype(np.float32)
    y = rng.standard_normal((130,)).astype(np.float32)
    tx, ty = nt.Tensor.from_numpy(x, "cuda"), nt.Tensor.from_numpy(y, "cuda")
    assert np.array_equal(nt.argmax(tx, 1).numpy(), x.argmax(axis=1)) and nt.argmax(tx, 1).dtype == nt.int64
    assert np.array_equal(nt.argmin(tx, 0, keepdim=True).numpy(), x.argmin(axis=0)[None, :])
    assert int(nt.argmax(tx).numpy()) == int(x.argmax())
    for fn, ref in ((nt.eq, np.equal), (nt.gt, np.greater), (nt.geq, np.greater_equal), (nt.lt, np.less),
                    (nt.leq, np.less_equal)):
        got = fn(tx, ty)
        assert got.dtype == nt.bool_ and np.array_equal(got.numpy(), ref(x, y))
    assert np.array_equal(nt.eq(tx, tx).numpy(), np.ones_like(x, dtype=bool))
    nt.manual_seed(7)
    r = nt.randint(-3, 9, (1000,), device="cuda")
    assert r.dtype == nt.int64 and r.numpy().min() >= -3 and r.numpy().max() < 9 and len(np.unique(r.numpy())) >= 11
    nt.manual_seed(7)
    u = nt.rand(1000, device="cuda").numpy()
    assert np.array_equal(r.numpy(), (u * np.float32(12) + np.float32(-3)).astype(np.int64))  # the reference's recipe
    assert np.array_equal(nt.eye(5, device="cuda").numpy(), np.eye(5, dtype=np.float32))
    assert np.array_equal(nt.arange(6, 2, 3, device="cuda").numpy(), 2 + 3 * np.arange(6))
    assert nt.randint(0, 2, device="cuda").shape == ()
