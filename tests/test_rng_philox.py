"""The checker of the optional device generator (Philox4x32-10, oracle/nt_oracle.c) against the
known-answer vectors published with the algorithm's reference library (Random123, kat_vectors:
`philox4x32 10 <counter> <key> <expected>`), and the stream layout the library documents."""

import numpy as np

KAT = [
    ([0, 0, 0, 0], [0, 0], [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]),
    ([0xFFFFFFFF] * 4, [0xFFFFFFFF] * 2, [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]),
    ([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0],
     [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]),
]


def test_known_answers(port):
    for ctr, key, want in KAT:
        assert port.philox(ctr, key) == want


def test_stream_layout(port):
    seed, offset = 0x0123456789ABCDEF, (1 << 32) - 2   # the block counter carries into the second word
    u = port.philox_uniform(seed, offset, 13)
    assert u.dtype == np.float32 and (u >= 0).all() and (u < 1).all()
    for b in range(4):
        at = offset + b
        words = port.philox([at & 0xFFFFFFFF, at >> 32, 0, 0], [seed & 0xFFFFFFFF, seed >> 32])
        for j in range(4):
            if 4 * b + j < 13:
                assert u[4 * b + j] == np.float32((words[j] >> 8) * 2.0 ** -24)
    # a later call continues where the previous one stopped, on a fresh block
    assert np.array_equal(port.philox_uniform(seed, offset + 2, 5), u[8:13])
    d = port.philox_uniform(seed, 7, 3, np.float64)
    words = port.philox([7, 0, 0, 0], [seed & 0xFFFFFFFF, seed >> 32])
    assert d[0] == (((words[1] << 32) | words[0]) >> 11) * 2.0 ** -53
    assert d[1] == (((words[3] << 32) | words[2]) >> 11) * 2.0 ** -53


def test_uniformity(port):
    u = port.philox_uniform(5, 0, 1 << 18).astype(np.float64)
    assert abs(u.mean() - 0.5) < 3e-3 and abs(u.var() - 1 / 12) < 2e-3
    hist, _ = np.histogram(u, bins=64, range=(0, 1))
    assert hist.min() > 0.9 * u.size / 64 and hist.max() < 1.1 * u.size / 64
