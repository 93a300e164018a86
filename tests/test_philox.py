"""Known-answer and statistical checks of the counter-based Gaussian stream (CPU)."""
import numpy as np

from dizo_b200.ops import philox


def test_philox_known_answers():
    # Random123 known-answer vectors for Philox4x32-10
    out = philox.philox4x32(0, 0, 0, 0, 0, 0)
    assert [int(x) for x in out] == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    out = philox.philox4x32(0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF, 0xFFFFFFFF)
    assert [int(x) for x in out] == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    out = philox.philox4x32(0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344, 0xA4093822, 0x299F31D0)
    assert [int(x) for x in out] == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_gaussian_moments():
    z = philox.gaussian(seed=1234, tensor_id=3, numel=1 << 20).astype(np.float64)
    assert abs(z.mean()) < 4e-3
    assert abs(z.var() - 1.0) < 5e-3
    assert abs((z ** 3).mean()) < 2e-2
    assert abs((z ** 4).mean() - 3.0) < 5e-2
    assert abs(np.corrcoef(z[0::2], z[1::2])[0, 1]) < 5e-3


def test_gaussian_is_layout_invariant():
    full = philox.gaussian(7, 11, 4096 * 3)
    # contiguous shard
    assert np.array_equal(philox.gaussian(7, 11, 4096, elem_base=4096), full[4096:8192])
    # column shard of a [96, 128] matrix
    part = philox.gaussian_cols(7, 11, rows=96, local_cols=32, full_cols=128, col0=64)
    assert np.array_equal(part.reshape(96, 32), full.reshape(96, 128)[:, 64:96])
    # different tensors / seeds decorrelate
    other = philox.gaussian(7, 12, 4096 * 3)
    assert abs(np.corrcoef(full, other)[0, 1]) < 0.05


def test_z_stream_statistics_with_reduced_rounds():
    """The perturbation stream runs Philox4x32 with Z_PHILOX_ROUNDS rounds: uniform 16-bit indices,
    unit-variance normals, no correlation between neighbouring counters, tensors or seeds."""
    import numpy as np
    from dizo_b200.ops import philox as P
    assert P.Z_PHILOX_ROUNDS == 7
    n = 1 << 22
    z = P.gaussian(123, 5, n)
    assert abs(z.mean()) < 5 / np.sqrt(n) and abs(z.var() - 1.0) < 0.01
    assert abs(np.mean(z ** 3)) < 0.01 and abs(np.mean(z ** 4) - 3.0) < 0.05
    # neighbouring elements / neighbouring 8-element groups (consecutive counters)
    for lag in (1, 2, 7, 8, 9, 64, 4096):
        c = float(np.mean(z[:-lag] * z[lag:]))
        assert abs(c) < 5 / np.sqrt(n), (lag, c)
    # other tensor id, other seed, nearby seed
    for other in (P.gaussian(123, 6, n), P.gaussian(124, 5, n), P.gaussian(123 + (1 << 32), 5, n)):
        assert abs(float(np.mean(z * other))) < 5 / np.sqrt(n)
    # uniformity of the raw 16-bit indices over 4096 coarse bins
    grp = np.arange(n >> 3, dtype=np.uint32)
    words = np.stack(P.philox4x32(grp, np.uint32(5), np.uint32(0), np.uint32(0), 123, 0, rounds=P.Z_PHILOX_ROUNDS), -1)
    idx = np.concatenate([(words & np.uint32(0xFFFF)).ravel(), (words >> np.uint32(16)).ravel()])
    counts = np.bincount(idx >> 4, minlength=4096).astype(np.float64)
    expect = idx.size / 4096
    chi2 = float(((counts - expect) ** 2 / expect).sum())
    assert abs(chi2 - 4095) < 6 * np.sqrt(2 * 4095), chi2
    # every bit position of the 32-bit words is balanced
    for bit in range(32):
        frac = float(((words >> np.uint32(bit)) & np.uint32(1)).mean())
        assert abs(frac - 0.5) < 5 * 0.5 / np.sqrt(words.size), (bit, frac)
