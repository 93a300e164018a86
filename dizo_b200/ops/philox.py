"""NumPy statement of the framework's Gaussian stream (the oracle for ``csrc/philox.cuh``).

``z(seed, tensor_id, e)`` is a pure function of the seed, the tensor's stream id and the
element index ``e`` inside the *full* tensor:

    words = Philox4x32-7(counter=(e >> 3, tensor_id, stream, 0), key=(seed_lo, seed_hi))
    w     = words[(e & 7) >> 1];  u = w & 0xffff for even e, w >> 16 for odd e
    i = u & 1023 (quantile bin), k = u >> 10 (position inside the bin)
    z = bfloat16(a'_i + b_i * (1 + (2k + 1)/128))          one fused multiply-add, one rounding

(:func:`gauss_table_entries`: the inverse normal CDF, piecewise linear over 1024 equal-probability bins).
The CUDA kernels hold the same 1024 (a', b) pairs in shared memory and evaluate the same fused
multiply-add, so the host stream equals the device stream bit for bit.  The
reference instead calls ``torch.manual_seed(seed)`` and ``torch.normal`` per tensor
(large_models/trainer.py:1438-1444); bit-matching that generator is not a goal.
"""
from __future__ import annotations

import numpy as np

M0 = np.uint64(0xD2511F53)
M1 = np.uint64(0xCD9E8D57)
W0 = np.uint32(0x9E3779B9)
W1 = np.uint32(0xBB67AE85)
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0, k1, rounds: int = 10):
    """Vectorised Philox4x32; all inputs broadcastable uint32 arrays."""
    c0 = np.asarray(c0, dtype=np.uint32)
    shape = np.broadcast(c0, c1, c2, c3).shape
    c0 = np.broadcast_to(c0, shape).astype(np.uint32)
    c1 = np.broadcast_to(np.asarray(c1, dtype=np.uint32), shape).astype(np.uint32)
    c2 = np.broadcast_to(np.asarray(c2, dtype=np.uint32), shape).astype(np.uint32)
    c3 = np.broadcast_to(np.asarray(c3, dtype=np.uint32), shape).astype(np.uint32)
    k0 = np.uint32(k0)
    k1 = np.uint32(k1)
    with np.errstate(over="ignore"):
        for _ in range(rounds):
            p0 = M0 * c0.astype(np.uint64)
            p1 = M1 * c2.astype(np.uint64)
            hi0 = (p0 >> np.uint64(32)).astype(np.uint32)
            lo0 = (p0 & _MASK).astype(np.uint32)
            hi1 = (p1 >> np.uint64(32)).astype(np.uint32)
            lo1 = (p1 & _MASK).astype(np.uint32)
            n0 = hi1 ^ c1 ^ k0
            n2 = hi0 ^ c3 ^ k1
            c0, c1, c2, c3 = n0, lo1, n2, lo0
            k0 = np.uint32((int(k0) + int(W0)) & 0xFFFFFFFF)
            k1 = np.uint32((int(k1) + int(W1)) & 0xFFFFFFFF)
    return c0, c1, c2, c3


_TABLE = None
_TABLE_BITS = None


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns (uint16), round to nearest even."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    with np.errstate(over="ignore"):
        r = (b + np.uint32(0x7FFF) + ((b >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)
    return r.astype(np.uint16)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << np.uint32(16)).view(np.float32)


def f64_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float64 -> bf16 with ONE rounding (nearest even).  NumPy / PyTorch convert through float32,
    which rounds twice; here the float32 step rounds to odd, which makes the second rounding exact.
    This is the host statement of the device's ``fma.rn.bf16x2`` result rounding."""
    x = np.ascontiguousarray(x, dtype=np.float64)
    f = x.astype(np.float32)
    inexact = f.astype(np.float64) != x
    too_big = np.abs(f.astype(np.float64)) > np.abs(x)
    f = np.where(inexact & too_big, np.nextafter(f, np.float32(0)), f).astype(np.float32)
    b = f.view(np.uint32) | inexact.astype(np.uint32)         # sticky bit
    return f32_to_bf16_bits(b.view(np.float32))


GAUSS_BINS = 1024     # equal-probability bins of the piecewise-linear inverse CDF
GAUSS_SUB = 64        # positions inside a bin


def gauss_table_entries() -> np.ndarray:
    """uint32[1024]: per quantile bin i the pair (a'_i, b_i) as bf16 bit patterns (a' in the low half, b in
    the high half) with z = a'_i + b_i * m_k, m_k = 1 + (2k + 1)/128: the line with the mean and variance of
    the 64 quantiles Phi^-1((i + (k + 0.5)/64)/1024), k = 0..63, of bin i (computed in float64), shifted by
    1.5 b so that m_k comes straight from the index bits.  This is what the kernels hold in shared memory."""
    global _TABLE_BITS
    if _TABLE_BITS is None:
        from scipy.special import ndtri
        i = np.arange(GAUSS_BINS, dtype=np.float64)[:, None]
        k = np.arange(GAUSS_SUB, dtype=np.float64)[None, :]
        q = ndtri((i + (k + 0.5) / GAUSS_SUB) / GAUSS_BINS)                 # [1024, 64]
        f = (2 * k + 1) / 128.0 - 0.5                                        # m_k - 1.5, mean zero
        # line with the bin's own mean and variance (equal to the least-squares line except in the two
        # tail bins, where it keeps the stream's variance at 1 instead of flattening the tail)
        a = q.mean(1)
        b = np.sqrt(q.var(1) / (f * f).mean())
        b_bits = f64_to_bf16_bits(b)
        a_bits = f64_to_bf16_bits(a - 1.5 * bf16_bits_to_f32(b_bits).astype(np.float64))
        _TABLE_BITS = a_bits.astype(np.uint32) | (b_bits.astype(np.uint32) << np.uint32(16))
    return _TABLE_BITS


def gauss_from_u16(u: np.ndarray) -> np.ndarray:
    """16-bit indices -> normals (float32 holding bf16 values): bf16(b * m + a') with one rounding."""
    u = u.astype(np.uint32)
    e = gauss_table_entries()[u & np.uint32(GAUSS_BINS - 1)]
    a = bf16_bits_to_f32((e & np.uint32(0xFFFF)).astype(np.uint16)).astype(np.float64)
    b = bf16_bits_to_f32((e >> np.uint32(16)).astype(np.uint16)).astype(np.float64)
    m = 1.0 + (2.0 * (u >> np.uint32(10)).astype(np.float64) + 1.0) / 128.0
    return bf16_bits_to_f32(f64_to_bf16_bits(b * m + a))                     # product and sum exact in float64


def gauss_table() -> np.ndarray:
    """float32[65536]: the normal for every 16-bit index (a view of the stream's quantile function)."""
    global _TABLE
    if _TABLE is None:
        _TABLE = gauss_from_u16(np.arange(65536, dtype=np.uint32))
    return _TABLE


def gauss_words(words: np.ndarray) -> np.ndarray:
    """[..., 4] uint32 -> [..., 8] float32 normals (two 16-bit indices per word)."""
    w = words.astype(np.uint32)
    tab = gauss_table()
    out = np.empty(w.shape[:-1] + (8,), dtype=np.float32)
    out[..., 0::2] = tab[w & np.uint32(0xFFFF)]
    out[..., 1::2] = tab[w >> np.uint32(16)]
    return out


def perturb_bf16(theta_bits: np.ndarray, coef: float, z: np.ndarray) -> np.ndarray:
    """bf16 bits of ``theta + bf16(coef) * z`` rounded once: the packed perturbation of the sweep
    kernel (``perturb8_packed`` in csrc/philox.cuh).  ``z`` holds bf16-representable values."""
    c = bf16_bits_to_f32(f32_to_bf16_bits(np.float32(coef).reshape(1)))[0].astype(np.float64)
    v = bf16_bits_to_f32(theta_bits).astype(np.float64)
    return f64_to_bf16_bits(v + c * z.astype(np.float64))     # 8+8-bit product and the sum are exact in float64


# Rounds of the perturbation stream z.  Philox4x32 is specified with 10 rounds by default and is
# "Crush-resistant" from 7 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11); the
# sweep spends a third of its instructions in the rounds, so z and the stochastic-rounding stream of the
# update use 7.  The scalar draws of the gamma search keep 10.  Must equal Z_PHILOX_ROUNDS in csrc/philox.cuh.
Z_PHILOX_ROUNDS = 7


def gaussian(seed: int, tensor_id: int, numel: int, elem_base: int = 0, stream: int = 0) -> np.ndarray:
    """z for elements [elem_base, elem_base + numel) of tensor ``tensor_id`` (fp32)."""
    assert elem_base % 8 == 0
    g0 = elem_base >> 3
    ngroups = (numel + 7) >> 3
    grp = (np.arange(g0, g0 + ngroups, dtype=np.uint64) & _MASK).astype(np.uint32)
    c = philox4x32(grp, np.uint32(tensor_id), np.uint32(stream), np.uint32(0),
                   seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF, rounds=Z_PHILOX_ROUNDS)
    words = np.stack(c, axis=-1)
    return gauss_words(words).reshape(-1)[:numel]


def gaussian_cols(seed: int, tensor_id: int, rows: int, local_cols: int, full_cols: int,
                  col0: int, elem_base: int = 0) -> np.ndarray:
    """z for a column slice [col0, col0+local_cols) of a [rows, full_cols] tensor."""
    full = gaussian(seed, tensor_id, rows * full_cols, elem_base).reshape(rows, full_cols)
    return np.ascontiguousarray(full[:, col0:col0 + local_cols]).reshape(-1)


def scalar_gaussian(seed: int, index: int, it: int) -> float:
    """The gamma-search draw for constraint ``index`` at search iteration ``it``."""
    c = philox4x32(np.uint32(index), np.uint32(it), np.uint32(2), np.uint32(0),
                   seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    words = np.stack([np.atleast_1d(x) for x in c], axis=-1)
    return float(gauss_words(words)[0, 0])
