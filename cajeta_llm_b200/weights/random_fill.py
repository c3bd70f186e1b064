"""The random-weights generator on the host: element ``i`` of a tensor from ``(key, i)``.

It restates, in numpy, the few integer operations of ``csrc/random_fill.cu`` - two rounds
of the splitmix64 finaliser, eight 16-bit integers summed and centred, one float32 multiply -
so that a tensor drawn on the CPU and the same tensor drawn on a GPU hold the same bits
(tested).  A value depends on the seed, the tensor's name and the element's index in the
row-major tensor only.  The distribution is the bell of a sum of eight uniform integers
(Irwin-Hall): mean 0, the standard deviation asked for, tails bounded at 4.9 of them.
(The reference has random weights only as test fixtures, selftest/ToyModel.cajeta:116-120.)
"""
from __future__ import annotations

import hashlib
import math

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
# standard deviation of 2 * sum(u_0..u_7) - 8 * 65535 with u uniform on 0..65535
_UNIT = 2.0 * math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)
CHUNK = 1 << 18


def tensor_key(seed: int, name: str) -> int:
    """64 bits from (seed, tensor name)."""
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little")


def scale_for(std: float) -> np.float32:
    """The float32 factor that turns the centred integer into a value of standard deviation ``std``."""
    return np.float32(std / _UNIT)


def _mix64(z: np.ndarray, t: np.ndarray) -> None:
    """The splitmix64 finaliser, in place (``t`` is scratch of the same shape)."""
    np.right_shift(z, np.uint64(30), out=t)
    z ^= t
    z *= _M1
    np.right_shift(z, np.uint64(27), out=t)
    z ^= t
    z *= _M2
    np.right_shift(z, np.uint64(31), out=t)
    z ^= t


def _add_sum16(h: np.ndarray, t: np.ndarray, acc: np.ndarray) -> None:
    """acc += the four 16-bit fields of h."""
    m = np.uint64(0xFFFF)
    for shift in (0, 16, 32, 48):
        np.right_shift(h, np.uint64(shift), out=t)
        t &= m
        acc += t


def fill(count: int, key: int, std: float, start: int = 0) -> np.ndarray:
    """Elements ``start .. start + count`` of the tensor with this key, float32."""
    out = np.empty((count,), dtype=np.float32)
    scale = scale_for(std)
    n_buf = min(CHUNK, max(count, 1))
    z, t, acc = (np.empty((n_buf,), dtype=np.uint64) for _ in range(3))
    with np.errstate(over="ignore"):
        for lo in range(0, count, CHUNK):
            n = min(CHUNK, count - lo)
            zz, tt, aa = z[:n], t[:n], acc[:n]
            zz[:] = np.arange(start + lo, start + lo + n, dtype=np.uint64)
            zz *= np.uint64(GOLDEN)
            zz += np.uint64(key)
            _mix64(zz, tt)
            aa[:] = 0
            _add_sum16(zz, tt, aa)
            zz += np.uint64(GOLDEN)
            _mix64(zz, tt)
            _add_sum16(zz, tt, aa)
            centred = 2 * aa.astype(np.int64) - 8 * 65535
            out[lo:lo + n] = centred.astype(np.float32) * scale
    return out
