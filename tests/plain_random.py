"""The random-weights generator restated with Python integers, one element at a time.

It shares no code with the package: the key is the first 8 bytes (little endian) of
SHA-256 of "<seed>:<tensor name>"; element i takes two rounds of the splitmix64 finaliser
over key + i * golden, reads the 128 bits as eight 16-bit integers, centres twice their
sum, and multiplies, in float32, by the float32 of std / (2 sqrt(8 (65536^2 - 1) / 12)).
A stored bfloat16 value is that float32 rounded to nearest even.  (The reference has random
weights only as test fixtures, selftest/ToyModel.cajeta:116-120; this generator is the
engine's own.)
"""
import hashlib
import math
import struct

M64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def key_of(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix(z: int) -> int:
    z ^= z >> 30
    z = (z * 0xBF58476D1CE4E5B9) & M64
    z ^= z >> 27
    z = (z * 0x94D049BB133111EB) & M64
    return z ^ (z >> 31)


def _f32(x: float) -> float:
    return struct.unpack("<f", struct.pack("<f", x))[0]


def value(seed: int, name: str, index: int, std: float) -> float:
    """Element ``index`` (row-major) of tensor ``name`` as the float32 the generator computes."""
    h1 = _mix((key_of(seed, name) + index * GOLDEN) & M64)
    h2 = _mix((h1 + GOLDEN) & M64)
    total = sum((h >> s) & 0xFFFF for h in (h1, h2) for s in (0, 16, 32, 48))
    centred = 2 * total - 8 * 65535
    scale = _f32(std / (2.0 * math.sqrt(8.0 * (65536.0 ** 2 - 1.0) / 12.0)))
    return _f32(float(centred) * scale)           # the product of two float32 values, rounded once


def to_bfloat16(x: float) -> float:
    """Round a float32 value to bfloat16, to nearest even."""
    (u,) = struct.unpack("<I", struct.pack("<f", x))
    u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000
    return struct.unpack("<f", struct.pack("<I", u))[0]
