"""The random-weights formula, restated with Python integers and ``struct`` rounding only.

A tensor of the random-weights mode is a closed formula of (seed, tensor name, element index); the
reference builds its toy models from closed formulas for the same reason
(crates/bfi-models/src/lib.rs:52-79: any implementation can rebuild them).  This file shares no
code with the product package: the product computes the same values with numpy on the CPU and with
a CUDA kernel on the GPU, and the tests compare all three bit for bit.
"""
import hashlib
import math
import struct

MASK = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def f32(x: float) -> float:
    """``x`` rounded to the nearest float32 (ties to even), as a Python float."""
    return struct.unpack("<f", struct.pack("<f", x))[0]


def key_of(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode("utf-8")).digest()[:8], "little")


def mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK
    return z ^ (z >> 31)


def fields16(x: int) -> int:
    return (x & 0xFFFF) + ((x >> 16) & 0xFFFF) + ((x >> 32) & 0xFFFF) + (x >> 48)


def value(seed: int, name: str, index: int, role: str) -> float:
    """Element ``index`` (row-major) of tensor ``name`` as float32: N(0, 0.02) for matrices and
    tables, 1 + N(0, 0.1) for norm weights."""
    std, offset = (0.1, 1.0) if role == "norm" else (0.02, 0.0)
    scale = f32(std / (131072.0 * math.sqrt(2.0 / 3.0)))
    base = (key_of(seed, name) + (2 * index + 1) * GOLDEN) & MASK
    s = fields16(mix64(base)) + fields16(mix64((base + GOLDEN) & MASK))
    c = 2 * s - 8 * 65535
    return f32(offset + f32(float(c) * scale))


def bf16_bits(x: float) -> int:
    """The bfloat16 nearest to float32 ``x`` (ties to even), as its 16 bits."""
    b = struct.unpack("<I", struct.pack("<f", x))[0]
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16) & 0xFFFF
