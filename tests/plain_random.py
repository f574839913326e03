"""The tests' own statement of the library's weight generator, element by element in plain
Python integers (no NumPy in the draw, no code shared with ``supersonic_b200``):

    key   = mix(seed XOR fnv1a64(name))
    z_j   = mix(key + (3 i + j + 1) * 0x9E3779B97F4A7C15 mod 2^64),  j = 0, 1, 2
    n     = (2 * (sum of the twelve 16-bit fields of z_0..z_2) - 12 * 65535) / 131072
    value = mean + std * n   (float64), rounded to float32, then to bfloat16 (nearest even)

The reference has no random weights; this recipe is the library's (``csrc/random_fill.cu``).
"""
import struct

M = (1 << 64) - 1


def fnv1a64(text):
    h = 0xCBF29CE484222325
    for b in text.encode("utf-8"):
        h = ((h ^ b) * 0x100000001B3) & M
    return h


def mix(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & M
    return z ^ (z >> 31)


def normal(seed, name, i):
    key = mix((seed & M) ^ fnv1a64(name))
    s = 0
    for j in range(3):
        z = mix((key + (3 * i + j + 1) * 0x9E3779B97F4A7C15) & M)
        s += (z & 0xFFFF) + ((z >> 16) & 0xFFFF) + ((z >> 32) & 0xFFFF) + (z >> 48)
    return (2 * s - 12 * 65535) / 131072.0


def to_float32(x):
    return struct.unpack("<f", struct.pack("<f", x))[0]


def to_bfloat16_bits(x):
    """Round a float32-representable number to bfloat16, nearest even; returns the 16 bits."""
    (u,) = struct.unpack("<I", struct.pack("<f", x))
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) & 0xFFFF


def value_bits(seed, name, i, mean, std):
    return to_bfloat16_bits(to_float32(mean + std * normal(seed, name, i)))
