"""Draw keys for temperature sampling.

A draw is identified by (seed, stream, index): the request's seed, its stream number (by
default the order in which it was submitted) and the index of the output token.  The key is a
64-bit mix of the three; the sampling kernel finishes the hash (splitmix64) and takes the top
24 bits as a uniform number in [0, 1).  ``uniform_from_key`` restates the kernel's arithmetic
for tests.  The reference has no random sampling (src/cloud_engine/scheduler.py:69-71).
"""

from __future__ import annotations

MASK = (1 << 64) - 1


def draw_key(seed: int, stream: int, index: int) -> int:
    x = (
        (seed & MASK) * 0x9E3779B97F4A7C15
        + (stream & MASK) * 0xD1B54A32D192ED03
        + (index & MASK) * 0x8CB92BA72F3D8DD7
        + 0x632BE59BD9B4E019
    ) & MASK
    return x


def as_signed(key: int) -> int:
    """The same 64 bits as a signed integer (what an int64 tensor stores)."""
    return key - (1 << 64) if key >= (1 << 63) else key


def uniform_from_key(key: int) -> float:
    x = key & MASK
    x ^= x >> 30
    x = (x * 0xBF58476D1CE4E5B9) & MASK
    x ^= x >> 27
    x = (x * 0x94D049BB133111EB) & MASK
    x ^= x >> 31
    return (x >> 40) / 16777216.0
