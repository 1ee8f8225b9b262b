"""The reference's random streams, one draw at a time — TEST INFRASTRUCTURE.

A scalar restatement of crates/quabla-python/src/tensor.rs:327-345 (SplitMix64,
open-unit uniform, Box-Muller normal), :1426-1433 (split_key), :1436-1472
(random_normal, glorot_normal), :1482-1534 (random_uniform with float32
rounding and clamping), :1539-1543 (fold_in_key).  Slow on purpose: it is the
check of the vectorised generators the product ships.
"""

from __future__ import annotations

import math

import numpy as np

MASK = (1 << 64) - 1


class Stream:
    def __init__(self, key: int) -> None:
        self.state = key & MASK

    def next(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & MASK
        v = self.state
        v = ((v ^ (v >> 30)) * 0xBF58476D1CE4E5B9) & MASK
        v = ((v ^ (v >> 27)) * 0x94D049BB133111EB) & MASK
        return v ^ (v >> 31)

    def open_unit(self) -> float:
        return ((self.next() >> 11) + 0.5) * (1.0 / float(1 << 53))

    def standard_normal(self) -> float:
        radius = math.sqrt(-2.0 * math.log(self.open_unit()))
        angle = math.tau * self.open_unit()
        return radius * math.cos(angle)


def split_key(key: int, count: int) -> list[int]:
    stream = Stream(key)
    return [stream.next() for _ in range(count)]


def fold_in_key(key: int, data: int) -> int:
    state = (key ^ Stream(data).next()) & MASK
    return Stream(state).next()


def random_normal(shape, key: int, mean: float = 0.0, stddev: float = 1.0) -> np.ndarray:
    stream = Stream(key)
    count = int(np.prod(shape, dtype=np.int64))
    return np.array([mean + stddev * stream.standard_normal() for _ in range(count)]).reshape(shape)


def glorot_normal(shape, key: int) -> np.ndarray:
    return random_normal(shape, key, 0.0, math.sqrt(2.0 / (shape[0] + shape[1])))


def random_uniform(shape, key: int, minval: float = 0.0, maxval: float = 1.0, dtype=np.float64) -> np.ndarray:
    width = maxval - minval
    if np.dtype(dtype) == np.float64:
        low, high = minval, float(np.nextafter(maxval, -np.inf))
    else:
        low32 = np.float32(minval)
        if float(low32) < minval:
            low32 = np.nextafter(low32, np.float32(np.inf))
        high32 = np.float32(maxval)
        if float(high32) >= maxval:
            high32 = np.nextafter(high32, np.float32(-np.inf))
        low, high = float(low32), float(high32)
    stream = Stream(key)
    out = []
    for _ in range(int(np.prod(shape, dtype=np.int64))):
        unit = (stream.next() >> 11) / float(1 << 53)
        value = minval + width * unit
        if np.dtype(dtype) == np.float32:
            value = float(np.float32(value))
        out.append(min(max(value, low), high))
    return np.array(out, dtype=dtype).reshape(shape)
