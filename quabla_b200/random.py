"""Keys and samplers with the reference's streams, so that seeded weights and
collocation points are bit-identical to `quabla.random`.

SplitMix64 (crates/quabla-python/src/tensor.rs:327-345): the i-th output of
the stream seeded by `key` is mix(key + (i+1) * 0x9e3779b97f4a7c15), which
lets NumPy generate whole arrays at once.
  uniform  [minval, maxval): (bits >> 11) / 2^53 scaled, float32 by rounding
           and clamping into the interval (tensor.rs:1482-1534);
  normal   Box-Muller cosine branch from two open-unit draws per sample,
           u = ((bits >> 11) + 0.5) / 2^53 (tensor.rs:336-345, 1436-1454);
  glorot   normal * sqrt(2 / (fan_in + fan_out)) (python/quabla/random.py:197-204);
  split    the next `num` outputs of the stream (tensor.rs:1426-1433);
  fold_in  mix(key ^ mix-stream(data)) (tensor.rs:1539-1543).
"""

from __future__ import annotations

import math
import operator

import numpy as np

_MASK = (1 << 64) - 1
_GAMMA = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB


class Key:
    """An explicit random key: an unsigned 64-bit stream seed."""

    __slots__ = ("_value",)

    def __init__(self, value: int) -> None:
        self._value = operator.index(value) & _MASK

    @property
    def value(self) -> int:
        return self._value

    def __repr__(self) -> str:
        return f"Key({self._value})"

    def __eq__(self, other) -> bool:
        return isinstance(other, Key) and other._value == self._value

    def __hash__(self) -> int:
        return hash(("Key", self._value))


def _mix_scalar(z: int) -> int:
    z = ((z ^ (z >> 30)) * _M1) & _MASK
    z = ((z ^ (z >> 27)) * _M2) & _MASK
    return z ^ (z >> 31)


def _stream(key: int, count: int) -> np.ndarray:
    """The first `count` outputs of the SplitMix64 stream seeded by `key`."""
    with np.errstate(over="ignore"):
        z = np.uint64(key) + np.arange(1, count + 1, dtype=np.uint64) * np.uint64(_GAMMA)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
        return z ^ (z >> np.uint64(31))


def _key_value(key) -> int:
    if isinstance(key, Key):
        return key._value
    if isinstance(key, bool) or not isinstance(key, int):
        raise TypeError(f"expected a Key from quabla_b200.random.key, got {type(key).__name__}")
    return key & _MASK


def _shape(shape) -> tuple[int, ...]:
    if isinstance(shape, int):
        return (operator.index(shape),)
    return tuple(operator.index(s) for s in shape)


def _float_dtype(dtype, what: str) -> np.dtype:
    dtype = np.dtype(dtype)
    if dtype not in (np.float32, np.float64):
        raise TypeError(f"{what} requires dtype float32 or float64, got {dtype}")
    return dtype


def key(seed: int) -> Key:
    return Key(seed)


def split(key: Key, num: int = 2) -> tuple[Key, ...]:
    num = operator.index(num)
    if num < 1:
        raise ValueError(f"split requires num >= 1, got {num}")
    return tuple(Key(int(v)) for v in _stream(_key_value(key), num))


def fold_in(key: Key, data: int) -> Key:
    data = operator.index(data) & _MASK
    state = _key_value(key) ^ _mix_scalar((data + _GAMMA) & _MASK)
    return Key(_mix_scalar((state + _GAMMA) & _MASK))


def uniform(key: Key, shape=(), dtype=np.float64, minval: float = 0.0, maxval: float = 1.0) -> np.ndarray:
    dtype = _float_dtype(dtype, "uniform")
    minval, maxval = float(minval), float(maxval)
    width = maxval - minval
    if not (minval < maxval and math.isfinite(width)):
        raise ValueError(f"random_uniform requires finite minval < maxval, got [{minval}, {maxval})")
    shape = _shape(shape)
    count = int(np.prod(shape, dtype=np.int64))
    unit = (_stream(_key_value(key), count) >> np.uint64(11)).astype(np.float64) / float(1 << 53)
    value = minval + width * unit
    if dtype == np.float64:
        low, high = minval, np.nextafter(maxval, -np.inf)
    else:
        low32 = np.float32(minval)
        if float(low32) < minval:
            low32 = np.nextafter(low32, np.float32(np.inf))
        high32 = np.float32(maxval)
        if float(high32) >= maxval:
            high32 = np.nextafter(high32, np.float32(-np.inf))
        if low32 > high32:
            raise ValueError(f"no float32 value lies in [{minval}, {maxval})")
        low, high = float(low32), float(high32)
        value = value.astype(np.float32).astype(np.float64)
    return np.clip(value, low, high).astype(dtype).reshape(shape)


def _normal(key: Key, shape, dtype, stddev: float, what: str) -> np.ndarray:
    dtype = _float_dtype(dtype, what)
    shape = _shape(shape)
    count = int(np.prod(shape, dtype=np.int64))
    bits = (_stream(_key_value(key), 2 * count) >> np.uint64(11)).astype(np.float64)
    unit = (bits + 0.5) * (1.0 / float(1 << 53))
    radius = np.sqrt(-2.0 * np.log(unit[0::2]))
    angle = math.tau * unit[1::2]
    samples = 0.0 + stddev * (radius * np.cos(angle))
    return samples.astype(dtype).reshape(shape)


def normal(key: Key, shape=(), dtype=np.float64) -> np.ndarray:
    return _normal(key, shape, dtype, 1.0, "normal")


def glorot_normal(key: Key, shape, dtype=np.float64) -> np.ndarray:
    shape = _shape(shape)
    if len(shape) < 2 or any(s <= 0 for s in shape):
        raise ValueError(f"glorot_normal requires a weight shape of rank >= 2 with positive extents, got {shape}")
    receptive = math.prod(shape[:-2])
    fan_in, fan_out = shape[-2] * receptive, shape[-1] * receptive
    return _normal(key, shape, dtype, math.sqrt(2.0 / (fan_in + fan_out)), "glorot_normal")
