"""Learning-rate schedules for the device trainer: `schedule(step) -> float` evaluated on the host.

The surface follows the reference's `python/quabla/_schedules.py:30-176` (itself modelled on the optax
schedules of the same names): `constant`, `exponential_decay`, `cosine_decay`, `warmup_cosine_decay`
and `piecewise_constant`, same argument order, same `ValueError`s.  `step` is the number of completed
optimizer updates, so the first update runs at `schedule(0)`; `optim.Trainer` evaluates the schedule
before every `qb200_plan_optimizer_step` and passes the rate in the call's `qb200_opt_config`
(the reference does the same through its executor's `learning_rate` setter,
python/quabla/optim.py:520-550).

Each schedule is a small callable object that prints and pickles its configuration; nothing here
touches the device.
"""

from __future__ import annotations

import math
import operator
import sys
from typing import Sequence

__all__ = ["constant", "exponential_decay", "cosine_decay", "warmup_cosine_decay", "piecewise_constant"]


def _real(value, name: str) -> float:
    value = float(value)
    if math.isnan(value) or math.isinf(value):
        raise ValueError(f"{name} must be finite")
    return value


def _count(value, name: str, minimum: int) -> int:
    value = operator.index(value)
    if value < minimum:
        raise ValueError(f"{name} must be a positive integer" if minimum > 0 else f"{name} must be nonnegative")
    return value


class _Schedule:
    """Base: printable, picklable."""

    __slots__ = ()

    def __repr__(self) -> str:
        fields = ", ".join(f"{name}={getattr(self, name)!r}" for name in self.__slots__)
        return f"{type(self).__name__}({fields})"

    def __getstate__(self):
        return {name: getattr(self, name) for name in self.__slots__}

    def __setstate__(self, state):
        for name, value in state.items():
            object.__setattr__(self, name, value)


class constant(_Schedule):
    """`value` at every step."""

    __slots__ = ("value",)

    def __init__(self, value: float) -> None:
        self.value = _real(value, "value")

    def __call__(self, step: int) -> float:
        return self.value


class exponential_decay(_Schedule):
    """`init_value * decay_rate ** ((step - transition_begin) / transition_steps)`.

    `init_value` until `transition_begin`; `staircase` floors the exponent; `end_value` is a floor when
    `decay_rate < 1` and a cap otherwise.  The product is formed in logarithms when the bare power
    overflows or goes subnormal, so a representable rate is returned even then.
    """

    __slots__ = ("init_value", "transition_steps", "decay_rate", "transition_begin", "staircase", "end_value")

    def __init__(self, init_value: float, transition_steps: int, decay_rate: float, transition_begin: int = 0,
                 staircase: bool = False, end_value: float | None = None) -> None:
        self.init_value = _real(init_value, "init_value")
        self.transition_steps = _count(transition_steps, "transition_steps", 1)
        self.decay_rate = _real(decay_rate, "decay_rate")
        if self.decay_rate <= 0.0:
            raise ValueError("decay_rate must be positive")
        self.transition_begin = _count(transition_begin, "transition_begin", 0)
        self.staircase = bool(staircase)
        self.end_value = None if end_value is None else _real(end_value, "end_value")

    def _scaled(self, exponent: float) -> float:
        start = self.init_value
        if start == 0.0:
            return start
        try:
            power = self.decay_rate ** exponent
        except OverflowError:
            power = math.inf
        if math.isfinite(power) and power >= sys.float_info.min:
            return start * power
        # |start| * rate^e = exp(ln|start| + e ln rate): the sum can be in range when the power is not.
        magnitude = math.log(abs(start)) + exponent * math.log(self.decay_rate)
        try:
            return math.copysign(math.exp(magnitude), start)
        except OverflowError:
            if self.end_value is None:
                raise
            return math.copysign(math.inf, start)

    def __call__(self, step: int) -> float:
        elapsed = step - self.transition_begin
        if elapsed <= 0:
            rate = self.init_value
        else:
            exponent = elapsed / self.transition_steps
            rate = self._scaled(float(math.floor(exponent)) if self.staircase else exponent)
        if self.end_value is None:
            return rate
        return max(rate, self.end_value) if self.decay_rate < 1.0 else min(rate, self.end_value)


class cosine_decay(_Schedule):
    """`init_value * (c + alpha * (1 - c))`, `c = (1 + cos(pi * min(step, decay_steps) / decay_steps)) / 2`.

    Equal to optax's `(1 - alpha) * c + alpha`, written so that both end points are exact:
    `init_value` at step 0 and `alpha * init_value` from `decay_steps` on.
    """

    __slots__ = ("init_value", "decay_steps", "alpha")

    def __init__(self, init_value: float, decay_steps: int, alpha: float = 0.0) -> None:
        self.init_value = _real(init_value, "init_value")
        self.decay_steps = _count(decay_steps, "decay_steps", 1)
        self.alpha = _real(alpha, "alpha")

    def weight(self, step: int) -> float:
        """The cosine factor c in [0, 1]: 1 at step 0, 0 from `decay_steps` on."""
        if step <= 0:
            return 1.0
        if step >= self.decay_steps:
            return 0.0
        return 0.5 * (1.0 + math.cos(math.pi * step / self.decay_steps))

    def __call__(self, step: int) -> float:
        c = self.weight(step)
        return self.init_value * (c + self.alpha * (1.0 - c))


class warmup_cosine_decay(_Schedule):
    """Linear warm-up from `init_value` to `peak_value` over `warmup_steps`, then cosine decay to `end_value`.

    `decay_steps` counts from step 0 (it includes the warm-up): the rate is `peak_value` at
    `warmup_steps` and `end_value` from `decay_steps` on.  Both segments are convex combinations of
    their end points, so opposite-signed huge end points do not overflow and a zero end point is exact.
    """

    __slots__ = ("init_value", "peak_value", "warmup_steps", "decay_steps", "end_value")

    def __init__(self, init_value: float, peak_value: float, warmup_steps: int, decay_steps: int,
                 end_value: float = 0.0) -> None:
        self.init_value = _real(init_value, "init_value")
        self.peak_value = _real(peak_value, "peak_value")
        self.end_value = _real(end_value, "end_value")
        self.warmup_steps = _count(warmup_steps, "warmup_steps", 0)
        self.decay_steps = operator.index(decay_steps)
        if self.decay_steps <= self.warmup_steps:
            raise ValueError("decay_steps must exceed warmup_steps")

    def __call__(self, step: int) -> float:
        if step < self.warmup_steps:
            w = step / self.warmup_steps
            return self.init_value * (1.0 - w) + self.peak_value * w
        span = self.decay_steps - self.warmup_steps
        done = min(step - self.warmup_steps, span)
        c = 1.0 if done <= 0 else 0.0 if done >= span else 0.5 * (1.0 + math.cos(math.pi * done / span))
        return self.peak_value * c + self.end_value * (1.0 - c)


class piecewise_constant(_Schedule):
    """`values[i]` while `boundaries[i - 1] <= step < boundaries[i]`; one more value than boundaries."""

    __slots__ = ("boundaries", "values")

    def __init__(self, boundaries: Sequence[int], values: Sequence[float]) -> None:
        self.boundaries = tuple(operator.index(b) for b in boundaries)
        self.values = tuple(_real(v, "values") for v in values)
        if len(self.values) != len(self.boundaries) + 1:
            raise ValueError("values must have one more entry than boundaries")
        if any(b < 0 for b in self.boundaries) or any(a >= b for a, b in zip(self.boundaries, self.boundaries[1:])):
            raise ValueError("boundaries must be nonnegative and strictly increasing")

    def __call__(self, step: int) -> float:
        index = 0
        for boundary in self.boundaries:
            if step < boundary:
                break
            index += 1
        return self.values[index]
