"""Learning-rate schedules: closed-form values at chosen steps, the end-point and extreme-scale
behaviour the reference's tests ask for (tests/python/test_optim_api.py:485-600), and validation."""

import math
import pickle

import pytest

from quabla_b200.optim import constant, cosine_decay, exponential_decay, piecewise_constant, warmup_cosine_decay


def _check(schedule, expected, rel=1e-15):
    for step, value in expected.items():
        got = schedule(step)
        assert math.isclose(got, value, rel_tol=rel, abs_tol=1e-15), (schedule, step, got, value)


def test_constant_and_piecewise_constant():
    _check(constant(0.25), {0: 0.25, 1000: 0.25})
    stairs = piecewise_constant([4, 9], [1.0, 0.5, 0.125])
    _check(stairs, {0: 1.0, 3: 1.0, 4: 0.5, 8: 0.5, 9: 0.125, 10**6: 0.125})
    assert piecewise_constant([], [3.0])(17) == 3.0


def test_exponential_decay_values():
    _check(exponential_decay(2.0, 8, 0.25), {0: 2.0, 4: 1.0, 8: 0.5, 16: 0.125})
    _check(exponential_decay(2.0, 8, 0.25, staircase=True), {7: 2.0, 8: 0.5, 15: 0.5, 16: 0.125})
    _check(exponential_decay(2.0, 8, 0.25, transition_begin=3), {0: 2.0, 3: 2.0, 11: 0.5})
    _check(exponential_decay(1.0, 5, 0.5, end_value=0.4), {5: 0.5, 10: 0.4, 500: 0.4})
    _check(exponential_decay(1.0, 5, 3.0, end_value=5.0), {5: 3.0, 10: 5.0})


def test_exponential_decay_at_extreme_scales():
    # The bare power overflows or vanishes; the product is representable.
    for start, rate, step in ((1e300, 0.5, 1100), (1e-300, 2.0, 1024), (-1e300, 0.5, 1100)):
        want = math.ldexp(start, step if rate > 1 else -step)
        for bound in (None, (1e300 if rate > 1 else 1e-300) * (1 if start > 0 else -1)):
            if bound is not None and start < 0:
                continue  # a floor above a negative rate would clip it
            got = exponential_decay(start, 1, rate, end_value=bound)(step)
            assert math.isclose(got, want, rel_tol=1e-12), (start, rate, got, want)
    assert exponential_decay(1.0, 1, 2.0, end_value=3.0)(1024) == 3.0
    assert exponential_decay(0.0, 1, 2.0, end_value=3.0)(1024) == 0.0
    with pytest.raises(OverflowError):
        exponential_decay(1.0, 1, 2.0)(1025)


def test_cosine_decay_values_and_exact_end_points():
    c = cosine_decay(3.0, 60, alpha=0.2)
    quarter = 0.5 * (1 + math.cos(math.pi / 3))  # step 20 of 60: cos(60 degrees) = 1/2
    _check(c, {0: 3.0, 20: 3.0 * (0.8 * quarter + 0.2), 30: 3.0 * 0.6, 60: 0.6, 61: 0.6, 10**9: 0.6})
    huge = cosine_decay(1.0, 4, alpha=1e20)
    assert huge(0) == 1.0 and huge(4) == 1e20


def test_warmup_cosine_decay_values_and_exact_end_points():
    w = warmup_cosine_decay(0.0, 2.0, 4, 24, end_value=0.5)
    _check(w, {0: 0.0, 1: 0.5, 4: 2.0, 14: 1.25, 24: 0.5, 99: 0.5})
    _check(warmup_cosine_decay(0.3, 1.0, 0, 10), {0: 1.0, 5: 0.5, 10: 0.0})
    for peak in (0.0, 1e-320):
        s = warmup_cosine_decay(1.0, peak, 2, 4, end_value=0.1)
        for step, value in ((0, 1.0), (2, peak), (3, 0.05), (4, 0.1), (5, 0.1)):
            assert math.isclose(s(step), value, rel_tol=1e-14, abs_tol=1e-320)
    wide = warmup_cosine_decay(1e308, -1e308, 2, 4)
    assert [wide(k) for k in (0, 1, 2, 4)] == [1e308, 0.0, -1e308, 0.0]


def test_invalid_configurations_are_refused():
    for build in (lambda: exponential_decay(1.0, 0, 0.5), lambda: exponential_decay(1.0, 10, 0.0),
                  lambda: exponential_decay(1.0, 10, 0.5, transition_begin=-1),
                  lambda: exponential_decay(math.inf, 10, 0.5), lambda: cosine_decay(1.0, 0),
                  lambda: cosine_decay(1.0, 10, alpha=math.nan), lambda: warmup_cosine_decay(0.0, 1.0, 10, 10),
                  lambda: warmup_cosine_decay(0.0, 1.0, -1, 10), lambda: piecewise_constant([5, 5], [1.0, 2.0, 3.0]),
                  lambda: piecewise_constant([5], [1.0]), lambda: piecewise_constant([-1], [1.0, 2.0]),
                  lambda: constant(math.inf)):
        with pytest.raises(ValueError):
            build()
    with pytest.raises(TypeError):
        cosine_decay(1.0, 2.5)


def test_schedules_print_and_pickle():
    s = warmup_cosine_decay(0.0, 0.05, 3, 12, end_value=0.005)
    again = pickle.loads(pickle.dumps(s))
    assert [again(k) for k in range(15)] == [s(k) for k in range(15)]
    assert "warmup_steps=3" in repr(s)
