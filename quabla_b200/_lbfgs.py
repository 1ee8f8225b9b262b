"""Full-batch L-BFGS refinement over the device value-and-gradient plan.

The surface follows the reference's `optim.LBFGS` (python/quabla/_lbfgs.py:219-355):
the same constructor arguments, `minimize(fun, params, *args) -> (params, info)` and the
same `info` keys and stop reasons.  The reference evaluates the loss with its CPU
interpreter; here every evaluation is one `qb200_plan_execute` of the traced loss
on the GPU (parameters uploaded, loss and flat gradient read back), and the
quasi-Newton algebra runs on the host in float64 over one flat vector.

Algorithm (Nocedal and Wright, Numerical Optimization, 2nd ed.): two-loop
recursion with the initial scaling gamma = s'y / y'y, strong Wolfe line search by
bracketing and zoom with safeguarded cubic interpolation.
"""

from __future__ import annotations

import math
import operator
from collections import deque
from typing import Any, Callable

import numpy as np

ARMIJO = 1e-4      # sufficient-decrease constant c1
CURVATURE = 0.9    # curvature constant c2 (quasi-Newton value)
LINE_SEARCH_EVALUATIONS = 25
PAIR_ANGLE = 1e-10  # keep (s, y) only if cos(s, y) exceeds this
EDGE = 0.1          # interpolated trials stay this fraction away from the bracket ends


def _cubic_trial(a, fa, ga, b, fb, gb):
    """Minimiser of the cubic through (a, fa, ga) and (b, fb, gb), clamped inside the bracket."""
    low, high = (a, b) if a <= b else (b, a)
    span = high - low
    d1 = ga + gb - 3.0 * (fa - fb) / (a - b)
    radicand = d1 * d1 - ga * gb
    trial = None
    if radicand >= 0.0 and math.isfinite(radicand):
        d2 = math.copysign(math.sqrt(radicand), b - a)
        denominator = gb - ga + 2.0 * d2
        if denominator != 0.0:
            trial = b - (b - a) * (gb + d2 - d1) / denominator
    if trial is None or not math.isfinite(trial):
        trial = 0.5 * (low + high)
    return min(max(trial, low + EDGE * span), high - EDGE * span)


class _LineFunction:
    """phi(alpha) = f(x + alpha d) with its slope; remembers the point of every evaluation."""

    def __init__(self, evaluate, x, direction):
        self.evaluate, self.x, self.direction = evaluate, x, direction

    def __call__(self, alpha):
        point, value, gradient = self.evaluate(self.x + alpha * self.direction)
        return alpha, value, float(gradient @ self.direction), (point, gradient)


def _usable(trial):
    return math.isfinite(trial[1]) and math.isfinite(trial[2])


def _zoom(phi, f0, slope0, low, high, budget):
    """Shrinks [low, high] (low has the smaller acceptable value) to a strong Wolfe point."""
    best = None
    while budget > 0:
        alpha = _cubic_trial(low[0], low[1], low[2], high[0], high[1], high[2]) if _usable(high) else 0.5 * (low[0] + high[0])
        trial = phi(alpha)
        budget -= 1
        if not _usable(trial) or trial[1] > f0 + ARMIJO * alpha * slope0 or trial[1] >= low[1]:
            high = trial
        else:
            if abs(trial[2]) <= -CURVATURE * slope0:
                return trial, budget
            if trial[2] * (high[0] - low[0]) >= 0.0:
                high = low
            low = trial
            best = trial
        if abs(high[0] - low[0]) <= 1e-16 * max(1.0, abs(low[0])):
            break
    # Out of budget: accept the best sufficient-decrease point seen, if any.
    if best is None and low[0] > 0.0 and low[1] < f0:
        best = low
    return best, budget


def _strong_wolfe(phi, f0, slope0, first_step, budget):
    previous = (0.0, f0, slope0, None)
    alpha = first_step
    first = True
    while budget > 0:
        trial = phi(alpha)
        budget -= 1
        if not _usable(trial):
            # Backtrack out of a non-finite region.
            alpha = 0.5 * (previous[0] + alpha)
            if alpha - previous[0] <= 1e-16:
                break
            continue
        if trial[1] > f0 + ARMIJO * alpha * slope0 or (not first and trial[1] >= previous[1]):
            return _zoom(phi, f0, slope0, previous, trial, budget)
        if abs(trial[2]) <= -CURVATURE * slope0:
            return trial, budget
        if trial[2] >= 0.0:
            return _zoom(phi, f0, slope0, trial, previous, budget)
        previous = trial
        alpha *= 2.0
        first = False
    return None, budget


def _two_loop(gradient, pairs):
    """-H g with H the L-BFGS inverse-Hessian approximation of the stored pairs."""
    q = gradient.copy()
    alphas = []
    for s, y, rho in reversed(pairs):
        a = rho * float(s @ q)
        alphas.append(a)
        q -= a * y
    if pairs:
        s, y, _ = pairs[-1]
        q *= float(s @ y) / float(y @ y)
    for (s, y, rho), a in zip(pairs, reversed(alphas)):
        b = rho * float(y @ q)
        q += (a - b) * s
    return -q


class _Layout:
    """Parameter pytree <-> one float64 host vector."""

    def __init__(self, params):
        from . import _trace as tr

        leaves, self._rebuild = tr.flatten(params)
        self._arrays = [np.asarray(leaf) for leaf in leaves]
        if not self._arrays:
            raise ValueError("L-BFGS requires at least one parameter")
        for a in self._arrays:
            if a.dtype not in (np.float32, np.float64):
                raise TypeError(f"L-BFGS parameters must be float32 or float64 arrays, got {a.dtype}")
        self.exact = all(a.dtype == np.float64 for a in self._arrays)

    def vector(self, tree):
        from . import _trace as tr

        leaves, _ = tr.flatten(tree)
        return np.concatenate([np.asarray(leaf, dtype=np.float64).reshape(-1) for leaf in leaves])

    def tree(self, vector):
        leaves, offset = [], 0
        for a in self._arrays:
            leaves.append(vector[offset:offset + a.size].reshape(a.shape).astype(a.dtype))
            offset += a.size
        return self._rebuild(leaves)


class LBFGS:
    """Full-batch L-BFGS minimiser for a scalar loss over a parameter pytree.

    `minimize(fun, params, *args, device="cuda")` traces `fun(params, *args)` once, compiles it to a
    device plan and returns `(params, info)`; `info` holds `iterations`, `evaluations`, `loss`,
    `grad_norm` (infinity norm), `reason` and `converged`.  `reason` is "gradient_tolerance",
    "change_tolerance" (relative, no floor of 1), "max_iterations", "max_evaluations" or
    "line_search_failed"; the first two set `converged`.
    """

    def __init__(self, history: int = 10, max_iterations: int = 500, max_evaluations: int | None = None,
                 tolerance_grad: float = 1e-7, tolerance_change: float = 1e-9, line_search: str = "strong_wolfe") -> None:
        self.history = operator.index(history)
        self.max_iterations = operator.index(max_iterations)
        if self.history <= 0 or self.max_iterations <= 0:
            raise ValueError("history and max_iterations must be positive")
        if max_evaluations is not None:
            max_evaluations = operator.index(max_evaluations)
            if max_evaluations <= 0:
                raise ValueError("max_evaluations must be positive")
        self.max_evaluations = max_evaluations
        self.tolerance_grad = float(tolerance_grad)
        self.tolerance_change = float(tolerance_change)
        if not (math.isfinite(self.tolerance_grad) and math.isfinite(self.tolerance_change)
                and self.tolerance_grad >= 0 and self.tolerance_change >= 0):
            raise ValueError("tolerances must be finite and nonnegative")
        if line_search != "strong_wolfe":
            raise ValueError('line_search must be "strong_wolfe"')
        self.line_search = line_search

    # The evaluator is separate so that the quasi-Newton logic can be exercised without a device.
    def minimize_with(self, value_and_grad: Callable[[Any], tuple[float, Any]], params: Any):
        """`value_and_grad(params_tree) -> (loss, gradient_tree)`; returns `(params, info)`."""
        layout = _Layout(params)
        evaluations = 0

        def evaluate(x):
            nonlocal evaluations
            evaluations += 1
            point = layout.tree(x)
            loss, gradients = value_and_grad(point)
            if np.size(loss) != 1:
                raise ValueError("L-BFGS loss must be a scalar")
            if not layout.exact:
                x = layout.vector(point)  # the float32 point that was actually evaluated
            return x, float(np.asarray(loss).reshape(())), layout.vector(gradients)

        x, f, g = evaluate(layout.vector(params))
        if not (math.isfinite(f) and np.all(np.isfinite(g))):
            raise ValueError("L-BFGS initial loss and gradient must be finite")
        pairs: deque = deque(maxlen=self.history)
        iterations = 0
        while True:
            grad_norm = abs(float(np.max(np.abs(g)))) if g.size else 0.0
            if grad_norm <= self.tolerance_grad:
                reason = "gradient_tolerance"
                break
            if iterations >= self.max_iterations:
                reason = "max_iterations"
                break
            budget = LINE_SEARCH_EVALUATIONS
            if self.max_evaluations is not None:
                budget = min(budget, self.max_evaluations - evaluations)
            if budget <= 0:
                reason = "max_evaluations"
                break
            direction = _two_loop(g, pairs)
            slope = float(g @ direction)
            if not (slope < 0 and math.isfinite(slope)):
                pairs.clear()
                direction = -(g / grad_norm)  # scaled first, so tiny gradients keep a non-zero slope
                slope = float(g @ direction)
                if not (slope < 0 and math.isfinite(slope)):
                    reason = "line_search_failed"
                    break
            step = 1.0 if pairs else min(1.0, 1.0 / math.sqrt(-slope))
            accepted, _ = _strong_wolfe(_LineFunction(evaluate, x, direction), f, slope, step, budget)
            if accepted is None or accepted[3] is None:
                if pairs:
                    pairs.clear()  # retry along steepest descent before giving up
                    continue
                exhausted = self.max_evaluations is not None and evaluations >= self.max_evaluations
                reason = "max_evaluations" if exhausted else "line_search_failed"
                break
            x_new, g_new = accepted[3]
            f_new = accepted[1]
            s, y = x_new - x, g_new - g
            sy = float(s @ y)
            if sy > PAIR_ANGLE * math.sqrt(float(s @ s) * float(y @ y)):
                pairs.append((s, y, 1.0 / sy))
            f_old, x, f, g = f, x_new, f_new, g_new
            iterations += 1
            if abs(f_old - f) <= self.tolerance_change * max(abs(f_old), abs(f)):
                grad_norm = abs(float(np.max(np.abs(g))))
                reason = "change_tolerance"
                break
        info = {"iterations": iterations, "evaluations": evaluations, "loss": f, "grad_norm": grad_norm,
                "reason": reason, "converged": reason in ("gradient_tolerance", "change_tolerance")}
        return layout.tree(x), info

    def minimize(self, fun: Callable[..., Any], params: Any, *args: Any, device: str = "cuda"):
        """Minimise `fun(params, *args)` over `params`, evaluating on the GPU."""
        if not callable(fun):
            raise TypeError("fun must be callable")
        from ._devices import require_device
        from ._transforms import CompiledLoss

        _, ordinal = require_device(device, "LBFGS")
        arguments = (params, *args)
        compiled = CompiledLoss(fun, arguments, (0,), ordinal, retained=list(range(1, len(arguments))))
        compiled.bind(arguments)

        def value_and_grad(point):
            leaves = compiled.leaves_of((point,))[0]
            for name, value in zip(compiled.param_names, leaves):
                if name in compiled._active:
                    compiled.plan.bind(name, value)
            compiled.plan.execute()
            value, trees = compiled.gradients((point, *args))
            return value, trees[0]

        try:
            return self.minimize_with(value_and_grad, params)
        finally:
            compiled.plan.close()
