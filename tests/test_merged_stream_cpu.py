"""The merged second-order stream on the host: the symbolic rewrite of a residual that uses second
derivatives only through one weighted sum, and the plan descriptions the tracer builds from it."""

import math
import random

import numpy as np
import pytest

from quabla_b200 import _symbolic as sx

from _util import traced


class _Net:
    def substituted(self, mapping):
        return self


NET = _Net()
X, Y, Z = (1.0, 0.0, 0.0), (0.0, 1.0, 0.0), (0.0, 0.0, 1.0)
U, UX = sx.net(NET, ()), sx.net(NET, (X,))
UXX, UYY, UZZ = sx.net(NET, (X, X)), sx.net(NET, (Y, Y)), sx.net(NET, (Z, Z))
COL = sx.sym(("col", "p", 0))
MERGED = sx.Expr("net", (NET, sx.MERGED_WORD))


def _same_value(root, targets, rewritten, weights):
    rng = random.Random(7)
    values = {leaf: rng.uniform(-2, 2) for leaf in sx.leaves([root], "net") + sx.leaves([root], "sym")}
    merged_values = dict(values)
    merged_values[MERGED] = sum(weights[t] * values[t] for t in targets)
    a = sx.evaluate(root, lambda leaf: values[leaf])
    b = sx.evaluate(rewritten, lambda leaf: merged_values[leaf])
    return math.isclose(a, b, rel_tol=1e-12, abs_tol=1e-12)


@pytest.mark.parametrize("root,targets,expected", [
    ((UXX + UYY + sx.const(2.0) * sx.unary("sin", COL)) ** 2, [UXX, UYY], {UXX: 1.0, UYY: 1.0}),
    ((UX - sx.const(0.1) * (UXX + UYY + UZZ) - COL) ** 2, [UXX, UYY, UZZ], {UXX: -0.1, UYY: -0.1, UZZ: -0.1}),
    ((UXX + UYY) ** 2 + (sx.const(3.0) * UXX + sx.const(3.0) * UYY) * U, [UXX, UYY], {UXX: 1.0, UYY: 1.0}),
    ((UXX + sx.const(4.0) * UYY) / sx.const(2.0) + sx.unary("exp", UXX * sx.const(0.25) + UYY), [UXX, UYY],
     {UXX: 0.5, UYY: 2.0}),
    (UXX + UYY, [UXX, UYY], {UXX: 1.0, UYY: 1.0}),
])
def test_weighted_sums_are_merged(root, targets, expected):
    out = sx.merge_weighted_sum(root, targets, MERGED)
    assert out is not None
    rewritten, weights = out
    # The weight vector is fixed up to a common factor (whichever sum the traversal closes first).
    scale = weights[targets[0]] / expected[targets[0]]
    assert {t: w / scale for t, w in weights.items()} == pytest.approx(expected)
    assert not set(sx.leaves([rewritten], "net")) & set(targets)
    assert _same_value(root, targets, rewritten, weights)


@pytest.mark.parametrize("root,targets", [
    ((UXX + sx.const(2.0) * UYY) ** 2 + (UXX + UYY), [UXX, UYY]),   # two sums that are not proportional
    ((UXX * U + UYY) ** 2, [UXX, UYY]),                              # a non-constant coefficient
    (UXX ** 2 + UYY ** 2, [UXX, UYY]),                               # each second derivative on its own
    ((UXX - UXX + UYY) ** 2, [UXX, UYY]),                            # a target that cancels
    ((UXX + UYY) ** 2 + UZZ, [UXX, UYY, UZZ]),                       # sums over different supports
])
def test_other_uses_are_left_alone(root, targets):
    assert sx.merge_weighted_sum(root, targets, MERGED) is None


def test_traced_workloads_carry_the_merged_stream_where_it_applies():
    _, compiled, _ = traced("poisson2d", 64)
    interior = compiled.spec.sets[0]
    assert interior.streams == 4 and [m for _, m in interior.directions] == [1, 1]
    assert interior.merge_weights == [1.0, 1.0]
    assert interior.program.grad_regs[1] == interior.program.grad_regs[2] == -1  # u_x, u_y are not in the residual
    assert interior.program.grad_regs[3] >= 0
    assert compiled.spec.unmerged is not None and compiled.spec.unmerged.sets[0].streams == 5
    assert compiled.spec.unmerged.sets[0].merge_weights is None

    _, compiled, _ = traced("heat3d", 32)
    interior = compiled.spec.sets[0]
    assert interior.streams == 6 and len(interior.directions) == 4
    time = [i for i, (d, _) in enumerate(interior.directions) if d[3] == 1.0]
    assert [w for i, w in enumerate(interior.merge_weights) if i not in time] == pytest.approx([-0.1] * 3)
    assert interior.merge_weights[time[0]] == 0.0
    assert compiled.spec.unmerged.sets[0].streams == 8

    for name in ("poisson1d", "burgers", "beam"):  # one second-order direction, or none: nothing to merge
        _, compiled, _ = traced(name, 16)
        assert compiled.spec.unmerged is None
        assert all(s.merge_weights is None for s in compiled.spec.sets)


def test_the_switch_keeps_one_stream_per_direction(monkeypatch):
    monkeypatch.setenv("QB200_MERGE", "0")
    _, compiled, _ = traced("poisson2d", 64)
    assert compiled.spec.unmerged is None and compiled.spec.sets[0].streams == 5


def test_the_oracle_evaluates_the_reference_formulation():
    from oracle import contracted

    w, compiled, inputs = traced("poisson2d", 96)
    loss_a, grads_a = contracted.value_and_grad(compiled.spec, inputs)
    loss_b, grads_b = contracted.value_and_grad(compiled.spec.unmerged, inputs)
    assert loss_a == loss_b and all(np.array_equal(a, b) for a, b in zip(grads_a, grads_b))
    merged_only = compiled.spec.unmerged.__class__(**{**compiled.spec.__dict__, "unmerged": None})
    with pytest.raises(ValueError):
        contracted.value_and_grad(merged_only, inputs)
