"""Shared helpers of the test-suite."""

from __future__ import annotations

import numpy as np

from quabla_b200 import workloads
from quabla_b200._transforms import CompiledLoss

# Parity gates: loss and every gradient leaf within these relative errors of the
# CPU oracle (1e-10 float64, 1e-5 float32), measured leaf-wise as
# max|a - b| / max(max|b|, tiny).
TOLERANCE = {np.dtype(np.float64): 1e-10, np.dtype(np.float32): 1e-5}


def relative_error(actual, expected) -> float:
    actual = np.asarray(actual, dtype=np.float64)
    expected = np.asarray(expected, dtype=np.float64)
    scale = max(float(np.max(np.abs(expected))), 1e-300)
    return float(np.max(np.abs(actual - expected))) / scale


def traced(name: str, points: int | None):
    """(workload, traced loss without a device plan, named inputs)."""
    w = workloads.make(name, points)
    args = (w.params, *w.data)
    compiled = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    return w, compiled, compiled.named_inputs(args)
