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


def traced(name: str, points: int | None, activation: str = "tanh"):
    """(workload, traced loss without a device plan, named inputs)."""
    w = workloads.make(name, points, activation=activation)
    args = (w.params, *w.data)
    compiled = CompiledLoss(w.loss, args, (0,), 0, build_plan=False)
    return w, compiled, compiled.named_inputs(args)


def load_golden(name: str):
    """(workload at the fixture's size, fixture dict) of tests/golden/<name>.npz."""
    import hashlib
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"{name}.npz")
    fixture = dict(np.load(path, allow_pickle=False))
    w = workloads.make(name, int(fixture["points"]))
    digest = hashlib.sha256()
    for layer in w.params:
        digest.update(np.ascontiguousarray(layer["b"]).tobytes())
        digest.update(np.ascontiguousarray(layer["w"]).tobytes())
    assert digest.hexdigest() == str(fixture["digest"]), "seeded parameters changed since the fixture was made"
    for i, a in enumerate(w.data):
        assert a.tobytes() == fixture[f"data{i}"].tobytes(), "seeded points changed since the fixture was made"
    return w, fixture


def check_against_golden(fixture, value, grads_by_name: dict, tolerance: float) -> None:
    """grads_by_name maps 'params/<layer>/<w|b>' to arrays."""
    assert relative_error(value, fixture["loss"]) <= tolerance
    full = bool(fixture["full"])
    for name, got in grads_by_name.items():
        _, layer, kind = name.split("/")
        key = f"grad/{layer}/{kind}"
        flat = np.asarray(got, dtype=np.float64).reshape(-1)
        if full:
            assert relative_error(flat, fixture[key].reshape(-1)) <= tolerance, name
        else:
            norm = float(fixture[key + "/norm"])
            assert abs(np.sqrt((flat * flat).sum()) - norm) <= tolerance * max(norm, 1e-300), name
            assert abs(flat.sum() - float(fixture[key + "/sum"])) <= tolerance * max(norm, 1e-300) * np.sqrt(flat.size), name
            head = fixture[key + "/head"].astype(np.float64)
            scale = max(float(np.max(np.abs(flat))), 1e-300)
            assert np.max(np.abs(flat[: head.size] - head)) <= tolerance * scale, name
