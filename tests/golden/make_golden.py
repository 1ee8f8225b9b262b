"""Generates tests/golden/*.npz from the literal oracle.

The reference cannot be imported or built in this environment, so the golden
vectors are outputs of oracle/literal (the NumPy restatement of the reference's
graph transforms and CPU interpreter, itself pinned by tests/test_oracle_pins.py)
on tiny seeded cases of the five workloads.  Run from the repository root:

    python tests/golden/make_golden.py

Each file holds the data arrays, a SHA-256 of the (seed-regenerated) parameter
bytes, the loss, and per gradient leaf either the full array (small networks)
or its sum, Euclidean norm and first 16 entries (wide networks).
"""

import hashlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)

from oracle import literal  # noqa: E402
from quabla_b200 import workloads  # noqa: E402

CASES = {"poisson1d": 16, "poisson2d": 16, "burgers": 8, "heat3d": 4, "beam": 8}
FULL_LIMIT = 20000  # gradient scalars stored in full below this parameter count


def parameter_digest(params) -> str:
    h = hashlib.sha256()
    for layer in params:
        h.update(np.ascontiguousarray(layer["b"]).tobytes())
        h.update(np.ascontiguousarray(layer["w"]).tobytes())
    return h.hexdigest()


def main() -> None:
    here = os.path.dirname(os.path.abspath(__file__))
    for name, points in CASES.items():
        w = workloads.make(name, points, api=literal)
        value, grads = literal.value_and_grad(w.loss)(w.params, *w.data)
        out = {"points": np.array(points), "loss": np.asarray(value), "digest": np.array(parameter_digest(w.params))}
        for i, a in enumerate(w.data):
            out[f"data{i}"] = a
        full = w.parameter_count <= FULL_LIMIT
        out["full"] = np.array(full)
        for layer, tree in enumerate(grads):
            for kind in ("b", "w"):
                g = np.asarray(tree[kind])
                key = f"grad/{layer}/{kind}"
                if full:
                    out[key] = g
                else:
                    flat = g.reshape(-1).astype(np.float64)
                    out[key + "/sum"] = np.array(flat.sum())
                    out[key + "/norm"] = np.array(np.sqrt((flat * flat).sum()))
                    out[key + "/head"] = g.reshape(-1)[:16]
        np.savez_compressed(os.path.join(here, f"{name}.npz"), **out)
        print(name, "loss", float(value))


if __name__ == "__main__":
    main()
