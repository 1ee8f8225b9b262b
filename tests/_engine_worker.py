"""Child process of tests/test_gpu_engine_switches.py: one workload's value and gradients on the
device against the CPU oracle, with whatever QB200_* switches the parent put in the environment
(the library reads them once per process).  Prints one JSON line."""

import json
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from oracle import contracted  # noqa: E402
from quabla_b200 import _lib  # noqa: E402
from quabla_b200._plan import Plan  # noqa: E402

from _util import relative_error, traced  # noqa: E402


def main() -> None:
    name, points = sys.argv[1], int(sys.argv[2])
    w, compiled, inputs = traced(name, points)
    expected_loss, expected_grads = contracted.value_and_grad(compiled.spec, inputs)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.execute()
    outputs = plan.outputs()
    errors = [relative_error(outputs[0], expected_loss)]
    for got, expected in zip(outputs[1:], expected_grads):
        errors.append(relative_error(got.reshape(expected.shape), expected))
    print(json.dumps({"engine": plan.query(_lib.Q_ENGINE), "launches": plan.query(_lib.Q_KERNEL_LAUNCHES),
                      "max_error": float(np.max(errors)), "loss": float(outputs[0]),
                      "streams": compiled.spec.sets[0].streams}))
    plan.close()


if __name__ == "__main__":
    main()
