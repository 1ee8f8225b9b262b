"""The reference's optimizer element rules on the host — TEST INFRASTRUCTURE.

adam_update follows adam_element (crates/quabla-core/src/tensor_ir/
device_optimizer.rs:241-274) one rounded operation at a time in `dtype`, with
the coefficients formed in float64 and rounded once
(device_optimizer.rs:97-150, cuda_optimizer.rs:340-359): this is what a device
plan of that dtype must reproduce bit for bit.  sgd_update is sgd_element
(device_optimizer.rs:276-285).
"""

from __future__ import annotations

import numpy as np


def adam_update(p, g, m, v, step: int, lr: float, b1: float, b2: float, eps: float, weight_decay: float, dtype):
    t = np.dtype(dtype).type
    k = dict(lr=t(lr), b1=t(b1), b2=t(b2), omb1=t(1.0 - b1), omb2=t(1.0 - b2), eps=t(eps),
             c1=t(1.0 - b1 ** float(step)), c2=t(1.0 - b2 ** float(step)), wd=t(weight_decay))
    p, g, m, v = (np.asarray(a, dtype=dtype) for a in (p, g, m, v))
    with np.errstate(all="ignore"):
        first = m * k["b1"] + g * k["omb1"]
        second = v * k["b2"] + (g * g) * k["omb2"]
        delta = (first / k["c1"]) / (np.sqrt(second / k["c2"]) + k["eps"])
        if weight_decay != 0.0:
            delta = delta + k["wd"] * p
        new_p = p - delta * k["lr"]
    return new_p.astype(dtype), first.astype(dtype), second.astype(dtype)


def sgd_update(p, g, lr: float, dtype):
    t = np.dtype(dtype).type
    p, g = np.asarray(p, dtype=dtype), np.asarray(g, dtype=dtype)
    return (p - g * t(lr)).astype(dtype)
