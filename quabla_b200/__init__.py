"""quabla_b200: a B200-native (sm_100a) backend for Quabla's data-parallel PINN
training step, behind the reference's Python surface.

    import quabla_b200 as qb
    step = qb.jit(qb.value_and_grad(loss), device="cuda:0")
    trainer = qb.optim.Trainer(loss, params, qb.optim.Adam(1e-3), x, xb, device="cuda:0")

Host arrays are NumPy arrays; every computation runs in hand-written CUDA
kernels behind the C ABI of include/qb200.h.  There is no CPU fallback.
"""

import numpy as _np

from . import optim, random  # noqa: F401
from ._errors import QuablaError, TracerError, UnsupportedOperationError  # noqa: F401
from ._io import load, save  # noqa: F401
from ._plantext import plan_spec_from_text  # noqa: F401
from ._transforms import (cos, erf, erfc, exp, expm1, gelu, grad, hessian, jit, jvp, log, log1p, mean,  # noqa: F401,A004
                          reshape, sigmoid, silu, sin, softplus, sqrt, stack, sum, tan, tanh, trace, value_and_grad, vmap)

float32 = _np.float32
float64 = _np.float64

__version__ = "0.1.0"


def array(value, dtype=None):
    """A host array; floating data defaults to float64 as in the reference."""
    out = _np.asarray(value, dtype=dtype)
    if dtype is None and out.dtype.kind in "iuf" and out.dtype != _np.float32:
        out = out.astype(_np.float64)
    return out


def zeros(shape, dtype=float64):
    return _np.zeros(shape, dtype=dtype)


def ones(shape, dtype=float64):
    return _np.ones(shape, dtype=dtype)


def linspace(start, stop, num, dtype=float64):
    return _np.linspace(start, stop, num, dtype=dtype)


from . import distributed  # noqa: E402,F401
