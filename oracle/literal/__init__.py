"""Literal oracle — TEST INFRASTRUCTURE, not product.

A NumPy restatement of how the reference turns a Python loss into numbers:
tracing into a tensor IR (ir.py), the graph transforms behind grad / vmap /
hessian (transforms.py), and the CPU interpreter with float64 compute and one
rounding per node (interp.py).  api.py exposes it with the reference's call
shapes, so one loss function can be evaluated by this oracle and by the CUDA
backend.  It materialises the [B, in, out] weight-gradient products exactly as
the reference plan does, so it is meant for small point counts.
"""

from .api import (Tracer, array, cos, erf, erfc, exp, expm1, gelu, grad, hessian, jvp, log1p, mean, relu, sigmoid,  # noqa: F401,A004
                  silu, sin, softplus, sum, tan, tanh, trace, value_and_grad, value_and_grad_data_parallel, vmap,
                  where, zeros)
