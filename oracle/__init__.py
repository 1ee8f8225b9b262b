"""CPU oracle for the PINN training step — TEST INFRASTRUCTURE, not product.

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may
import this package.  It restates the reference's algorithm for the path:

  oracle/literal/     NumPy restatement of the reference's tensor IR subset,
                      its symbolic VJP/JVP/vmap transforms, plan compilation
                      and CPU interpreter (float64 compute, one rounding per
                      node), rule by rule with file:line citations;
  oracle/contracted.c float64 C evaluation of the same loss and gradients in
                      contracted form, usable at the benchmark sizes;
  oracle/rng.py       the reference's SplitMix64 key stream and samplers;
  oracle/adam.py      the reference's Adam/SGD element rule on the host.

Parity is pinned: the reference cannot be built here (no Rust toolchain), so
the pins are the reference's own closed-form known answers and structural
counts, reproduced in tests/test_oracle_*.py.
"""
