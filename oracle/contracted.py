"""ctypes front end of oracle/contracted.c — TEST INFRASTRUCTURE.

`value_and_grad(spec, inputs)` evaluates a plan description (the same
`PlanSpec` the product compiles) in float64 on the CPU: loss, and one gradient
per parameter leaf in the spec's parameter order.  For a float32 spec the
inputs and the program constants are first rounded to float32, so both sides
see the same numbers; everything after that is double.
"""

from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_HERE, "_ref", "libqbo_contracted.so")
WEIGHT, BIAS = 0, 1


class _Net(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("sizes", C.POINTER(C.c_int)),
                ("W", C.POINTER(C.POINTER(C.c_double))), ("b", C.POINTER(C.POINTER(C.c_double))),
                ("activation", C.c_int)]


class _Set(C.Structure):
    _fields_ = [("n", C.c_int64), ("ncols", C.c_int), ("table", C.POINTER(C.c_double)), ("ndirs", C.c_int),
                ("dirs", C.POINTER(C.c_double)), ("orders", C.POINTER(C.c_int)), ("code", C.POINTER(C.c_int32)),
                ("n_instr", C.c_int), ("consts", C.POINTER(C.c_double)), ("value_reg", C.c_int),
                ("grad_regs", C.POINTER(C.c_int32)), ("weight", C.c_double)]


def build(force: bool = False) -> str:
    stale = force or not os.path.exists(_LIB) or os.path.getmtime(_LIB) < os.path.getmtime(
        os.path.join(_HERE, "contracted.c"))
    if stale:
        subprocess.check_call(["make", "-C", _HERE, "-B", "_ref/libqbo_contracted.so"], stdout=subprocess.DEVNULL)
    return _LIB


_lib = None


def _load() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _lib.qbo_set_value_and_grad.restype = C.c_int
        _lib.qbo_point_jets.restype = C.c_int
        _lib.qbo_max_threads.restype = C.c_int
    return _lib


def max_threads() -> int:
    return int(_load().qbo_max_threads())


def _dp(a: np.ndarray):
    return a.ctypes.data_as(C.POINTER(C.c_double))


def _round(values, dtype) -> np.ndarray:
    return np.ascontiguousarray(np.asarray(values, dtype=dtype).astype(np.float64))


class _Problem:
    """Host arrays of one spec, kept alive while C reads them."""

    def __init__(self, spec, inputs: dict) -> None:
        self.spec = spec
        dtype = np.dtype(spec.dtype)
        n_layers = len(spec.sizes) - 1
        self.sizes = (C.c_int * (n_layers + 1))(*spec.sizes)
        self.W = [None] * n_layers
        self.b = [None] * n_layers
        for name, layer, kind in spec.parameters:
            value = _round(inputs[name], dtype).reshape(-1)
            if kind == WEIGHT:
                self.W[layer] = value
            else:
                self.b[layer] = value
        self.Wp = (C.POINTER(C.c_double) * n_layers)(*[_dp(w) for w in self.W])
        self.bp = (C.POINTER(C.c_double) * n_layers)(
            *[_dp(b) if b is not None else C.POINTER(C.c_double)() for b in self.b])
        activation = {"tanh": 0, "sin": 1, "sigmoid": 2, "softplus": 3, "silu": 4, "gelu": 5}[
            getattr(spec, "activation", "tanh")]
        self.net = _Net(n_layers, self.sizes, self.Wp, self.bp, activation)
        self.sets = []
        self.keep = []
        for s in spec.sets:
            columns = []
            for input_index, column in s.columns:
                name, rows, cols, _ = spec.inputs[input_index]
                columns.append(_round(inputs[name], dtype).reshape(rows, cols)[:, column])
            table = np.ascontiguousarray(np.stack(columns, axis=1))
            dirs = np.ascontiguousarray(np.array([v for v, _ in s.directions], dtype=np.float64).reshape(-1))
            dirs = _round(dirs, dtype) if dirs.size else np.zeros(1)
            orders = (C.c_int * max(1, len(s.directions)))(*[o for _, o in s.directions])
            code = np.ascontiguousarray(np.array(s.program.code, dtype=np.int32))
            consts = _round(s.program.consts, dtype) if s.program.consts else np.zeros(1)
            grad_regs = np.ascontiguousarray(np.array(s.program.grad_regs, dtype=np.int32))
            self.keep.append((table, dirs, orders, code, consts, grad_regs))
            self.sets.append(_Set(
                s.n_points, table.shape[1], _dp(table), len(s.directions), _dp(dirs), orders,
                code.ctypes.data_as(C.POINTER(C.c_int32)), s.program.n_instr, _dp(consts), s.program.value_reg,
                grad_regs.ctypes.data_as(C.POINTER(C.c_int32)), float(_set_weight(s.weight, dtype))))


def _set_weight(weight: float, dtype) -> float:
    # A Mean's 1/n meets the strong dtype as a weak scalar and is rounded to it
    # (crates/quabla-core/src/tensor_ir/op/vjp.rs:292-298, tensor_ir.rs:6995-7004);
    # for 1/2^k this is exact either way.
    return float(np.asarray(weight, dtype=dtype))


def value_and_grad(spec, inputs: dict, cotangent: float = 1.0, threads: int = 1, forward_only: bool = False,
                   point_slices: list | None = None):
    """(loss, [gradient per spec parameter]) in float64.

    point_slices, when given, restricts set k to points [lo, hi) (for bounded
    timing samples); weights are unchanged.

    A spec whose sets carry a merged second-order stream (the forward-Laplacian recurrence of the
    device kernels) is evaluated in its `unmerged` form, one second-order stream per direction:
    the oracle always computes the formulation pinned against the reference's known answers."""
    spec = getattr(spec, "unmerged", None) or spec
    if any(getattr(s, "merge_weights", None) is not None for s in spec.sets):
        raise ValueError("the oracle evaluates unmerged specs only")
    lib = _load()
    problem = _Problem(spec, inputs)
    n_layers = len(spec.sizes) - 1
    gW = [np.zeros(spec.sizes[l] * spec.sizes[l + 1]) for l in range(n_layers)]
    gb = [np.zeros(spec.sizes[l + 1]) if problem.b[l] is not None else None for l in range(n_layers)]
    gWp = (C.POINTER(C.c_double) * n_layers)(*[_dp(g) for g in gW])
    gbp = (C.POINTER(C.c_double) * n_layers)(*[_dp(g) if g is not None else C.POINTER(C.c_double)() for g in gb])
    loss = C.c_double(0.0)
    for k, s in enumerate(problem.sets):
        if point_slices is not None:
            lo, hi = point_slices[k]
            table = problem.keep[k][0][lo:hi]
            s.table = _dp(np.ascontiguousarray(table))
            problem.keep.append(table)
            s.n = hi - lo
        status = lib.qbo_set_value_and_grad(C.byref(problem.net), C.byref(s), C.c_double(cotangent), C.byref(loss),
                                            gWp, gbp, int(forward_only), int(threads))
        if status != 0:
            raise RuntimeError("oracle/contracted.c rejected the description")
    grads = []
    for name, layer, kind in spec.parameters:
        if kind == WEIGHT:
            grads.append(gW[layer].reshape(spec.sizes[layer], spec.sizes[layer + 1]))
        else:
            grads.append(gb[layer])
    return loss.value, grads


def point_jets(spec, inputs: dict, set_index: int, point: int) -> np.ndarray:
    """Network output streams [u, derivative streams...] of one point."""
    lib = _load()
    problem = _Problem(spec, inputs)
    s = problem.sets[set_index]
    table = problem.keep[set_index][0]
    out = np.zeros(spec.sets[set_index].streams)
    row = np.ascontiguousarray(table[point])
    if lib.qbo_point_jets(C.byref(problem.net), C.byref(s), _dp(row), _dp(out)) != 0:
        raise RuntimeError("oracle/contracted.c failed")
    return out
