"""Per-point symbolic expressions: the host side of the fusion pass.

A PINN loss is, per collocation point, a scalar expression over the point's
coordinates, auxiliary per-point data, and derivatives of the network output
along input directions.  The reference obtains those derivatives by graph
transforms (symbolic VJP/JVP of the traced tensor program,
crates/quabla-core/src/tensor_ir.rs:2999-3906) and then executes the resulting
node list; here derivatives of the network are kept as opaque leaves
(`NetJet`) that the device kernels produce by propagating Taylor jets, and
only the small residual expression around them is differentiated symbolically
and compiled to a register program (qb200_desc_set_program).

Expressions are hash-consed and lightly simplified on construction, so common
sub-expressions are shared and the compiled programs stay short.
"""

from __future__ import annotations

import math
from typing import Callable, Iterable

# Opcodes of the register program; numbering fixed by qb200_op in include/qb200.h.
OP_CONST, OP_COL, OP_JET, OP_ADD, OP_SUB, OP_MUL, OP_DIV, OP_NEG, OP_SIN, OP_COS, OP_EXP, OP_TANH, OP_POWI, \
    OP_SQRT, OP_LOG, OP_LOG1P, OP_EXPM1, OP_ERF, OP_ERFC, OP_TAN = range(20)

_UNARY_OPS = {"neg": OP_NEG, "sin": OP_SIN, "cos": OP_COS, "exp": OP_EXP, "tanh": OP_TANH, "sqrt": OP_SQRT,
              "log": OP_LOG, "log1p": OP_LOG1P, "expm1": OP_EXPM1, "erf": OP_ERF, "erfc": OP_ERFC, "tan": OP_TAN}
_BINARY_OPS = {"add": OP_ADD, "sub": OP_SUB, "mul": OP_MUL, "div": OP_DIV}

MAX_REGS = 64
MAX_INSTR = 1024


class UnsupportedExpression(ValueError):
    """The expression is outside what the fused kernels evaluate."""


class Expr:
    """A node of a per-point scalar expression DAG.

    kind is one of: const, sym, net, the unary and binary operator names, powi.
      const: args = (float,)
      sym:   args = (key,)            a differentiation variable or a table column
      net:   args = (net, word)       derivative of the network output; word is a
                                      sorted tuple of direction tuples
      powi:  args = (Expr, int)
    """

    __slots__ = ("kind", "args", "_hash")
    _table: dict = {}

    def __new__(cls, kind: str, args: tuple):
        key = (kind, args)
        found = cls._table.get(key)
        if found is not None:
            return found
        node = object.__new__(cls)
        node.kind = kind
        node.args = args
        node._hash = hash(key)
        cls._table[key] = node
        return node

    def __hash__(self) -> int:
        return self._hash

    def __eq__(self, other) -> bool:  # identity: nodes are interned
        return self is other

    def __repr__(self) -> str:
        if self.kind == "const":
            return repr(self.args[0])
        if self.kind == "sym":
            return f"sym{self.args[0]!r}"
        if self.kind == "net":
            return f"net{self.args[1]!r}"
        return f"{self.kind}({', '.join(map(repr, self.args))})"

    # -- arithmetic ---------------------------------------------------------
    def __add__(self, other):
        return add(self, as_expr(other))

    def __radd__(self, other):
        return add(as_expr(other), self)

    def __sub__(self, other):
        return sub(self, as_expr(other))

    def __rsub__(self, other):
        return sub(as_expr(other), self)

    def __mul__(self, other):
        return mul(self, as_expr(other))

    def __rmul__(self, other):
        return mul(as_expr(other), self)

    def __truediv__(self, other):
        return div(self, as_expr(other))

    def __rtruediv__(self, other):
        return div(as_expr(other), self)

    def __neg__(self):
        return neg(self)

    def __pos__(self):
        return self

    def __pow__(self, exponent):
        if isinstance(exponent, bool) or not isinstance(exponent, int):
            if isinstance(exponent, float) and exponent == int(exponent):
                exponent = int(exponent)
            else:
                raise UnsupportedExpression("only integer powers of a per-point value are supported")
        return powi(self, exponent)


def const(value: float) -> Expr:
    value = float(value)
    if value == 0.0:
        value = 0.0  # one zero: -0.0 and 0.0 hash alike but print differently
    return Expr("const", (value,))


ZERO = const(0.0)
ONE = const(1.0)


def sym(key) -> Expr:
    return Expr("sym", (key,))


def net(network, word: tuple) -> Expr:
    return Expr("net", (network, tuple(sorted(word))))


def as_expr(value) -> Expr:
    if isinstance(value, Expr):
        return value
    if isinstance(value, bool):
        raise UnsupportedExpression("a bool is not a per-point value")
    if isinstance(value, (int, float)):
        return const(value)
    item = getattr(value, "item", None)
    if callable(item) and getattr(value, "shape", None) in ((), []):
        return const(item())
    raise UnsupportedExpression(f"cannot use {type(value).__name__} as a per-point value")


def is_const(e: Expr) -> bool:
    return e.kind == "const"


def add(a: Expr, b: Expr) -> Expr:
    if is_const(a) and is_const(b):
        return const(a.args[0] + b.args[0])
    if a is ZERO:
        return b
    if b is ZERO:
        return a
    return Expr("add", (a, b))


def sub(a: Expr, b: Expr) -> Expr:
    if is_const(a) and is_const(b):
        return const(a.args[0] - b.args[0])
    if b is ZERO:
        return a
    if a is ZERO:
        return neg(b)
    if a is b:
        return ZERO
    return Expr("sub", (a, b))


def mul(a: Expr, b: Expr) -> Expr:
    if is_const(a) and is_const(b):
        return const(a.args[0] * b.args[0])
    if a is ZERO or b is ZERO:
        return ZERO
    if a is ONE:
        return b
    if b is ONE:
        return a
    if is_const(b):  # constants first, a canonical order that helps sharing
        a, b = b, a
    return Expr("mul", (a, b))


def div(a: Expr, b: Expr) -> Expr:
    if is_const(b):
        if b.args[0] == 0.0:
            raise ZeroDivisionError("per-point division by the constant zero")
        if is_const(a):
            return const(a.args[0] / b.args[0])
        if b is ONE:
            return a
    if a is ZERO:
        return ZERO
    return Expr("div", (a, b))


def neg(a: Expr) -> Expr:
    if is_const(a):
        return const(-a.args[0])
    if a.kind == "neg":
        return a.args[0]
    return Expr("neg", (a,))


def powi(a: Expr, n: int) -> Expr:
    n = int(n)
    if n == 0:
        return ONE
    if n == 1:
        return a
    if is_const(a):
        return const(a.args[0] ** n)
    return Expr("powi", (a, n))


_CONST_FUNCS: dict[str, Callable[[float], float]] = {
    "sin": math.sin, "cos": math.cos, "exp": math.exp, "tanh": math.tanh, "sqrt": math.sqrt, "log": math.log,
    "log1p": math.log1p, "expm1": math.expm1, "erf": math.erf, "erfc": math.erfc, "tan": math.tan,
}

TWO_OVER_SQRT_PI = 2.0 / math.sqrt(math.pi)


def unary(kind: str, a) -> Expr:
    a = as_expr(a)
    if kind == "neg":
        return neg(a)
    if is_const(a):
        return const(_CONST_FUNCS[kind](a.args[0]))
    return Expr(kind, (a,))


def children(e: Expr) -> tuple:
    if e.kind in ("const", "sym", "net"):
        return ()
    if e.kind == "powi":
        return (e.args[0],)
    return e.args


def topological(roots: Iterable[Expr]) -> list[Expr]:
    order: list[Expr] = []
    seen: set = set()
    for root in roots:
        stack = [(root, False)]
        while stack:
            node, expanded = stack.pop()
            if expanded:
                order.append(node)
                continue
            if node in seen:
                continue
            seen.add(node)
            stack.append((node, True))
            for child in reversed(children(node)):
                if child not in seen:
                    stack.append((child, False))
    return order


def derivative(root: Expr, leaf_rule: Callable[[Expr], Expr]) -> Expr:
    """d(root)/d(variable); leaf_rule gives the derivative of sym and net leaves."""
    d: dict[Expr, Expr] = {}
    for e in topological([root]):
        k = e.kind
        if k == "const":
            r = ZERO
        elif k in ("sym", "net"):
            r = leaf_rule(e)
        elif k == "add":
            r = add(d[e.args[0]], d[e.args[1]])
        elif k == "sub":
            r = sub(d[e.args[0]], d[e.args[1]])
        elif k == "mul":
            a, b = e.args
            r = add(mul(d[a], b), mul(a, d[b]))
        elif k == "div":
            a, b = e.args
            # d(a/b) = da/b - (a/b) * db/b
            r = sub(div(d[a], b), mul(div(e, b), d[b])) if d[b] is not ZERO else div(d[a], b)
        elif k == "neg":
            r = neg(d[e.args[0]])
        elif k == "powi":
            a, n = e.args
            r = mul(mul(const(n), powi(a, n - 1)), d[a])
        elif k == "sin":
            r = mul(unary("cos", e.args[0]), d[e.args[0]])
        elif k == "cos":
            r = neg(mul(unary("sin", e.args[0]), d[e.args[0]]))
        elif k == "exp":
            r = mul(e, d[e.args[0]])
        elif k == "tanh":
            r = mul(sub(ONE, mul(e, e)), d[e.args[0]])
        elif k == "sqrt":
            r = div(d[e.args[0]], mul(const(2.0), e))
        elif k == "log":
            r = div(d[e.args[0]], e.args[0])
        # The chains below are the reference's (unary_math_chain, tensor_ir/elementwise.rs:416-450).
        elif k == "log1p":
            r = div(d[e.args[0]], add(ONE, e.args[0]))
        elif k == "expm1":
            r = mul(unary("exp", e.args[0]), d[e.args[0]])
        elif k in ("erf", "erfc"):
            a = e.args[0]
            bell = mul(const(TWO_OVER_SQRT_PI if k == "erf" else -TWO_OVER_SQRT_PI), unary("exp", neg(mul(a, a))))
            r = mul(bell, d[a])
        elif k == "tan":
            r = mul(add(ONE, mul(e, e)), d[e.args[0]])
        else:  # pragma: no cover
            raise UnsupportedExpression(f"no derivative rule for {k}")
        d[e] = r
    return d[root]


def substitute(root: Expr, mapping: dict) -> Expr:
    """Replace leaves by expressions; net leaves have their input maps rewritten too."""
    out: dict[Expr, Expr] = {}
    for e in topological([root]):
        k = e.kind
        if e in mapping:
            r = mapping[e]
        elif k in ("const", "sym"):
            r = e
        elif k == "net":
            network, word = e.args
            r = net(network.substituted(mapping), word)
        elif k == "powi":
            r = powi(out[e.args[0]], e.args[1])
        elif k in _BINARY_OPS:
            r = {"add": add, "sub": sub, "mul": mul, "div": div}[k](out[e.args[0]], out[e.args[1]])
        else:
            r = unary(k, out[e.args[0]])
        out[e] = r
    return out[root]


MERGED_WORD = ("merged",)  # word of the net leaf that stands for a weighted sum of second derivatives


def merge_weighted_sum(root: Expr, targets: list[Expr], merged_leaf: Expr):
    """Rewrite `root` so that the leaves `targets` appear only through `merged_leaf`.

    Succeeds when `root` depends on the targets only through sums  sum_t c_t * t  with constant
    coefficients that are all proportional to one weight vector w (u_xx + u_yy;
    0.1 * (u_xx + u_yy + u_zz) - u_t; ...).  Returns (new_root, {target: w_t}) with
    merged_leaf = sum_t w_t * t, or None when some target is used in another way (multiplied by a
    non-constant, alone inside a nonlinear function with different weights, ...).
    """
    target_set = set(targets)
    weights: dict[Expr, float] = {}

    def close(coeffs: dict, rest: Expr):
        """The node  rest + sum coeffs[t] * t  as  rest + k * merged_leaf, fixing or checking w."""
        if not coeffs:
            return rest
        if not weights:
            if set(coeffs) != target_set or any(c == 0.0 for c in coeffs.values()):
                return None
            weights.update(coeffs)
            return add(rest, merged_leaf)
        if set(coeffs) != set(weights):
            return None
        first = next(iter(weights))
        k = coeffs[first] / weights[first]
        for t, c in coeffs.items():
            if abs(c - k * weights[t]) > 1e-12 * max(abs(c), abs(k * weights[t])):
                return None
        return add(rest, mul(const(k), merged_leaf))

    # value[e] = (coeffs, rest): e == rest + sum coeffs[t] * t with `rest` free of targets (rebuilt).
    value: dict[Expr, tuple[dict, Expr]] = {}
    for e in topological([root]):
        k = e.kind
        if e in target_set:
            value[e] = ({e: 1.0}, ZERO)
            continue
        if k in ("const", "sym", "net"):
            value[e] = ({}, e)
            continue
        parts = [value[c] for c in children(e)]
        if k in ("add", "sub"):
            (ca, ra), (cb, rb) = parts
            sign = 1.0 if k == "add" else -1.0
            coeffs = dict(ca)
            for t, c in cb.items():
                coeffs[t] = coeffs.get(t, 0.0) + sign * c
            value[e] = ({t: c for t, c in coeffs.items() if c != 0.0} if any(coeffs.values()) else {},
                        add(ra, rb) if k == "add" else sub(ra, rb))
            if len(value[e][0]) != len(coeffs):  # a target cancelled: give up rather than reason about it
                return None
            continue
        if k == "neg":
            (ca, ra), = parts
            value[e] = ({t: -c for t, c in ca.items()}, neg(ra))
            continue
        if k == "mul":
            (ca, ra), (cb, rb) = parts
            if ca and not cb and is_const(rb):
                ca, ra, cb, rb = cb, rb, ca, ra
            if cb and not ca and is_const(ra):
                factor = ra.args[0]
                value[e] = ({t: factor * c for t, c in cb.items()}, mul(ra, rb))
                continue
        if k == "div":
            (ca, ra), (cb, rb) = parts
            if ca and not cb and is_const(rb):
                factor = 1.0 / rb.args[0]
                value[e] = ({t: factor * c for t, c in ca.items()}, div(ra, rb))
                continue
        # Any other use is nonlinear in the children: each child that carries targets is closed here.
        closed = []
        for coeffs, rest in parts:
            node = close(coeffs, rest)
            if node is None:
                return None
            closed.append(node)
        if k == "powi":
            rebuilt = powi(closed[0], e.args[1])
        elif k in _BINARY_OPS:
            rebuilt = {"add": add, "sub": sub, "mul": mul, "div": div}[k](closed[0], closed[1])
        else:
            rebuilt = unary(k, closed[0])
        value[e] = ({}, rebuilt)
    new_root = close(*value[root])
    if new_root is None or not weights:
        return None
    return new_root, weights


def leaves(roots: Iterable[Expr], kind: str) -> list[Expr]:
    return [e for e in topological(roots) if e.kind == kind]


class Program:
    """A compiled register program: what qb200_desc_set_program takes."""

    def __init__(self, code: list[int], consts: list[float], n_regs: int, value_reg: int, grad_regs: list[int]):
        self.code = code
        self.consts = consts
        self.n_regs = n_regs
        self.value_reg = value_reg
        self.grad_regs = grad_regs

    @property
    def n_instr(self) -> int:
        return len(self.code) // 4


def compile_program(value: Expr, grads: list[Expr | None], column_of: Callable[[Expr], int],
                    stream_of: Callable[[Expr], int]) -> Program:
    """Lower `value` and the per-stream derivatives to one register program.

    column_of maps a sym leaf to its point-table column, stream_of a net leaf
    to its output stream.  Registers are reused once a value is dead; outputs
    stay live to the end.
    """
    outputs = [value] + [g for g in grads if g is not None and g is not ZERO]
    order = topological(outputs)
    last_use: dict[Expr, int] = {}
    for position, e in enumerate(order):
        for child in children(e):
            last_use[child] = position
    keep = set(outputs)
    consts: list[float] = []
    const_index: dict[float, int] = {}
    free: list[int] = []
    n_regs = 0
    reg: dict[Expr, int] = {}
    code: list[int] = []
    for position, e in enumerate(order):
        k = e.kind
        operands = [reg[c] for c in children(e)]
        # Release operands that die here before taking the destination, so an
        # instruction may overwrite its own operand.
        for child in set(children(e)):
            if last_use[child] == position and child not in keep:
                free.append(reg[child])
        if free:
            dst = free.pop()
        else:
            dst = n_regs
            n_regs += 1
        reg[e] = dst
        if k == "const":
            v = e.args[0]
            if v not in const_index:
                const_index[v] = len(consts)
                consts.append(v)
            code += [OP_CONST, dst, const_index[v], 0]
        elif k == "sym":
            code += [OP_COL, dst, column_of(e), 0]
        elif k == "net":
            code += [OP_JET, dst, stream_of(e), 0]
        elif k == "powi":
            code += [OP_POWI, dst, operands[0], e.args[1]]
        elif k in _BINARY_OPS:
            code += [_BINARY_OPS[k], dst, operands[0], operands[1]]
        else:
            code += [_UNARY_OPS[k], dst, operands[0], 0]
    if n_regs > MAX_REGS:
        raise UnsupportedExpression(f"the residual needs {n_regs} registers, at most {MAX_REGS} are available")
    if len(code) // 4 > MAX_INSTR:
        raise UnsupportedExpression(f"the residual compiles to {len(code) // 4} instructions, at most {MAX_INSTR}")
    grad_regs = [reg[g] if (g is not None and g is not ZERO) else -1 for g in grads]
    return Program(code, consts, n_regs, reg[value], grad_regs)


def evaluate(root: Expr, leaf_value: Callable[[Expr], float]) -> float:
    """Host evaluation in double, for tests of the symbolic layer itself."""
    out: dict[Expr, float] = {}
    for e in topological([root]):
        k = e.kind
        if k == "const":
            r = e.args[0]
        elif k in ("sym", "net"):
            r = leaf_value(e)
        elif k == "add":
            r = out[e.args[0]] + out[e.args[1]]
        elif k == "sub":
            r = out[e.args[0]] - out[e.args[1]]
        elif k == "mul":
            r = out[e.args[0]] * out[e.args[1]]
        elif k == "div":
            r = out[e.args[0]] / out[e.args[1]]
        elif k == "neg":
            r = -out[e.args[0]]
        elif k == "powi":
            r = out[e.args[0]] ** e.args[1]
        else:
            r = _CONST_FUNCS[k](out[e.args[0]])
        out[e] = r
    return out[root]
