"""Graph-to-graph transforms of the reference — TEST INFRASTRUCTURE (literal oracle).

symbolic_vjp     crates/quabla-core/src/tensor_ir.rs:3359-3906 with the per-op
                 rules of tensor_ir/op/vjp.rs:19-431 (same node order);
symbolic_jvp     tensor_ir.rs:2999-3319 with tensor_ir/op/jvp.rs:16-346;
inline           tensor_ir.rs:2533-2577;
inline_batched   tensor_ir.rs:2612-2690 with tensor_ir/op/batch.rs:21-205.
"""

from __future__ import annotations

import math

import numpy as np

from .ir import F64, Graph, Node


# -- helpers shared by the reverse rules (tensor_ir.rs:7828-7839, 9249-9372) -------
def _accumulate(g: Graph, cotangents: list, target: int, contribution: int) -> None:
    existing = cotangents[target]
    cotangents[target] = contribution if existing is None else g.add(existing, contribution)


def _full_like(g: Graph, value: float, target: int) -> int:
    node = g.node(target)
    constant = g.constant_like(value, node.dtype, node.weak)
    return constant if node.shape == () else g.broadcast_to(constant, node.shape)


def _broadcast_like(g: Graph, value: int, target: int) -> int:
    return g.mul(value, _full_like(g, 1.0, target))


def _expand_reduced_axis(g: Graph, value: int, target: int, axis: int) -> int:
    shape = list(g.shape(target))
    expanded = list(shape)
    expanded[axis] = 1
    return g.broadcast_to(g.reshape(value, expanded), shape)


def _reduce_to_shape(g: Graph, value: int, source: tuple, target: tuple) -> int:
    offset = len(source) - len(target)
    reduced = value
    for axis in reversed(range(len(source))):
        if axis < offset or (target[axis - offset] == 1 and source[axis] != 1):
            reduced = g.sum_axis(reduced, axis)
    return g.reshape(reduced, target)


def _transpose_last_two(g: Graph, value: int, shape: tuple) -> int:
    axes = list(range(len(shape)))
    axes[-1], axes[-2] = axes[-2], axes[-1]
    return g.transpose(value, axes)


def _unary_chain(g: Graph, kind: str, operand: int, value: int):
    """(mode, node): the scaling a unary op applies to a tangent or cotangent
    (unary_math_chain, tensor_ir/elementwise.rs:416-450)."""
    if kind == "exp":
        return "times", value
    if kind == "tanh":
        one = g.scalar_constant(1.0)
        squared = g.mul(value, value)
        return "times", g.sub(one, squared)
    if kind == "sin":
        return "times", g.unary(operand, "cos")
    if kind == "cos":
        return "negated", g.unary(operand, "sin")
    if kind == "log1p":
        one = g.scalar_constant(1.0)
        return "over", g.add(one, operand)
    if kind == "expm1":
        return "times", g.unary(operand, "exp")
    if kind in ("erf", "erfc"):
        # sign * 2 / sqrt(pi) * exp(-(x * x))  (erf_derivative, tensor_ir/elementwise.rs:487-500)
        squared = g.mul(operand, operand)
        zero = g.scalar_constant(0.0)
        bell = g.unary(g.sub(zero, squared), "exp")
        scale = g.scalar_constant((2.0 if kind == "erf" else -2.0) / math.sqrt(math.pi))
        return "times", g.mul(scale, bell)
    if kind == "tan":
        one = g.scalar_constant(1.0)
        return "times", g.add(one, g.mul(value, value))
    raise ValueError(kind)


def _apply_chain(g: Graph, chain, seed: int) -> int:
    mode, derivative = chain
    if mode == "over":
        return g.div(seed, derivative)
    product = g.mul(seed, derivative)
    if mode == "times":
        return product
    zero = g.scalar_constant(0.0)
    return g.sub(zero, product)


def _reachable(src: Graph, outputs) -> list:
    seen = [False] * len(src.nodes)
    pending = list(outputs)
    while pending:
        i = pending.pop()
        if not seen[i]:
            seen[i] = True
            pending.extend(src.node(i).inputs)
    return seen


# -- reverse mode ----------------------------------------------------------------------
def _push_vjp(src: Graph, node_id: int, upstream: int, g: Graph, values: list, cot: list) -> None:
    node = src.node(node_id)
    op, ins = node.op, node.inputs
    shape_of = lambda i: src.shape(i)  # noqa: E731
    if op in ("scalar_constant", "constant"):
        return
    if op == "cast":
        _accumulate(g, cot, ins[0], g.cast(upstream, src.node(ins[0]).dtype))
    elif op == "add":
        lhs = _reduce_to_shape(g, upstream, node.shape, shape_of(ins[0]))
        rhs = _reduce_to_shape(g, upstream, node.shape, shape_of(ins[1]))
        _accumulate(g, cot, ins[0], lhs)
        _accumulate(g, cot, ins[1], rhs)
    elif op == "sub":
        lhs = _reduce_to_shape(g, upstream, node.shape, shape_of(ins[0]))
        zero = g.scalar_constant(0.0)
        negated = g.sub(zero, upstream)
        rhs = _reduce_to_shape(g, negated, node.shape, shape_of(ins[1]))
        _accumulate(g, cot, ins[0], lhs)
        _accumulate(g, cot, ins[1], rhs)
    elif op == "div":
        lv, rv = values[ins[0]], values[ins[1]]
        lhs = g.div(upstream, rv)
        quotient = g.div(lv, rv)
        product = g.mul(lhs, quotient)
        zero = g.scalar_constant(0.0)
        rhs = g.sub(zero, product)
        lhs = _reduce_to_shape(g, lhs, node.shape, shape_of(ins[0]))
        rhs = _reduce_to_shape(g, rhs, node.shape, shape_of(ins[1]))
        _accumulate(g, cot, ins[0], lhs)
        _accumulate(g, cot, ins[1], rhs)
    elif op == "mul":
        lhs = g.mul(upstream, values[ins[1]])
        rhs = g.mul(upstream, values[ins[0]])
        lhs = _reduce_to_shape(g, lhs, node.shape, shape_of(ins[0]))
        rhs = _reduce_to_shape(g, rhs, node.shape, shape_of(ins[1]))
        _accumulate(g, cot, ins[0], lhs)
        _accumulate(g, cot, ins[1], rhs)
    elif op == "sum":
        _accumulate(g, cot, ins[0], _broadcast_like(g, upstream, values[ins[0]]))
    elif op == "broadcast":
        _accumulate(g, cot, ins[0], _reduce_to_shape(g, upstream, node.shape, shape_of(ins[0])))
    elif op == "sum_axis":
        _accumulate(g, cot, ins[0], _expand_reduced_axis(g, upstream, values[ins[0]], node.attrs[0]))
    elif op == "matmul":
        lt = _transpose_last_two(g, values[ins[0]], shape_of(ins[0]))
        rt = _transpose_last_two(g, values[ins[1]], shape_of(ins[1]))
        lhs = g.matmul(upstream, rt)
        rhs = g.matmul(lt, upstream)
        lhs = _reduce_to_shape(g, lhs, g.shape(lhs), shape_of(ins[0]))
        rhs = _reduce_to_shape(g, rhs, g.shape(rhs), shape_of(ins[1]))
        _accumulate(g, cot, ins[0], lhs)
        _accumulate(g, cot, ins[1], rhs)
    elif op == "reshape":
        _accumulate(g, cot, ins[0], g.reshape(upstream, shape_of(ins[0])))
    elif op == "mean":
        contribution = _broadcast_like(g, upstream, values[ins[0]])
        count = int(np.prod(shape_of(ins[0]), dtype=np.int64))
        scale = g.scalar_constant(1.0 / count)
        _accumulate(g, cot, ins[0], g.mul(contribution, scale))
    elif op == "mean_axis":
        contribution = _expand_reduced_axis(g, upstream, values[ins[0]], node.attrs[0])
        scale = g.scalar_constant(1.0 / shape_of(ins[0])[node.attrs[0]])
        _accumulate(g, cot, ins[0], g.mul(contribution, scale))
    elif op == "powi":
        exponent = node.attrs[0]
        if exponent != 0:
            coefficient = g.scalar_constant(float(exponent))
            lower = g.powi(values[ins[0]], exponent - 1)
            derivative = g.mul(coefficient, lower)
            contribution = g.mul(upstream, derivative)
            contribution = _reduce_to_shape(g, contribution, node.shape, shape_of(ins[0]))
            _accumulate(g, cot, ins[0], contribution)
    elif op == "transpose":
        axes = node.attrs[0]
        inverse = [0] * len(axes)
        for position, axis in enumerate(axes):
            inverse[axis] = position
        _accumulate(g, cot, ins[0], g.transpose(upstream, inverse))
    elif op == "unary":
        chain = _unary_chain(g, node.attrs[0], values[ins[0]], values[node_id])
        contribution = _apply_chain(g, chain, upstream)
        contribution = _reduce_to_shape(g, contribution, node.shape, shape_of(ins[0]))
        _accumulate(g, cot, ins[0], contribution)
    elif op == "greater":
        return  # a Bool result carries no cotangent
    elif op == "where":
        # where_select(condition, upstream, 0) to the true branch, where_select(condition, 0, upstream) to the
        # false branch, each reduced to its operand's shape (op/vjp.rs:124-148).
        zero = g.scalar_constant(0.0)
        on_true = g.where(values[ins[0]], upstream, zero)
        on_false = g.where(values[ins[0]], zero, upstream)
        _accumulate(g, cot, ins[1], _reduce_to_shape(g, on_true, node.shape, shape_of(ins[1])))
        _accumulate(g, cot, ins[2], _reduce_to_shape(g, on_false, node.shape, shape_of(ins[2])))
    elif op == "concat":
        start = 0
        for i in ins:
            extent = shape_of(i)[node.attrs[0]]
            _accumulate(g, cot, i, g.slice(upstream, node.attrs[0], start, extent))
            start += extent
    elif op == "slice":
        axis, start, _ = node.attrs
        _accumulate(g, cot, ins[0], g.pad_slice(upstream, shape_of(ins[0]), axis, start))
    elif op == "pad_slice":
        axis, start = node.attrs
        _accumulate(g, cot, ins[0], g.slice(upstream, axis, start, shape_of(ins[0])[axis]))
    else:
        raise NotImplementedError(f"no VJP rule for {op}")


def symbolic_vjp(src: Graph, outputs: list):
    """outputs: [(node id, cotangent input name or None for a ones seed)].
    Returns (graph, primal ids by source node, seed ids, gradients by input name)."""
    g = Graph()
    values = []
    for node in src.nodes:
        if node.op == "input":
            values.append(g.input(node.attrs[0], node.shape, node.dtype))
        else:
            values.append(g.rebuild_like(node, lambda i: values[i]))
    cot = [None] * len(src.nodes)
    seeds = []
    for output, name in outputs:
        node = src.node(output)
        if name is not None:
            seed = g.input(name, node.shape, node.dtype)
        else:
            one = g.constant_like(1.0, node.dtype, False)
            seed = one if node.shape == () else g.broadcast_to(one, node.shape)
        _accumulate(g, cot, output, seed)
        seeds.append(seed)
    for node_id in reversed(range(len(src.nodes))):
        upstream = cot[node_id]
        if upstream is None or src.node(node_id).op == "input":
            continue
        _push_vjp(src, node_id, upstream, g, values, cot)
    gradients = {}
    for node_id, node in enumerate(src.nodes):
        if node.op == "input":
            gradients[node.attrs[0]] = cot[node_id] if cot[node_id] is not None else _full_like(g, 0.0, values[node_id])
    return g, values, seeds, gradients


# -- forward mode ------------------------------------------------------------------------
def _push_jvp(g: Graph, node: Node, pairs: list):
    op, ins = node.op, node.inputs
    if op == "scalar_constant":
        return (g.constant_like(node.attrs[0], node.dtype, node.weak), g.constant_like(0.0, node.dtype, node.weak))
    if op == "constant":
        primal = g.push("constant", (), node.attrs, node.shape, node.dtype, node.weak)
        return primal, _full_like(g, 0.0, primal)
    if op == "cast":
        v, t = pairs[ins[0]]
        return (g.push("cast", (v,), (), node.shape, node.dtype, node.weak),
                g.push("cast", (t,), (), node.shape, node.dtype, node.weak))
    if op in ("add", "sub"):
        (lv, lt), (rv, rt) = pairs[ins[0]], pairs[ins[1]]
        f = g.add if op == "add" else g.sub
        return f(lv, rv), f(lt, rt)
    if op == "div":
        (lv, lt), (rv, rt) = pairs[ins[0]], pairs[ins[1]]
        quotient = g.div(lv, rv)
        scaled = g.mul(quotient, rt)
        numerator = g.sub(lt, scaled)
        return quotient, g.div(numerator, rv)
    if op == "mul":
        (lv, lt), (rv, rt) = pairs[ins[0]], pairs[ins[1]]
        left = g.mul(lt, rv)
        right = g.mul(lv, rt)
        return g.mul(lv, rv), g.add(left, right)
    if op == "unary":
        v, t = pairs[ins[0]]
        kind = node.attrs[0]
        if kind in ("sin", "cos", "log1p", "expm1", "erf", "erfc"):  # kinds that emit their derivative first
            chain = _unary_chain(g, kind, v, None)
            value = g.unary(v, kind)
        else:
            value = g.unary(v, kind)
            chain = _unary_chain(g, kind, v, value)
        return value, _apply_chain(g, chain, t)
    if op == "greater":
        value = g.greater(pairs[ins[0]][0], pairs[ins[1]][0])
        return value, value  # a Bool node has no tangent; the slot is never read
    if op == "where":
        # Both the values and the tangents are selected by the primal condition (op/jvp.rs:116-128).
        condition = pairs[ins[0]][0]
        (tv, tt), (fv, ft) = pairs[ins[1]], pairs[ins[2]]
        return g.where(condition, tv, fv), g.where(condition, tt, ft)
    if op == "matmul":
        (lv, lt), (rv, rt) = pairs[ins[0]], pairs[ins[1]]
        left = g.matmul(lt, rv)
        right = g.matmul(lv, rt)
        return g.matmul(lv, rv), g.add(left, right)
    if op in ("sum", "mean"):
        v, t = pairs[ins[0]]
        f = g.sum if op == "sum" else g.mean
        return f(v), f(t)
    if op in ("sum_axis", "mean_axis"):
        v, t = pairs[ins[0]]
        f = g.sum_axis if op == "sum_axis" else g.mean_axis
        return f(v, node.attrs[0]), f(t, node.attrs[0])
    if op == "reshape":
        v, t = pairs[ins[0]]
        return g.reshape(v, node.shape), g.reshape(t, node.shape)
    if op == "transpose":
        v, t = pairs[ins[0]]
        return g.transpose(v, node.attrs[0]), g.transpose(t, node.attrs[0])
    if op == "broadcast":
        v, t = pairs[ins[0]]
        return g.broadcast_to(v, node.shape), g.broadcast_to(t, node.shape)
    if op == "powi":
        v, t = pairs[ins[0]]
        exponent = node.attrs[0]
        value = g.powi(v, exponent)
        if exponent == 0:
            return value, _full_like(g, 0.0, v)
        coefficient = g.scalar_constant(float(exponent))
        lower = g.powi(v, exponent - 1)
        derivative = g.mul(coefficient, lower)
        return value, g.mul(t, derivative)
    if op == "concat":
        vs = [pairs[i][0] for i in ins]
        ts = [pairs[i][1] for i in ins]
        return g.concat(vs, node.attrs[0]), g.concat(ts, node.attrs[0])
    if op == "slice":
        v, t = pairs[ins[0]]
        return g.slice(v, *node.attrs), g.slice(t, *node.attrs)
    if op == "pad_slice":
        v, t = pairs[ins[0]]
        return g.pad_slice(v, node.shape, *node.attrs), g.pad_slice(t, node.shape, *node.attrs)
    raise NotImplementedError(f"no JVP rule for {op}")


def symbolic_jvp(src: Graph, outputs: list, tangent_names: dict):
    """tangent_names: input name -> name of its tangent input in the new graph;
    other inputs get a zero tangent.  Returns (graph, values, tangents)."""
    g = Graph()
    reachable = _reachable(src, outputs)
    pairs = []
    for node_id, node in enumerate(src.nodes):
        if node.op == "input":
            value = g.input(node.attrs[0], node.shape, node.dtype)
            if node.attrs[0] in tangent_names:
                tangent = g.input(tangent_names[node.attrs[0]], node.shape, node.dtype)
            else:
                tangent = _full_like(g, 0.0, value)
            pairs.append((value, tangent))
        elif not reachable[node_id]:
            pairs.append((None, None))
        else:
            pairs.append(_push_jvp(g, node, pairs))
    return g, [pairs[o][0] for o in outputs], [pairs[o][1] for o in outputs]


# -- splicing --------------------------------------------------------------------------------
def inline(g: Graph, callee: Graph, bindings: dict, outputs: list) -> list:
    reachable = _reachable(callee, outputs)
    remap = {}
    for node_id, node in enumerate(callee.nodes):
        if not reachable[node_id]:
            continue
        if node.op == "input":
            remap[node_id] = bindings[node.attrs[0]]
        else:
            remap[node_id] = g.rebuild_like(node, lambda i: remap[i])
    return [remap[o] for o in outputs]


def _pad_batched(g: Graph, node_id: int, rank: int) -> int:
    shape = g.shape(node_id)
    example_rank = len(shape) - 1
    if example_rank >= rank:
        return node_id
    padded = (shape[0],) + (1,) * (rank - example_rank) + shape[1:]
    node = g.node(node_id)
    return g.push("reshape", (node_id,), (), padded, node.dtype, node.weak)


def _batched_op(g: Graph, callee: Graph, node: Node, remap: dict, mapped: list, batch: int):
    """(op, inputs, attrs) of the batched node (batched_op, op/batch.rs:21-205)."""
    op, ins = node.op, node.inputs
    rank = len(node.shape)
    if op in ("cast", "powi", "unary", "reshape"):
        return op, tuple(remap[i] for i in ins), node.attrs
    if op in ("add", "sub", "mul", "div", "matmul", "broadcast", "greater", "where"):
        local = []
        for i in ins:
            spliced = remap[i]
            local.append(_pad_batched(g, spliced, rank) if mapped[i] else spliced)
        return op, tuple(local), node.attrs
    if op in ("sum", "mean"):
        count = int(np.prod(callee.shape(ins[0]), dtype=np.int64))
        spliced = remap[ins[0]]
        source = g.node(spliced)
        flat = g.push("reshape", (spliced,), (), (batch, count), source.dtype, source.weak)
        return ("sum_axis" if op == "sum" else "mean_axis"), (flat,), (1,)
    if op in ("sum_axis", "mean_axis"):
        return op, (remap[ins[0]],), (node.attrs[0] + 1,)
    if op == "transpose":
        return op, (remap[ins[0]],), ((0,) + tuple(a + 1 for a in node.attrs[0]),)
    if op == "concat":
        items = []
        for i in ins:
            spliced = remap[i]
            if not mapped[i]:
                source = g.node(spliced)
                spliced = g.push("broadcast", (spliced,), (), (batch,) + source.shape, source.dtype, source.weak)
            items.append(spliced)
        return op, tuple(items), (node.attrs[0] + 1,)
    if op == "slice":
        axis, start, length = node.attrs
        return op, (remap[ins[0]],), (axis + 1, start, length)
    if op == "pad_slice":
        axis, start = node.attrs
        return op, (remap[ins[0]],), (axis + 1, start)
    raise NotImplementedError(f"no batching rule for {op}")


def inline_batched(g: Graph, callee: Graph, bindings: dict, batch: int, outputs: list) -> list:
    """bindings: input name -> (node, mapped).  Returns [(node, mapped)] per output."""
    reachable = _reachable(callee, outputs)
    remap = {}
    mapped = [False] * len(callee.nodes)
    for node_id, node in enumerate(callee.nodes):
        if not reachable[node_id]:
            continue
        if node.op == "input":
            remap[node_id], mapped[node_id] = bindings[node.attrs[0]]
        elif any(mapped[i] for i in node.inputs):
            op, ins, attrs = _batched_op(g, callee, node, remap, mapped, batch)
            if op == "pad_slice":
                shape = (batch,) + node.shape
            else:
                shape = (batch,) + node.shape
            remap[node_id] = g.push(op, ins, attrs, shape, node.dtype, node.weak)
            mapped[node_id] = True
        else:
            remap[node_id] = g.rebuild_like(node, lambda i: remap[i])
    return [(remap[o], mapped[o]) for o in outputs]
