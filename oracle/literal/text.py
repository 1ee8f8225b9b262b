"""The reference's program text for a literal-oracle graph — TEST INFRASTRUCTURE.

`lower_text` prints one line per node, `%id = op(operands, attributes) : tensor<dims x dtype>`, exactly as
`TensorIr::lower_text` does (crates/quabla-core/src/tensor_ir.rs:6605-6836; format pinned by
crates/quabla-core/tests/snapshots/tensor_op_transforms.txt): inputs carry their name, scalar constants their
value, dense constants no elements, axis ops their axis, `powi` its exponent, `transpose` its axes, `slice` and
`pad_slice` their window.  The literal IR's op names differ from the reference's in three places, mapped here:
sum_axis / mean_axis print as `sum` / `mean` with an axis, unary prints the kind's own name.
"""

from __future__ import annotations

from .ir import BOOL, Graph


def _number(value: float) -> str:
    """Rust's `{}` for an f64: integers without a fraction digit, otherwise the shortest round-trip form."""
    if value != value:
        return "NaN"
    if value in (float("inf"), float("-inf")):
        return "inf" if value > 0 else "-inf"
    if value == int(value) and abs(value) < 1e16:
        return str(int(value)) if not (value == 0 and str(value).startswith("-")) else "-0"
    text = repr(float(value))
    if "e" in text or "E" in text:
        mantissa, exponent = text.lower().split("e")
        return f"{mantissa}e{int(exponent)}"
    return text


def tensor_type(shape: tuple, dtype: str) -> str:
    dtype = "i1" if dtype == BOOL else dtype
    if not shape:
        return f"tensor<{dtype}>"
    return "tensor<" + "x".join(str(int(d)) for d in shape) + f"x{dtype}>"


def lower_text(graph: Graph) -> str:
    lines = []
    for index, node in enumerate(graph.nodes):
        kind = tensor_type(node.shape, node.dtype)
        ins = node.inputs
        op = node.op
        if op == "input":
            body = f"input[name={node.attrs[0]}]"
        elif op == "scalar_constant":
            body = f"constant[value={_number(node.attrs[0])}]"
        elif op == "constant":
            body = "constant[dense]"
        elif op in ("cast", "sum", "mean", "reshape", "broadcast"):
            body = f"{op}(%{ins[0]})"
        elif op in ("add", "sub", "mul", "div", "matmul", "greater"):
            body = f"{op}(%{ins[0]}, %{ins[1]})"
        elif op == "where":
            body = f"where(%{ins[0]}, %{ins[1]}, %{ins[2]})"
        elif op in ("sum_axis", "mean_axis"):
            body = f"{op[:-5]}(%{ins[0]}, axis={node.attrs[0]})"
        elif op == "powi":
            body = f"powi(%{ins[0]}, {node.attrs[0]})"
        elif op == "unary":
            body = f"{node.attrs[0]}(%{ins[0]})"
        elif op == "transpose":
            axes = node.attrs[0]
            body = f"transpose(%{ins[0]}, axes=[" + ", ".join(str(int(a)) for a in axes) + "])"
        elif op == "slice":
            axis, start, length = node.attrs
            body = f"slice(%{ins[0]}, axis={axis}, start={start}, length={length})"
        elif op == "pad_slice":
            axis, start = node.attrs
            body = f"pad_slice(%{ins[0]}, axis={axis}, start={start})"
        elif op == "concat":
            body = "concat(" + ", ".join(f"%{i}" for i in ins) + f") axis={node.attrs[0]}"
        else:
            raise NotImplementedError(op)
        lines.append(f"%{index} = {body} : {kind}")
    return "\n".join(lines)


def dense_constants(graph: Graph) -> dict:
    """{node id: array} of the dense constants, whose elements the text leaves out."""
    return {index: node.attrs[0] for index, node in enumerate(graph.nodes) if node.op == "constant"}
