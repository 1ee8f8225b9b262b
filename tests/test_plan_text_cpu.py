"""The reference's program text as a wire format: the literal oracle prints the traced loss of each workload as
`TensorIr::lower_text` would (crates/quabla-core/src/tensor_ir.rs:6605-6836), the recogniser turns that text into a
plan description without the Python tracer, and the description must compute what the literal oracle computes."""

import numpy as np
import pytest

from oracle import contracted, literal
from oracle.literal import api as literal_api
from oracle.literal.text import dense_constants, lower_text
from quabla_b200 import workloads
from quabla_b200._errors import UnsupportedOperationError
from quabla_b200._plantext import parse, plan_spec_from_text

from _util import relative_error


def loss_text(name, points, activation="tanh"):
    """(text, dense constants, parameter names, named inputs, literal value, literal gradients by name)."""
    w = workloads.make(name, points, api=literal, activation=activation)
    args = (w.params, *w.data)
    transform = literal.value_and_grad(w.loss)
    trace, names, leaves, _, _, _, _ = transform._graph(args)
    value, grads = transform(*args)
    parameter_count = len(literal_api._flatten([w.params])[0])
    parameter_names = names[:parameter_count]
    inputs = {n: np.asarray(l) for n, l in zip(names, leaves)}
    grad_leaves = literal_api._flatten([grads])[0]
    return (lower_text(trace.graph), dense_constants(trace.graph), parameter_names, inputs, value,
            dict(zip(parameter_names, grad_leaves)), w)


def test_the_printer_writes_the_reference_format():
    text, *_ = loss_text("poisson1d", 16)
    lines = text.splitlines()
    assert lines[0] == "%0 = input[name=arg/0] : tensor<16xf64>"
    assert any(l.endswith("= constant[value=1] : tensor<f64>") for l in lines)
    assert any("= constant[value=3.141592653589793] : tensor<f64>" in l for l in lines)
    assert any("transpose(%" in l and "axes=[1, 0]" in l for l in lines)
    assert any(l.split(" = ")[1].startswith("powi(%") and ", 2) : tensor<16xf64>" in l for l in lines)
    assert lines[-1].startswith(f"%{len(lines) - 1} = add(")
    assert len(parse(text)) == len(lines)


@pytest.mark.parametrize("name,points,activation", [
    ("poisson1d", 16, "tanh"), ("poisson2d", 8, "tanh"), ("burgers", 8, "tanh"), ("heat3d", 4, "tanh"),
    ("beam", 6, "tanh"), ("poisson1d", 16, "sin")])
def test_recognised_text_computes_what_the_literal_oracle_computes(name, points, activation):
    text, constants, parameter_names, inputs, value, grads, w = loss_text(name, points, activation)
    spec, parameters, data = plan_spec_from_text(text, parameter_names, constants=constants)
    assert spec.sizes == w.sizes and spec.activation == activation
    assert [n for n, _ in parameters] == parameter_names
    got_value, got_grads = contracted.value_and_grad(spec, inputs)
    tolerance = 1e-12 if np.dtype(w.dtype) == np.float64 else 3e-6
    assert relative_error(got_value, value) <= tolerance
    for (pname, _, _), got in zip(spec.parameters, got_grads):
        assert relative_error(got, np.asarray(grads[pname]).reshape(got.shape)) <= tolerance, pname


def test_recognised_streams_of_the_first_configuration():
    text, constants, parameter_names, *_ = loss_text("poisson1d", 16)
    spec, _, _ = plan_spec_from_text(text, parameter_names)
    interior, boundary = spec.sets
    assert interior.n_points == 16 and interior.directions == [((1.0,), 2)]  # u_xx from ninety adjoint nodes
    assert boundary.n_points == 2 and boundary.directions == []


def test_what_is_not_a_pinn_loss_is_refused():
    text, constants, parameter_names, *_ = loss_text("poisson1d", 16)
    with pytest.raises(UnsupportedOperationError, match="outside the PINN family"):
        plan_spec_from_text(text.replace("= sin(", "= arcsinh("), parameter_names)
    with pytest.raises(UnsupportedOperationError, match="is not `%k = op"):
        plan_spec_from_text(text + "\nnot a node", parameter_names)
    with pytest.raises(UnsupportedOperationError, match="is not an input"):
        plan_spec_from_text(text, ["params/9/w"])
    # A loss that uses a hidden activation directly is no derivative of the network.
    lines = text.splitlines()
    hidden = next(i for i, l in enumerate(lines) if "= tanh(" in l)
    broken = lines + [f"%{len(lines)} = sum(%{hidden}) : tensor<f64>"]
    with pytest.raises(UnsupportedOperationError):
        plan_spec_from_text("\n".join(broken), parameter_names)
    # Dense constants are not in the text.
    text2, constants2, names2, *_ = loss_text("poisson2d", 8)
    with pytest.raises(UnsupportedOperationError, match="dense constant"):
        plan_spec_from_text(text2, names2)
