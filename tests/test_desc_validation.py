"""Plan descriptions are validated before any device work (the reference's rule:
validation errors precede device work, cuda_optimizer.rs:207-212, cuda.rs:3349-3368), so the
error paths of qb200_plan_create can be exercised without a GPU."""

import ctypes as C
import copy

import numpy as np
import pytest

from quabla_b200 import _lib
from quabla_b200._plan import PlanSpec, SetSpec, build_desc
from quabla_b200 import _symbolic as sx
from quabla_b200._symbolic import Program

INVALID, UNSUPPORTED = 1, 2


def _program(streams: int) -> Program:
    # value = jet 0 squared; gradient wrt stream 0 = 2 * jet 0, others zero.
    code = [sx.OP_JET, 0, 0, 0, sx.OP_MUL, 1, 0, 0, sx.OP_ADD, 2, 0, 0]
    return Program(code=code, consts=[], n_regs=3, value_reg=1, grad_regs=[2] + [-1] * (streams - 1))


def _spec() -> PlanSpec:
    spec = PlanSpec(dtype=np.dtype(np.float64), sizes=[2, 8, 1])
    spec.parameters = [("p/0/w", 0, _lib.WEIGHT), ("p/0/b", 0, _lib.BIAS), ("p/1/w", 1, _lib.WEIGHT)]
    spec.inputs = [("x", 16, 2, True)]
    spec.sets = [SetSpec(n_points=16, weight=1.0 / 16, columns=[(0, 0), (0, 1)],
                         directions=[((1.0, 0.0), 2)], program=_program(3))]
    return spec


def _create(spec) -> tuple[int, str]:
    lib = _lib.load()
    desc = build_desc(spec)
    try:
        plan = C.c_void_p()
        status = lib.qb200_plan_create(desc, 0, C.byref(plan))
        message = lib.qb200_last_error().decode()
        if status == 0:
            lib.qb200_plan_destroy(plan)
        return status, message
    finally:
        lib.qb200_desc_destroy(desc)


def _check(mutate, status, fragment):
    spec = _spec()
    mutate(spec)
    got, message = _create(spec)
    assert got == status, message
    assert fragment in message, message


def test_a_valid_description_passes_validation():
    # Without a GPU the call then fails at the device, never at validation.
    status, message = _create(_spec())
    assert status in (0, 3), message  # QB200_OK or QB200_CUDA_ERROR


@pytest.mark.parametrize("mutate,status,fragment", [
    (lambda s: setattr(s, "sizes", [2, 8, 3]), UNSUPPORTED, "one scalar per point"),
    (lambda s: setattr(s, "sizes", [32, 8, 1]), UNSUPPORTED, "input width"),
    (lambda s: s.parameters.pop(2), INVALID, "exactly one weight"),
    (lambda s: s.parameters.append(("p/0/w", 1, _lib.BIAS)), INVALID, "duplicate parameter"),
    (lambda s: s.parameters.append(("x", 1, _lib.BIAS)), INVALID, "both a parameter and an input"),
    (lambda s: setattr(s, "sets", []), INVALID, "no point set"),
    (lambda s: setattr(s.sets[0], "n_points", 0), INVALID, "point count"),
    (lambda s: setattr(s.sets[0], "n_points", 15), INVALID, "rows for"),
    (lambda s: setattr(s.sets[0], "weight", float("nan")), INVALID, "finite"),
    (lambda s: setattr(s.sets[0], "columns", [(0, 0)]), INVALID, "network inputs"),
    (lambda s: setattr(s.sets[0], "columns", [(0, 0), (0, 2)]), INVALID, "column 2"),
    (lambda s: setattr(s.sets[0], "directions", [((1.0, 0.0), 5)]), UNSUPPORTED, "derivative order"),
    (lambda s: setattr(s.sets[0], "directions", [((1.0, 0.0), 4)] * 5), UNSUPPORTED, "streams exceed"),
])
def test_description_errors_are_reported_before_device_work(mutate, status, fragment):
    def wrapped(spec):
        mutate(spec)
        # keep the program's gradient-register count in step with the streams where the case is not about it
        streams = spec.sets[0].streams if spec.sets else 0
        if spec.sets and streams <= 17 and all(1 <= k <= 4 for _, k in spec.sets[0].directions):
            spec.sets[0].program = _program(streams)

    _check(wrapped, status, fragment)


def test_program_errors():
    def unknown_opcode(spec):
        p = copy.deepcopy(spec.sets[0].program)
        p.code[0] = 99
        spec.sets[0].program = p

    _check(unknown_opcode, UNSUPPORTED, "unknown opcode")

    def read_before_write(spec):
        p = copy.deepcopy(spec.sets[0].program)
        p.code[4:8] = [sx.OP_MUL, 1, 2, 2]  # register 2 is written later
        spec.sets[0].program = p

    _check(read_before_write, INVALID, "read before it is written")

    def value_never_written(spec):
        p = copy.deepcopy(spec.sets[0].program)
        p.n_regs, p.value_reg = 4, 3
        spec.sets[0].program = p

    _check(value_never_written, INVALID, "value register")

    def wrong_gradient_count(spec):
        p = copy.deepcopy(spec.sets[0].program)
        p.grad_regs = [2]
        spec.sets[0].program = p

    _check(wrong_gradient_count, INVALID, "gradient registers")


def test_activation_is_checked():
    lib = _lib.load()
    desc = C.c_void_p()
    _lib.check(lib.qb200_desc_create(_lib.F32, C.byref(desc)))
    for code in _lib.ACTIVATIONS.values():
        assert lib.qb200_desc_set_activation(desc, code) == 0
    for code in (-1, 6, 7):
        assert lib.qb200_desc_set_activation(desc, code) == UNSUPPORTED
        assert "tanh (0), sin (1), sigmoid (2), softplus (3), silu (4) or gelu (5)" in lib.qb200_last_error().decode()
    lib.qb200_desc_destroy(desc)


def test_merged_stream_declaration_is_validated():
    lib = _lib.load()

    def declare(weights, *, directions=2, after_program=False):
        desc = C.c_void_p()
        assert lib.qb200_desc_create(_lib.F64, C.byref(desc)) == 0
        try:
            sizes = (C.c_int32 * 3)(2, 8, 1)
            assert lib.qb200_desc_set_network(desc, sizes, 3) == 0
            index = C.c_int32()
            assert lib.qb200_desc_add_input(desc, b"x", 16, 2, 1, C.byref(index)) == 0
            set_index = C.c_int32()
            assert lib.qb200_desc_add_set(desc, 16, 1.0 / 16, C.byref(set_index)) == 0
            for j in range(directions):
                vec = (C.c_double * 2)(*[1.0 if k == j else 0.0 for k in range(2)])
                assert lib.qb200_desc_set_add_direction(desc, set_index.value, vec, 1) == 0
            if after_program:
                p = _program(1 + directions)
                assert lib.qb200_desc_set_program(desc, set_index.value, (C.c_int32 * len(p.code))(*p.code), p.n_instr,
                                                  (C.c_double * 1)(), 0, p.n_regs, p.value_reg,
                                                  (C.c_int32 * len(p.grad_regs))(*p.grad_regs), len(p.grad_regs)) == 0
            array = (C.c_double * max(1, len(weights)))(*weights) if weights is not None else None
            status = lib.qb200_desc_set_merge_second_order(desc, set_index.value, array, len(weights or ()))
            return status, lib.qb200_last_error().decode()
        finally:
            lib.qb200_desc_destroy(desc)

    assert declare([1.0, 1.0])[0] == 0
    assert declare([1.0, 0.0])[0] == 0  # a direction may stay out of the sum
    for weights, kwargs, fragment in (([1.0], {}, "1 merge weights for 2 directions"),
                                      ([1.0, 1.0, 1.0], {}, "3 merge weights for 2 directions"),
                                      (None, {}, "merge weights are missing"),
                                      ([1.0, float("nan")], {}, "not finite"),
                                      ([1.0, float("inf")], {}, "not finite"),
                                      ([1.0, 1.0], {"after_program": True}, "before the program")):
        status, message = declare(weights, **kwargs)
        assert status == INVALID and fragment in message, (weights, message)


def test_a_merged_set_counts_its_extra_stream():
    # Two first-order directions plus the merged stream: the program addresses stream 3.
    spec = _spec()
    code = [sx.OP_JET, 0, 3, 0, sx.OP_MUL, 1, 0, 0, sx.OP_ADD, 2, 0, 0]
    program = Program(code=code, consts=[], n_regs=3, value_reg=1, grad_regs=[-1, -1, -1, 2])
    spec.sets = [SetSpec(n_points=16, weight=1.0 / 16, columns=[(0, 0), (0, 1)],
                         directions=[((1.0, 0.0), 1), ((0.0, 1.0), 1)], program=program, merge_weights=[1.0, 1.0])]
    assert spec.sets[0].streams == 4
    status, message = _create(spec)
    assert status in (0, 3), message
    spec.sets[0].merge_weights = None  # without the declaration stream 3 does not exist
    status, message = _create(spec)
    assert status == INVALID, message
