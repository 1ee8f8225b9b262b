"""ctypes binding of libqb200.so (the C ABI declared in include/qb200.h).

The library is the only compute path: if it is missing it is built with nvcc,
and if that fails the import error is raised to the caller.  There is no CPU
fallback behind this module.
"""

from __future__ import annotations

import ctypes as C
import os

from . import _build

OK, INVALID, UNSUPPORTED, CUDA_ERROR, NCCL_ERROR, NOT_BOUND, TOO_LARGE = range(7)
F32, F64 = 0, 1
WEIGHT, BIAS = 0, 1
ACT_TANH, ACT_SIN, ACT_SIGMOID, ACT_SOFTPLUS, ACT_SILU, ACT_GELU = range(6)
ACTIVATIONS = {"tanh": ACT_TANH, "sin": ACT_SIN, "sigmoid": ACT_SIGMOID, "softplus": ACT_SOFTPLUS, "silu": ACT_SILU,
               "gelu": ACT_GELU}
SGD, ADAM = 0, 1
REDUCE_SUM, REDUCE_MEAN = 0, 1
(Q_DEVICE_BUFFER_COUNT, Q_NONFINITE_CLIP_SEEN, Q_STREAM, Q_PARAMETER_COUNT, Q_OUTPUT_COUNT,
 Q_KERNEL_LAUNCHES, Q_FLAT_DEVICE_PTR, Q_SCRATCH_BYTES, Q_STEP_COUNT, Q_ENGINE, Q_SET0_NANOSECONDS,
 Q_ALLREDUCE_NANOSECONDS, Q_GEMM_NANOSECONDS, Q_GEMM_LAUNCHES, Q_GEMM_FLOPS, Q_LANES,
 Q_GEMM_PIPE_FLOPS) = range(17)
OPT_KERNEL_TIMERS, OPT_SINGLE_LANE = 0, 1


class OptConfig(C.Structure):
    """qb200_opt_config."""

    _fields_ = [
        ("rule", C.c_int32),
        ("has_clip", C.c_int32),
        ("learning_rate", C.c_double),
        ("beta1", C.c_double),
        ("beta2", C.c_double),
        ("epsilon", C.c_double),
        ("weight_decay", C.c_double),
        ("clip_norm", C.c_double),
    ]


class DpTiming(C.Structure):
    """qb200_dp_timing."""

    _fields_ = [
        ("replica_enqueue", C.c_double),
        ("collective", C.c_double),
        ("output_readback", C.c_double),
    ]


class BackendError(RuntimeError):
    """A qb200 call failed; `status` is the qb200_status code."""

    def __init__(self, status: int, message: str) -> None:
        super().__init__(message)
        self.status = status


# Every symbol include/qb200.h declares: name -> (restype, argtypes).
_P = C.c_void_p
_I32 = C.c_int32
_I64 = C.c_int64
SIGNATURES = {
    "qb200_last_error": (C.c_char_p, []),
    "qb200_version": (C.c_char_p, []),
    "qb200_device_count": (_I32, []),
    "qb200_desc_create": (_I32, [_I32, C.POINTER(_P)]),
    "qb200_desc_destroy": (None, [_P]),
    "qb200_desc_set_network": (_I32, [_P, C.POINTER(_I32), _I32]),
    "qb200_desc_set_activation": (_I32, [_P, _I32]),
    "qb200_desc_add_parameter": (_I32, [_P, C.c_char_p, _I32, _I32]),
    "qb200_desc_add_input": (_I32, [_P, C.c_char_p, _I64, _I64, _I32, C.POINTER(_I32)]),
    "qb200_desc_add_set": (_I32, [_P, _I64, C.c_double, C.POINTER(_I32)]),
    "qb200_desc_set_add_column": (_I32, [_P, _I32, _I32, _I32]),
    "qb200_desc_set_add_direction": (_I32, [_P, _I32, C.POINTER(C.c_double), _I32]),
    "qb200_desc_set_merge_second_order": (_I32, [_P, _I32, C.POINTER(C.c_double), _I32]),
    "qb200_desc_set_program": (_I32, [_P, _I32, C.POINTER(_I32), _I32, C.POINTER(C.c_double), _I32, _I32, _I32,
                                      C.POINTER(_I32), _I32]),
    "qb200_plan_create": (_I32, [_P, _I32, C.POINTER(_P)]),
    "qb200_plan_destroy": (None, [_P]),
    "qb200_plan_bind": (_I32, [_P, C.c_char_p, _P, C.c_size_t]),
    "qb200_plan_execute": (_I32, [_P]),
    "qb200_plan_read_output": (_I32, [_P, _I32, _P, C.c_size_t]),
    "qb200_plan_optimizer_step": (_I32, [_P, C.POINTER(OptConfig)]),
    "qb200_plan_loss": (_I32, [_P, _P]),
    "qb200_plan_read_input": (_I32, [_P, C.c_char_p, _P, C.c_size_t]),
    "qb200_plan_sample_uniform": (_I32, [_P, C.c_char_p, _I32, C.c_uint64, C.c_double, C.c_double]),
    "qb200_plan_read_moments": (_I32, [_P, _I32, _P, C.c_size_t]),
    "qb200_plan_write_moments": (_I32, [_P, _I32, _P, C.c_size_t, _I64]),
    "qb200_plan_query": (_I32, [_P, _I32, C.POINTER(_I64)]),
    "qb200_plan_set_option": (_I32, [_P, _I32, _I64]),
    "qb200_plan_synchronize": (_I32, [_P]),
    "qb200_plan_inject_wait_timeout": (_I32, [_P]),
    "qb200_nccl_unique_id": (_I32, [_P]),
    "qb200_plan_attach_comm": (_I32, [_P, _P, _I32, _I32, _I32]),
    "qb200_plan_detach_comm": (_I32, [_P]),
    "qb200_dp_create": (_I32, [_P, C.POINTER(_I32), _I32, C.POINTER(_P)]),
    "qb200_dp_destroy": (None, [_P]),
    "qb200_dp_bind_sharded": (_I32, [_P, C.c_char_p, _P, C.c_size_t]),
    "qb200_dp_bind_replicated": (_I32, [_P, C.c_char_p, _P, C.c_size_t]),
    "qb200_dp_step": (_I32, [_P, _I32, C.POINTER(DpTiming)]),
    "qb200_dp_read_output": (_I32, [_P, _I32, _P, C.c_size_t]),
    "qb200_dp_optimizer_step": (_I32, [_P, C.POINTER(OptConfig)]),
    "qb200_dp_replica": (_P, [_P, _I32]),
    "qb200_dp_replica_count": (_I32, [_P]),
    "qb200_dp_inject_host_failure": (_I32, [_P, _I32]),
    "qb200_optimizer_apply": (_I32, [_I32, _P, _P, _P, _P, _I64, C.POINTER(OptConfig), _I64, _P]),
    "qb200_weight_gradient": (_I32, [_I32, _P, _P, _I64, _I32, _I32, _P, _P]),
    "qb200_weight_gradient_static": (_I32, [_I32, _P, _P, _I64, _I32, _I32, _P, _P]),
    "qb200_matmul_3xtf32": (_I32, [_P, _P, _P, _P, _I64, _I32, _I32, _I64, _P]),
}

_library = None


def library_path() -> str:
    return _build.LIBRARY


def load() -> C.CDLL:
    """The loaded library; builds it first when the .so is absent."""
    global _library
    if _library is not None:
        return _library
    path = _build.LIBRARY
    if not os.path.exists(path):
        _build.build()
    lib = C.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        function = getattr(lib, name)  # AttributeError names the missing symbol
        function.restype = restype
        function.argtypes = argtypes
    _library = lib
    return lib


def check(status: int) -> None:
    if status != OK:
        message = load().qb200_last_error()
        raise BackendError(status, (message or b"").decode("utf-8", "replace"))
