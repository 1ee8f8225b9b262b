"""qb200_weight_gradient_static: the weight gradient for hosts that cannot
allocate device memory (a plugin in a runtime that owns the pool, a loop that
may not touch the allocator).  Its scratch is an array inside the library, so
the check that matters is that it returns exactly what the allocating entry
point returns, also when a second call follows a first one that left other
data in the shared array.

Collected last on purpose: a run that stops at the first failure has then
already run every other test.
"""

import ctypes as C

import numpy as np
import pytest

from quabla_b200 import _lib

pytestmark = pytest.mark.gpu


def _ptr(tensor):
    return C.c_void_p(tensor.data_ptr())


def _both(lib, torch, dtype_name, rows, d_in, d_out, seed):
    dtype = getattr(torch, dtype_name)
    code = _lib.F32 if dtype_name == "float32" else _lib.F64
    generator = torch.Generator(device="cuda").manual_seed(seed)
    acts = torch.randn(rows, d_in, dtype=dtype, device="cuda", generator=generator)
    cots = torch.randn(rows, d_out, dtype=dtype, device="cuda", generator=generator)
    pooled = torch.full((d_in, d_out), float("nan"), dtype=dtype, device="cuda")
    fixed = torch.full((d_in, d_out), float("nan"), dtype=dtype, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.qb200_weight_gradient(code, _ptr(acts), _ptr(cots), rows, d_in, d_out, _ptr(pooled), stream))
    _lib.check(lib.qb200_weight_gradient_static(code, _ptr(acts), _ptr(cots), rows, d_in, d_out, _ptr(fixed), stream))
    torch.cuda.synchronize()
    return pooled.cpu().numpy(), fixed.cpu().numpy(), (acts.double().T @ cots.double()).cpu().numpy()


@pytest.mark.parametrize("dtype_name", ["float32", "float64"])
def test_static_scratch_variant_equals_the_allocating_one_on_two_calls_in_a_row(cuda_device, dtype_name):
    import torch

    lib = _lib.load()
    # First a call that fills many slices of the shared array, then a smaller one
    # with a different shape, which would pick up leftovers if it read any.
    # 128 x 128 and 256 x 256 take the tensor-core contraction in float32 (both entry points share one
    # dispatch), the other shapes the FP64 tensor-core or the plain kernel.
    for rows, d_in, d_out, seed in ((50000, 64, 64, 1), (4097, 17, 5, 2), (30000, 128, 128, 3), (9000, 256, 256, 4),
                                    (100, 128, 64, 5)):
        pooled, fixed, exact = _both(lib, torch, dtype_name, rows, d_in, d_out, seed)
        assert np.isfinite(fixed).all()
        # Same kernels, same split, same order of additions: identical bits.
        assert fixed.tobytes() == pooled.tobytes()
        tolerance = (2e-6 if dtype_name == "float32" else 1e-14) * np.sqrt(rows) * 4
        assert np.max(np.abs(fixed - exact)) <= tolerance


def test_static_scratch_variant_refuses_what_does_not_fit(cuda_device):
    import torch

    lib = _lib.load()
    rows, d_in, d_out = 200000, 512, 512  # 49 slices x 1 MiB of float32 > 16 MiB
    acts = torch.zeros(8, dtype=torch.float32, device="cuda")
    out = torch.zeros(8, dtype=torch.float32, device="cuda")
    status = lib.qb200_weight_gradient_static(_lib.F32, _ptr(acts), _ptr(acts), rows, d_in, d_out, _ptr(out), None)
    assert status == _lib.TOO_LARGE
    assert b"16777216" in lib.qb200_last_error()
