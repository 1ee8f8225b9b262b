"""The stand-alone entry points over caller-owned device arrays."""

import ctypes as C

import numpy as np
import pytest

from quabla_b200 import _lib
from quabla_b200._plan import opt_config

pytestmark = pytest.mark.gpu


def _ptr(tensor):
    return C.c_void_p(tensor.data_ptr())


@pytest.mark.parametrize("dtype_name,rows,d_in,d_out", [
    ("float64", 1, 1, 1), ("float64", 127, 3, 17), ("float64", 5000, 16, 16), ("float32", 129, 17, 1),
    ("float32", 40000, 64, 64), ("float32", 8192, 2, 64), ("float64", 12289, 128, 65),
])
def test_weight_gradient_matches_a_float64_contraction(cuda_device, dtype_name, rows, d_in, d_out):
    import torch

    lib = _lib.load()
    dtype = getattr(torch, dtype_name)
    generator = torch.Generator(device="cuda").manual_seed(rows + d_in)
    acts = torch.randn(rows, d_in, dtype=dtype, device="cuda", generator=generator)
    cots = torch.randn(rows, d_out, dtype=dtype, device="cuda", generator=generator)
    grad = torch.full((d_in, d_out), float("nan"), dtype=dtype, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    code = _lib.F32 if dtype_name == "float32" else _lib.F64
    _lib.check(lib.qb200_weight_gradient(code, _ptr(acts), _ptr(cots), rows, d_in, d_out, _ptr(grad), stream))
    torch.cuda.synchronize()
    expected = (acts.double().T @ cots.double()).cpu().numpy()
    # float32: each 4096-row slice is summed in float32 (relative ~1e-6 of the
    # term magnitudes), slices in double; float64 is limited by summation order.
    scale = np.sqrt(rows)
    tolerance = (2e-6 if dtype_name == "float32" else 1e-14) * scale * 4
    assert np.max(np.abs(grad.cpu().numpy() - expected)) <= tolerance


def test_weight_gradient_rejects_bad_arguments(cuda_device):
    lib = _lib.load()
    assert lib.qb200_weight_gradient(_lib.F32, None, None, 1, 1, 1, None, None) == _lib.INVALID
    assert lib.qb200_weight_gradient(7, C.c_void_p(8), C.c_void_p(8), 1, 1, 1, C.c_void_p(8), None) == _lib.INVALID


@pytest.mark.parametrize("dtype_name", ["float32", "float64"])
def test_optimizer_apply_matches_the_host_rule_bit_for_bit(cuda_device, dtype_name):
    import torch

    from oracle import adam as host

    lib = _lib.load()
    dtype = np.dtype(dtype_name)
    rng = np.random.default_rng(3)
    count = 10007
    p = rng.standard_normal(count).astype(dtype)
    g = (rng.standard_normal(count) * 10.0 ** rng.integers(-6, 3, count)).astype(dtype)
    m = np.zeros(count, dtype=dtype)
    v = np.zeros(count, dtype=dtype)
    dp, dg, dm, dv = (torch.from_numpy(a.copy()).cuda() for a in (p, g, m, v))
    config = opt_config("adam", 3e-3, 0.9, 0.999, 1e-8, 0.01)
    code = _lib.F32 if dtype_name == "float32" else _lib.F64
    for step in range(1, 4):
        _lib.check(lib.qb200_optimizer_apply(code, _ptr(dp), _ptr(dg), _ptr(dm), _ptr(dv), count, C.byref(config),
                                             step, C.c_void_p(torch.cuda.current_stream().cuda_stream)))
        torch.cuda.synchronize()
        p, m, v = host.adam_update(p, g, m, v, step, 3e-3, 0.9, 0.999, 1e-8, 0.01, dtype)
        assert dp.cpu().numpy().tobytes() == p.tobytes()
        assert dm.cpu().numpy().tobytes() == m.tobytes()
        assert dv.cpu().numpy().tobytes() == v.tobytes()


@pytest.mark.parametrize("M,N,K", [(1, 64, 32), (127, 64, 64), (129, 128, 96), (1000, 192, 64), (4096, 256, 256)])
def test_matmul_3xtf32_keeps_float32_accuracy(cuda_device, M, N, K):
    import torch

    lib = _lib.load()
    generator = torch.Generator(device="cuda").manual_seed(M + N + K)
    a = torch.randn(M, K, device="cuda", generator=generator)
    w = torch.randn(K, N, device="cuda", generator=generator) / K**0.5
    bias = torch.randn(N, device="cuda", generator=generator)
    out = torch.full((M, N), float("nan"), device="cuda")
    biased = M // 2
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.qb200_matmul_3xtf32(_ptr(a), _ptr(w), _ptr(bias), _ptr(out), M, N, K, biased, stream))
    expected = a.double() @ w.double()
    expected[:biased] += bias.double()
    error = (out.double() - expected).abs().max().item() / expected.abs().max().item()
    assert error <= 2e-6  # plain TF32 would be ~1e-3


def test_matmul_3xtf32_rejects_unsupported_shapes(cuda_device):
    lib = _lib.load()
    eight = C.c_void_p(8)
    assert lib.qb200_matmul_3xtf32(eight, eight, None, eight, 4, 48, 32, 0, None) == _lib.UNSUPPORTED
    assert lib.qb200_matmul_3xtf32(eight, eight, None, eight, 4, 64, 20, 0, None) == _lib.UNSUPPORTED
    assert lib.qb200_matmul_3xtf32(None, eight, None, eight, 4, 64, 32, 0, None) == _lib.INVALID


@pytest.mark.parametrize("rows,d_in,d_out", [(4096, 128, 64), (10000, 256, 256), (33, 128, 128)])
def test_weight_gradient_on_the_tensor_cores(cuda_device, rows, d_in, d_out):
    # Shapes with d_in % 128 == 0 and d_out % 64 == 0 take the tcgen05 kernel in float32.
    import torch

    lib = _lib.load()
    generator = torch.Generator(device="cuda").manual_seed(rows)
    acts = torch.randn(rows, d_in, device="cuda", generator=generator)
    cots = torch.randn(rows, d_out, device="cuda", generator=generator)
    grad = torch.full((d_in, d_out), float("nan"), device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.qb200_weight_gradient(_lib.F32, _ptr(acts), _ptr(cots), rows, d_in, d_out, _ptr(grad), stream))
    torch.cuda.synchronize()
    expected = acts.double().T @ cots.double()
    error = (grad.double() - expected).abs().max().item() / expected.abs().max().item()
    assert error <= 2e-6


@pytest.mark.parametrize("rows,d_in,d_out", [(20000, 128, 128), (5001, 256, 64), (33, 64, 128), (70000, 2, 128),
                                             (70000, 128, 1)])
def test_float64_weight_gradient_variants(cuda_device, rows, d_in, d_out):
    # 128-wide shapes run on the FP64 tensor-core kernel, narrow sides on the SIMT kernel.
    import torch

    lib = _lib.load()
    generator = torch.Generator(device="cuda").manual_seed(rows)
    acts = torch.randn(rows, d_in, dtype=torch.float64, device="cuda", generator=generator)
    cots = torch.randn(rows, d_out, dtype=torch.float64, device="cuda", generator=generator)
    grad = torch.full((d_in, d_out), float("nan"), dtype=torch.float64, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.qb200_weight_gradient(_lib.F64, _ptr(acts), _ptr(cots), rows, d_in, d_out, _ptr(grad), stream))
    torch.cuda.synchronize()
    expected = (acts.T @ cots).cpu().numpy()
    assert np.max(np.abs(grad.cpu().numpy() - expected)) <= 1e-14 * np.sqrt(rows) * 8


@pytest.mark.parametrize("M,N,K", [(300000, 256, 256), (70001, 128, 64)])
def test_matmul_3xtf32_over_many_tiles(cuda_device, M, N, K):
    # Persistent CTAs walk several output tiles each; the stage ring runs across tile boundaries.
    import torch

    lib = _lib.load()
    generator = torch.Generator(device="cuda").manual_seed(M)
    a = torch.randn(M, K, device="cuda", generator=generator)
    w = torch.randn(K, N, device="cuda", generator=generator) / K ** 0.5
    c = torch.full((M, N), float("nan"), device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    _lib.check(lib.qb200_matmul_3xtf32(_ptr(a), _ptr(w), None, _ptr(c), M, N, K, 0, stream))
    expected = a.double() @ w.double()
    error = (c.double() - expected).abs().max().item() / expected.abs().max().item()
    assert error <= 2e-6


@pytest.mark.parametrize("dtype", [np.float32, np.float64])
def test_device_resampling_equals_the_host_generator_bit_for_bit(cuda_device, dtype):
    import quabla_b200 as qb
    from quabla_b200 import workloads
    from quabla_b200._plan import Plan

    from _util import traced

    name = "poisson2d" if dtype == np.float32 else "burgers"
    w, compiled, inputs = traced(name, 5000)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    data_name, rows, cols, _ = compiled.spec.inputs[0]
    bounds = [(-1.0, 1.0), (0.0, 0.3)][:cols] if cols <= 2 else [(0.0, 1.0)] * cols
    key = qb.random.key(20240607)
    for j, (low, high) in enumerate(bounds):
        plan.sample_uniform(data_name, j, qb.random.fold_in(key, j), low, high)
    got = plan.read_input(data_name, (rows, cols))
    for j, (low, high) in enumerate(bounds):
        expected = qb.random.uniform(qb.random.fold_in(key, j), (rows,), dtype, low, high)
        assert got[:, j].tobytes() == expected.tobytes()
    with pytest.raises(_lib.BackendError):
        plan.sample_uniform(data_name, cols, key, 0.0, 1.0)
    with pytest.raises(_lib.BackendError):
        plan.sample_uniform(data_name, 0, key, 1.0, 1.0)
    plan.close()


def test_trainer_resample_trains_on_the_same_batch_as_a_host_draw(cuda_device):
    import quabla_b200 as qb
    from quabla_b200 import workloads

    w = workloads.make("poisson2d", 1024)
    key = qb.random.key(7)
    bounds = [(0.0, 1.0), (0.0, 1.0)]
    rows = w.data[0].shape[0]
    host_batch = np.stack([qb.random.uniform(qb.random.fold_in(key, j), (rows,), np.float32, *bounds[j])
                           for j in range(2)], axis=1)
    a = qb.optim.Trainer(w.loss, w.params, qb.optim.Adam(1e-3), *w.data, device="cuda:0", batch_argnums=(0,))
    b = qb.optim.Trainer(w.loss, w.params, qb.optim.Adam(1e-3), *w.data, device="cuda:0", batch_argnums=(0,))
    a.step(host_batch)
    b.resample(0, key, bounds)
    b.step()
    assert np.asarray(a.value).tobytes() == np.asarray(b.value).tobytes()
    for pa, pb in zip(a.params, b.params):
        assert pa["w"].tobytes() == pb["w"].tobytes() and pa["b"].tobytes() == pb["b"].tobytes()
