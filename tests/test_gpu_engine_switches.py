"""The layer-wise engine's GEMM variants (tcgen05 with tensor-map loads, FP64 MMA, SIMT) all meet the
parity gate.  The switches are read once per process, so every
variant runs in a child process."""

import json
import os
import subprocess
import sys

import numpy as np
import pytest

from _util import TOLERANCE

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def _run(name, points, **switches):
    env = dict(os.environ)
    env.update(switches)
    out = subprocess.run([sys.executable, os.path.join(HERE, "_engine_worker.py"), name, str(points)], env=env,
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    return json.loads(out.stdout.strip().splitlines()[-1])


@pytest.mark.parametrize("switches", [{}, {"QB200_TC_COR": "bf16"}, {"QB200_TC_COR": "tf32"}, {"QB200_TC": "0"}],
                         ids=["tcgen05, scheme by size", "tcgen05, bf16 corrections", "tcgen05, tf32 corrections", "simt"])
def test_wide_float32_network_on_every_gemm_variant(cuda_device, switches):
    result = _run("heat3d", 640, **switches)
    assert result["engine"] == (0 if switches.get("QB200_TC") == "0" else 3)
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32)]


@pytest.mark.parametrize("switches", [{}, {"QB200_DMMA": "0"}], ids=["fp64 mma", "simt"])
def test_wide_float64_network_on_every_gemm_variant(cuda_device, switches):
    result = _run("burgers", 1536, **switches)
    assert result["engine"] == 0
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float64)]


@pytest.mark.parametrize("name,points", [("heat3d", 900), ("burgers", 1100)])
@pytest.mark.parametrize("switches", [{"QB200_FIRST_FUSED": "0"}, {"QB200_HEAD_FUSED": "0"},
                                      {"QB200_FIRST_FUSED": "0", "QB200_HEAD_FUSED": "0"}],
                         ids=["first layer apart", "output layer apart", "both apart"])
def test_narrow_layers_in_kernels_of_their_own(cuda_device, name, points, switches):
    # By default the jet kernels form the first layer's product and weight gradient and the output layer's; the
    # separate kernels remain for shapes those cannot take and must give the same answer.
    result = _run(name, points, **switches)
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32 if name == "heat3d" else np.float64)]


@pytest.mark.parametrize("name,points,chunk,engine", [("heat3d", 1800, "512", 3), ("burgers", 1500, "256", 0)])
def test_point_sets_cut_into_chunks(cuda_device, name, points, chunk, engine):
    # Several chunks per point set, the last one ragged (its rows are not a multiple of the GEMM tile).
    result = _run(name, points, QB200_CHUNK_POINTS=chunk)
    assert result["engine"] == engine
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32 if name == "heat3d" else np.float64)]


@pytest.mark.parametrize("corrections", ["bf16", "tf32"])
def test_narrow_network_forced_onto_the_layerwise_engine(cuda_device, corrections):
    # Width 64 float32 through the layer-wise kernels: tcgen05 GEMMs with 64-column tiles.
    result = _run("poisson2d", 3000, QB200_ENGINE="layerwise", QB200_TC_COR=corrections)
    assert result["engine"] == 3
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32)]


@pytest.mark.parametrize("name,points", [("poisson2d", 3000), ("beam", 2500)])
@pytest.mark.parametrize("switches", [{}, {"QB200_FUSED_TILE": "32"}, {"QB200_FUSED": "simt"}],
                         ids=["two CTAs per SM", "one CTA per SM", "simt"])
def test_fused_engine_variants(cuda_device, name, points, switches):
    # Ragged point counts: the last tile of both tile sizes is partial.
    result = _run(name, points, **switches)
    assert result["engine"] == (1 if switches.get("QB200_FUSED") == "simt" else 2)
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32)]


def test_two_lanes_are_repeatable_and_agree_with_one_lane(cuda_device, monkeypatch):
    # float64 plans of the layer-wise engine send consecutive chunks down two streams with their own scratch and
    # accumulators (added in lane order): the result must not depend on how the lanes overlapped, and must agree
    # with the single-lane order of additions to rounding.
    from quabla_b200 import _lib
    from quabla_b200._plan import Plan

    from _util import relative_error, traced

    w, compiled, inputs = traced("burgers", 20480)

    def run(lanes):
        monkeypatch.setenv("QB200_LANES", lanes)
        plan = Plan(compiled.spec, 0)
        for key, value in inputs.items():
            plan.bind(key, value)
        assert plan.query(_lib.Q_LANES) == int(lanes)
        results = []
        for _ in range(3):
            plan.execute()
            results.append([o.copy() for o in plan.outputs()])
        plan.close()
        for later in results[1:]:
            for a, b in zip(results[0], later):
                assert a.tobytes() == b.tobytes()
        return results[0]

    two, one = run("2"), run("1")
    for a, b in zip(two, one):
        assert relative_error(a, b) <= 1e-12


@pytest.mark.parametrize("scheme,passes", [("tf32", 6.0), ("bf16", 14.0 / 3.0)])
def test_gemm_timers_report_flops_and_tensor_pipe_passes(cuda_device, monkeypatch, scheme, passes):
    # With QB200_OPT_KERNEL_TIMERS the plan reports, for the layer GEMMs of the last execute, launches, device time,
    # 2MNK and the tensor-pipe passes behind them at the bfloat16 rate: 6 per FLOP for three tf32 products, 4 where
    # the two correction products are bfloat16 instructions (forward and data gradient; the weight gradient keeps 6).
    from quabla_b200 import _lib
    from quabla_b200._plan import Plan

    from _util import traced

    monkeypatch.setenv("QB200_TC_COR", scheme)
    w, compiled, inputs = traced("heat3d", 1024)
    plan = Plan(compiled.spec, 0)
    for key, value in inputs.items():
        plan.bind(key, value)
    plan.set_option(_lib.OPT_KERNEL_TIMERS, 1)
    plan.execute()
    plan.synchronize()
    launches = plan.query(_lib.Q_GEMM_LAUNCHES)
    flops = plan.query(_lib.Q_GEMM_FLOPS)
    pipe = plan.query(_lib.Q_GEMM_PIPE_FLOPS)
    nanoseconds = plan.query(_lib.Q_GEMM_NANOSECONDS)
    plan.close()
    # Five 256 x 256 layers: forward, data gradient (not for the first of them... the first hidden layer has no GEMM
    # at all) and weight gradient each.
    assert launches == 15
    rows = 1024 * compiled.spec.sets[0].streams
    assert flops == 15 * 2 * rows * 256 * 256
    assert nanoseconds > 0
    assert abs(pipe / flops - passes) < 1e-9
