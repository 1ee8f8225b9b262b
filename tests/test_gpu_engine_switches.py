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


@pytest.mark.parametrize("switches", [{}, {"QB200_TC": "0"}], ids=["tcgen05", "simt"])
def test_wide_float32_network_on_every_gemm_variant(cuda_device, switches):
    result = _run("heat3d", 640, **switches)
    assert result["engine"] == (0 if switches.get("QB200_TC") == "0" else 3)
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float32)]


@pytest.mark.parametrize("switches", [{}, {"QB200_DMMA": "0"}], ids=["fp64 mma", "simt"])
def test_wide_float64_network_on_every_gemm_variant(cuda_device, switches):
    result = _run("burgers", 1536, **switches)
    assert result["engine"] == 0
    assert result["max_error"] <= TOLERANCE[np.dtype(np.float64)]


def test_narrow_network_forced_onto_the_layerwise_engine(cuda_device):
    # Width 64 float32 through the layer-wise kernels: tcgen05 GEMMs with 64-column tiles.
    result = _run("poisson2d", 3000, QB200_ENGINE="layerwise")
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
