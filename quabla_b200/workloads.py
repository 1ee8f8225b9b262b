"""The five PINN training workloads the backend is measured and tested on.

Each workload is written against the public surface exactly as a user of the
reference would write it (the surface module is a parameter, so the same
source can be traced by another implementation of that surface) (a per-point network, `grad`/`hessian` under `vmap`,
`mean` of squared residuals), with seeded synthetic inputs:

  weights  W_l = glorot_normal(split(key(seed), layers)[l], [d_l, d_{l+1}]),
           zero biases (docs/guide/11-pinn-tutorial.md section 11.2 convention);
  points   column j of point set s = uniform(fold_in(key(seed), 1000*s + j),
           [N_s], lo_j, hi_j, dtype).

`points` scales every point set by the same factor, for parity tests at sizes
a CPU oracle finishes quickly.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Callable

import numpy as np

import quabla_b200 as qb


@dataclass
class Workload:
    name: str
    description: str
    sizes: list[int]
    dtype: Any
    seed: int
    loss: Callable
    params: list
    data: tuple
    interior_points: int
    streams: int                 # interior streams S (primal + derivative streams)
    extra: list[tuple[int, int]] = field(default_factory=list)  # (points, streams) of the other sets

    @property
    def parameter_count(self) -> int:
        return sum(m * n + n for m, n in zip(self.sizes[:-1], self.sizes[1:]))

    def flops_per_point(self, streams: int) -> float:
        """Matmul FLOPs of one point through forward, dgrad and wgrad:
        6*S*Q + 2*d0*d1*(1+S) with Q = sum_{l>=1} d_l*d_{l+1}."""
        q = sum(m * n for m, n in zip(self.sizes[1:-1], self.sizes[2:]))
        return 6.0 * streams * q + 2.0 * self.sizes[0] * self.sizes[1] * (1 + streams)

    @property
    def flops_per_step(self) -> float:
        total = self.flops_per_point(self.streams) * self.interior_points
        for points, streams in self.extra:
            total += self.flops_per_point(streams) * points
        return total


def init_mlp(key, sizes, dtype=np.float64):
    keys = qb.random.split(key, len(sizes) - 1)
    return [{"w": qb.random.glorot_normal(k, (m, n), dtype=dtype), "b": qb.zeros((n,), dtype=dtype)}
            for k, m, n in zip(keys, sizes[:-1], sizes[1:])]


def make_u(api, activation: str = "tanh"):
    """The network as a scalar function of one point (scalar or vector), written
    against `api` (this package, or any module with the same surface); hidden
    layers use `api.tanh` or `api.sin`."""
    act = getattr(api, activation)

    def mlp(params, x):
        h = x
        for layer in params[:-1]:
            h = act(h @ layer["w"] + layer["b"])
        last = params[-1]
        return h @ last["w"] + last["b"]

    def u(params, p):
        return mlp(params, p.reshape(1, -1)).reshape(())

    return u


def _column(seed: int, set_index: int, j: int, n: int, lo: float, hi: float, dtype) -> np.ndarray:
    return qb.random.uniform(qb.random.fold_in(qb.random.key(seed), 1000 * set_index + j), (n,), dtype, lo, hi)


def _points(seed: int, set_index: int, n: int, bounds, dtype) -> np.ndarray:
    return np.stack([_column(seed, set_index, j, n, lo, hi, dtype) for j, (lo, hi) in enumerate(bounds)], axis=1)


def _scaled(n: int, points: int | None, full: int) -> int:
    if points is None:
        return n
    return max(4, int(round(n * points / full)))


# -- 1: 1-D Poisson, float64 ---------------------------------------------------
def poisson1d(points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    api = qb if api is None else api
    u = make_u(api, activation)
    sizes, dtype, seed = [1, 16, 16, 1], np.float64, 0
    n = _scaled(128, points, 128)

    def loss(params, x, xb):
        u_xx = api.vmap(api.grad(api.grad(lambda t: u(params, t))))
        residual = u_xx(x) + math.pi**2 * api.sin(math.pi * x)
        boundary = api.vmap(lambda t: u(params, t))(xb)
        return api.mean(residual**2) + api.mean(boundary**2)

    x = _column(seed, 0, 0, n, -1.0, 1.0, dtype)
    xb = np.array([-1.0, 1.0], dtype=dtype)
    return Workload("poisson1d", "1D Poisson, tanh MLP 1-16-16-1, float64", sizes, dtype, seed, loss,
                    init_mlp(qb.random.key(seed), sizes, dtype), (x, xb), n, 3, [(2, 1)])


# -- 2: 2-D Poisson on the unit square, float32 -----------------------------------
def poisson2d(points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    api = qb if api is None else api
    u = make_u(api, activation)
    sizes, dtype, seed = [2, 64, 64, 64, 64, 1], np.float32, 1
    n = _scaled(65536, points, 65536)
    nb = _scaled(4096, points, 65536)
    nb -= nb % 4

    def loss(params, p, pb):
        laplacian = api.vmap(lambda q: api.trace(api.hessian(lambda s: u(params, s))(q)))(p)
        forcing = 2.0 * math.pi**2 * api.sin(math.pi * p[:, 0]) * api.sin(math.pi * p[:, 1])
        boundary = api.vmap(lambda q: u(params, q))(pb)
        return api.mean((laplacian + forcing) ** 2) + api.mean(boundary**2)

    p = _points(seed, 0, n, [(0.0, 1.0), (0.0, 1.0)], dtype)
    free = _column(seed, 1, 0, nb, 0.0, 1.0, dtype)
    edge = np.arange(nb) % 4  # 0: x=0, 1: x=1, 2: y=0, 3: y=1
    pb = np.empty((nb, 2), dtype=dtype)
    pb[:, 0] = np.where(edge == 0, 0.0, np.where(edge == 1, 1.0, free))
    pb[:, 1] = np.where(edge == 2, 0.0, np.where(edge == 3, 1.0, free))
    return Workload("poisson2d", "2D Poisson on the unit square, tanh MLP 2-64x4-1, float32", sizes, dtype, seed, loss,
                    init_mlp(qb.random.key(seed), sizes, dtype), (p, pb), n, 5, [(nb, 1)])


# -- 3: viscous Burgers (x, t), float64 --------------------------------------------
def burgers(points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    api = qb if api is None else api
    u = make_u(api, activation)
    sizes, dtype, seed = [2] + [128] * 8 + [1], np.float64, 2
    n = _scaled(262144, points, 262144)
    n_ic = _scaled(8192, points, 262144)
    n_bc = _scaled(8192, points, 262144)
    n_bc -= n_bc % 2
    nu = 0.01 / math.pi

    def loss(params, p, p_ic, target_ic, p_bc):
        def residual(q):
            value, g = api.value_and_grad(lambda s: u(params, s))(q)
            u_xx = api.hessian(lambda s: u(params, s))(q)[0, 0]
            return g[1] + value * g[0] - nu * u_xx

        interior = api.vmap(residual)(p)
        initial = api.vmap(lambda q: u(params, q))(p_ic) - target_ic
        wall = api.vmap(lambda q: u(params, q))(p_bc)
        return api.mean(interior**2) + api.mean(initial**2) + api.mean(wall**2)

    p = _points(seed, 0, n, [(-1.0, 1.0), (0.0, 1.0)], dtype)
    p_ic = np.stack([_column(seed, 1, 0, n_ic, -1.0, 1.0, dtype), np.zeros(n_ic, dtype=dtype)], axis=1)
    target_ic = (-np.sin(math.pi * p_ic[:, 0].astype(np.float64))).astype(dtype)
    p_bc = np.stack([np.where(np.arange(n_bc) % 2 == 0, -1.0, 1.0).astype(dtype),
                     _column(seed, 2, 1, n_bc, 0.0, 1.0, dtype)], axis=1)
    return Workload("burgers", "viscous Burgers (x,t), tanh MLP 2-128x8-1, float64", sizes, dtype, seed, loss,
                    init_mlp(qb.random.key(seed), sizes, dtype), (p, p_ic, target_ic, p_bc), n, 4,
                    [(n_ic, 1), (n_bc, 1)])


# -- 4: 3-D heat equation (x, y, z, t), float32 -------------------------------------
def heat3d(points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    api = qb if api is None else api
    u = make_u(api, activation)
    sizes, dtype, seed = [4] + [256] * 6 + [1], np.float32, 3
    n = _scaled(1048576, points, 1048576)
    alpha, decay = 0.1, 0.3 * math.pi**2
    source_scale = -decay + alpha * 3.0 * math.pi**2  # (d/dt - alpha*Laplacian) of the exact solution

    def loss(params, p):
        def residual(q):
            g = api.grad(lambda s: u(params, s))(q)
            h = api.hessian(lambda s: u(params, s))(q)
            source = source_scale * api.exp(-decay * q[3]) * api.sin(math.pi * q[0]) * api.sin(math.pi * q[1]) \
                * api.sin(math.pi * q[2])
            return g[3] - alpha * (h[0, 0] + h[1, 1] + h[2, 2]) - source

        return api.mean(api.vmap(residual)(p) ** 2)

    p = _points(seed, 0, n, [(0.0, 1.0)] * 4, dtype)
    return Workload("heat3d", "3D heat equation (x,y,z,t), tanh MLP 4-256x6-1, float32", sizes, dtype, seed, loss,
                    init_mlp(qb.random.key(seed), sizes, dtype), (p,), n, 8, [])


# -- 5: Euler-Bernoulli beam, 4th order, float32 --------------------------------------
def beam(points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    api = qb if api is None else api
    u = make_u(api, activation)
    sizes, dtype, seed = [1] + [64] * 4 + [1], np.float32, 4
    n = _scaled(1048576, points, 1048576)

    def loss(params, x, xb):
        f = lambda t: u(params, t)  # noqa: E731
        u_xxxx = api.vmap(api.grad(api.grad(api.grad(api.grad(f)))))
        residual = u_xxxx(x) - math.pi**4 * api.sin(math.pi * x)
        value = api.vmap(f)(xb)
        slope = api.vmap(api.grad(f))(xb)
        return api.mean(residual**2) + api.mean(value**2) + api.mean(slope**2)

    x = _column(seed, 0, 0, n, 0.0, 1.0, dtype)
    xb = np.array([0.0, 1.0], dtype=dtype)
    return Workload("beam", "4th-order Euler-Bernoulli beam, tanh MLP 1-64x4-1, float32", sizes, dtype, seed, loss,
                    init_mlp(qb.random.key(seed), sizes, dtype), (x, xb), n, 5, [(2, 2)])


WORKLOADS = {"poisson1d": poisson1d, "poisson2d": poisson2d, "burgers": burgers, "heat3d": heat3d, "beam": beam}
ORDER = ["poisson1d", "poisson2d", "burgers", "heat3d", "beam"]


def make(name: str, points: int | None = None, api=None, activation: str = "tanh") -> Workload:
    """`api` selects the module the loss is written against (default: this package);
    `activation` ("tanh" or "sin") the hidden layers' activation."""
    return WORKLOADS[name](points, api, activation)
