"""Langevin step (BAOAB) against a line-by-line restatement of LangevinSimulation.timestep
(src/mlcg/simulation/langevin.py:100-144): on CPU with the oracle primitives, on the GPU with the CUDA kernels."""
import numpy as np
import pytest
import torch

import mlcg_b200
from mlcg_b200 import backend, nn as bnn
from mlcg_b200.simulation import LangevinSimulation

from helpers import prior_setup


def reference_timestep(x, v, f, masses, bmr, noise, dt, vscale, noisescale, force_fn):
    v_new = v + 0.5 * dt * f / masses[:, None]
    x_new = x + v_new * dt * 0.5
    v_new = v_new * vscale + noisescale * (bmr[:, None] * noise)
    x_new = x_new + v_new * dt * 0.5
    pot, f_new = force_fn(x_new)
    v_new = v_new + 0.5 * dt * f_new / masses[:, None]
    return x_new, v_new, pot, f_new


def run_case(device, dtype, steps=4):
    data, priors = prior_setup(14, 3, 4, torch.Generator().manual_seed(3))
    models = torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})
    model = bnn.SumOut(models).eval().to(device)
    data = data.to(device)
    data.pos = data.pos.to(dtype)
    N = data.pos.shape[0]
    gen = torch.Generator().manual_seed(11)
    masses = (0.5 + torch.rand(N, generator=gen)).to(device=device, dtype=dtype)
    dt, friction, beta = 0.002, 1.0, 1.0 / (0.0019872041 * 300)
    sim = LangevinSimulation(model, dt=dt, friction=friction, beta=beta)
    v0 = LangevinSimulation.sample_maxwell_boltzmann(torch.full((N,), beta, dtype=dtype), masses.cpu(), gen).to(device)
    sim.attach(data, masses, velocities=v0.clone())

    def force_fn(x):
        d = mlcg_b200.AtomicData(pos=x.clone(), atom_types=data.atom_types, batch=data.batch, n_atoms=data.n_atoms,
                                 neighbor_list=data.neighbor_list)
        o = model(d)
        return o.out["energy"].detach(), o.out["forces"].detach()

    x_ref, v_ref = sim.data.pos.clone(), v0.clone()
    pot, f = sim.calculate_potential_and_forces(sim.data)
    f_ref = f.clone()
    vscale, noisescale = np.exp(-dt * friction), np.sqrt(1 - np.exp(-dt * friction) ** 2)
    for _ in range(steps):
        noise = torch.randn(N, 3, generator=gen).to(device=device, dtype=dtype)
        _, pot, f = sim.timestep(sim.data, f, noise=noise)
        x_ref, v_ref, pot_ref, f_ref = reference_timestep(x_ref, v_ref, f_ref, masses, sim.beta_mass_ratio, noise, dt, vscale, noisescale, force_fn)
        tol = 1e-10 if dtype == torch.float64 else 2e-4
        assert torch.allclose(sim.data.pos, x_ref, rtol=tol, atol=tol)
        assert torch.allclose(sim.velocities, v_ref, rtol=tol, atol=tol * 10)
        assert torch.allclose(pot, pot_ref, rtol=max(tol, 1e-5), atol=max(tol, 1e-4))


def test_langevin_step_cpu_wiring():
    from oracle.primitives import OracleBackend
    old = backend.set_backend(OracleBackend())
    try:
        run_case("cpu", torch.float64)
    finally:
        backend.set_backend(old)


def test_maxwell_boltzmann_moments():
    """tests/unit/simulation/test_simulation.py:451-471 checks the same moments for the reference sampler."""
    gen = torch.Generator().manual_seed(0)
    masses = torch.full((200000,), 2.0)
    betas = torch.full((200000,), 0.5)
    v = LangevinSimulation.sample_maxwell_boltzmann(betas, masses, gen)
    assert abs(float(v.mean())) < 5e-3 and abs(float(v.var()) - 1.0) < 1e-2     # variance 1/(beta m) = 1


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_langevin_step_gpu(dtype):
    run_case("cuda:0", dtype)
