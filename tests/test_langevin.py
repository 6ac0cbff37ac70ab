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


def test_langevin_step_cpu_wiring(monkeypatch):
    from oracle.primitives import OracleBackend
    monkeypatch.setattr(backend, "_backend", OracleBackend())
    run_case("cpu", torch.float64)


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


def _md_case(device, B=2, n=70, seed=5):
    """SchNet + four priors on `B` chains of `n` beads, practically without friction (no noise enters: the integrator is
    then deterministic, so two runs can be compared)."""
    from mlcg_b200.data import collate
    gen = torch.Generator().manual_seed(seed)
    data, priors = prior_setup(n, B, 4, gen)
    torch.manual_seed(seed)
    cut = bnn.CosineCutoff(0.0, 12.0)
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, 128, trainable=False), cut, [128], hidden_channels=128, embedding_size=4,
                             num_filters=128, num_interactions=2)
    models = {k: bnn.GradientsOut(p, "forces") for k, p in priors.items()}
    models["SchNet"] = bnn.GradientsOut(net, "forces")
    model = bnn.SumOut(torch.nn.ModuleDict(models)).eval().to(device)
    data = data.to(device)
    masses = torch.full((data.pos.shape[0],), 12.0 / 418.39, device=device)
    # (a short time step: the comparison of two runs must not depend on how fast rounding differences grow)
    sim = LangevinSimulation(model, dt=0.0005, friction=1e-12, beta=1.0 / (0.0019872041 * 300))
    sim.attach(data, masses, velocities=torch.zeros_like(data.pos))
    return sim, model


@pytest.mark.gpu
def test_simulation_replayed_from_a_cuda_graph():
    """One MD step recorded into a CUDA graph (fixed edge capacity: no host read in the step) and replayed gives the
    trajectory of the step-by-step loop; the trajectory buffer holds the positions at the save points."""
    from mlcg_b200.neighbor_list import edge_plan_for
    steps, every = 12, 3
    sim, model = _md_case("cuda:0")
    assert sim.noisescale < 1e-6
    x0 = sim.data.pos.clone()
    sim.simulate(steps, save_interval=every)
    traj_plain, pot_plain = sim.trajectory.clone(), sim.potentials.clone()
    moved = float((traj_plain[-1] - x0).abs().max())
    assert torch.equal(traj_plain[-1], sim.data.pos) and moved > 1e-4, moved

    sim2, model2 = _md_case("cuda:0")
    E = edge_plan_for(sim2.data, 12.0)[0].E
    bnn.set_edge_capacity(model2, int(1.5 * E))
    sim2.simulate(steps, save_interval=every, cuda_graph=True)
    assert sim2.trajectory.shape == traj_plain.shape
    diff = float((sim2.trajectory - traj_plain).abs().max())
    assert diff < 1e-3 and diff < 0.05 * moved, (diff, moved)
    assert torch.allclose(sim2.potentials, pot_plain, rtol=1e-4, atol=1e-2), (sim2.potentials, pot_plain)
    # an edge capacity that the graph outgrows is reported at the next save point
    sim3, model3 = _md_case("cuda:0")
    bnn.set_edge_capacity(model3, E - 2)
    with pytest.raises(RuntimeError, match="capacity"):
        sim3.simulate(steps, save_interval=every, cuda_graph=True)
    backend.get_backend().check_pending()


def test_simulation_trajectory_buffer_cpu_wiring(monkeypatch):
    from oracle.primitives import OracleBackend
    monkeypatch.setattr(backend, "_backend", OracleBackend())
    data, priors = prior_setup(14, 3, 4, torch.Generator().manual_seed(3))
    model = bnn.SumOut(torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})).eval()
    data.pos = data.pos.to(torch.float64)
    sim = LangevinSimulation(model, dt=0.002, friction=1.0, beta=1.0 / (0.0019872041 * 300), rng=torch.Generator().manual_seed(1))
    sim.attach(data, torch.ones(data.pos.shape[0], dtype=torch.float64))
    sim.simulate(7, save_interval=3)
    assert sim.trajectory.shape == (2, data.pos.shape[0], 3) and sim.potentials.shape == (2, 3)
    assert bool(torch.isfinite(sim.trajectory).all()) and not torch.equal(sim.trajectory[0], sim.trajectory[1])
