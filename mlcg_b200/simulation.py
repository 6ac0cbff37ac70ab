"""Langevin dynamics driver with mlcg's step semantics (src/mlcg/simulation/langevin.py, base.py).

Only what the hot path needs: ``LangevinSimulation.timestep`` (BAOAB, one force evaluation per step,
langevin.py:100-144), Maxwell-Boltzmann initial velocities (:69-98), ``calculate_potential_and_forces``
(base.py:517-539) and a plain ``simulate`` loop that keeps positions on the device.  File export,
checkpointing, logging and the CLI of ``_Simulation`` are mlcg's and are not reproduced here.
"""
from typing import Optional, Tuple

import numpy as np
import torch

from .backend import get_backend
from .data import ENERGY_KEY, FORCE_KEY


class LangevinSimulation:
    def __init__(self, model: torch.nn.Module, dt: float = 5e-4, friction: float = 1e-3, beta: float = 1.0,
                 rng: Optional[torch.Generator] = None):
        assert friction > 0
        self.model = model
        self.dt, self.friction = float(dt), float(friction)
        self.beta = beta
        self.vscale = float(np.exp(-self.dt * self.friction))
        self.noisescale = float(np.sqrt(1 - self.vscale * self.vscale))
        self.rng = rng

    @staticmethod
    def sample_maxwell_boltzmann(betas: torch.Tensor, masses: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        """Velocities ~ N(0, 1/(beta m)) per coordinate (langevin.py:69-98)."""
        scale = torch.sqrt(1 / (betas * masses))
        return torch.randn((masses.shape[0], 3), dtype=scale.dtype, device=scale.device, generator=generator) * scale[:, None]

    def attach(self, data, masses: torch.Tensor, velocities: Optional[torch.Tensor] = None):
        """``data``: collated structures on the device; one beta for all or one per structure."""
        self.data = data
        self.masses = masses.to(data.pos.dtype).contiguous()
        beta = torch.as_tensor(self.beta, dtype=data.pos.dtype, device=data.pos.device)
        betas = beta.expand(data.pos.shape[0]) if beta.dim() == 0 else beta[data.batch]
        if velocities is None:
            velocities = self.sample_maxwell_boltzmann(betas, self.masses, self.rng)
        self.velocities = velocities.to(data.pos.dtype).contiguous()
        self.beta_mass_ratio = torch.sqrt(1.0 / betas / self.masses).contiguous()     # langevin.py:176-180
        self.data.pos = self.data.pos.detach().contiguous().clone()

    def calculate_potential_and_forces(self, data) -> Tuple[torch.Tensor, torch.Tensor]:
        data.out = {}
        data = self.model(data)
        out = data.out if ENERGY_KEY in data.out else data.out[self.model.name]   # SumOut totals, or a single GradientsOut model
        return out[ENERGY_KEY].detach(), out[FORCE_KEY].detach()

    def timestep(self, data, forces: torch.Tensor, noise: Optional[torch.Tensor] = None):
        """(data at t, forces at t) -> (data at t+1, potential, forces at t+1); positions and velocities updated in place.
        ``noise`` (standard normal, ``[N,3]``) is drawn from ``self.rng`` when not given."""
        be = get_backend()
        if noise is None:
            noise = torch.randn(data.pos.shape, dtype=data.pos.dtype, device=data.pos.device, generator=self.rng)
        be.langevin_first_half(data.pos, self.velocities, forces, self.masses, self.beta_mass_ratio, noise, self.dt, self.vscale, self.noisescale)
        potential, forces = self.calculate_potential_and_forces(data)
        be.langevin_second_half(self.velocities, forces, self.masses, self.dt)
        return data, potential, forces

    def simulate(self, n_timesteps: int, save_interval: Optional[int] = None, cuda_graph: bool = False):
        """``n_timesteps`` BAOAB steps.  ``save_interval``: positions after every that many steps are kept in a trajectory
        buffer on the device (``self.trajectory`` ``[n_saves, N, 3]``, ``self.potentials`` ``[n_saves, B]``), where the
        simulation is also checked for non-finite positions and for kernel status reports, as the reference does when it
        saves (base.py:864-938) — once, at the end, without it.  ``cuda_graph``: record one step (noise, both halves of the
        integrator, graph construction, every model and prior) into a CUDA graph and replay it; every SchNet of the model
        needs a fixed edge capacity for that (:func:`mlcg_b200.nn.set_edge_capacity`), so that no step reads the edge count
        on the host."""
        data = self.data
        be = get_backend()
        n_saves = n_timesteps // save_interval if save_interval else 0
        if n_saves:
            self.trajectory = torch.empty((n_saves,) + tuple(data.pos.shape), dtype=data.pos.dtype, device=data.pos.device)
            self.potentials = None
        potential, forces = self.calculate_potential_and_forces(data)
        step_graph, done = None, 0

        def check():
            be.check_pending()
            if not bool(torch.isfinite(data.pos).all()):
                raise RuntimeError(f"mlcg_b200: simulation blew up before step {done}: non-finite positions")

        def save(k):
            self.trajectory[k].copy_(data.pos)
            if self.potentials is None:
                self.potentials = torch.empty((n_saves,) + tuple(potential.shape), dtype=potential.dtype, device=potential.device)
            self.potentials[k].copy_(potential)
            check()

        if cuda_graph and n_timesteps > 3:
            # two plain steps first: every lazily created buffer and kernel attribute exists before the recording starts
            forces = forces.clone()
            for _ in range(2):
                data, potential, f = self.timestep(data, forces)
                forces.copy_(f)
                done += 1
                if save_interval and done % save_interval == 0:
                    save(done // save_interval - 1)
            check()
            potential = potential.clone()
            step_graph = torch.cuda.CUDAGraph()
            if self.rng is not None:
                step_graph.register_generator_state(self.rng)
            with torch.cuda.graph(step_graph):
                _, p, f = self.timestep(data, forces)
                forces.copy_(f)
                potential.copy_(p)
            # (recording does not run the step; every step from here on is a replay)
        while done < n_timesteps:
            if step_graph is not None:
                step_graph.replay()
            else:
                data, potential, forces = self.timestep(data, forces)
            done += 1
            if save_interval and done % save_interval == 0:
                save(done // save_interval - 1)
        check()
        return data, potential, forces
