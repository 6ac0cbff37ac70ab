"""TEST INFRASTRUCTURE — CPU oracle for the SchNet energy / force path (not shipped).

A functional, dense-tensor restatement in plain torch of what mlcg evaluates, written against a
``state_dict`` with mlcg's own key names so that the reference's weights, this repository's weights
and the golden fixtures are interchangeable.  Every function cites the reference lines it follows.
Runs in whatever dtype the inputs have (float32 for parity, float64 for derivative checks).

Third-party pieces that are not in the reference tree are restated from their published behaviour:
``torch_geometric.nn.MessagePassing.propagate`` with ``aggr="add"`` and default flow gathers
``x[edge_index[0]]`` and sums messages at ``edge_index[1]``; ``torch_geometric.utils.scatter`` with
``reduce="sum"`` is an index-add over ``dim 0`` (torch-geometric 2.6.1).

Parity status: pinned — ``tests/golden/make_golden.py`` runs the reference's own modules (loaded by
path, third-party calls shimmed) and the fixtures it writes are checked in ``tests/test_oracle_golden.py``.
"""
import math
from typing import Dict, Optional

import torch

Tensor = torch.Tensor


# ----------------------------------------------------------------------------- cutoffs and bases
def cosine_cutoff(d: Tensor, lower: float, upper: float) -> Tensor:
    """src/mlcg/nn/cutoff.py:110-153."""
    if lower > 0:
        c = 0.5 * (torch.cos(math.pi * (2 * (d - lower) / (upper - lower) + 1.0)) + 1.0)
        c = c * (d < upper).to(d.dtype)
        return c * (d > lower).to(d.dtype)
    c = 0.5 * (torch.cos(d * math.pi / upper) + 1.0)
    return c * (d < upper).to(d.dtype)


def cutoff_value(d: Tensor, spec: Dict) -> Tensor:
    """``spec["cutoff"]`` is ``"cosine"`` or ``"identity"`` (cutoff.py:40-72 returns ones)."""
    if spec["cutoff"] == "identity":
        return torch.ones_like(d)
    return cosine_cutoff(d, spec["lower"], spec["upper"])


def gaussian_params(lower: float, upper: float, num_rbf: int, dtype=torch.float32):
    """src/mlcg/nn/radial_basis/gaussian.py:64-75."""
    offset = torch.linspace(lower, upper, num_rbf)
    coeff = -0.5 / (offset[1] - offset[0]) ** 2
    return offset.to(dtype), coeff.to(dtype)


def expnormal_params(lower: float, upper: float, num_rbf: int, dtype=torch.float32):
    """src/mlcg/nn/radial_basis/exp_normal.py:80-94."""
    start = torch.exp(torch.scalar_tensor(-upper + lower))
    means = torch.linspace(start, 1, num_rbf)
    betas = torch.tensor([(2 / num_rbf * (1 - start)) ** -2] * num_rbf)
    return means.to(dtype), betas.to(dtype)


def radial_basis(d: Tensor, spec: Dict, sd: Dict[str, Tensor]) -> Tensor:
    """Gaussian: gaussian.py:83-102; exp-normal: exp_normal.py:104-124. Output ``[E, R]``."""
    dd = d.unsqueeze(-1)
    env = cutoff_value(dd, spec["rbf_cutoff"])
    if spec["kind"] == "gaussian":
        return torch.exp(sd["rbf_layer.coeff"] * torch.pow(dd - sd["rbf_layer.offset"], 2)) * env
    alpha = 5.0 / (spec["rbf_cutoff"]["upper"] - spec["rbf_cutoff"]["lower"])
    inner = torch.exp(alpha * (-dd + spec["rbf_cutoff"]["lower"])) - sd["rbf_layer.means"]
    return env * torch.exp(-sd["rbf_layer.betas"] * inner ** 2)


# ----------------------------------------------------------------------------- geometry
def edge_distances(pos: Tensor, edge_index: Tensor) -> Tensor:
    """src/mlcg/geometry/internal_coordinates.py:72-100 without cell shifts."""
    dr = pos[edge_index[1]] - pos[edge_index[0]]
    return dr.norm(p=2, dim=1)


def index_sum(src: Tensor, index: Tensor, size: int) -> Tensor:
    """``scatter(..., reduce="sum")`` / ``aggr="add"``: out[index[k]] += src[k]."""
    out = torch.zeros((size,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
    return out.index_add_(0, index, src)


# ----------------------------------------------------------------------------- network
def _act(name: str):
    return {"tanh": torch.tanh, "silu": torch.nn.functional.silu, "relu": torch.relu}[name]


def filter_network(rbf: Tensor, sd: Dict[str, Tensor], prefix: str, act) -> Tensor:
    """MLP([R, F, F], last_bias=False): src/mlcg/nn/mlp.py:41-58, built at schnet.py:446-450."""
    h = act(rbf @ sd[prefix + "layers.0.weight"].t() + sd[prefix + "layers.0.bias"])
    return h @ sd[prefix + "layers.2.weight"].t()


def cfconv(x: Tensor, edge_index: Tensor, d: Tensor, rbf: Tensor, sd, prefix: str, spec, act) -> Tensor:
    """src/mlcg/nn/schnet.py:312-368."""
    C = cutoff_value(d, spec["cutoff"])
    W = filter_network(rbf, sd, prefix + "filter_network.", act) * C.view(-1, 1)
    xl = x @ sd[prefix + "lin1.weight"].t()
    msg = xl[edge_index[0]] * W
    agg = index_sum(msg, edge_index[1], x.shape[0])
    return agg @ sd[prefix + "lin2.weight"].t() + sd[prefix + "lin2.bias"]


def interaction_block(x, edge_index, d, rbf, sd, prefix: str, spec, act) -> Tensor:
    """src/mlcg/nn/schnet.py:229-262."""
    y = act(cfconv(x, edge_index, d, rbf, sd, prefix + "conv.", spec, act))
    return y @ sd[prefix + "lin.weight"].t() + sd[prefix + "lin.bias"]


def output_network(x: Tensor, sd, act) -> Tensor:
    """MLP([H, *widths, 1], last_bias=False): schnet.py:463-468, mlp.py:41-58."""
    idx = sorted({int(k.split(".")[2]) for k in sd if k.startswith("output_network.layers.")})
    for n, i in enumerate(idx):
        x = x @ sd[f"output_network.layers.{i}.weight"].t()
        b = sd.get(f"output_network.layers.{i}.bias")
        if b is not None:
            x = x + b
        if n < len(idx) - 1:
            x = act(x)
    return x


def schnet_energy(sd: Dict[str, Tensor], spec: Dict, pos: Tensor, atom_types: Tensor, batch: Tensor,
                  edge_index: Tensor, num_structures: Optional[int] = None) -> Tensor:
    """``SchNet.forward`` (src/mlcg/nn/schnet.py:116-162) for a given edge list; energy ``[B]``.

    ``spec`` = ``{"kind": "gaussian"|"expnormal", "rbf_cutoff": {...}, "cutoff": {...},
    "activation": "tanh", "num_interactions": L}``.
    """
    act = _act(spec.get("activation", "tanh"))
    x = sd["embedding_layer.weight"][atom_types]
    d = edge_distances(pos, edge_index)
    rbf = radial_basis(d, spec, sd)
    for l in range(spec["num_interactions"]):
        x = x + interaction_block(x, edge_index, d, rbf, sd, f"interaction_blocks.{l}.", spec, act)
    e = output_network(x, sd, act)
    B = int(batch[-1]) + 1 if num_structures is None else num_structures
    return index_sum(e, batch, B).flatten()


def energy_and_forces(energy_fn, pos: Tensor, create_graph: bool = False):
    """``GradientsOut.forward`` (src/mlcg/nn/gradients.py:191-230): forces = -d(sum E)/d pos."""
    pos = pos.detach().clone().requires_grad_(True)
    e = energy_fn(pos)
    (g,) = torch.autograd.grad(e.sum(), pos, create_graph=create_graph)
    return e, -g, pos


# ----------------------------------------------------------------------------- priors
def angles_cos(pos: Tensor, m: Tensor) -> Tensor:
    """internal_coordinates.py:145-183."""
    a = pos[m[0]] - pos[m[1]]
    b = pos[m[2]] - pos[m[1]]
    return (a * b).sum(dim=1) / a.norm(p=2, dim=1) / b.norm(p=2, dim=1)


def torsions(pos: Tensor, m: Tensor) -> Tensor:
    """internal_coordinates.py:186-252."""
    b1 = pos[m[1]] - pos[m[0]]
    b2 = pos[m[2]] - pos[m[1]]
    b3 = pos[m[3]] - pos[m[2]]
    b1 = b1 / b1.norm(p=2, dim=1)[:, None]
    b2 = b2 / b2.norm(p=2, dim=1)[:, None]
    b3 = b3 / b3.norm(p=2, dim=1)[:, None]
    n1 = torch.cross(b1, b2, dim=1)
    n2 = torch.cross(b2, b3, dim=1)
    m1 = torch.cross(n1, b2, dim=1)
    return torch.atan2(-(m1 * n2).sum(-1), (n1 * n2).sum(-1))


def harmonic_energy(feature: Tensor, x0: Tensor, k: Tensor, mapping_batch: Tensor, B: int) -> Tensor:
    """harmonic.py:110-120: k (x - x0)^2, no factor one half, summed per structure."""
    return index_sum(k * (feature - x0) ** 2, mapping_batch, B)


def bonds_energy(pos, atom_types, mapping, mapping_batch, B, x0_table, k_table):
    """HarmonicBonds: harmonic.py:78-88 (table lookup by bead types), :229-242."""
    t = (atom_types[mapping[0]], atom_types[mapping[1]])
    return harmonic_energy(edge_distances(pos, mapping), x0_table[t], k_table[t], mapping_batch, B)


def angles_energy(pos, atom_types, mapping, mapping_batch, B, x0_table, k_table):
    """HarmonicAngles: harmonic.py:284-297; the feature and x0 are cosines."""
    t = (atom_types[mapping[0]], atom_types[mapping[1]], atom_types[mapping[2]])
    return harmonic_energy(angles_cos(pos, mapping), x0_table[t], k_table[t], mapping_batch, B)


def dihedral_energy(pos, atom_types, mapping, mapping_batch, B, v0_table, k1_table, k2_table):
    """Dihedral / FourierSeries: fourier_series.py:105-198. ``k1_table`` is ``[n_degs, T, T, T, T]``."""
    t = tuple(atom_types[mapping[i]] for i in range(4))
    theta = torsions(pos, mapping)
    n_degs = k1_table.shape[0]
    y = v0_table[t]
    for n in range(1, n_degs + 1):
        y = y + k1_table[n - 1][t] * torch.sin(n * theta) + k2_table[n - 1][t] * torch.cos(n * theta)
    return index_sum(y, mapping_batch, B)


def repulsion_energy(pos, atom_types, mapping, mapping_batch, B, sigma_table):
    """Repulsion: repulsion.py:88-140, (sigma/d)^6 over the pair list as given."""
    t = (atom_types[mapping[0]], atom_types[mapping[1]])
    rr = (sigma_table[t] / edge_distances(pos, mapping)) ** 2
    return index_sum(rr * rr * rr, mapping_batch, B)
