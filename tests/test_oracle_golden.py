"""The CPU oracle against the fixtures produced by the reference's own modules (tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import radius_ref, schnet_ref


def _spec(case):
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": case["upper"]}
    return {"kind": case["kind"], "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": case["L"]}


SCHNET_CASES = ["schnet_gaussian_f32", "schnet_expnormal_f32", "schnet_expnormal_trainable_f64"]


@pytest.mark.parametrize("name", SCHNET_CASES)
def test_edges_match_reference(golden, name):
    c = golden[name]
    ptr = radius_ref.batch_to_ptr(c["batch"].numpy())
    for fn in (radius_ref.radius_graph_c, radius_ref.radius_graph_numpy):
        ei = fn(c["pos"].numpy(), ptr, c["upper"], 1000, False, "cluster")
        assert np.array_equal(ei, c["edge_index"].numpy())


@pytest.mark.parametrize("name", SCHNET_CASES)
def test_energy_forces_match_reference(golden, name):
    c = golden[name]
    sd, spec = c["state_dict"], _spec(c)
    fn = lambda p: schnet_ref.schnet_energy(sd, spec, p, c["atom_types"], c["batch"], c["edge_index"], c["B"])
    e, f, _ = schnet_ref.energy_and_forces(fn, c["pos"])
    tol = 1e-12 if c["pos"].dtype == torch.float64 else 2e-6
    assert torch.allclose(e, c["energy"], rtol=tol, atol=tol)
    assert torch.allclose(f, c["forces"], rtol=tol, atol=10 * tol)


@pytest.mark.parametrize("name", SCHNET_CASES)
def test_force_matching_gradients_match_reference(golden, name):
    """Second-order pass: d MSE(forces, target) / d parameters (src/mlcg/pl/model.py:113-131)."""
    c = golden[name]
    spec = _spec(c)
    sd = {k: v.clone().requires_grad_(k in c["param_grads"]) for k, v in c["state_dict"].items()}
    fn = lambda p: schnet_ref.schnet_energy(sd, spec, p, c["atom_types"], c["batch"], c["edge_index"], c["B"])
    _, f, _ = schnet_ref.energy_and_forces(fn, c["pos"], create_graph=True)
    loss = torch.nn.functional.mse_loss(f, c["target_forces"])
    loss.backward()
    tol = 1e-10 if c["pos"].dtype == torch.float64 else 1e-5
    assert torch.allclose(loss.detach(), c["loss"], rtol=tol)
    for k, g in c["param_grads"].items():
        assert torch.allclose(sd[k].grad, g, rtol=10 * tol, atol=tol * float(g.abs().max() + 1e-30)), k


FULLWIDTH = ["chain100", "chain10", "chain268", "chain73", "chain73_trainable"]


@pytest.mark.parametrize("name", FULLWIDTH)
def test_fullwidth_oracle_matches_reference(golden_fullwidth, name):
    """The restatement at the widths the benchmark runs (128 hidden channels and filters, 128 exp-normal or 50 Gaussian
    functions): edges, energies, forces, force-matching loss and parameter gradients against the reference's own modules."""
    from helpers import fullwidth_case
    c = fullwidth_case(golden_fullwidth, name)
    ptr = radius_ref.batch_to_ptr(c["batch"].numpy())
    assert np.array_equal(radius_ref.radius_graph_c(c["pos"].numpy(), ptr, c["upper"], 1000, False, "cluster"), c["edge_index"].numpy())
    spec = _spec(c)
    sd = {k: v.clone().requires_grad_(k in c["param_grads"]) for k, v in c["state_dict"].items()}
    fn = lambda p: schnet_ref.schnet_energy(sd, spec, p, c["atom_types"], c["batch"], c["edge_index"], c["B"])
    e, f, _ = schnet_ref.energy_and_forces(fn, c["pos"], create_graph=True)
    assert torch.allclose(e.detach(), c["energy"], rtol=1e-5, atol=1e-5)
    assert float((f.detach() - c["forces"]).abs().max()) < 1e-4
    loss = torch.nn.functional.mse_loss(f, c["target_forces"])
    loss.backward()
    assert torch.allclose(loss.detach(), c["loss"], rtol=1e-5)
    for k, g in c["param_grads"].items():
        assert torch.allclose(sd[k].grad, g, rtol=1e-3, atol=1e-4 * float(g.abs().max() + 1e-30)), k


def test_priors_match_reference(golden):
    c = golden["priors_f32"]
    pos, t, B = c["pos"], c["atom_types"], c["B"]
    fns = {
        "bonds": lambda p: schnet_ref.bonds_energy(p, t, c["mappings"]["bonds"], c["mapping_batch"]["bonds"], B,
                                                   c["tables"]["bonds"]["x_0"], c["tables"]["bonds"]["k"]),
        "angles": lambda p: schnet_ref.angles_energy(p, t, c["mappings"]["angles"], c["mapping_batch"]["angles"], B,
                                                     c["tables"]["angles"]["x_0"], c["tables"]["angles"]["k"]),
        "dihedrals": lambda p: schnet_ref.dihedral_energy(p, t, c["mappings"]["dihedrals"], c["mapping_batch"]["dihedrals"], B,
                                                          c["tables"]["dihedrals"]["v_0"], c["tables"]["dihedrals"]["k1s"],
                                                          c["tables"]["dihedrals"]["k2s"]),
        "repulsion": lambda p: schnet_ref.repulsion_energy(p, t, c["mappings"]["repulsion"], c["mapping_batch"]["repulsion"], B,
                                                           c["tables"]["repulsion"]["sigma"]),
    }
    for k, fn in fns.items():
        e, f, _ = schnet_ref.energy_and_forces(fn, pos)
        assert torch.allclose(e, c["energy"][k], rtol=1e-5), k
        assert torch.allclose(f, c["forces"][k], rtol=1e-4, atol=1e-4 * float(c["forces"][k].abs().max())), k


def test_cutoff_endpoints(golden):
    """tests/unit/nn/test_cutoff.py:27-43: one at the lower end, zero at and beyond the upper end."""
    c = golden["cutoff"]
    v0 = schnet_ref.cosine_cutoff(c["d"], 0.0, 5.0)
    v1 = schnet_ref.cosine_cutoff(c["d"], 1.0, 5.0)
    assert torch.allclose(v0, c["lower0"], atol=1e-7) and torch.allclose(v1, c["lower1"], atol=1e-7)
    assert v0[0] == 1.0 and v0[4] == 0.0 and v0[5] == 0.0
    assert v1[0] == 0.0 and abs(float(v1[1])) < 1e-6  # below and at the lower bound the strict mask gives zero
