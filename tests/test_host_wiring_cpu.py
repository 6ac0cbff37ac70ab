"""Host-side logic on CPU: the package's modules and autograd wiring, with the kernel primitives
replaced by their oracle restatements (``oracle/primitives.py``).  What is checked here is the
Python layer — edge plans, operator composition, derivative formulas, module/state_dict layout —
not the CUDA kernels (those are compared with the same oracle in the ``-m gpu`` tests)."""
import pytest
import torch

import mlcg_b200
from mlcg_b200 import autograd as ag
from mlcg_b200 import backend, nn as bnn
from oracle.primitives import OracleBackend

from helpers import attentive_schnet_from_case, data_from_case, periodic_prior_cases, prior_setup, regularized_schnet_from_case, schnet_from_case


@pytest.fixture(autouse=True)
def oracle_backend(monkeypatch):
    """Swap the package's back-end object for the oracle's for the duration of one test (the package has no such switch)."""
    monkeypatch.setattr(backend, "_backend", OracleBackend())
    yield


CASES = ["schnet_gaussian_f32", "schnet_expnormal_f32", "schnet_expnormal_trainable_f64"]


@pytest.mark.parametrize("name", CASES)
def test_schnet_energy_forces_vs_reference(golden, name):
    c = golden[name]
    model = bnn.GradientsOut(schnet_from_case(c), "forces").eval()
    out = model(data_from_case(c))
    tol = 1e-10 if c["pos"].dtype == torch.float64 else 2e-6
    assert torch.allclose(out.out["SchNet"]["energy"], c["energy"], rtol=tol, atol=tol)
    assert torch.allclose(out.out["SchNet"]["forces"], c["forces"], rtol=tol, atol=10 * tol)


@pytest.mark.parametrize("name", CASES)
def test_force_matching_step_vs_reference(golden, name):
    c = golden[name]
    net = schnet_from_case(c)
    model = bnn.GradientsOut(net, "forces").train()
    out = model(data_from_case(c))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"])
    loss.backward()
    tol = 1e-9 if c["pos"].dtype == torch.float64 else 1e-5
    assert torch.allclose(loss.detach(), c["loss"], rtol=tol)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        assert grads[k].grad is not None, k
        assert torch.allclose(grads[k].grad, g, rtol=10 * tol, atol=tol * float(g.abs().max() + 1e-30)), k


@pytest.mark.parametrize("name", ["shared", "independent"])
def test_rbf_regularized_schnet_vs_reference(golden_regularized, name):
    """`RBFRegularizedSchNet` (src/mlcg/nn/schnet.py:676-803): state_dict keys, energies, forces, the `radial_filters` output
    and the gradients of a force-matching loss, factors outside [0, 1] included (both clamps act)."""
    c = golden_regularized[name]
    net = regularized_schnet_from_case(c)
    assert set(net.state_dict().keys()) == set(c["state_dict"].keys())
    out = bnn.GradientsOut(net, "forces").eval()(data_from_case(c))
    assert torch.allclose(out.out["SchNet"]["energy"], c["energy"], rtol=2e-6, atol=2e-6)
    assert torch.allclose(out.out["SchNet"]["forces"], c["forces"], rtol=2e-6, atol=2e-5)
    assert torch.equal(out.out["SchNet"]["radial_filters"], c["radial_filters"])
    out = bnn.GradientsOut(net, "forces").train()(data_from_case(c))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"])
    loss.backward()
    assert torch.allclose(loss.detach(), c["loss"], rtol=1e-5)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        assert grads[k].grad is not None, k
        assert torch.allclose(grads[k].grad, g, rtol=1e-4, atol=1e-5 * float(g.abs().max() + 1e-30)), k


@pytest.mark.parametrize("name", ["orthorhombic", "slab", "triclinic"])
def test_periodic_structures_vs_reference(golden_periodic, name):
    """Neighbour-list dictionary of periodic structures and a SchNet evaluated on it (torch_impl.py:252-329,
    internal_coordinates.py:72-100) against the reference's outputs."""
    from mlcg_b200.neighbor_list import atomic_data2neighbor_list
    c = golden_periodic[name]
    mk = lambda: mlcg_b200.AtomicData(pos=c["pos"].clone(), atom_types=c["atom_types"], batch=c["batch"], n_atoms=torch.full((c["B"],), c["n"]),
                                      cell=c["cells"].clone(), pbc=c["pbc"].clone())
    for key, cap, loop in (("1000", 1000, False), ("12", 12, False)):
        nl = atomic_data2neighbor_list(mk(), c["upper"], self_interaction=loop, max_num_neighbors=cap)
        assert torch.equal(nl["index_mapping"], c[f"index_mapping_{key}"])
        assert torch.allclose(nl["cell_shifts"], c[f"cell_shifts_{key}"], rtol=1e-6, atol=1e-6)
        assert torch.equal(nl["mapping_batch"], c[f"mapping_batch_{key}"])
    cut = bnn.CosineCutoff(0.0, c["upper"])
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, c["R"], trainable=False), cut, [c["H"]], hidden_channels=c["H"], embedding_size=c["T"],
                             num_filters=c["H"], num_interactions=c["L"])
    net.load_state_dict(c["state_dict"])
    out = bnn.GradientsOut(net, "forces").eval()(mk())
    assert torch.allclose(out.out["SchNet"]["energy"], c["energy"], rtol=2e-6, atol=2e-6)
    assert torch.allclose(out.out["SchNet"]["forces"], c["forces"], rtol=2e-6, atol=2e-5)


@pytest.mark.parametrize("name", ["normal_exact", "v2_favor", "normal_favor_single"])
def test_attentive_schnet_vs_reference(golden_attentive, name):
    """`AttentiveSchNet` (src/mlcg/nn/schnet.py:478-674, src/mlcg/nn/attention.py): state_dict keys, energies, forces and the
    force-matching gradients of the small parameters, for both block versions and both attention kernels."""
    c = golden_attentive[name]
    net = attentive_schnet_from_case(c)
    assert set(net.state_dict().keys()) == set(c["state_dict"].keys())
    out = bnn.GradientsOut(net, "forces").eval()(data_from_case(c))
    assert torch.allclose(out.out["SchNet"]["energy"], c["energy"], rtol=5e-6, atol=5e-6)
    assert torch.allclose(out.out["SchNet"]["forces"], c["forces"], rtol=1e-5, atol=5e-5)
    out = bnn.GradientsOut(net, "forces").train()(data_from_case(c))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"])
    loss.backward()
    assert torch.allclose(loss.detach(), c["loss"], rtol=1e-5)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        assert grads[k].grad is not None, k
        assert torch.allclose(grads[k].grad, g, rtol=1e-3, atol=2e-5 * float(g.abs().max() + 1e-30)), k


def test_state_dict_keys_match_reference(golden):
    c = golden["schnet_expnormal_f32"]
    assert set(schnet_from_case(c).state_dict().keys()) == set(c["state_dict"].keys())


def test_neighbor_list_dictionary_format(golden):
    c = golden["schnet_gaussian_f32"]
    nl = mlcg_b200.atomic_data2neighbor_list(data_from_case(c), c["upper"], False, 1000)
    assert set(nl) >= {"tag", "order", "index_mapping", "cell_shifts", "rcut", "self_interaction", "mapping_batch"}
    assert nl["order"] == 2 and nl["rcut"] == c["upper"] and nl["self_interaction"] is False
    assert torch.equal(nl["index_mapping"], c["edge_index"])
    assert torch.equal(nl["mapping_batch"], c["batch"][c["edge_index"][0]])
    assert nl["cell_shifts"].shape == (c["edge_index"].shape[1], 3) and not nl["cell_shifts"].any()
    assert mlcg_b200.neighbor_list.validate_neighborlist(nl)


def _plans(golden):
    c = golden["schnet_gaussian_f32"]
    ei = c["edge_index"]
    N = c["pos"].shape[0]
    sym = ag.EdgePlan.from_centre_sorted(ei[0].int(), ei[1].int(), ag._ptr_from_index(ei[0], N), N, symmetric=True)
    perm = torch.randperm(ei.shape[1], generator=torch.Generator().manual_seed(0))
    keep = perm[: int(0.8 * len(perm))]                   # shuffled and no longer symmetric
    gen = ag.EdgePlan.from_edge_index(ei[:, keep].contiguous(), N)
    return c, sym, gen


def test_symmetric_plan_equals_general_plan(golden):
    c, sym, _ = _plans(golden)
    N = c["pos"].shape[0]
    general = ag.EdgePlan.from_edge_index(c["edge_index"], N)
    assert torch.equal(sym.ptr_in, general.ptr_in) and torch.equal(sym.perm_in, general.perm_in)
    assert torch.equal(sym.nbr_in, general.nbr_in) and general.perm_out is None


@pytest.mark.parametrize("which", ["symmetric", "general"])
def test_bilinear_family_gradcheck(golden, which):
    c, sym, gen = _plans(golden)
    plan = sym if which == "symmetric" else gen
    g = torch.Generator().manual_seed(1)
    a = torch.randn(plan.N, 3, dtype=torch.float64, generator=g, requires_grad=True)
    b = torch.randn(plan.N, 3, dtype=torch.float64, generator=g, requires_grad=True)
    V = torch.randn(plan.E, 3, dtype=torch.float64, generator=g, requires_grad=True)
    for fn, args in [(lambda a, V: ag.SegIn.apply(a, V, plan, False), (a, V)), (lambda a, V: ag.SegOut.apply(a, V, plan), (a, V)),
                     (lambda a, b: ag.EdgeMul.apply(a, b, plan), (a, b))]:
        assert torch.autograd.gradcheck(fn, args, eps=1e-6, atol=1e-6)
        assert torch.autograd.gradgradcheck(fn, args, eps=1e-6, atol=1e-6)
    # SegIn against the definition: sum at row1 of a[row0] * V
    ref = torch.zeros(plan.N, 3, dtype=torch.float64).index_add_(0, plan.row1.long(), a[plan.row0.long()] * V)
    assert torch.allclose(ag.SegIn.apply(a, V, plan, False), ref)


@pytest.mark.parametrize("which", ["symmetric", "general"])
def test_distance_gradcheck(golden, which):
    """The recipe of the reference's native-op test (test_radius.py:126-150): gradcheck and gradgradcheck."""
    c, sym, gen = _plans(golden)
    plan = sym if which == "symmetric" else gen
    pos = c["pos"].double().clone().requires_grad_(True)
    fn = lambda p: ag.edge_distances(p, plan)
    assert torch.autograd.gradcheck(fn, (pos,), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradgradcheck(fn, (pos,), eps=1e-6, atol=1e-6)


@pytest.mark.parametrize("kind", ["gaussian", "expnormal"])
def test_rbf_operator_chain_gradcheck(kind):
    cut = bnn.CosineCutoff(0.0, 8.0)
    rbf = (bnn.GaussianBasis(cut, 6) if kind == "gaussian" else bnn.ExpNormalBasis(cut, 6, trainable=False)).double()
    d = (0.5 + 7.0 * torch.rand(9, dtype=torch.float64, generator=torch.Generator().manual_seed(2))).requires_grad_(True)
    assert torch.autograd.gradcheck(rbf, (d,), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradgradcheck(rbf, (d,), eps=1e-6, atol=1e-6)


def test_gemm_family_gradcheck():
    g = torch.Generator().manual_seed(3)
    X = torch.randn(7, 4, dtype=torch.float64, generator=g, requires_grad=True)
    W = torch.randn(5, 4, dtype=torch.float64, generator=g, requires_grad=True)
    b = torch.randn(5, dtype=torch.float64, generator=g, requires_grad=True)
    assert torch.autograd.gradcheck(ag.MatmulNT.apply, (X, W, b), eps=1e-6, atol=1e-6)
    assert torch.autograd.gradgradcheck(ag.MatmulNT.apply, (X, W, b), eps=1e-6, atol=1e-6)


def test_priors_eval_and_train_paths_vs_reference(golden):
    c = golden["priors_f32"]
    import itertools
    T = c["tables"]["bonds"]["x_0"].shape[0]
    data, priors = prior_setup(12, 2, T, torch.Generator().manual_seed(0))
    # replace geometry, lists and tables by the golden ones
    for k, p in priors.items():
        p.load_state_dict(c["tables"][k])
    for mode in ("eval", "train"):
        for k, p in priors.items():
            d = mlcg_b200.AtomicData(pos=c["pos"].clone(), atom_types=c["atom_types"], batch=c["batch"], n_atoms=torch.full((c["B"],), 12),
                                     neighbor_list={k: mlcg_b200.make_neighbor_list(k, c["mappings"][k].shape[0], c["mappings"][k], c["mapping_batch"][k])})
            m = bnn.GradientsOut(p, "forces")
            m = m.eval() if mode == "eval" else m.train()
            o = m(d)
            assert torch.allclose(o.out[k]["energy"], c["energy"][k], rtol=1e-5), (mode, k)
            f = o.out[k]["forces"].detach()
            assert torch.allclose(f, c["forces"][k], rtol=1e-4, atol=1e-4 * float(c["forces"][k].abs().max())), (mode, k)


@pytest.mark.parametrize("box", ["orthorhombic", "slab", "triclinic"])
def test_priors_on_periodic_data_vs_reference(golden_priors_periodic, box):
    """Bonds, angles, dihedrals and repulsion pairs that cross the box: the reference applies its cell shifts whenever the data
    carry ``pbc`` and ``cell`` (harmonic.py:214-242 with base.py:5-62)."""
    c, cases = periodic_prior_cases(golden_priors_periodic, box)
    for mode in ("eval", "train"):
        for k, p, data in cases:
            m = bnn.GradientsOut(p, "forces")
            o = (m.eval() if mode == "eval" else m.train())(data)
            assert torch.allclose(o.out[k]["energy"].detach(), c["energy"][k], rtol=2e-5), (mode, k)
            assert torch.allclose(o.out[k]["forces"].detach(), c["forces"][k], rtol=1e-4, atol=1e-4 * float(c["forces"][k].abs().max())), (mode, k)


def test_two_priors_of_one_class_on_one_data_object():
    """Each prior gathers its own per-term parameters: a second prior of the same class and name with other statistics, a
    changed parameter table and changed bead types must all be seen (nothing stale is reused)."""
    data, priors = prior_setup(12, 2, 3, torch.Generator().manual_seed(4))
    a = priors["bonds"]
    b = bnn.HarmonicBonds({k: {"k": 2.0 * v["k"], "x_0": v["x_0"] + 0.5} for k, v in
                           {key: {"k": float(a.k[key]), "x_0": float(a.x_0[key])} for key in a.allowed_interaction_keys}.items()})
    run = lambda p: bnn.GradientsOut(p, "forces").eval()(data).out["bonds"]["energy"].clone()
    ea, eb = run(a), run(b)
    assert not torch.allclose(ea, eb)
    assert set(data.neighbor_list["bonds"].keys()) == {"tag", "order", "index_mapping", "cell_shifts", "rcut", "self_interaction", "mapping_batch"}
    assert torch.allclose(run(a), ea)                       # the first prior again: its own parameters
    with torch.no_grad():
        a.k.mul_(3.0)                                        # a table edited in place
    assert torch.allclose(run(a), 3.0 * ea, rtol=1e-5)
    data.atom_types = (data.atom_types + 1) % 3              # other bead types on the same lists
    want = ag_free_bond_energy(a, data)
    assert torch.allclose(run(a), want, rtol=1e-5)


def ag_free_bond_energy(prior, data):
    m = data.neighbor_list["bonds"]["index_mapping"]
    t0, t1 = data.atom_types[m[0]], data.atom_types[m[1]]
    d = (data.pos[m[1]] - data.pos[m[0]]).norm(dim=1)
    y = prior.k[t0, t1] * (d - prior.x_0[t0, t1]) ** 2
    return torch.zeros(int(data.batch.max()) + 1).index_add_(0, data.neighbor_list["bonds"]["mapping_batch"], y)


def test_sumout_additivity(golden):
    """tests/unit/nn/test_outs.py:160-166: SumOut totals equal the sum of the components (atol 1e-5 relative here)."""
    data, priors = prior_setup(12, 3, 4, torch.Generator().manual_seed(5))
    models = torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})
    out = bnn.SumOut(models).eval()(data)
    e = sum(out.out[k]["energy"] for k in priors)
    f = sum(out.out[k]["forces"] for k in priors)
    assert torch.allclose(out.out["energy"], e, rtol=1e-6) and torch.allclose(out.out["forces"], f, rtol=1e-6)


def test_no_cpu_fallback(monkeypatch):
    """Without the test substitution the package refuses CPU tensors instead of computing on the host."""
    monkeypatch.setattr(backend, "_backend", None)
    try:
        be = backend.get_backend()
    except Exception:
        return  # library not built on this machine: operators cannot run at all, which is the point
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        be.edge_mul(torch.zeros(2, 4), torch.zeros(2, 4), torch.zeros(1, dtype=torch.int32), torch.zeros(1, dtype=torch.int32))


def test_condensed_priors_give_the_same_energies_and_forces():
    """src/mlcg/simulation/specialize_prior.py:75-206: several priors of one class merged into one Static prior over the
    concatenated index lists; the total energy and forces of a collated batch do not change."""
    import itertools
    from mlcg_b200.data import collate
    from mlcg_b200.specialize_prior import StaticPrior, condense_all_priors_for_simulation
    gen = torch.Generator().manual_seed(9)
    T, n, B = 3, 11, 3
    r = lambda: float(torch.rand(1, generator=gen))
    tab2 = lambda: {k: {"k": 50 + 100 * r(), "x_0": 3.5 + 0.6 * r()} for k in itertools.product(range(T), repeat=2)}
    tab3 = {k: {"k": 20 + 60 * r(), "x_0": -0.8 + r()} for k in itertools.product(range(T), repeat=3)}
    def tab4(nd):
        return {k: {"v_0": r(), "k1s": {f"k1_{i}": r() - 0.5 for i in range(1, nd + 1)}, "k2s": {f"k2_{i}": r() - 0.5 for i in range(1, nd + 1)}}
                for k in itertools.product(range(T), repeat=4)}
    priors = {"bonds_even": bnn.HarmonicBonds(tab2()), "bonds_odd": bnn.HarmonicBonds(tab2()), "angles": bnn.HarmonicAngles(tab3),
              "dih_short": bnn.Dihedral(tab4(2), n_degs=2, name="dih_short"), "dih_long": bnn.Dihedral(tab4(3), n_degs=3, name="dih_long"),
              "repulsion": bnn.Repulsion({k: {"sigma": 3.0 + 2.0 * r()} for k in itertools.product(range(T), repeat=2)})}
    for k, p in priors.items():
        p.name = k
    idx = torch.arange(n)
    bonds = torch.stack([idx[:-1], idx[1:]])
    full = torch.cartesian_prod(idx, idx).t()
    per = {"bonds_even": bonds[:, ::2], "bonds_odd": bonds[:, 1::2], "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
           "dih_short": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])[:, :4],
           "dih_long": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])[:, 4:], "repulsion": full[:, (full[0] - full[1]).abs() >= 3]}
    from helpers import random_walk_chain
    data_list = []
    for b in range(B):
        nls = {k: mlcg_b200.make_neighbor_list(k, m.shape[0], m.clone()) for k, m in per.items()}
        data_list.append(mlcg_b200.AtomicData(pos=random_walk_chain(n, gen, jitter=0.3), atom_types=torch.randint(0, T, (n,), generator=gen),
                                              neighbor_list=nls))
    model = bnn.SumOut(torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})).eval()
    ref = model(collate(data_list))
    cmodel, cdata = condense_all_priors_for_simulation(model, data_list)
    assert set(cmodel.models.keys()) == {"bonds", "angles", "dihedrals", "repulsion"}
    assert all(isinstance(cmodel.models[k].model, StaticPrior) for k in ("bonds", "angles", "dihedrals"))
    assert set(cdata[0].neighbor_list.keys()) == {"bonds", "angles", "dihedrals", "repulsion"}
    out = cmodel.eval()(collate(cdata))
    assert torch.allclose(out.out["energy"], ref.out["energy"], rtol=1e-5)
    assert torch.allclose(out.out["forces"], ref.out["forces"], rtol=1e-4, atol=1e-4 * float(ref.out["forces"].abs().max()))
    # and a second pass finds nothing left to merge
    again, _ = condense_all_priors_for_simulation(cmodel, cdata)
    assert set(again.models.keys()) == set(cmodel.models.keys())


def test_condensed_priors_equal_the_reference_s(golden_condensed_priors):
    """The reference's own specialize_prior.py:75-206 produced the fixture (tests/golden/make_golden.py, mode `condensed`):
    same keys in the same order, same Static class names, identical parameter buffers and rewritten index mappings, and the
    merged model's energies and forces on the collated structures."""
    from helpers import condensed_prior_case
    from mlcg_b200.data import collate
    from mlcg_b200.specialize_prior import condense_all_priors_for_simulation
    g = golden_condensed_priors
    model, data_list = condensed_prior_case(g)
    cmodel, cdata = condense_all_priors_for_simulation(model, data_list)
    assert list(cmodel.models.keys()) == g["model_keys"]
    for k, m in cmodel.models.items():
        assert type(m.model).__name__ == g["class_names"][k]
        ours = m.model.state_dict()
        assert set(ours.keys()) == set(g["buffers"][k].keys())
        for bk, bv in g["buffers"][k].items():
            assert ours[bk].shape == bv.shape and torch.equal(ours[bk], bv), (k, bk)
    for d, ref in zip(cdata, g["condensed_mappings"]):
        assert set(d.neighbor_list.keys()) == set(ref.keys())
        for k, m in ref.items():
            assert torch.equal(d.neighbor_list[k]["index_mapping"], m)
    out = cmodel.eval()(collate(cdata))
    assert torch.allclose(out.out["energy"], g["energy"], rtol=1e-5)
    assert torch.allclose(out.out["forces"], g["forces"], rtol=1e-4, atol=1e-4 * float(g["forces"].abs().max()))
    for k, e in g["per_model_energy"].items():
        assert torch.allclose(out.out[k]["energy"], e, rtol=1e-5, atol=1e-4)
