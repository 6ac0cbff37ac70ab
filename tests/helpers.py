"""Shared builders for the tests: models from golden cases, synthetic chains, prior set-ups."""
import itertools

import torch

import mlcg_b200
from mlcg_b200 import nn as bnn


def schnet_from_case(case, dtype=None, device="cpu", trainable=None):
    """mlcg_b200 StandardSchNet with the architecture and weights of a golden case."""
    cut = bnn.CosineCutoff(0.0, case["upper"])
    trainable = case.get("trainable", "rbf_layer.means" in case.get("param_grads", {})) if trainable is None else trainable
    rbf = bnn.GaussianBasis(cut, case["R"], trainable=trainable) if case["kind"] == "gaussian" else bnn.ExpNormalBasis(cut, case["R"], trainable=trainable)
    emb = case["state_dict"]["embedding_layer.weight"].shape[0]
    model = bnn.StandardSchNet(rbf, cut, [case["H"]], hidden_channels=case["H"], embedding_size=emb, num_filters=case["H"],
                               num_interactions=case["L"])
    model = model.to(case["pos"].dtype)          # cast first: loading float64 weights into float32 would round them
    assert set(model.state_dict().keys()) == set(case["state_dict"].keys())
    model.load_state_dict(case["state_dict"])
    dtype = case["pos"].dtype if dtype is None else dtype
    return model.to(device=device, dtype=dtype)


def fullwidth_case(golden_fullwidth, name):
    """A case of ``reference_vectors_fullwidth.pt`` with its complete ``state_dict`` (the case that repeats another case's
    structures with a trainable basis stores the basis parameters only; the other weights are those of ``chain73``)."""
    c = dict(golden_fullwidth[name])
    if name == "chain73_trainable":
        c["state_dict"] = {**golden_fullwidth["chain73"]["state_dict"], **c["state_dict"]}
    return c


def regularized_schnet_from_case(case, device="cpu"):
    """mlcg_b200 RBFRegularizedSchNet with the architecture and weights of a golden case."""
    cut = bnn.CosineCutoff(0.0, case["upper"])
    model = bnn.RBFRegularizedSchNet(bnn.ExpNormalBasis(cut, case["R"], trainable=False), cut, [case["H"]], hidden_channels=case["H"],
                                     embedding_size=case["T"], num_filters=case["H"], num_interactions=case["L"],
                                     independent_regularizations=case["independent"])
    model.load_state_dict(case["state_dict"])
    return model.to(device)


def attentive_schnet_from_case(case, device="cpu"):
    """mlcg_b200 AttentiveSchNet with the architecture and weights of a golden case."""
    cut = bnn.CosineCutoff(0.0, case["upper"])
    att = bnn.FavorAttention(dimv=case["state_dict"]["interaction_blocks.0.attention_block.attention_block.omega"].shape[1],
                             dimqk=case["H"]) if case["favor"] else bnn.ExactAttention()
    model = bnn.AttentiveSchNet(bnn.ExpNormalBasis(cut, case["R"], trainable=False), cut, [16], num_features_in=case["H"],
                                num_features_out=case["H"], num_residual_q=1, num_residual_k=1, num_residual_v=1, attention_block=att,
                                hidden_channels=case["H"], embedding_size=case["T"], num_filters=case["F"], num_interactions=case["L"],
                                attention_version=case["version"])
    model.load_state_dict(case["state_dict"])
    return model.to(device)


def data_from_case(case, device="cpu", dtype=None):
    dtype = case["pos"].dtype if dtype is None else dtype
    return mlcg_b200.AtomicData(pos=case["pos"].clone().to(device=device, dtype=dtype), atom_types=case["atom_types"].to(device),
                                batch=case["batch"].to(device), n_atoms=torch.full((case["B"],), case["n"]).to(device), neighbor_list={})


def random_walk_chain(n, gen, step=3.8, jitter=0.0, min_dist=None):
    """3.8 A random walk; with ``min_dist`` a step is redrawn while the new bead is closer than that to any
    bead except its predecessor (back-tracking five beads after 200 failures)."""
    pos = torch.zeros(n, 3)
    i, fails = 1, 0
    while i < n:
        v = torch.randn(3, generator=gen)
        cand = pos[i - 1] + step * v / v.norm()
        if min_dist is not None and i > 1 and bool(((pos[: i - 1] - cand).norm(dim=1) < min_dist).any()):
            fails += 1
            if fails > 200:
                i, fails = max(1, i - 5), 0
            continue
        pos[i] = cand
        i, fails = i + 1, 0
    if jitter:
        pos = pos + jitter * torch.randn(n, 3, generator=gen)
    return pos


def prior_setup(n, B, T, gen, min_sep=3):
    """Chains with bonds / angles / dihedrals / repulsion lists and random parameter tables over T types."""
    pos = torch.cat([random_walk_chain(n, gen, jitter=0.3) for _ in range(B)])
    types_ = torch.randint(0, T, (B * n,), generator=gen)
    batch = torch.arange(B).repeat_interleave(n)
    idx = torch.arange(n)
    per = {"bonds": torch.stack([idx[:-1], idx[1:]]), "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
           "dihedrals": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])}
    full = torch.cartesian_prod(idx, idx).t()
    per["repulsion"] = full[:, (full[0] - full[1]).abs() >= min_sep]
    nls = {}
    for k, m in per.items():
        nls[k] = mlcg_b200.make_neighbor_list(k, m.shape[0], torch.cat([m + b * n for b in range(B)], dim=1),
                                              torch.arange(B).repeat_interleave(m.shape[1]))
    r = lambda: float(torch.rand(1, generator=gen))
    bond = {k: {"k": 50 + 100 * r(), "x_0": 3.5 + 0.6 * r()} for k in itertools.product(range(T), repeat=2)}
    ang = {k: {"k": 20 + 60 * r(), "x_0": -0.8 + r()} for k in itertools.product(range(T), repeat=3)}
    dih = {k: {"v_0": r(), "k1s": {f"k1_{i}": r() - 0.5 for i in (1, 2, 3)}, "k2s": {f"k2_{i}": r() - 0.5 for i in (1, 2, 3)}}
           for k in itertools.product(range(T), repeat=4)}
    rep = {k: {"sigma": 3.0 + 2.0 * r()} for k in itertools.product(range(T), repeat=2)}
    priors = {"bonds": bnn.HarmonicBonds(bond), "angles": bnn.HarmonicAngles(ang), "dihedrals": bnn.Dihedral(dih, n_degs=3),
              "repulsion": bnn.Repulsion(rep)}
    data = mlcg_b200.AtomicData(pos=pos, atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list=nls)
    return data, priors


def periodic_prior_cases(golden_priors_periodic, box, device="cpu"):
    """(name, prior module, data) for the four priors on one box of ``reference_vectors_priors_periodic.pt``."""
    g = golden_priors_periodic
    c = g[box]
    st = g["stats"]
    priors = {"bonds": bnn.HarmonicBonds(st["bonds"]), "angles": bnn.HarmonicAngles(st["angles"]), "dihedrals": bnn.Dihedral(st["dihedrals"], n_degs=3),
              "repulsion": bnn.Repulsion(st["repulsion"])}
    out = []
    for k, p in priors.items():
        p.load_state_dict(g["tables"][k])
        nl = {k: mlcg_b200.make_neighbor_list(k, c["mappings"][k].shape[0], c["mappings"][k].to(device), c["mapping_batch"][k].to(device))}
        data = mlcg_b200.AtomicData(pos=c["pos"].clone().to(device), atom_types=c["atom_types"].to(device), batch=c["batch"].to(device),
                                    n_atoms=torch.full((g["B"],), g["n"]).to(device), neighbor_list=nl, cell=c["cells"].clone().to(device),
                                    pbc=c["pbc"].clone().to(device))
        out.append((k, p.to(device), data))
    return c, out


def condensed_prior_case(golden_condensed_priors):
    """The model and the structures of ``reference_vectors_condensed_priors.pt`` built from this package's classes: two
    named bond priors, angles, two dihedral priors of different length, repulsion; three structures of different length."""
    g = golden_condensed_priors
    st = g["stats"]
    priors = {"bonds_even": bnn.GeneralBonds(st["bonds_even"], name="bonds_even"), "bonds_odd": bnn.GeneralBonds(st["bonds_odd"], name="bonds_odd"),
              "angles": bnn.HarmonicAngles(st["angles"]), "dih_short": bnn.Dihedral(st["dih_short"], n_degs=2, name="dih_short"),
              "dih_long": bnn.Dihedral(st["dih_long"], n_degs=3, name="dih_long"), "repulsion": bnn.Repulsion(st["repulsion"])}
    data_list = []
    for s in g["structures"]:
        nls = {k: mlcg_b200.make_neighbor_list(k, m.shape[0], m.clone()) for k, m in s["mappings"].items()}
        data_list.append(mlcg_b200.AtomicData(pos=s["pos"].clone(), atom_types=s["atom_types"].clone(), neighbor_list=nls))
    model = bnn.SumOut(torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()}))
    return model, data_list
