"""Generate the golden fixtures in this folder by running the reference's own Python modules.

Run once, in a container where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/mlcg

The reference package cannot be imported as a whole (its ``__init__`` files need torch_geometric,
torch_cluster, ase, mdtraj, e3nn, ... which are not installed), so the hot-path files are loaded by
path under synthetic parent packages, and the three third-party calls they make are replaced by the small
stand-ins of ``oracle/mlcg_loader.py`` (``MessagePassing.propagate``, ``utils.scatter``, ``torch_cluster.radius_graph`` and
``torch_cluster.radius``).

Everything else that runs — SchNet, CFConv, MLP, the radial bases, the cutoffs, compute_distances /
angles / torsions, the prior classes, GradientsOut — is the reference's unmodified code.
The fixtures are plain ``torch.save`` dictionaries of tensors and floats.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
from oracle import mlcg_loader, radius_ref  # noqa: E402


def install_shims(ref_src: str):
    """The stand-ins and parent packages of ``oracle/mlcg_loader.py``, over the checkout at ``ref_src``."""
    mlcg_loader.install(os.path.join(ref_src, "src", "mlcg"))


def chain(n, step=3.8, jitter=0.0, gen=None):
    v = torch.randn(n, 3, generator=gen)
    v = step * v / v.norm(dim=1, keepdim=True)
    return torch.cumsum(v, 0) + jitter * torch.randn(n, 3, generator=gen)


def nl(mapping, mapping_batch):
    return dict(tag="t", order=mapping.shape[0], index_mapping=mapping, mapping_batch=mapping_batch,
                cell_shifts=None, rcut=None, self_interaction=False)


def main(ref_src):
    install_shims(ref_src)
    schnet = importlib.import_module("mlcg.nn.schnet")
    from mlcg.nn.radial_basis import GaussianBasis, ExpNormalBasis
    from mlcg.nn.cutoff import CosineCutoff
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    harmonic = importlib.import_module("mlcg.nn.prior.harmonic")
    repulsion = importlib.import_module("mlcg.nn.prior.repulsion")
    fourier = importlib.import_module("mlcg.nn.prior.fourier_series")

    gen = torch.Generator().manual_seed(1234)
    out = {}

    def schnet_case(name, kind, B, n, n_types, upper, R, H, L, trainable, dtype):
        torch.manual_seed(7)
        cut = CosineCutoff(0.0, upper)
        rbf = GaussianBasis(cut, R, trainable=trainable) if kind == "gaussian" else ExpNormalBasis(cut, R, trainable=trainable)
        model = schnet.StandardSchNet(rbf, cut, [H], hidden_channels=H, embedding_size=n_types, num_filters=H,
                                      num_interactions=L).to(dtype)
        # biases are zero after the reference's Xavier reset; perturb them so they are exercised
        with torch.no_grad():
            for k, p in model.named_parameters():
                if k.endswith("bias"):
                    p.copy_(0.1 * torch.randn(p.shape, generator=gen).to(dtype))
        pos = torch.cat([chain(n, jitter=0.3, gen=gen) for _ in range(B)]).to(dtype)
        types_ = torch.randint(0, n_types, (B * n,), generator=gen)
        batch = torch.arange(B).repeat_interleave(n)
        mk = lambda: AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
        res = GradientsOut(model, "forces").eval()(mk())
        case = dict(kind=kind, upper=upper, R=R, H=H, L=L, B=B, n=n, pos=pos, atom_types=types_, batch=batch,
                    state_dict={k: v.detach().clone() for k, v in model.state_dict().items()},
                    edge_index=res.neighbor_list.get("SchNet", {}).get("index_mapping") if False else None,
                    energy=res.out["SchNet"]["energy"].detach(), forces=res.out["SchNet"]["forces"].detach())
        # the edge list the model used (rebuilt here the way SchNet.neighbor_list does)
        case["edge_index"] = model.neighbor_list(mk(), upper, model.max_num_neighbors)["SchNet"]["index_mapping"]
        # force-matching step: second-order pass, gradients of the MSE force loss w.r.t. every parameter
        target = torch.randn(pos.shape, generator=gen).to(dtype)
        tr = GradientsOut(model, "forces").train()
        model.zero_grad()
        o = tr(mk())
        loss = torch.nn.functional.mse_loss(o.out["SchNet"]["forces"], target)
        loss.backward()
        case["target_forces"] = target
        case["loss"] = loss.detach()
        case["param_grads"] = {k: p.grad.detach().clone() for k, p in model.named_parameters() if p.grad is not None}
        out[name] = case
        print(name, "E", case["energy"].tolist()[:2], "edges", case["edge_index"].shape[1], "loss", float(loss))

    schnet_case("schnet_gaussian_f32", "gaussian", 3, 10, 10, 30.0, 16, 32, 2, False, torch.float32)
    schnet_case("schnet_expnormal_f32", "expnormal", 2, 30, 20, 15.0, 24, 32, 3, False, torch.float32)
    schnet_case("schnet_expnormal_trainable_f64", "expnormal", 2, 12, 5, 12.0, 8, 16, 2, True, torch.float64)

    # ---- priors on two 12-bead chains, 4 bead types, random parameter tables
    n, B, T = 12, 2, 4
    pos = torch.cat([chain(n, jitter=0.3, gen=gen) for _ in range(B)])
    types_ = torch.randint(0, T, (B * n,), generator=gen)
    batch = torch.arange(B).repeat_interleave(n)
    idx = torch.arange(n)
    per = {"bonds": torch.stack([idx[:-1], idx[1:]]), "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
           "dihedrals": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])}
    full = torch.cartesian_prod(idx, idx).t()
    per["repulsion"] = full[:, (full[0] - full[1]).abs() >= 3]
    nls = {}
    for k, m in per.items():
        nls[k] = nl(torch.cat([m + b * n for b in range(B)], dim=1), torch.arange(B).repeat_interleave(m.shape[1]))
    r = lambda *s: torch.rand(*s, generator=gen)
    import itertools
    bond_stats = {k: {"k": float(50 + 100 * r(1)), "x_0": float(3.5 + 0.6 * r(1))} for k in itertools.product(range(T), repeat=2)}
    ang_stats = {k: {"k": float(20 + 60 * r(1)), "x_0": float(-0.8 + 1.0 * r(1))} for k in itertools.product(range(T), repeat=3)}
    dih_stats = {k: {"v_0": float(r(1)), "k1s": {f"k1_{i}": float(r(1) - 0.5) for i in (1, 2, 3)},
                     "k2s": {f"k2_{i}": float(r(1) - 0.5) for i in (1, 2, 3)}} for k in itertools.product(range(T), repeat=4)}
    rep_stats = {k: {"sigma": float(3.0 + 2.0 * r(1))} for k in itertools.product(range(T), repeat=2)}
    priors = {"bonds": harmonic.HarmonicBonds(bond_stats), "angles": harmonic.HarmonicAngles(ang_stats),
              "dihedrals": fourier.Dihedral(dih_stats, n_degs=3), "repulsion": repulsion.Repulsion(rep_stats)}
    pc = dict(pos=pos, atom_types=types_, batch=batch, B=B, mappings={k: v["index_mapping"] for k, v in nls.items()},
              mapping_batch={k: v["mapping_batch"] for k, v in nls.items()}, tables={}, energy={}, forces={})
    for k, p in priors.items():
        d = AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list=dict(nls))
        o = GradientsOut(p, "forces")(d)
        pc["energy"][k] = o.out[k]["energy"].detach()
        pc["forces"][k] = o.out[k]["forces"].detach()
        pc["tables"][k] = {bk: bv.clone() for bk, bv in p.state_dict().items()}
        print(k, pc["energy"][k].tolist())
    out["priors_f32"] = pc

    # ---- cutoff endpoint values the reference's tests pin (tests/unit/nn/test_cutoff.py:27-43)
    c0, c1 = CosineCutoff(0.0, 5.0), CosineCutoff(1.0, 5.0)
    dd = torch.tensor([0.0, 1.0, 2.5, 4.999, 5.0, 6.0])
    out["cutoff"] = dict(d=dd, lower0=c0(dd), lower1=c1(dd))

    torch.save(out, os.path.join(HERE, "reference_vectors.pt"))
    print("wrote", os.path.join(HERE, "reference_vectors.pt"), os.path.getsize(os.path.join(HERE, "reference_vectors.pt")), "bytes")


def main_periodic(ref_src):
    """Periodic structures: `torch_neighbor_list_pbc` / `atomic_data2neighbor_list` (src/mlcg/neighbor_list/torch_impl.py:252-329,
    neighbor_list.py:27-102) and a SchNet evaluated on them, for an orthorhombic box, a box periodic along two directions
    only, and a sheared (triclinic) box; two structures per batch."""
    install_shims(ref_src)
    schnet = importlib.import_module("mlcg.nn.schnet")
    from mlcg.nn.radial_basis import ExpNormalBasis
    from mlcg.nn.cutoff import CosineCutoff
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    nlmod = importlib.import_module("mlcg.neighbor_list.neighbor_list")
    gen = torch.Generator().manual_seed(777)
    out = {}
    boxes = {"orthorhombic": (torch.tensor([[9.0, 0, 0], [0, 11.0, 0], [0, 0, 13.0]]), [True, True, True]),
             "slab": (torch.tensor([[9.0, 0, 0], [0, 11.0, 0], [0, 0, 13.0]]), [True, True, False]),
             "triclinic": (torch.tensor([[9.0, 0, 0], [2.5, 10.0, 0], [1.5, -2.0, 12.0]]), [True, True, True])}
    for name, (cell, pbc) in boxes.items():
        torch.manual_seed(3)
        B, n, T, upper, R, H, L = 2, 18, 4, 7.5, 16, 32, 2
        cells = torch.stack([cell, cell * 1.1])
        frac = torch.rand(B, n, 3, generator=gen) * 1.2 - 0.1           # some points outside the cell
        pos = torch.einsum("bnk,bkd->bnd", frac, cells).reshape(-1, 3)
        types_ = torch.randint(0, T, (B * n,), generator=gen)
        batch = torch.arange(B).repeat_interleave(n)
        mk = lambda: AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={},
                                cell=cells.clone(), pbc=torch.tensor([pbc] * B))
        case = dict(cells=cells, pbc=torch.tensor([pbc] * B), pos=pos, atom_types=types_, batch=batch, B=B, n=n, upper=upper, R=R, H=H, L=L, T=T)
        for cap in (1000, 12):
            nl_ = nlmod.atomic_data2neighbor_list(mk(), upper, self_interaction=False, max_num_neighbors=cap)
            case[f"index_mapping_{cap}"] = nl_["index_mapping"].clone()
            case[f"cell_shifts_{cap}"] = nl_["cell_shifts"].clone()
            case[f"mapping_batch_{cap}"] = nl_["mapping_batch"].clone()
        nl_self = nlmod.atomic_data2neighbor_list(mk(), upper, self_interaction=True, max_num_neighbors=1000)
        case["index_mapping_self"], case["cell_shifts_self"] = nl_self["index_mapping"].clone(), nl_self["cell_shifts"].clone()
        cut = CosineCutoff(0.0, upper)
        model = schnet.StandardSchNet(ExpNormalBasis(cut, R, trainable=False), cut, [H], hidden_channels=H, embedding_size=T,
                                      num_filters=H, num_interactions=L)
        with torch.no_grad():
            for k, p in model.named_parameters():
                if k.endswith("bias"):
                    p.copy_(0.1 * torch.randn(p.shape, generator=gen))
        res = GradientsOut(model, "forces").eval()(mk())
        case["state_dict"] = {k: v.detach().clone() for k, v in model.state_dict().items()}
        case["energy"], case["forces"] = res.out["SchNet"]["energy"].detach(), res.out["SchNet"]["forces"].detach()
        out[name] = case
        print(name, "edges", case["index_mapping_1000"].shape[1], case["index_mapping_12"].shape[1], "E", case["energy"].tolist())
    path = os.path.join(HERE, "reference_vectors_periodic.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_attentive(ref_src):
    """`AttentiveSchNet` (src/mlcg/nn/schnet.py:478-674, src/mlcg/nn/attention.py): both block versions, softmax and FAVOR+
    attention, two structures per batch (so the structure mask acts) and one (the unmasked branch)."""
    install_shims(ref_src)
    schnet = importlib.import_module("mlcg.nn.schnet")
    attention = importlib.import_module("mlcg.nn.attention")
    from mlcg.nn.radial_basis import ExpNormalBasis
    from mlcg.nn.cutoff import CosineCutoff
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    gen = torch.Generator().manual_seed(2468)
    out = {}
    # (the reference's non-local part is always 128 wide, so hidden_channels has to be 128; filters and bases are kept small,
    # and of the force-matching gradients only those of the small parameters are stored, to keep the file small)
    for name, version, favor, B in (("normal_exact", "normal", False, 2), ("v2_favor", "2", True, 2), ("normal_favor_single", "normal", True, 1)):
        torch.manual_seed(11)
        n, T, upper, R, H, L, F = 16, 4, 12.0, 8, 128, 1, 32
        cut = CosineCutoff(0.0, upper)
        att = attention.FavorAttention(dimv=24, dimqk=H) if favor else attention.ExactAttention()
        model = schnet.AttentiveSchNet(ExpNormalBasis(cut, R, trainable=False), cut, [16], num_features_in=H, num_features_out=H,
                                       num_residual_q=1, num_residual_k=1, num_residual_v=1, attention_block=att, hidden_channels=H,
                                       embedding_size=T, num_filters=F, num_interactions=L, attention_version=version)
        with torch.no_grad():
            for k, p in model.named_parameters():
                if k.endswith("bias"):
                    p.copy_(0.1 * torch.randn(p.shape, generator=gen))
        pos = torch.cat([chain(n, jitter=0.3, gen=gen) for _ in range(B)])
        types_ = torch.randint(0, T, (B * n,), generator=gen)
        batch = torch.arange(B).repeat_interleave(n)
        mk = lambda: AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
        res = GradientsOut(model, "forces").eval()(mk())
        case = dict(version=version, favor=favor, upper=upper, R=R, H=H, L=L, T=T, F=F, B=B, n=n, pos=pos, atom_types=types_,
                    batch=batch, state_dict={k: v.detach().clone() for k, v in model.state_dict().items()},
                    energy=res.out["SchNet"]["energy"].detach(), forces=res.out["SchNet"]["forces"].detach())
        target = torch.randn(pos.shape, generator=gen)
        tr = GradientsOut(model, "forces").train()
        model.zero_grad()
        loss = torch.nn.functional.mse_loss(tr(mk()).out["SchNet"]["forces"], target)
        loss.backward()
        case["target_forces"], case["loss"] = target, loss.detach()
        case["param_grads"] = {k: p.grad.detach().clone() for k, p in model.named_parameters() if p.grad is not None and p.numel() <= 4096}
        out[name] = case
        print(name, "E", case["energy"].tolist(), "loss", float(loss), "params", len(case["param_grads"]))
    path = os.path.join(HERE, "reference_vectors_attentive.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_regularized(ref_src):
    """`RBFRegularizedSchNet` (src/mlcg/nn/schnet.py:676-803) with shared and with per-block factors, random factors in
    [-0.2, 1.2] so that both clamps act; written to a file of its own."""
    install_shims(ref_src)
    schnet = importlib.import_module("mlcg.nn.schnet")
    from mlcg.nn.radial_basis import ExpNormalBasis
    from mlcg.nn.cutoff import CosineCutoff
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    gen = torch.Generator().manual_seed(4321)
    out = {}
    for name, independent in (("shared", False), ("independent", True)):
        torch.manual_seed(9)
        B, n, T, upper, R, H, L = 2, 20, 4, 12.0, 16, 32, 2
        cut = CosineCutoff(0.0, upper)
        model = schnet.RBFRegularizedSchNet(ExpNormalBasis(cut, R, trainable=False), cut, [H], hidden_channels=H, embedding_size=T,
                                            num_filters=H, num_interactions=L, independent_regularizations=independent)
        with torch.no_grad():
            for k, p in model.named_parameters():
                if k.endswith("bias"):
                    p.copy_(0.1 * torch.randn(p.shape, generator=gen))
                if k.endswith(".w"):
                    p.copy_(-0.2 + 1.4 * torch.rand(p.shape, generator=gen))
        pos = torch.cat([chain(n, jitter=0.3, gen=gen) for _ in range(B)])
        types_ = torch.randint(0, T, (B * n,), generator=gen)
        batch = torch.arange(B).repeat_interleave(n)
        mk = lambda: AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
        res = GradientsOut(model, "forces").eval()(mk())
        case = dict(independent=independent, upper=upper, R=R, H=H, L=L, T=T, B=B, n=n, pos=pos, atom_types=types_, batch=batch,
                    state_dict={k: v.detach().clone() for k, v in model.state_dict().items()},
                    energy=res.out["SchNet"]["energy"].detach(), forces=res.out["SchNet"]["forces"].detach(),
                    radial_filters=res.out["SchNet"]["radial_filters"].detach().clone())
        target = torch.randn(pos.shape, generator=gen)
        tr = GradientsOut(model, "forces").train()
        model.zero_grad()
        loss = torch.nn.functional.mse_loss(tr(mk()).out["SchNet"]["forces"], target)
        loss.backward()
        case["target_forces"], case["loss"] = target, loss.detach()
        case["param_grads"] = {k: p.grad.detach().clone() for k, p in model.named_parameters() if p.grad is not None}
        out[name] = case
        print(name, "E", case["energy"].tolist(), "loss", float(loss))
    path = os.path.join(HERE, "reference_vectors_regularized.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_priors_periodic(ref_src):
    """The four priors on periodic data (harmonic.py:214-242, fourier_series.py:95-101,477-483, repulsion.py:78-134 with
    base.py:5-62): chains wrapped into their cell, so that bonds, angles, dihedrals and repulsion pairs cross the box; an
    orthorhombic box periodic along all directions, the same box periodic along two, and a sheared box (where the reference's
    shift convention, as written, is not the minimum image; it is followed as written)."""
    install_shims(ref_src)
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    harmonic = importlib.import_module("mlcg.nn.prior.harmonic")
    repulsion = importlib.import_module("mlcg.nn.prior.repulsion")
    fourier = importlib.import_module("mlcg.nn.prior.fourier_series")
    import itertools
    gen = torch.Generator().manual_seed(8642)
    n, B, T = 14, 2, 3
    idx = torch.arange(n)
    per = {"bonds": torch.stack([idx[:-1], idx[1:]]), "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
           "dihedrals": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])}
    full = torch.cartesian_prod(idx, idx).t()
    per["repulsion"] = full[:, (full[0] - full[1]).abs() >= 3]
    r = lambda *s: torch.rand(*s, generator=gen)
    bond_stats = {k: {"k": float(50 + 100 * r(1)), "x_0": float(3.5 + 0.6 * r(1))} for k in itertools.product(range(T), repeat=2)}
    ang_stats = {k: {"k": float(20 + 60 * r(1)), "x_0": float(-0.8 + 1.0 * r(1))} for k in itertools.product(range(T), repeat=3)}
    dih_stats = {k: {"v_0": float(r(1)), "k1s": {f"k1_{i}": float(r(1) - 0.5) for i in (1, 2, 3)},
                     "k2s": {f"k2_{i}": float(r(1) - 0.5) for i in (1, 2, 3)}} for k in itertools.product(range(T), repeat=4)}
    rep_stats = {k: {"sigma": float(3.0 + 2.0 * r(1))} for k in itertools.product(range(T), repeat=2)}
    priors = {"bonds": harmonic.HarmonicBonds(bond_stats), "angles": harmonic.HarmonicAngles(ang_stats),
              "dihedrals": fourier.Dihedral(dih_stats, n_degs=3), "repulsion": repulsion.Repulsion(rep_stats)}
    boxes = {"orthorhombic": (torch.tensor([[13.0, 0, 0], [0, 15.0, 0], [0, 0, 17.0]]), [True, True, True]),
             "slab": (torch.tensor([[13.0, 0, 0], [0, 15.0, 0], [0, 0, 17.0]]), [True, True, False]),
             "triclinic": (torch.tensor([[13.0, 0, 0], [3.0, 15.0, 0], [2.0, -2.5, 17.0]]), [True, True, True])}
    out = dict(tables={k: {bk: bv.clone() for bk, bv in p.state_dict().items()} for k, p in priors.items()}, n=n, B=B, T=T,
               stats=dict(bonds=bond_stats, angles=ang_stats, dihedrals=dih_stats, repulsion=rep_stats))
    for name, (cell, pbc) in boxes.items():
        cells = torch.stack([cell, cell * 1.15])
        free = torch.cat([chain(n, jitter=0.3, gen=gen) + 6.0 for _ in range(B)]).view(B, n, 3)
        # wrap into the cell along the periodic directions (fractional coordinates modulo 1)
        frac = torch.einsum("bnd,bdk->bnk", free, torch.linalg.inv(cells))
        frac = torch.where(torch.tensor(pbc)[None, None, :], frac - torch.floor(frac), frac)
        pos = torch.einsum("bnk,bkd->bnd", frac, cells).reshape(-1, 3)
        types_ = torch.randint(0, T, (B * n,), generator=gen)
        batch = torch.arange(B).repeat_interleave(n)
        nls = {k: nl(torch.cat([m + b * n for b in range(B)], dim=1), torch.arange(B).repeat_interleave(m.shape[1])) for k, m in per.items()}
        case = dict(cells=cells, pbc=torch.tensor([pbc] * B), pos=pos, atom_types=types_, batch=batch, energy={}, forces={},
                    mappings={k: v["index_mapping"] for k, v in nls.items()}, mapping_batch={k: v["mapping_batch"] for k, v in nls.items()})
        for k, p in priors.items():
            d = AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list=dict(nls),
                           cell=cells.clone(), pbc=case["pbc"].clone())
            o = GradientsOut(p, "forces")(d)
            case["energy"][k], case["forces"][k] = o.out[k]["energy"].detach(), o.out[k]["forces"].detach()
            free_d = AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list=dict(nls))
            e_open = GradientsOut(p, "forces")(free_d).out[k]["energy"].detach()
            print(name, k, "periodic", [round(v, 3) for v in case["energy"][k].tolist()], "open", [round(v, 3) for v in e_open.tolist()])
        out[name] = case
    path = os.path.join(HERE, "reference_vectors_priors_periodic.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def main_condensed(ref_src):
    """src/mlcg/simulation/specialize_prior.py:75-206 run as it stands: two bond priors, one angle prior, two dihedral priors of
    different expansion length and a repulsion prior over three structures of different length; the merged Static priors'
    buffers, the rewritten neighbour lists, and the energies and forces of the merged model on the collated structures."""
    install_shims(ref_src)
    import itertools
    import types
    from mlcg.nn.gradients import GradientsOut, SumOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    harmonic = importlib.import_module("mlcg.nn.prior.harmonic")
    repulsion = importlib.import_module("mlcg.nn.prior.repulsion")
    fourier = importlib.import_module("mlcg.nn.prior.fourier_series")
    base = importlib.import_module("mlcg.nn.prior.base")
    # what the package __init__ files would have exported for `from ..nn import ...` / `from ..nn.prior import ...`
    prior_pkg, nn_pkg = sys.modules["mlcg.nn.prior"], sys.modules["mlcg.nn"]
    for name in ("HarmonicBonds", "HarmonicAngles", "HarmonicImpropers", "GeneralBonds", "GeneralAngles", "Harmonic"):
        setattr(prior_pkg, name, getattr(harmonic, name))
    prior_pkg.Dihedral, prior_pkg._Prior = fourier.Dihedral, base._Prior
    nn_pkg.GradientsOut, nn_pkg.SumOut, nn_pkg.Dihedral = GradientsOut, SumOut, fourier.Dihedral
    sim = types.ModuleType("mlcg.simulation")
    sim.__path__ = [os.path.join(ref_src, "src", "mlcg", "simulation")]
    sys.modules["mlcg.simulation"] = sim
    sp = importlib.import_module("mlcg.simulation.specialize_prior")
    make_neighbor_list = importlib.import_module("mlcg.neighbor_list.neighbor_list").make_neighbor_list

    gen = torch.Generator().manual_seed(97531)
    T, lengths = 3, (11, 9, 14)
    r = lambda: float(torch.rand(1, generator=gen))
    tab2 = lambda: {k: {"k": 50 + 100 * r(), "x_0": 3.5 + 0.6 * r()} for k in itertools.product(range(T), repeat=2)}
    tab3 = {k: {"k": 20 + 60 * r(), "x_0": -0.8 + r()} for k in itertools.product(range(T), repeat=3)}
    def tab4(nd):
        return {k: {"v_0": r(), "k1s": {f"k1_{i}": r() - 0.5 for i in range(1, nd + 1)}, "k2s": {f"k2_{i}": r() - 0.5 for i in range(1, nd + 1)}}
                for k in itertools.product(range(T), repeat=4)}
    stats = {"bonds_even": tab2(), "bonds_odd": tab2(), "angles": tab3, "dih_short": tab4(2), "dih_long": tab4(3),
             "repulsion": {k: {"sigma": 3.0 + 2.0 * r()} for k in itertools.product(range(T), repeat=2)}}
    priors = {"bonds_even": harmonic.GeneralBonds(stats["bonds_even"], name="bonds_even"), "bonds_odd": harmonic.GeneralBonds(stats["bonds_odd"], name="bonds_odd"),
              "angles": harmonic.HarmonicAngles(stats["angles"]),
              "dih_short": fourier.Dihedral(stats["dih_short"], n_degs=2, name="dih_short"), "dih_long": fourier.Dihedral(stats["dih_long"], n_degs=3, name="dih_long"),
              "repulsion": repulsion.Repulsion(stats["repulsion"])}
    data_list, raw = [], []
    for n in lengths:
        idx = torch.arange(n)
        bonds = torch.stack([idx[:-1], idx[1:]])
        full = torch.cartesian_prod(idx, idx).t()
        dih = torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])
        per = {"bonds_even": bonds[:, ::2], "bonds_odd": bonds[:, 1::2], "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
               "dih_short": dih[:, :4], "dih_long": dih[:, 4:], "repulsion": full[:, (full[0] - full[1]).abs() >= 3]}
        pos, types_ = chain(n, jitter=0.3, gen=gen), torch.randint(0, T, (n,), generator=gen)
        nls = {k: make_neighbor_list(tag=k, order=m.shape[0], index_mapping=m.clone()) for k, m in per.items()}
        data_list.append(AtomicData(pos=pos.clone(), atom_types=types_, n_atoms=torch.tensor([n]), neighbor_list=nls))
        raw.append(dict(pos=pos, atom_types=types_, mappings={k: m.clone() for k, m in per.items()}))
    model = SumOut(torch.nn.ModuleDict({k: GradientsOut(p, "forces") for k, p in priors.items()}))
    cmodel, cdata = sp.condense_all_priors_for_simulation(model, data_list)

    def collated(dl):   # what torch_geometric's collate does to these fields: concatenation, index mappings shifted by the bead offsets
        off, cat = 0, dict(pos=[], atom_types=[], batch=[], nls={})
        for b, d in enumerate(dl):
            n = d.pos.shape[0]
            cat["pos"].append(d.pos); cat["atom_types"].append(d.atom_types); cat["batch"].append(torch.full((n,), b))
            for k, v in d.neighbor_list.items():
                e = cat["nls"].setdefault(k, dict(m=[], mb=[], order=v["order"]))
                e["m"].append(v["index_mapping"] + off); e["mb"].append(torch.full((v["index_mapping"].shape[1],), b))
            off += n
        nls = {k: nl(torch.cat(e["m"], dim=1), torch.cat(e["mb"])) | {"order": e["order"], "tag": k} for k, e in cat["nls"].items()}
        return AtomicData(pos=torch.cat(cat["pos"]), atom_types=torch.cat(cat["atom_types"]), batch=torch.cat(cat["batch"]),
                          n_atoms=torch.tensor([d.pos.shape[0] for d in dl]), neighbor_list=nls)

    res = cmodel.eval()(collated(cdata))
    ref = model.eval()(collated(data_list))
    print("keys", list(cmodel.models.keys()), "energy", res.out["energy"].tolist(), "separate", ref.out["energy"].tolist())
    out = dict(T=T, lengths=lengths, stats=stats, structures=raw, model_keys=list(cmodel.models.keys()),
               buffers={k: {bk: bv.clone() for bk, bv in m.model.state_dict().items()} for k, m in cmodel.models.items()},
               class_names={k: type(m.model).__name__ for k, m in cmodel.models.items()},
               condensed_mappings=[{k: v["index_mapping"].clone() for k, v in d.neighbor_list.items()} for d in cdata],
               energy=res.out["energy"].detach(), forces=res.out["forces"].detach(),
               energy_separate=ref.out["energy"].detach(), forces_separate=ref.out["forces"].detach(),
               per_model_energy={k: res.out[k]["energy"].detach() for k in cmodel.models.keys()})
    path = os.path.join(HERE, "reference_vectors_condensed_priors.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


def avoiding_chain(n, gen, step=3.8, min_dist=4.0):
    """3.8 A random walk; a step is redrawn while the new bead is closer than ``min_dist`` to any bead except its predecessor
    (five beads back after 200 failures)."""
    pos = torch.zeros(n, 3)
    i, fails = 1, 0
    while i < n:
        v = torch.randn(3, generator=gen)
        cand = pos[i - 1] + step * v / v.norm()
        if i > 1 and bool(((pos[: i - 1] - cand).norm(dim=1) < min_dist).any()):
            fails += 1
            if fails > 200:
                i, fails = max(1, i - 5), 0
            continue
        pos[i] = cand
        i, fails = i + 1, 0
    return pos


def main_fullwidth(ref_src):
    """SchNet at the widths and shapes of the benchmark configurations (hidden = filters = 128, which is what the fused
    tensor-core route of this package needs): energies, forces, the force-matching loss and its parameter gradients, from the
    reference's unmodified modules.

    * ``chain100``: 3 x 100-bead self-avoiding chains, 20 types, 128 exp-normal functions, 15 A, 3 blocks;
    * ``chain10``: 16 x 10-bead chains with 0.3 A jitter, types 0..9 in order, 50 Gaussians on 0-30 A, 2 blocks;
    * ``chain268``: one 268-bead self-avoiding chain, 20 types, 128 exp-normal functions, 12 A, 3 blocks;
    * ``chain73``: 4 x 73-bead walks, 20 types, 128 exp-normal functions, 10 A, 3 blocks, target forces N(0,1);
    * ``chain73_trainable``: the same structures with the reference's default ``trainable=True`` basis (only the loss, the
      forces and the gradients of the basis parameters are stored).
    """
    install_shims(ref_src)
    schnet = importlib.import_module("mlcg.nn.schnet")
    from mlcg.nn.radial_basis import GaussianBasis, ExpNormalBasis
    from mlcg.nn.cutoff import CosineCutoff
    from mlcg.nn.gradients import GradientsOut
    from mlcg.data.atomic_data import AtomicData
    sys.modules["mlcg.data"].AtomicData = AtomicData
    gen = torch.Generator().manual_seed(97531)
    out = {}

    def case(name, kind, chains, types_, upper, R, L, n_types, trainable=False, keep=None, weights_of=None):
        torch.manual_seed(13)
        H = 128
        cut = CosineCutoff(0.0, upper)
        rbf = GaussianBasis(cut, R, trainable=trainable) if kind == "gaussian" else ExpNormalBasis(cut, R, trainable=trainable)
        model = schnet.StandardSchNet(rbf, cut, [H], hidden_channels=H, embedding_size=n_types, num_filters=H, num_interactions=L)
        if weights_of is not None:
            model.load_state_dict(out[weights_of]["state_dict"])
        else:
            with torch.no_grad():
                for k, p in model.named_parameters():
                    if k.endswith("bias"):
                        p.copy_(0.1 * torch.randn(p.shape, generator=gen))
        B, n = len(chains), chains[0].shape[0]
        pos = torch.cat(chains)
        batch = torch.arange(B).repeat_interleave(n)
        mk = lambda: AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
        res = GradientsOut(model, "forces").eval()(mk())
        c = dict(kind=kind, upper=upper, R=R, H=H, L=L, B=B, n=n, pos=pos, atom_types=types_, batch=batch, trainable=trainable,
                 state_dict={k: v.detach().clone() for k, v in model.state_dict().items()},
                 energy=res.out["SchNet"]["energy"].detach(), forces=res.out["SchNet"]["forces"].detach())
        c["edge_index"] = model.neighbor_list(mk(), upper, model.max_num_neighbors)["SchNet"]["index_mapping"]
        target = torch.randn(pos.shape, generator=gen)
        tr = GradientsOut(model, "forces").train()
        model.zero_grad()
        loss = torch.nn.functional.mse_loss(tr(mk()).out["SchNet"]["forces"], target)
        loss.backward()
        c["target_forces"], c["loss"] = target, loss.detach()
        c["param_grads"] = {k: p.grad.detach().clone() for k, p in model.named_parameters() if p.grad is not None and (keep is None or keep(k))}
        # the same float32 weights and positions evaluated in double precision: the value every float32 evaluation rounds towards
        mk64 = lambda: AtomicData(pos=pos.clone().double(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
        res64 = GradientsOut(model.double(), "forces").eval()(mk64())
        c["energy_f64"], c["forces_f64"] = res64.out["SchNet"]["energy"].detach(), res64.out["SchNet"]["forces"].detach()
        if keep is not None:       # the weights are those of the case this one repeats: do not store them twice
            c["state_dict"] = {k: v for k, v in c["state_dict"].items() if keep(k)}
        out[name] = c
        print(name, "E", [round(v, 4) for v in c["energy"].tolist()[:3]], "max|F|", float(c["forces"].abs().max()), "edges", c["edge_index"].shape[1],
              "loss", float(loss), "grads", len(c["param_grads"]))

    rt = lambda n, T: torch.randint(0, T, (n,), generator=gen)
    case("chain100", "expnormal", [avoiding_chain(100, gen) for _ in range(3)], rt(300, 20), 15.0, 128, 3, 20)
    case("chain10", "gaussian", [chain(10, jitter=0.3, gen=gen) for _ in range(16)], torch.arange(10).repeat(16), 30.0, 50, 2, 10)
    case("chain268", "expnormal", [avoiding_chain(268, gen)], rt(268, 20), 12.0, 128, 3, 20)
    walks, wt = [chain(73, gen=gen) for _ in range(4)], rt(292, 20)
    case("chain73", "expnormal", walks, wt, 10.0, 128, 3, 20)
    case("chain73_trainable", "expnormal", walks, wt, 10.0, 128, 3, 20, trainable=True, keep=lambda k: k.startswith("rbf_layer"),
         weights_of="chain73")
    path = os.path.join(HERE, "reference_vectors_fullwidth.pt")
    torch.save(out, path)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    extra = {"regularized": main_regularized, "periodic": main_periodic, "attentive": main_attentive, "fullwidth": main_fullwidth,
             "priors_periodic": main_priors_periodic, "condensed": main_condensed}
    if len(sys.argv) not in (2, 3) or (len(sys.argv) == 3 and sys.argv[2] not in extra):
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of ClementiGroup/mlcg> [regularized|periodic|attentive|fullwidth|priors_periodic|condensed]")
    (extra[sys.argv[2]] if len(sys.argv) == 3 else main)(sys.argv[1])
