"""Generate the golden fixtures in this folder by running the reference's own Python modules.

Run once, in a container where the reference checkout is available::

    python tests/golden/make_golden.py /path/to/mlcg

The reference package cannot be imported as a whole (its ``__init__`` files need torch_geometric,
torch_cluster, ase, mdtraj, e3nn, ... which are not installed), so the hot-path files are loaded by
path under synthetic parent packages, and the three third-party calls they make are replaced by small
stand-ins that restate the published behaviour:

* ``torch_geometric.nn.MessagePassing.propagate`` (``aggr="add"``): gather ``x[edge_index[0]]``, call
  ``message``, index-add at ``edge_index[1]``;
* ``torch_geometric.utils.scatter(reduce="sum")``: index-add over dim 0;
* ``torch_cluster.radius_graph``: the oracle in ``oracle/radius_ref.py`` (rule "cluster");
* ``torch_cluster.radius`` (periodic structures only): all points of the same structure within the radius, in index
  order, cut after ``max_num_neighbors``.

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
from oracle import radius_ref  # noqa: E402


def install_shims(ref_src: str):
    ref = os.path.join(ref_src, "src", "mlcg")

    def pkg(name, path):
        m = types.ModuleType(name)
        m.__path__ = [path]
        m.__package__ = name
        sys.modules[name] = m

    for name, sub in [("mlcg", ""), ("mlcg.nn", "nn"), ("mlcg.nn.prior", "nn/prior"), ("mlcg.geometry", "geometry"),
                      ("mlcg.data", "data"), ("mlcg.neighbor_list", "neighbor_list")]:
        pkg(name, os.path.join(ref, sub))

    class MessagePassing(torch.nn.Module):
        def __init__(self, aggr="add"):
            super().__init__()
            assert aggr == "add"
            self.aggr = aggr

        def propagate(self, edge_index, size=None, **kw):
            x = kw.pop("x")
            msg = self.message(x_j=x.index_select(0, edge_index[0]), **kw)
            out = torch.zeros(x.size(0), msg.size(1), dtype=msg.dtype, device=msg.device)
            return out.index_add_(0, edge_index[1], msg)

    def scatter(src, index, dim=0, reduce="sum", dim_size=None):
        assert dim == 0 and reduce == "sum"
        n = int(index.max()) + 1 if dim_size is None else dim_size
        out = torch.zeros((n,) + tuple(src.shape[1:]), dtype=src.dtype, device=src.device)
        return out.index_add_(0, index, src)

    class Data:
        def __init__(self, **kw):
            self.__dict__.update(kw)

        def __contains__(self, k):
            return self.__dict__.get(k) is not None

        def __getitem__(self, k):
            return self.__dict__[k]

        def __setitem__(self, k, v):
            self.__dict__[k] = v

    def radius_graph(x, r, batch=None, loop=False, max_num_neighbors=32, flow="source_to_target", num_workers=1):
        b = batch.numpy() if batch is not None else np.zeros(len(x), np.int64)
        ei = radius_ref.radius_graph_c(x.detach().numpy(), radius_ref.batch_to_ptr(b), r, max_num_neighbors, loop, "cluster")
        ei = torch.from_numpy(ei)
        return ei if flow == "target_to_source" else ei.flip(0)

    def radius(x, y, r, batch_x=None, batch_y=None, max_num_neighbors=32, num_workers=1):
        """torch_cluster.radius as its CUDA kernel states it: for every point of y, the points of x of the same structure
        with squared distance < r*r (float arithmetic of the inputs' dtype), in index order, at most max_num_neighbors;
        row 0 indexes y, row 1 indexes x."""
        xn, yn = x.detach().numpy(), y.detach().numpy()
        bx = batch_x.numpy() if batch_x is not None else np.zeros(len(xn), np.int64)
        by = batch_y.numpy() if batch_y is not None else np.zeros(len(yn), np.int64)
        r2 = xn.dtype.type(float(r) * float(r))
        rows = [[], []]
        for i in range(len(yn)):
            cand = np.nonzero(bx == by[i])[0]
            d = xn[cand] - yn[i]
            sq = d * d
            d2 = (sq[:, 0] + sq[:, 1]) + sq[:, 2]
            hit = cand[d2 < r2][:max_num_neighbors]
            rows[0].extend([i] * len(hit))
            rows[1].extend(hit.tolist())
        return torch.tensor(rows, dtype=torch.long).reshape(2, -1)

    mods = {n: types.ModuleType(n) for n in
            ["torch_geometric", "torch_geometric.nn", "torch_geometric.utils", "torch_geometric.data", "torch_cluster",
             "mdtraj", "mdtraj.core", "mdtraj.core.element", "ase", "ase.geometry", "ase.geometry.analysis", "ase.atoms",
             "ase.build", "ase.neighborlist", "mlcg.geometry.topology"]}
    mods["torch_geometric.nn"].MessagePassing = MessagePassing
    mods["torch_geometric.utils"].scatter = scatter
    mods["torch_geometric.data"].Data = Data
    mods["torch_cluster"].radius_graph = radius_graph
    mods["torch_cluster"].radius = radius
    mods["mdtraj.core.element"].Element = object
    mods["ase.geometry.analysis"].Analysis = object
    mods["ase"].Atoms = object
    mods["ase.atoms"].Atoms = object
    mods["mdtraj"].Topology = object
    mods["mlcg.geometry.topology"].Topology = object
    sys.modules.update(mods)


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


if __name__ == "__main__":
    extra = {"regularized": main_regularized, "periodic": main_periodic, "attentive": main_attentive}
    if len(sys.argv) not in (2, 3) or (len(sys.argv) == 3 and sys.argv[2] not in extra):
        sys.exit("usage: python tests/golden/make_golden.py <path to a checkout of ClementiGroup/mlcg> [regularized|periodic|attentive]")
    (extra[sys.argv[2]] if len(sys.argv) == 3 else main)(sys.argv[1])
