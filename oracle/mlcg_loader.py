"""TEST INFRASTRUCTURE — load the reference's own hot-path modules where its package cannot be imported as a whole.

``import mlcg`` needs torch_geometric, torch_cluster, ase, mdtraj, e3nn, pytorch_lightning, ... (none installed, no index
access), because its ``__init__`` files pull in every sub-package.  :func:`install` registers empty parent packages whose
``__path__`` points at a copy of the reference's ``mlcg`` package directory, so that ``importlib.import_module("mlcg.nn.schnet")``
and the like load the reference's files unmodified, and replaces the three third-party calls those files make by small
stand-ins that restate the published behaviour:

* ``torch_geometric.nn.MessagePassing.propagate`` (``aggr="add"``): gather ``x[edge_index[0]]``, call ``message``, index-add at
  ``edge_index[1]``;
* ``torch_geometric.utils.scatter(reduce="sum")``: index-add over dim 0;
* ``torch_cluster.radius_graph``: the oracle in ``oracle/radius_ref.py`` (rule "cluster");
* ``torch_cluster.radius`` (periodic structures only): all points of the same structure within the radius, in index order,
  cut after ``max_num_neighbors``.

Everything else that then runs — SchNet, CFConv, MLP, the radial bases, the cutoffs, compute_distances / angles / torsions, the
prior classes, GradientsOut, SumOut — is the reference's code.  Users: ``tests/golden/make_golden.py`` (fixtures, from a checkout)
and ``bench.py --impl reference`` / its CPU-baseline legs (from ``oracle/_ref/site``, where ``oracle/build_ref.py`` installs the
package with pip).  The product never imports this module.
"""
import importlib
import os
import sys
import types

import numpy as np
import torch

from . import radius_ref

HERE = os.path.dirname(os.path.abspath(__file__))
INSTALLED = os.path.join(HERE, "_ref", "site", "mlcg")      # where oracle/build_ref.py puts the reference's package


def available() -> bool:
    return os.path.isdir(INSTALLED)


def install(mlcg_dir: str = INSTALLED):
    """Register the stand-ins and the parent packages; ``mlcg_dir`` is the reference's ``mlcg`` package directory
    (``<checkout>/src/mlcg`` or the installed copy)."""
    ref = mlcg_dir

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
        with squared distance < r*r (`dist += diff * diff` over the coordinates, fused multiply-adds as nvcc contracts it), in
        index order, at most max_num_neighbors; row 0 indexes y, row 1 indexes x."""
        xn, yn = x.detach().numpy(), y.detach().numpy()
        bx = batch_x.numpy() if batch_x is not None else np.zeros(len(xn), np.int64)
        by = batch_y.numpy() if batch_y is not None else np.zeros(len(yn), np.int64)
        r2 = xn.dtype.type(float(r) * float(r))
        rows = [[], []]
        for i in range(len(yn)):
            cand = np.nonzero(bx == by[i])[0]
            d2 = radius_ref.squared_distance(xn[cand] - yn[i])
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


def modules():
    """The reference's classes the hot path is made of, as a namespace (call :func:`install` first)."""
    schnet = importlib.import_module("mlcg.nn.schnet")
    rb = importlib.import_module("mlcg.nn.radial_basis")
    cutoff = importlib.import_module("mlcg.nn.cutoff")
    gradients = importlib.import_module("mlcg.nn.gradients")
    atomic_data = importlib.import_module("mlcg.data.atomic_data")
    sys.modules["mlcg.data"].AtomicData = atomic_data.AtomicData
    harmonic = importlib.import_module("mlcg.nn.prior.harmonic")
    repulsion = importlib.import_module("mlcg.nn.prior.repulsion")
    fourier = importlib.import_module("mlcg.nn.prior.fourier_series")
    return types.SimpleNamespace(schnet=schnet, StandardSchNet=schnet.StandardSchNet, GaussianBasis=rb.GaussianBasis,
                                 ExpNormalBasis=rb.ExpNormalBasis, CosineCutoff=cutoff.CosineCutoff, GradientsOut=gradients.GradientsOut,
                                 SumOut=gradients.SumOut, AtomicData=atomic_data.AtomicData, HarmonicBonds=harmonic.HarmonicBonds,
                                 HarmonicAngles=harmonic.HarmonicAngles, Dihedral=fourier.Dihedral, Repulsion=repulsion.Repulsion)
