"""Radius-graph front end with mlcg's call signatures and neighbour-list dictionary format.

Mirrors ``src/mlcg/neighbor_list/neighbor_list.py`` (``atomic_data2neighbor_list`` :27-102,
``make_neighbor_list`` :105-163, ``validate_neighborlist`` :170-202), the ``radius_graph`` call made at
``src/mlcg/neighbor_list/torch_impl.py:216-224`` and the native op ``radius_distance``
(``src/opt_radius/mlcg_opt_radius/radius.py:187-199``), and ``torch_neighbor_list_pbc`` for periodic structures
(``src/mlcg/neighbor_list/torch_impl.py:102-163, 252-329``).
"""
from typing import Dict, Mapping, Optional, Tuple

import torch

from .autograd import EdgePlan, attach_plan, edge_distances
from .backend import STATUS_TRUNCATED, get_backend

RULE_NATIVE, RULE_CLUSTER = 0, 1
PLAN_KEY = "_mlcgb_plan"


def _as_3d(x: torch.Tensor) -> torch.Tensor:
    """Zero-pad 1-D / 2-D points to three coordinates (adding +0.0 leaves the squared distance unchanged)."""
    if x.dim() != 2 or not 1 <= x.shape[1] <= 3:
        raise ValueError("positions must be [N, dim] with dim in 1..3")
    if x.shape[1] == 3:
        return x
    return torch.cat([x, x.new_zeros(x.shape[0], 3 - x.shape[1])], dim=1)


def _structure_ptr(x, batch, batch_size):
    be = get_backend()
    N = x.shape[0]
    if batch is None:
        return torch.tensor([0, N], dtype=torch.int64, device=x.device)
    if batch.numel() != N:
        raise ValueError("batch must have one entry per point")
    if batch_size is None:
        batch_size = int(batch[-1]) + 1 if N > 0 else 1   # sorted batch vector: last entry is the maximum
    return be.batch_to_ptr(batch.to(torch.int64), batch_size)


def _graph(x, r, ptr, loop, max_num_neighbors, rule, want_distance=False, exclude=None, want_batch=False):
    be = get_backend()
    res = be.radius_graph(_as_3d(x), ptr, r, max_num_neighbors, loop, rule, want_distance=want_distance, want_batch=want_batch, exclude=exclude)
    truncated = bool(res["status"] & STATUS_TRUNCATED)
    # an exclusion list need not hold both directions of a pair: such a graph is not taken to be symmetric
    plan = EdgePlan.from_centre_sorted(res["row0"], res["row1"], res["offsets"], x.shape[0], symmetric=not truncated and exclude is None,
                                       loops=bool(loop))
    attach_plan(res["edge_index"], plan)
    res["plan"], res["truncated"] = plan, truncated
    return res


def radius_graph(x: torch.Tensor, r: float, batch: Optional[torch.Tensor] = None, loop: bool = False,
                 max_num_neighbors: int = 32, flow: str = "source_to_target", num_workers: int = 1,
                 batch_size: Optional[int] = None) -> torch.Tensor:
    """Same call and result as ``torch_cluster.radius_graph`` (torch_impl.py:216-224 passes
    ``flow="target_to_source"``: row 0 = centre, row 1 = neighbour, centre-major, neighbours ascending)."""
    assert flow in ("source_to_target", "target_to_source")
    res = _graph(x, r, _structure_ptr(x, batch, batch_size), loop, max_num_neighbors, RULE_CLUSTER)
    ei = res["edge_index"]
    if flow == "target_to_source":
        return ei
    out = ei.flip(0)
    return out


def radius_cuda(x: torch.Tensor, ptr_x: Optional[torch.Tensor], r: float, max_num_neighbors: int, ignore_same_index: bool,
                exclude_pair_xs: Optional[torch.Tensor] = None, ptr_exclude_pair_xs: Optional[torch.Tensor] = None
                ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``mlcg::radius_cuda`` (radius.cu:197-307): returns ``(edge_index [2,E], distance [E])``.  ``exclude_pair_xs`` /
    ``ptr_exclude_pair_xs`` as :func:`exclusion_pair_to_ptr` returns them: centre ``i`` never gets a neighbour listed in
    ``exclude_pair_xs[ptr_exclude_pair_xs[i]:ptr_exclude_pair_xs[i+1]]`` (radius.cu:112-133)."""
    if not x.is_cuda:
        raise RuntimeError("x must be CUDA tensor")
    if (exclude_pair_xs is None) != (ptr_exclude_pair_xs is None):
        raise RuntimeError("exclude_pair_xs and ptr_exclude_pair_xs go together")
    exclude = None
    if exclude_pair_xs is not None and exclude_pair_xs.numel() > 0:
        exclude = (exclude_pair_xs, ptr_exclude_pair_xs)
    if ptr_x is None:
        ptr_x = torch.tensor([0, x.shape[0]], dtype=torch.int64, device=x.device)
    res = _graph(x, r, ptr_x.to(torch.int64), not ignore_same_index, max_num_neighbors, RULE_NATIVE, want_distance=True, exclude=exclude)
    return res["edge_index"], res["distance"]


def exclusion_pair_to_ptr(exc_pair_index: torch.Tensor, num_nodes: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """``mlcg::exclusion_pair_to_ptr`` (exclusion_pairs.cpp:7-62): pairs ``[2, P]`` of ``(x, y)`` -> the ``x`` sorted by
    ``(y, x)`` and a pointer of length ``num_nodes + 1`` over ``y``.  Runs where the pairs live (the reference copies them to
    the host and back); torch's stable sort and bincount do the work."""
    if exc_pair_index.dtype != torch.int64 or exc_pair_index.dim() != 2 or exc_pair_index.shape[0] != 2:
        raise RuntimeError("exc_pair_index must be an int64 tensor of shape [2, P]")
    xs, ys = exc_pair_index[0], exc_pair_index[1]
    if xs.numel() and (int(ys.min()) < 0 or int(ys.max()) >= num_nodes):
        raise RuntimeError("pair index out of range")
    order = torch.argsort(xs, stable=True)
    order = order[torch.argsort(ys[order], stable=True)]
    y_ptr = torch.zeros(num_nodes + 1, dtype=torch.int64, device=exc_pair_index.device)
    if xs.numel():
        y_ptr[1:] = torch.cumsum(torch.bincount(ys, minlength=num_nodes), 0)
    return xs[order].contiguous(), y_ptr


def radius_distance(x: torch.Tensor, r: float, batch: Optional[torch.Tensor] = None, loop: bool = False,
                    max_num_neighbors: int = 32, batch_size: Optional[int] = None,
                    exclude_pair_indices: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``mlcg_opt_radius.radius.radius_distance`` (radius.py:187-199, :50-90): ``(distance, edge_index)``;
    ``exclude_pair_indices`` is a ``[2, P]`` tensor of ``(x, y)`` pairs: ``y`` never gets ``x`` as a neighbour."""
    if x.numel() == 0:
        return x.new_zeros(0), torch.empty(2, 0, dtype=torch.long, device=x.device)
    exclude = None
    if exclude_pair_indices is not None and exclude_pair_indices.numel() > 0:
        exclude = exclusion_pair_to_ptr(exclude_pair_indices.to(x.device), x.shape[0])
    res = _graph(x, r, _structure_ptr(x, batch, batch_size), loop, max_num_neighbors, RULE_NATIVE, exclude=exclude)
    # the distance goes through the differentiable geometry operators, so that derivatives of any
    # order with respect to x exist (the reference hand-writes two orders, radius.py:123-158)
    return edge_distances(_as_3d(x), res["plan"]), res["edge_index"]


def make_neighbor_list(tag: str, order: int, index_mapping: torch.Tensor, mapping_batch: Optional[torch.Tensor] = None,
                       cell_shifts: Optional[torch.Tensor] = None, rcut: Optional[float] = None,
                       self_interaction: Optional[bool] = None) -> Dict:
    """neighbor_list.py:105-163 — same keys, same checks."""
    if index_mapping.shape[0] != order:
        raise RuntimeError(f"index_mapping shape does not match the order:{index_mapping.shape[0]} != {order}")
    if mapping_batch is None:
        mapping_batch = torch.zeros((index_mapping.shape[1],) if len(index_mapping) > 0 else (0,), dtype=torch.long)
    plan = getattr(index_mapping, "_mlcgb_plan", None)
    im = torch.as_tensor(index_mapping, dtype=torch.long)
    if plan is not None:
        attach_plan(im, plan)
    return dict(tag=tag, order=order, index_mapping=im, cell_shifts=cell_shifts, rcut=rcut,
                self_interaction=self_interaction, mapping_batch=mapping_batch)


def validate_neighborlist(inp: Mapping) -> bool:
    """neighbor_list.py:170-202."""
    keys = {"tag", "order", "index_mapping", "cell_shifts", "rcut", "self_interaction", "mapping_batch"}
    if isinstance(inp, Mapping) and keys.issubset(inp.keys()):
        if isinstance(inp["tag"], str) and isinstance(inp["order"], int) and torch.is_tensor(inp["index_mapping"]):
            return True
    return False


def structure_pointer(data) -> torch.Tensor:
    """Structure boundaries ``ptr[B+1]`` of a collated batch, from ``n_atoms`` when it is there (no device->host read)."""
    pos = data.pos
    n_atoms = getattr(data, "n_atoms", None)
    if n_atoms is not None and torch.is_tensor(n_atoms) and n_atoms.dim() == 1:
        ptr = torch.zeros(n_atoms.numel() + 1, dtype=torch.int64, device=pos.device)
        torch.cumsum(n_atoms.to(device=pos.device, dtype=torch.int64), 0, out=ptr[1:])
        return ptr
    batch = getattr(data, "batch", None)
    if batch is None:
        batch = torch.zeros(pos.shape[0], dtype=torch.long, device=pos.device)
    return _structure_ptr(pos, batch, None)


def _is_periodic(data) -> bool:
    pbc = getattr(data, "pbc", None)
    return pbc is not None and bool(torch.any(pbc))


def pbc_repeats(cell: torch.Tensor, pbc: torch.Tensor, rcut: float) -> torch.Tensor:
    """Copies of a structure along each cell vector that a search within ``rcut`` needs, as compute_images works them out
    (torch_impl.py:113-120); zero along non-periodic directions.  ``[B,3]`` int64."""
    cell, pbc = cell.view((-1, 3, 3)), pbc.view((-1, 3))
    inv_distances = torch.linalg.inv(cell).transpose(2, 1).norm(2, dim=-1)
    num_repeats = torch.ceil(rcut * inv_distances).to(torch.long)
    return torch.where(pbc, num_repeats, torch.zeros_like(num_repeats))


def periodic_neighbor_list(data, rcut: float, self_interaction: bool = False, max_num_neighbors: int = 1000) -> Dict:
    """The neighbour-list dictionary of periodic structures (minimum images and beyond: every copy inside ``rcut``)."""
    if getattr(data, "cell", None) is None:
        raise ValueError("Periodic systems need to have a unit cell defined")
    pos = data.pos
    ptr = structure_pointer(data)
    cell = data.cell.to(pos.dtype).view((-1, 3, 3))
    res = get_backend().radius_graph_pbc(_as_3d(pos), ptr, cell, pbc_repeats(cell, data.pbc.to(pos.device), rcut), rcut, max_num_neighbors,
                                         self_interaction)
    mapping = res["edge_index"]
    return make_neighbor_list(tag=f"nonbounded rc:{rcut} order:{mapping.shape[0]}", order=mapping.shape[0], index_mapping=mapping,
                              mapping_batch=res["mapping_batch"], cell_shifts=res["cell_shifts"], rcut=rcut,
                              self_interaction=self_interaction)


def edge_plan_for(data, rcut: float, max_num_neighbors: int = 1000):
    """Radius graph of non-periodic data as (edge plan, structure pointer), without the neighbour-list dictionary around it
    (no ``mapping_batch``, no ``cell_shifts``): what the one-call evaluation needs and nothing else."""
    pbc = getattr(data, "pbc", None)
    if pbc is not None and bool(torch.any(pbc)):
        raise NotImplementedError("periodic structures are outside the scope of mlcg_b200's radius graph")
    ptr = structure_pointer(data)
    be = get_backend()
    res = be.radius_graph(_as_3d(data.pos), ptr, float(rcut), max_num_neighbors, False, RULE_CLUSTER, want_distance=False, want_batch=False)
    truncated = bool(res["status"] & STATUS_TRUNCATED)
    plan = EdgePlan.from_centre_sorted(res["row0"], res["row1"], res["offsets"], data.pos.shape[0], symmetric=not truncated, loops=False)
    return plan, ptr, res["edge_index"]


def atomic_data2neighbor_list(data, rcut: float, self_interaction: bool = False, max_num_neighbors: int = 1000,
                              nls_distance_method: str = "custom_kernel") -> Dict:
    """neighbor_list.py:27-102 for non-periodic data; every supported method name runs the same
    sm_100a kernel (there is no alternative back end in this package)."""
    rcut = float(rcut)
    if nls_distance_method not in ("torch", "custom_kernel", "nvalchemi_naive", "nvalchemi_cell", "nvalchemi_raw"):
        raise ValueError(f"Method {nls_distance_method} not supported for nls-distance computation ")
    if _is_periodic(data):
        return periodic_neighbor_list(data, rcut, self_interaction, max_num_neighbors)
    pos = data.pos
    batch = getattr(data, "batch", None)
    if batch is None:
        batch = torch.zeros(pos.shape[0], dtype=torch.long, device=pos.device)
    n_atoms = getattr(data, "n_atoms", None)
    if n_atoms is not None and torch.is_tensor(n_atoms) and n_atoms.dim() == 1:
        # structure boundaries without a device->host read of batch[-1]
        ptr = torch.zeros(n_atoms.numel() + 1, dtype=torch.int64, device=pos.device)
        torch.cumsum(n_atoms.to(device=pos.device, dtype=torch.int64), 0, out=ptr[1:])
    else:
        ptr = _structure_ptr(pos, batch, None)
    res = _graph(pos, rcut, ptr, self_interaction, max_num_neighbors, RULE_CLUSTER, want_batch=True)
    mapping = res["edge_index"]
    # The reference asserts batch[mapping[0]] == batch[mapping[1]] here (a device->host sync,
    # neighbor_list.py:89-91); the kernel only ever pairs points of one structure, by construction.
    cell_shifts = torch.zeros((mapping.shape[1], 3), dtype=pos.dtype, device=pos.device)
    nl = make_neighbor_list(tag=f"nonbounded rc:{rcut} order:{mapping.shape[0]}", order=mapping.shape[0], index_mapping=mapping,
                            mapping_batch=res["mapping_batch"], cell_shifts=cell_shifts, rcut=rcut,
                            self_interaction=self_interaction)
    nl["_mlcgb_zero_shifts"] = True
    nl["_mlcgb_ptr"] = ptr           # structure boundaries, for the per-structure energy sum
    return nl
