"""``torch.ops.mlcg.radius_cuda`` and ``torch.ops.mlcg.exclusion_pair_to_ptr`` — the two operators mlcg's native package
registers with torch's dispatcher (``src/opt_radius/mlcg_opt_radius/radius.cu:313-314``, ``exclusion_pairs.cpp:64-65``),
under the same names, with the same schemas, backed by this package's kernels.

The reference registers through ``torch::RegisterOperators().op(name, &function)``, which infers the schema from the C++
signature: positional arguments named ``_0 .. _6``.  The schemas below are those strings.  Argument meaning
(``radius.cu:197-203``): ``radius_cuda(x [N,dim], ptr_x [B+1] | None, r, max_num_neighbors, ignore_same_index,
exclude_pair_xs | None, ptr_exclude_pair_xs [N+1] | None) -> (edge_index [2,E], distance [E])``;
``exclusion_pair_to_ptr(exc_pair_index [2,P], num_nodes) -> (pair_xs [P], y_ptr [num_nodes+1])``.

A registered operator is what ``torch.compile`` treats as opaque (the reference wraps its neighbour search that way,
``src/mlcg/neighbor_list/torch_impl.py:8-23``); the fake implementations give the output shapes for tracing, with an
unbacked symbolic edge count.

If the process has already loaded mlcg's own extension, the names are taken: nothing is registered here and
:data:`REGISTERED` is ``False``.
"""
import torch

RADIUS_CUDA_SCHEMA = ("radius_cuda(Tensor _0, Tensor? _1, float _2, int _3, bool _4, Tensor? _5, Tensor? _6) "
                      "-> (Tensor _0, Tensor _1)")
EXCLUSION_PAIR_TO_PTR_SCHEMA = "exclusion_pair_to_ptr(Tensor _0, int _1) -> (Tensor _0, Tensor _1)"

REGISTERED = False
_library = None


def _taken(name: str) -> bool:
    try:
        getattr(torch.ops.mlcg, name)
        return True
    except (AttributeError, RuntimeError):
        return False


def _radius_cuda(x, ptr_x, r, max_num_neighbors, ignore_same_index, exclude_pair_xs, ptr_exclude_pair_xs):
    from .neighbor_list import radius_cuda
    return radius_cuda(x, ptr_x, r, max_num_neighbors, ignore_same_index, exclude_pair_xs, ptr_exclude_pair_xs)


def _radius_cuda_not_on_cuda(x, *args):
    raise RuntimeError("x must be CUDA tensor")       # the reference's CHECK_CUDA(x), radius.cu:205


def _radius_cuda_fake(x, ptr_x, r, max_num_neighbors, ignore_same_index, exclude_pair_xs, ptr_exclude_pair_xs):
    E = torch.library.get_ctx().new_dynamic_size()
    return x.new_empty((2, E), dtype=torch.int64), x.new_empty((E,))


def _exclusion_pair_to_ptr(exc_pair_index, num_nodes):
    from .neighbor_list import exclusion_pair_to_ptr
    return exclusion_pair_to_ptr(exc_pair_index, num_nodes)


def _exclusion_pair_to_ptr_fake(exc_pair_index, num_nodes):
    return exc_pair_index.new_empty((exc_pair_index.shape[1],)), exc_pair_index.new_empty((num_nodes + 1,))


def register() -> bool:
    """Define and implement the two operators (once per process).  Returns whether this package owns the names."""
    global REGISTERED, _library
    if REGISTERED:
        return True
    if _taken("radius_cuda") or _taken("exclusion_pair_to_ptr"):
        return False
    lib = torch.library.Library("mlcg", "FRAGMENT")
    lib.define(RADIUS_CUDA_SCHEMA)
    lib.define(EXCLUSION_PAIR_TO_PTR_SCHEMA)
    lib.impl("radius_cuda", _radius_cuda, "CUDA")
    lib.impl("radius_cuda", _radius_cuda_not_on_cuda, "CPU")
    lib.impl("exclusion_pair_to_ptr", _exclusion_pair_to_ptr, "CUDA")
    lib.impl("exclusion_pair_to_ptr", _exclusion_pair_to_ptr, "CPU")    # host-side list preparation, as in the reference
    torch.library.register_fake("mlcg::radius_cuda", _radius_cuda_fake, lib=lib)
    torch.library.register_fake("mlcg::exclusion_pair_to_ptr", _exclusion_pair_to_ptr_fake, lib=lib)
    _library = lib          # keeps the registrations alive
    REGISTERED = True
    return True


register()
