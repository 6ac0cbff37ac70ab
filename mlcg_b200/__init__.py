"""mlcg_b200 — sm_100a (B200) kernels behind mlcg's coarse-grained force-field hot path.

Radius graph, edge featurisation, filter network, continuous-filter convolution (with first and
second derivatives) and the classical prior terms, behind the Python interface of
``mlcg.nn`` / ``mlcg.neighbor_list``.  The compute back end is ``libmlcg_b200.so`` (C ABI in
``include/mlcg_b200.h``); there is no CPU path.
"""
from . import nn  # noqa: F401
from . import ops  # noqa: F401  (registers torch.ops.mlcg.radius_cuda / exclusion_pair_to_ptr)
from .data import AtomicData  # noqa: F401
from .graphed import GraphedForceField  # noqa: F401
from .neighbor_list import (atomic_data2neighbor_list, exclusion_pair_to_ptr, make_neighbor_list, radius_cuda,  # noqa: F401
                            radius_distance, radius_graph)

__version__ = "0.1.0"
