"""Energy + force evaluation of fixed-size batches replayed from a CUDA graph.

For small systems an evaluation is bound by the host's launch path (about a hundred dependent kernels of a few
microseconds each).  With a fixed edge capacity (:func:`mlcg_b200.nn.set_edge_capacity`) nothing in an evaluation reads
the device on the host, so the whole call — radius graph, pair plan, SchNet, priors, sums — can be recorded once and
replayed for every new set of positions of the same shape.
"""
from typing import Tuple

import torch

from .backend import get_backend
from .data import ENERGY_KEY, FORCE_KEY


class GraphedForceField:
    """``model`` (eval mode, e.g. ``GradientsOut(SchNet)`` or a ``SumOut``) recorded on ``data``'s shapes.

    ``data`` provides everything that stays fixed (bead types, batch, structure sizes, prior neighbour lists); its
    ``pos`` tensor becomes the input buffer.  Every SchNet of the model needs a fixed edge capacity beforehand.
    ``__call__(pos)`` copies the positions in, replays the graph and returns views of the output buffers
    ``(energy [B], forces [N,3])`` (valid until the next call).  ``check()`` reads the kernels' status words (edge
    capacity exceeded, ...) — call it now and then, e.g. whenever results are stored."""

    def __init__(self, model: torch.nn.Module, data, warmup: int = 2):
        if model.training:
            raise ValueError("GraphedForceField records eval-mode models (no autograd graph)")
        self.model, self.data = model, data
        self.data.pos = data.pos.detach().contiguous().clone()
        self._pos = self.data.pos
        be = get_backend()
        for _ in range(max(1, warmup)):           # lazily created buffers and kernel attributes exist before the recording
            self._evaluate()
        be.check_pending()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.energy, self.forces = self._evaluate()

    def _evaluate(self) -> Tuple[torch.Tensor, torch.Tensor]:
        data = self.data
        data.pos = self._pos
        data.out = {}
        data = self.model(data)
        out = data.out if ENERGY_KEY in data.out else data.out[self.model.name]
        return out[ENERGY_KEY], out[FORCE_KEY]

    def __call__(self, pos: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        self._pos.copy_(pos, non_blocking=True)
        self.graph.replay()
        return self.energy, self.forces

    @staticmethod
    def check() -> None:
        get_backend().check_pending()
