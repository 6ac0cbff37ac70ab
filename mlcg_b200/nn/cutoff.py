"""Cutoff envelopes with mlcg's class names and attributes (src/mlcg/nn/cutoff.py)."""
import math

import torch


class _Cutoff(torch.nn.Module):
    """Base class: holds ``cutoff_lower`` / ``cutoff_upper`` and validates them (cutoff.py:7-37)."""

    def __init__(self):
        super().__init__()
        self.cutoff_lower = None
        self.cutoff_upper = None

    def check_cutoff(self):
        if self.cutoff_upper < self.cutoff_lower:
            raise ValueError("Upper cutoff {} is less than lower cutoff {}".format(self.cutoff_upper, self.cutoff_lower))


class IdentityCutoff(_Cutoff):
    """Envelope of ones (cutoff.py:40-72)."""

    def __init__(self, cutoff_lower: float = 0, cutoff_upper: float = float("inf")):
        super().__init__()
        self.cutoff_lower, self.cutoff_upper = cutoff_lower, cutoff_upper
        self.check_cutoff()

    def forward(self, distances: torch.Tensor) -> torch.Tensor:
        return torch.ones_like(distances)


class CosineCutoff(_Cutoff):
    """0.5 (cos(pi d / upper) + 1) for a zero lower bound, the shifted form otherwise (cutoff.py:75-153)."""

    def __init__(self, cutoff_lower: float = 0.0, cutoff_upper: float = 5.0):
        super().__init__()
        self.cutoff_lower, self.cutoff_upper = cutoff_lower, cutoff_upper
        self.check_cutoff()

    def forward(self, distances: torch.Tensor) -> torch.Tensor:
        d, lo, hi = distances, self.cutoff_lower, self.cutoff_upper
        below = (d < hi).to(d.dtype)
        if lo > 0:
            env = 0.5 * (torch.cos(math.pi * (2 * (d - lo) / (hi - lo) + 1.0)) + 1.0)
            return env * below * (d > lo).to(d.dtype)
        return 0.5 * (torch.cos(d * math.pi / hi) + 1.0) * below


def cutoff_kind(cutoff: _Cutoff):
    """0 identity, 1 cosine, None for envelopes the kernels do not implement."""
    if type(cutoff) is IdentityCutoff or type(cutoff).__name__ == "IdentityCutoff":
        return 0
    if type(cutoff) is CosineCutoff or type(cutoff).__name__ == "CosineCutoff":
        return 1
    return None
