from .cutoff import CosineCutoff, IdentityCutoff
from .gradients import EnergyOut, GradientsOut, SumOut
from .mlp import MLP
from .prior import Dihedral, FourierSeries, Harmonic, HarmonicAngles, HarmonicBonds, Repulsion
from .radial_basis import ExpNormalBasis, GaussianBasis
from .schnet import CFConv, InteractionBlock, SchNet, StandardSchNet, set_edge_capacity, set_filter_precision
