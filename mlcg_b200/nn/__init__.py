from .cutoff import CosineCutoff, IdentityCutoff
from .gradients import EnergyOut, GradientsOut, SumOut
from .mlp import MLP
from .prior import Dihedral, FourierSeries, GeneralAngles, GeneralBonds, Harmonic, HarmonicAngles, HarmonicBonds, Repulsion, evaluate_priors, set_prior_determinism
from .radial_basis import ExpNormalBasis, GaussianBasis, RegularizedBasis, SymmetricTensor
from .attention import (AttentiveInteractionBlock, AttentiveInteractionBlock2, ExactAttention, FavorAttention, Nonlocalinteractionblock,  # noqa: F401
                        Residual, Residual_MLP, ResidualStack)
from .schnet import AttentiveSchNet, CFConv, InteractionBlock, RBFRegularizedSchNet, SchNet, StandardSchNet, set_edge_capacity, set_filter_precision
