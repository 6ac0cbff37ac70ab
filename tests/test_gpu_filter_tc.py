"""The fused tensor-core filter network against the oracle expression (float64 evaluation of the same float32 inputs)."""
import pytest
import torch

from mlcg_b200.backend import RbfSpec, get_backend
from oracle import schnet_ref
from oracle.primitives import OracleBackend

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def reference(d, kind, upper, R, A1, b1, A2):
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": upper}
    spec = {"kind": kind, "rbf_cutoff": cut}
    p0, p1 = (schnet_ref.gaussian_params(0.0, upper, R) if kind == "gaussian" else schnet_ref.expnormal_params(0.0, upper, R))
    sd = {"rbf_layer.offset": p0.double(), "rbf_layer.coeff": p1.double(), "rbf_layer.means": p0.double(), "rbf_layer.betas": p1.double()}
    dd = d if d.dtype == torch.float64 else d.double()
    rbf = schnet_ref.radial_basis(dd, spec, sd)
    h = torch.tanh(rbf @ A1.double().t() + b1.double())
    return (h @ A2.double().t()) * schnet_ref.cosine_cutoff(dd, 0.0, upper).view(-1, 1), p0, p1


@pytest.mark.parametrize("kind,R,upper", [("expnormal", 128, 15.0), ("gaussian", 50, 30.0), ("expnormal", 64, 12.0), ("gaussian", 100, 10.0)])
@pytest.mark.parametrize("E", [1, 127, 128, 1000, 40000])
@pytest.mark.parametrize("precision", [0, 1])
def test_filter_forward(kind, R, upper, E, precision):
    gen = torch.Generator().manual_seed(E + R)
    F = 128
    d = torch.rand(E, generator=gen) * (upper * 1.05) + 0.5
    lim1, lim2 = (6.0 / (R + F)) ** 0.5, (6.0 / (2 * F)) ** 0.5
    A1 = (torch.rand(F, R, generator=gen) * 2 - 1) * lim1
    A2 = (torch.rand(F, F, generator=gen) * 2 - 1) * lim2
    b1 = torch.randn(F, generator=gen) * 0.1
    want, p0, p1 = reference(d, kind, upper, R, A1, b1, A2)
    spec = RbfSpec(0 if kind == "gaussian" else 1, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.reshape(-1).to(DEV))
    W, status = get_backend().filter_forward(d.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV), precision)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    err = float((W.cpu().double() - want).abs().max())
    scale = float(want.abs().max()) + 1e-30
    if precision == 0:
        assert err < 3e-6 * max(scale, 1.0), (err, scale)        # float32-equivalent
    else:
        assert err < 3e-2 * max(scale, 1.0), (err, scale)        # bf16 operands
    assert not W[d.to(DEV) >= upper].any()                        # envelope: exactly zero beyond the cutoff


def test_filter_forward_is_row_independent():
    """A row of W depends on its own distance only: the same distance gives the same bits wherever it sits."""
    gen = torch.Generator().manual_seed(0)
    d = torch.rand(5000, generator=gen) * 14 + 0.5
    d2 = torch.cat([d.flip(0), d[:100]])
    R, F, upper = 128, 128, 15.0
    p0, p1 = schnet_ref.expnormal_params(0.0, upper, R)
    spec = RbfSpec(1, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.to(DEV))
    A1, A2, b1 = torch.randn(F, R, generator=gen) * 0.1, torch.randn(F, F, generator=gen) * 0.1, torch.zeros(F)
    be = get_backend()
    Wa, _ = be.filter_forward(d.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV), 0)
    Wb, _ = be.filter_forward(d2.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV), 0)
    assert torch.equal(Wa.flip(0), Wb[:5000]) and torch.equal(Wa[:100], Wb[5000:])


@pytest.mark.parametrize("kind,R,upper", [("expnormal", 128, 15.0), ("gaussian", 50, 30.0)])
@pytest.mark.parametrize("E", [100, 5000])
@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("gscale", [1.0, 1e4, 1e-6])
@pytest.mark.parametrize("saved", [False, True])
def test_filter_backward(kind, R, upper, E, precision, gscale, saved):
    """gd = d/dd sum(gW * W(d)) with gW = xl[row0] * gagg[row1]; checked against autograd of the float64 oracle.  ``saved``: the
    backward that reads the hidden layer the forward kept (two GEMMs per tile, two tiles in flight) instead of recomputing it."""
    gen = torch.Generator().manual_seed(E + R)
    F, N = 128, 300
    d = torch.rand(E, generator=gen) * (upper * 1.02) + 0.5
    lim1, lim2 = (6.0 / (R + F)) ** 0.5, (6.0 / (2 * F)) ** 0.5
    A1 = (torch.rand(F, R, generator=gen) * 2 - 1) * lim1
    A2 = (torch.rand(F, F, generator=gen) * 2 - 1) * lim2
    b1 = torch.randn(F, generator=gen) * 0.1
    row0 = torch.randint(0, N, (E,), generator=gen).int()
    row1 = torch.randint(0, N, (E,), generator=gen).int()
    xl = torch.randn(N, F, generator=gen)
    gagg = torch.randn(N, F, generator=gen) * gscale
    gW = (xl[row0.long()] * gagg[row1.long()]).double()
    dd = d.double().requires_grad_(True)
    W, p0, p1 = reference(dd, kind, upper, R, A1, b1, A2)
    (want,) = torch.autograd.grad((gW * W).sum(), dd)
    spec = RbfSpec(0 if kind == "gaussian" else 1, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.reshape(-1).to(DEV))
    hidden = None
    if saved:
        _, _, hidden = get_backend().filter_forward(d.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV), precision, save_hidden=True)
    gd, status = get_backend().filter_backward(d.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV), row0.to(DEV), row1.to(DEV),
                                               xl.to(DEV), gagg.to(DEV), precision, hidden=hidden)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    err = float((gd.cpu().double() - want).abs().max())
    scale = float(want.abs().max()) + 1e-30
    assert err < (2e-5 if precision == 0 else 5e-2) * scale, (err, scale)


@pytest.mark.parametrize("precision", [0, 1])
@pytest.mark.parametrize("E", [19000, 100003])
def test_filter_backward_many_tiles_per_block(E, precision):
    """Enough rows that every thread block walks several tiles (two, and five to six): the saved-hidden-layer backward keeps two
    tiles in flight and prefetches the indices of later ones, so its steady state, start and end are all exercised; compared
    with the float64 oracle and with the recomputing kernel."""
    kind, R, upper, F, N = "expnormal", 128, 15.0, 128, 4000
    gen = torch.Generator().manual_seed(E)
    d = torch.rand(E, generator=gen) * (upper * 1.02) + 0.5
    A1 = (torch.rand(F, R, generator=gen) * 2 - 1) * (6.0 / (R + F)) ** 0.5
    A2 = (torch.rand(F, F, generator=gen) * 2 - 1) * (6.0 / (2 * F)) ** 0.5
    b1 = torch.randn(F, generator=gen) * 0.1
    row0, row1 = torch.randint(0, N, (E,), generator=gen).int(), torch.randint(0, N, (E,), generator=gen).int()
    xl, gagg = torch.randn(N, F, generator=gen), torch.randn(N, F, generator=gen)
    gW = (xl[row0.long()] * gagg[row1.long()]).double()
    dd = d.double().requires_grad_(True)
    W, p0, p1 = reference(dd, kind, upper, R, A1, b1, A2)
    (want,) = torch.autograd.grad((gW * W).sum(), dd)
    spec = RbfSpec(1, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.reshape(-1).to(DEV))
    be = get_backend()
    args = (d.to(DEV), spec, 1, 0.0, upper, A1.to(DEV), b1.to(DEV), A2.to(DEV))
    Wg, _, hidden = be.filter_forward(*args, precision, save_hidden=True)
    tol = 3e-6 if precision == 0 else 3e-2
    assert float((Wg.cpu().double() - W.detach()).abs().max()) < tol * max(1.0, float(W.detach().abs().max()))
    more = (row0.to(DEV), row1.to(DEV), xl.to(DEV), gagg.to(DEV), precision)
    gd_saved, status = be.filter_backward(*args, *more, hidden=hidden)
    gd_again, _ = be.filter_backward(*args, *more, hidden=hidden)
    gd_recomputed, _ = be.filter_backward(*args, *more)
    torch.cuda.synchronize()
    assert int(status[0]) == 0
    scale = float(want.abs().max())
    tol = 2e-5 if precision == 0 else 5e-2
    assert torch.equal(gd_saved, gd_again)                                     # no dependence on timing
    assert float((gd_saved.cpu().double() - want).abs().max()) < tol * scale
    assert float((gd_recomputed.cpu().double() - want).abs().max()) < tol * scale


def test_pair_mode_equals_per_edge_mode():
    """Symmetric edge list: evaluating one row per unordered pair gives the same filters (bit for bit) and the same
    total distance gradient per pair as evaluating every directed edge."""
    from mlcg_b200 import autograd as ag
    from mlcg_b200.neighbor_list import _graph
    gen = torch.Generator().manual_seed(0)
    n, B, upper, R, F = 60, 6, 9.0, 128, 128
    pos = (torch.rand(B * n, 3, generator=gen) * 14).to(DEV)
    ptr = (torch.arange(B + 1) * n).to(DEV)
    res = _graph(pos, upper, ptr, False, 1000, 1)
    plan = res["plan"]
    assert plan.symmetric
    sel = plan.half_selection()
    assert sel.numel() * 2 == plan.E
    d = ag.EdgeDistanceOnce.apply(pos, plan)
    p0, p1 = schnet_ref.expnormal_params(0.0, upper, R)
    spec = RbfSpec(1, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.to(DEV))
    A1, A2, b1 = (torch.randn(F, R, generator=gen) * 0.1).to(DEV), (torch.randn(F, F, generator=gen) * 0.1).to(DEV), (torch.randn(F, generator=gen) * 0.1).to(DEV)
    be = get_backend()
    W_full, _ = be.filter_forward(d, spec, 1, 0.0, upper, A1, b1, A2, 0)
    W_pair, _ = be.filter_forward(d, spec, 1, 0.0, upper, A1, b1, A2, 0, sel, plan.perm_in)
    assert torch.equal(W_full, W_pair)
    # one stored row per pair, read by both edges through the pair index
    W_half, _ = be.filter_forward(d, spec, 1, 0.0, upper, A1, b1, A2, 0, sel)
    pair_of = plan.pair_index()
    assert W_half.shape[0] * 2 == plan.E
    assert torch.equal(pair_of.cpu(), OracleBackend().pair_index(sel.cpu(), plan.perm_in.cpu()))
    assert torch.equal(W_half[pair_of.long()], W_full)
    xs = torch.randn(B * n, F, generator=gen).to(DEV)
    agg_full = be.seg_mul_sum(xs, W_full, plan.ptr_out, plan.nbr_out, None, plan.N)
    agg_half = be.seg_mul_sum(xs, W_half, plan.ptr_out, plan.nbr_out, pair_of, plan.N)
    assert torch.equal(agg_full, agg_half)
    xl, gagg = torch.randn(B * n, F, generator=gen).to(DEV), torch.randn(B * n, F, generator=gen).to(DEV)
    g_full, _ = be.filter_backward(d, spec, 1, 0.0, upper, A1, b1, A2, plan.row0, plan.row1, xl, gagg, 0)
    g_pair, _ = be.filter_backward(d, spec, 1, 0.0, upper, A1, b1, A2, plan.row0, plan.row1, xl, gagg, 0, sel, plan.perm_in)
    tw = plan.perm_in.long()
    total_full = g_full + g_full[tw]
    total_pair = g_pair + g_pair[tw]
    assert bool((g_pair[tw[sel.long()]] == 0).all())
    assert float((total_full - total_pair).abs().max()) < 2e-5 * float(total_full.abs().max())
    # the same with the hidden layer kept by the forward (per pair and per edge)
    _, _, h_half = be.filter_forward(d, spec, 1, 0.0, upper, A1, b1, A2, 0, sel, save_hidden=True)
    g_pair_h, _ = be.filter_backward(d, spec, 1, 0.0, upper, A1, b1, A2, plan.row0, plan.row1, xl, gagg, 0, sel, plan.perm_in, hidden=h_half)
    assert bool((g_pair_h[tw[sel.long()]] == 0).all())
    assert float((g_pair_h - g_pair).abs().max()) < 2e-5 * float(total_full.abs().max())
    _, _, h_full = be.filter_forward(d, spec, 1, 0.0, upper, A1, b1, A2, 0, save_hidden=True)
    g_full_h, _ = be.filter_backward(d, spec, 1, 0.0, upper, A1, b1, A2, plan.row0, plan.row1, xl, gagg, 0, hidden=h_full)
    assert float((g_full_h - g_full).abs().max()) < 2e-5 * float(g_full.abs().max())


def test_weights_beyond_the_fp16_pair_range_are_reported():
    """|w| > 512 cannot be carried by the scaled fp16 operand pairs: the kernel says so through its status word, and with
    the tensor-core route switched off the same model evaluates on the CUDA cores."""
    from mlcg_b200 import nn as bnn
    import mlcg_b200
    gen = torch.Generator().manual_seed(0)
    torch.manual_seed(0)
    cut = bnn.CosineCutoff(0.0, 8.0)
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, 32, trainable=False), cut, [128], hidden_channels=128, embedding_size=5,
                             num_filters=128, num_interactions=1).to(DEV)
    with torch.no_grad():
        net.interaction_blocks[0].conv.filter_network.layers[0].weight[3, 5] = 2000.0
    model = bnn.GradientsOut(net, "forces").eval()
    B, n = 8, 20
    v = torch.randn(B, n, 3, generator=gen)
    pos = torch.cumsum(3.8 * v / v.norm(dim=2, keepdim=True), dim=1).reshape(B * n, 3).to(DEV)
    mk = lambda: mlcg_b200.AtomicData(pos=pos.clone(), atom_types=torch.randint(0, 5, (B * n,), generator=gen).to(DEV),
                                      batch=torch.arange(B).repeat_interleave(n).to(DEV), n_atoms=torch.full((B,), n).to(DEV))
    be = get_backend()
    be.check_pending()
    model(mk())
    with pytest.raises(RuntimeError, match="range of the fp16-pair"):
        be.check_pending()
    model(mk())                           # the report cleared the status word: the failure is raised again, not carried over
    with pytest.raises(RuntimeError, match="range of the fp16-pair"):
        be.check_pending()
    be.tensor_core_gemm = False
    try:
        out = model(mk())
        be.check_pending()
        assert bool(torch.isfinite(out.out["SchNet"]["forces"]).all())
    finally:
        be.tensor_core_gemm = True
