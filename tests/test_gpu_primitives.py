"""Each CUDA primitive, through the C ABI, against its oracle restatement on the same seeded inputs."""
import numpy as np
import pytest
import torch

from mlcg_b200 import autograd as ag
from mlcg_b200.backend import RbfSpec, get_backend
from oracle.primitives import OracleBackend

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ORA = OracleBackend()


def tol(dtype):
    return dict(rtol=1e-12, atol=1e-12) if dtype == torch.float64 else dict(rtol=2e-5, atol=2e-6)


def random_graph(N, deg, gen):
    """Symmetric-free random multigraph sorted by row0, plus its plan on CPU (built with torch ops)."""
    E = N * deg
    row0 = torch.sort(torch.randint(0, N, (E,), generator=gen)).values
    row1 = torch.randint(0, N, (E,), generator=gen)
    return torch.stack([row0, row1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("F", [128, 32, 20, 7, 1])
def test_seg_mul_sum_and_edge_mul(dtype, F):
    gen = torch.Generator().manual_seed(F)
    N = 300
    ei = random_graph(N, 9, gen)
    plan = ag.EdgePlan.from_edge_index(ei, N)
    a = torch.randn(N, F, dtype=dtype, generator=gen)
    V = torch.randn(ei.shape[1], F, dtype=dtype, generator=gen)
    be = get_backend()
    for ptr, nbr, perm in [(plan.ptr_in, plan.nbr_in, plan.perm_in), (plan.ptr_out, plan.nbr_out, plan.perm_out)]:
        want = ORA.seg_mul_sum(a, V, ptr, nbr, perm, N)
        got = be.seg_mul_sum(a.to(DEV), V.to(DEV), ptr.to(DEV), nbr.to(DEV), None if perm is None else perm.to(DEV), N)
        assert torch.allclose(got.cpu(), want, rtol=1e-5 if dtype == torch.float32 else 1e-12, atol=1e-5 if dtype == torch.float32 else 1e-12)
    want = ORA.edge_mul(a, a * 2, plan.row0, plan.row1)
    got = be.edge_mul(a.to(DEV), (a * 2).to(DEV), plan.row0.to(DEV), plan.row1.to(DEV))
    assert torch.equal(got.cpu(), want)
    # run-to-run reproducibility of the ordered sum
    again = be.seg_mul_sum(a.to(DEV), V.to(DEV), plan.ptr_in.to(DEV), plan.nbr_in.to(DEV), plan.perm_in.to(DEV), N)
    again2 = be.seg_mul_sum(a.to(DEV), V.to(DEV), plan.ptr_in.to(DEV), plan.nbr_in.to(DEV), plan.perm_in.to(DEV), N)
    assert torch.equal(again, again2)


def test_seg_mul_sum_empty_segments_and_no_edges():
    be = get_backend()
    N, F = 5, 8
    ptr = torch.tensor([0, 0, 3, 3, 3, 4], device=DEV)
    nbr = torch.tensor([1, 2, 4, 0], dtype=torch.int32, device=DEV)
    a = torch.arange(N * F, dtype=torch.float32, device=DEV).view(N, F)
    V = torch.ones(4, F, device=DEV)
    out = be.seg_mul_sum(a, V, ptr, nbr, None, N)
    assert torch.equal(out[0], torch.zeros(F, device=DEV)) and torch.equal(out[1], a[1] + a[2] + a[4]) and torch.equal(out[4], a[0])
    z = be.seg_mul_sum(a, torch.zeros(0, F, device=DEV), torch.zeros(N + 1, dtype=torch.int64, device=DEV),
                       torch.zeros(0, dtype=torch.int32, device=DEV), None, N)
    assert not z.any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_edge_geometry(dtype):
    gen = torch.Generator().manual_seed(0)
    N = 200
    ei = random_graph(N, 6, gen)
    plan = ag.EdgePlan.from_edge_index(ei, N)
    pos = torch.randn(N, 3, dtype=dtype, generator=gen)
    g = torch.randn(ei.shape[1], 3, dtype=dtype, generator=gen)
    be = get_backend()
    assert torch.equal(be.edge_diff(pos.to(DEV), plan.row0.to(DEV), plan.row1.to(DEV)).cpu(), ORA.edge_diff(pos, plan.row0, plan.row1))
    got = be.node_scatter_diff(g.to(DEV), plan.ptr_in.to(DEV), plan.perm_in.to(DEV), plan.ptr_out.to(DEV), None, N)
    assert torch.allclose(got.cpu(), ORA.node_scatter_diff(g, plan.ptr_in, plan.perm_in, plan.ptr_out, None, N), **tol(dtype))


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("cutoff_kind,lower", [(1, 0.0), (1, 1.5), (0, 0.0)])
@pytest.mark.parametrize("order", [0, 1, 2, 3])
def test_rbf_derivatives_float64(kind, cutoff_kind, lower, order):
    """Taylor-arithmetic kernel vs nested automatic differentiation of the oracle expression."""
    from oracle import schnet_ref
    upper, R = 9.0, 12
    p0, p1 = (schnet_ref.gaussian_params(lower, upper, R, torch.float64) if kind == 0 else schnet_ref.expnormal_params(lower, upper, R, torch.float64))
    spec = RbfSpec(kind, R, cutoff_kind, lower, upper, 5.0 / (upper - lower), p0, p1.reshape(-1))
    d = torch.linspace(0.3, 10.0, 57, dtype=torch.float64)
    want = ORA.rbf_expand(d, spec, order)
    spec_gpu = RbfSpec(kind, R, cutoff_kind, lower, upper, 5.0 / (upper - lower), p0.to(DEV), p1.reshape(-1).to(DEV))
    got = get_backend().rbf_expand(d.to(DEV), spec_gpu, order).cpu()
    scale = float(want.abs().max()) + 1e-30
    assert torch.allclose(got, want, rtol=1e-9, atol=1e-11 * scale)
    G = torch.randn(57, R, dtype=torch.float64, generator=torch.Generator().manual_seed(1))
    got_c = get_backend().rbf_contract(d.to(DEV), G.to(DEV), spec_gpu, order).cpu()
    assert torch.allclose(got_c, (G * want).sum(1), rtol=1e-9, atol=1e-10 * scale)


@pytest.mark.parametrize("kind", [0, 1])
@pytest.mark.parametrize("order", [0, 1, 2])
@pytest.mark.parametrize("with_c", [False, True])
def test_rbf_parameter_gradients_float64(kind, order, with_c):
    """mlcgb_rbf_param_contract vs automatic differentiation of the oracle expression with respect to offsets / coefficient
    (Gaussian, gaussian.py:64-75) and means / betas (exp-normal, exp_normal.py:80-94), for the distance-derivative orders a
    force-matching step needs; 5000 edges so that several blocks' partial sums are reduced."""
    from oracle import schnet_ref
    lower, upper, R, E = 0.0, 9.0, 20, 5000
    p0, p1 = (schnet_ref.gaussian_params(lower, upper, R, torch.float64) if kind == 0 else schnet_ref.expnormal_params(lower, upper, R, torch.float64))
    gen = torch.Generator().manual_seed(3 + order)
    p0 = p0 + 0.01 * torch.randn(R, dtype=torch.float64, generator=gen)          # (off the symmetric initial values)
    spec = RbfSpec(kind, R, 1, lower, upper, 5.0 / (upper - lower), p0, p1.reshape(-1))
    d = 0.3 + 9.5 * torch.rand(E, dtype=torch.float64, generator=gen)
    G = torch.randn(E, R, dtype=torch.float64, generator=gen)
    c = torch.randn(E, dtype=torch.float64, generator=gen) if with_c else None
    want0, want1 = ORA.rbf_param_contract(d, G, c, spec, order)
    spec_gpu = RbfSpec(kind, R, 1, lower, upper, 5.0 / (upper - lower), p0.to(DEV), p1.reshape(-1).to(DEV))
    got0, got1 = get_backend().rbf_param_contract(d.to(DEV), G.to(DEV), None if c is None else c.to(DEV), spec_gpu, order)
    assert got1.numel() == (1 if kind == 0 else R)
    for got, want in ((got0, want0), (got1, want1)):
        assert torch.allclose(got.cpu(), want, rtol=1e-9, atol=1e-10 * (float(want.abs().max()) + 1e-30))
    again0, again1 = get_backend().rbf_param_contract(d.to(DEV), G.to(DEV), None if c is None else c.to(DEV), spec_gpu, order)
    assert torch.equal(got0, again0) and torch.equal(got1, again1)              # fixed summation order


@pytest.mark.parametrize("kind", [0, 1])
def test_rbf_float32_matches_reference_expression(kind):
    from oracle import schnet_ref
    upper, R = 15.0, 128
    p0, p1 = (schnet_ref.gaussian_params(0.0, upper, R) if kind == 0 else schnet_ref.expnormal_params(0.0, upper, R))
    spec = RbfSpec(kind, R, 1, 0.0, upper, 5.0 / upper, p0, p1.reshape(-1))
    d = torch.rand(2000, generator=torch.Generator().manual_seed(0)) * 16.0
    want = ORA.rbf_expand(d, spec, 0)
    got = get_backend().rbf_expand(d.to(DEV), RbfSpec(kind, R, 1, 0.0, upper, 5.0 / upper, p0.to(DEV), p1.reshape(-1).to(DEV)), 0).cpu()
    assert torch.allclose(got, want, rtol=1e-5, atol=2e-6)
    assert not got[d >= upper].any()                       # envelope is exactly zero at and beyond the cutoff


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("M,N,K", [(1000, 128, 128), (333, 128, 50), (77, 20, 33), (5, 1, 3), (4096, 128, 128)])
def test_gemm_modes(dtype, M, N, K):
    gen = torch.Generator().manual_seed(M + N + K)
    be = get_backend()
    t = dict(rtol=1e-11, atol=1e-11) if dtype == torch.float64 else dict(rtol=1e-4, atol=1e-4)
    X, W, b = torch.randn(M, K, dtype=dtype, generator=gen), torch.randn(N, K, dtype=dtype, generator=gen), torch.randn(N, dtype=dtype, generator=gen)
    assert torch.allclose(be.gemm(0, X.to(DEV), W.to(DEV), b.to(DEV)).cpu(), (X.double() @ W.double().t() + b.double()).to(dtype), **t)
    assert torch.allclose(be.gemm(0, X.to(DEV), W.to(DEV)).cpu(), (X.double() @ W.double().t()).to(dtype), **t)
    G = torch.randn(M, N, dtype=dtype, generator=gen)
    assert torch.allclose(be.gemm(1, G.to(DEV), W.to(DEV)).cpu(), (G.double() @ W.double()).to(dtype), **t)
    t2 = dict(rtol=1e-10, atol=1e-10) if dtype == torch.float64 else dict(rtol=2e-4, atol=2e-3)
    assert torch.allclose(be.gemm(2, G.to(DEV), X.to(DEV)).cpu(), (G.double().t() @ X.double()).to(dtype), **t2)


def test_gemm_weight_gradient_over_many_edges_is_reproducible():
    gen = torch.Generator().manual_seed(0)
    G, X = torch.randn(200000, 128, generator=gen).to(DEV), torch.randn(200000, 128, generator=gen).to(DEV)
    be = get_backend()
    a, b = be.gemm(2, G, X), be.gemm(2, G, X)
    assert torch.equal(a, b)
    assert torch.allclose(a.cpu(), (G.double().t() @ X.double()).float().cpu(), rtol=1e-3, atol=0.05)


def test_segment_sum():
    x = torch.randn(1000, dtype=torch.float64, generator=torch.Generator().manual_seed(0))
    ptr = torch.tensor([0, 0, 10, 500, 500, 1000])
    assert torch.allclose(get_backend().segment_sum(x.to(DEV), ptr.to(DEV)).cpu(), ORA.segment_sum(x, ptr))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_prior_terms(dtype):
    from helpers import prior_setup
    data, priors = prior_setup(30, 5, 4, torch.Generator().manual_seed(0))
    pos = data.pos.to(dtype)
    for kind, name in enumerate(["bonds", "angles", "dihedrals", "repulsion"]):
        p = priors[name]
        nl = data.neighbor_list[name]
        params = p._params(data).to(dtype)
        e_ref, g_ref = ORA.prior_terms(kind, pos, nl["index_mapping"], nl["mapping_batch"], params, 5)
        e, g = get_backend().prior_terms(kind, pos.to(DEV), nl["index_mapping"].to(DEV), nl["mapping_batch"].to(DEV), params.to(DEV), 5)
        rt = 1e-10 if dtype == torch.float64 else 2e-5
        assert torch.allclose(e.cpu(), e_ref, rtol=rt), name
        assert torch.allclose(g.cpu(), g_ref, rtol=10 * rt, atol=rt * float(g_ref.abs().max())), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_edge_distance_and_its_backward(dtype):
    gen = torch.Generator().manual_seed(7)
    N = 150
    ei = random_graph(N, 8, gen)
    ei = ei[:, ei[0] != ei[1]]
    plan = ag.EdgePlan.from_edge_index(ei, N)
    pos = torch.randn(N, 3, dtype=dtype, generator=gen) * 3
    g = torch.randn(ei.shape[1], dtype=dtype, generator=gen)
    be = get_backend()
    d = be.edge_distance(pos.to(DEV), plan.row0.to(DEV), plan.row1.to(DEV))
    assert torch.allclose(d.cpu(), ORA.edge_distance(pos, plan.row0, plan.row1), **tol(dtype))
    import copy
    gplan = copy.copy(plan)
    for f in ("row0", "row1", "ptr_in", "perm_in", "ptr_out", "nbr_in", "nbr_out"):
        setattr(gplan, f, getattr(plan, f).to(DEV))
    gplan.perm_out = None if plan.perm_out is None else plan.perm_out.to(DEV)
    got = be.edge_distance_backward(pos.to(DEV), g.to(DEV), d, gplan)
    p = pos.clone().requires_grad_(True)
    (want,) = torch.autograd.grad((ORA.edge_distance(p, plan.row0, plan.row1) * g).sum(), p)
    assert torch.allclose(got.cpu(), want, rtol=1e-4 if dtype == torch.float32 else 1e-10, atol=1e-4 if dtype == torch.float32 else 1e-10)


@pytest.mark.parametrize("M,N,K", [(1000, 128, 128), (333, 128, 50), (5000, 50, 128), (128, 128, 128), (77, 64, 33), (40000, 128, 128)])
@pytest.mark.parametrize("heavy_tail", [False, True])
def test_tensor_core_gemm_matches_float64(M, N, K, heavy_tail):
    """The tcgen05 GEMMs (fp16 hi/lo pairs) against float64 products, rows spanning many orders of magnitude."""
    gen = torch.Generator().manual_seed(M + N + K)
    be = get_backend()
    assert be.tensor_core_gemm
    rows = torch.exp(torch.randn(M, 1, generator=gen) * (6.0 if heavy_tail else 0.0))
    X = torch.randn(M, K, generator=gen) * rows
    W = torch.randn(N, K, generator=gen) * 0.1
    b = torch.randn(N, generator=gen)
    def rel(got, want):
        return float(((got.cpu().double() - want).abs() / (want.abs().amax(dim=1, keepdim=True) + 1e-30)).max())
    want = X.double() @ W.double().t() + b.double()
    assert rel(be.gemm(0, X.to(DEV), W.to(DEV), b.to(DEV)), want) < 5e-6
    G = torch.randn(M, N, generator=gen) * rows
    assert rel(be.gemm(1, G.to(DEV), W.to(DEV)), G.double() @ W.double()) < 5e-6
    want_t = G.double().t() @ X.double()
    got_t = be.gemm(2, G.to(DEV), X.to(DEV)).cpu().double()
    assert float((got_t - want_t).abs().max()) < 2e-5 * float(want_t.abs().max())
    get_backend().check_pending()
    # and the CUDA-core kernel gives the same answers when the tensor-core route is switched off
    be.tensor_core_gemm = False
    try:
        assert rel(be.gemm(0, X.to(DEV), W.to(DEV), b.to(DEV)), want) < 5e-6
    finally:
        be.tensor_core_gemm = True


@pytest.mark.parametrize("M,N,K", [(1000, 128, 128), (128, 128, 128), (5003, 64, 128), (700, 128, 64)])
def test_tensor_core_gemm_fused_epilogues(M, N, K):
    """The epilogues of the pipelined row-wise GEMM (tanh, + aux, * (1 - aux^2)) against float64, both operand layouts."""
    gen = torch.Generator().manual_seed(M + N + K)
    be = get_backend()
    X = torch.randn(M, K, generator=gen)
    W = torch.randn(N, K, generator=gen) * 0.1          # mode 0: X W^T
    V = torch.randn(K, N, generator=gen) * 0.1          # mode 1: X V
    b = torch.randn(N, generator=gen) * 0.5
    aux = torch.tanh(torch.randn(M, N, generator=gen))
    assert be.gemm_fused_ok(0, X.to(DEV), W.to(DEV)) and be.gemm_fused_ok(1, X.to(DEV), V.to(DEV))
    lin0 = X.double() @ W.double().t() + b.double()
    lin1 = X.double() @ V.double()
    a64 = aux.double()
    cases = [(0, W, b, None, be.EPI_NONE, lin0), (0, W, b, None, be.EPI_TANH, torch.tanh(lin0)), (0, W, b, aux, be.EPI_ADD, lin0 + a64),
             (0, W, b, aux, be.EPI_TANH_GRAD, lin0 * (1 - a64 * a64)), (1, V, None, None, be.EPI_NONE, lin1),
             (1, V, None, aux, be.EPI_ADD, lin1 + a64), (1, V, None, aux, be.EPI_TANH_GRAD, lin1 * (1 - a64 * a64))]
    # input transform: A' = vec * (1 - A^2) with a vector over the columns of A (A = a tanh layer's output)
    T = torch.tanh(X)
    vec = torch.randn(K, generator=gen)
    Tp = vec.double() * (1 - T.double() ** 2)
    cases += [(1, V, None, vec, be.EPI_IN_TANH_GRAD_VEC, Tp @ V.double()), (0, W, b, vec, be.EPI_IN_TANH_GRAD_VEC, Tp @ W.double().t() + b.double())]
    for mode, B, bias, ax, epi, want in cases:
        A_in = T if epi == be.EPI_IN_TANH_GRAD_VEC else X
        got = be.gemm_fused(mode, A_in.to(DEV), B.to(DEV), None if bias is None else bias.to(DEV), None if ax is None else ax.to(DEV), epi)
        err = float((got.cpu().double() - want).abs().max())
        assert err < 5e-6 * max(1.0, float(want.abs().max())), (mode, epi, err)
    get_backend().check_pending()


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
@pytest.mark.parametrize("E,F", [(1000, 128), (37, 50), (0, 128), (5000, 64)])
def test_row_scale_and_row_dot(dtype, E, F):
    gen = torch.Generator().manual_seed(E + F)
    a, b, c = torch.randn(E, F, generator=gen, dtype=dtype), torch.randn(E, F, generator=gen, dtype=dtype), torch.randn(E, generator=gen, dtype=dtype)
    be = get_backend()
    assert torch.equal(be.row_scale(a.to(DEV), c.to(DEV)).cpu(), ORA.row_scale(a, c))
    tol = 1e-5 if dtype == torch.float32 else 1e-13
    assert torch.allclose(be.row_dot(a.to(DEV), b.to(DEV)).cpu(), ORA.row_dot(a, b), rtol=tol, atol=tol * F ** 0.5)


@pytest.mark.parametrize("K,M,N", [(40000, 128, 128), (1000, 128, 64), (333, 1, 128), (129, 64, 128)])
def test_weight_and_bias_gradient_in_one_pass(K, M, N):
    gen = torch.Generator().manual_seed(K + M + N)
    G = torch.randn(K, M, generator=gen) * torch.exp(torch.randn(K, 1, generator=gen))
    X = torch.randn(K, N, generator=gen)
    P, s = get_backend().gemm_tn_colsum(G.to(DEV), X.to(DEV))
    want_P, want_s = G.double().t() @ X.double(), G.double().sum(0)
    assert float((P.cpu().double() - want_P).abs().max()) < 2e-5 * float(want_P.abs().max())
    assert float((s.cpu().double() - want_s).abs().max()) < 1e-5 * float(G.abs().sum(0).max())
    get_backend().check_pending()


@pytest.mark.parametrize("M", [128, 1000, 51200])
def test_two_chained_layers_equal_two_fused_gemms(M):
    """mlcgb_gemm_tc_chain2 (the tail of an interaction block and its part of the force pass in one kernel, schnet.py:252-262
    with the residual sum at :150) against two calls of mlcgb_gemm_tc_fused — the same arithmetic, so bit for bit — and against
    float64."""
    gen = torch.Generator().manual_seed(M)
    be = get_backend()
    r = lambda *s: torch.randn(*s, generator=gen)
    A, X = r(M, 128).to(DEV), r(M, 128).to(DEV)
    Wa, Wb = (r(128, 128) / 11).to(DEV), (r(128, 128) / 11).to(DEV)
    ba, bb = (0.1 * r(128)).to(DEV), (0.1 * r(128)).to(DEV)
    mid, out = be.gemm_chain2(False, A, Wa, ba, Wb, bb, X)
    mid2 = be.gemm_fused(0, A, Wa, ba, None, 1)
    out2 = be.gemm_fused(0, mid2, Wb, bb, X, 2)
    assert torch.equal(mid, mid2) and torch.equal(out, out2)
    mid64 = torch.tanh(A.double() @ Wa.double().t() + ba.double())
    out64 = X.double() + mid64 @ Wb.double().t() + bb.double()
    assert float((mid.double() - mid64).abs().max()) < 5e-6 and float((out.double() - out64).abs().max()) < 1e-5
    # force pass: g -> (g W3) * (1 - a^2) -> . W2
    G = r(M, 128).to(DEV)
    _, gagg = be.gemm_chain2(True, G, Wb, None, Wa, None, mid)
    gy2 = be.gemm_fused(1, G, Wb, None, mid, 3)
    gagg2 = be.gemm_fused(1, gy2, Wa, None, None, 0)
    assert torch.equal(gagg, gagg2)
    g64 = ((G.double() @ Wb.double()) * (1 - mid64 ** 2)) @ Wa.double()
    assert float((gagg.double() - g64).abs().max()) < 1e-5 * max(1.0, float(g64.abs().max()))
    get_backend().check_pending()


@pytest.mark.parametrize("with_perm", [False, True])
def test_seg_mul_sum_rows_of_every_length(with_perm):
    """The float32 / 128-feature kernel (rows of V through a ring of asynchronous copies, sixteen per warp in flight): rows with
    no edge, fewer than a group of four, exactly 16, 17, 32, 33 and 100 edges, rows of V shared between edges; against the
    oracle and run to run."""
    gen = torch.Generator().manual_seed(5 + int(with_perm))
    degs = [0, 1, 2, 3, 4, 5, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 0, 7] * 9
    N = len(degs)
    ptr = torch.tensor([0] + degs).cumsum(0)
    E = int(ptr[-1])
    nbr = torch.cat([torch.randperm(N, generator=gen)[:d].sort().values if d <= N else torch.randint(0, N, (d,), generator=gen) for d in degs]).to(torch.int32)
    a = torch.randn(N, 128, generator=gen)
    P = E if not with_perm else E // 2 + 1
    V = torch.randn(P, 128, generator=gen)
    perm = torch.randint(0, P, (E,), generator=gen).to(torch.int32) if with_perm else None
    be = get_backend()
    dev = lambda t: None if t is None else t.to(DEV)
    got = be.seg_mul_sum(dev(a), dev(V), dev(ptr), dev(nbr), dev(perm), N)
    want = ORA.seg_mul_sum(a, V, ptr, nbr, perm, N)
    assert torch.allclose(got.cpu(), want, rtol=1e-5, atol=1e-4)
    assert not got[torch.tensor(degs) == 0].any()
    assert torch.equal(got, be.seg_mul_sum(dev(a), dev(V), dev(ptr), dev(nbr), dev(perm), N))


@pytest.mark.parametrize("dtype", [torch.float32, torch.float64])
def test_pair_family_is_closed_under_differentiation(dtype):
    """SegPair / PairMul (filters stored once per unordered pair) against SegIn / EdgeMul on the same symmetric list with every
    pair's row copied to both of its edges: values, first and second derivatives."""
    from mlcg_b200 import autograd as ag2
    gen = torch.Generator().manual_seed(9)
    B, n = 3, 12
    pos = torch.cat([torch.randn(n, 3, generator=gen) * 2.0 for _ in range(B)]).to(DEV)
    ptr = (torch.arange(B + 1) * n).to(DEV)
    res = get_backend().radius_graph(pos, ptr, 3.0, 1000, False, 1)
    row0, row1 = res["edge_index"][0].to(torch.int32), res["edge_index"][1].to(torch.int32)
    plan = ag2.EdgePlan.from_centre_sorted(row0.contiguous(), row1.contiguous(), res["offsets"], B * n, symmetric=True)
    P = plan.E // 2
    assert plan.half_selection() is not None and P > 10
    a = torch.randn(B * n, 16, dtype=dtype, generator=gen).to(DEV).requires_grad_(True)
    Vp = torch.randn(P, 16, dtype=dtype, generator=gen).to(DEV).requires_grad_(True)
    Ve = Vp[plan.pair_index().long()]                          # the same rows, one copy per directed edge
    out_p = ag2.SegPair.apply(a, Vp, plan)
    out_e = ag2.SegIn.apply(a, Ve, plan, True)
    t = dict(rtol=1e-5, atol=1e-5) if dtype == torch.float32 else dict(rtol=1e-12, atol=1e-12)
    assert torch.allclose(out_p, out_e, **t)
    w = torch.randn(B * n, 16, dtype=dtype, generator=gen).to(DEV)
    ga_p, gV_p = torch.autograd.grad((out_p * w).sum(), [a, Vp], create_graph=True)
    ga_e, gV_e = torch.autograd.grad((out_e * w).sum(), [a, Vp], create_graph=True)
    assert torch.allclose(ga_p, ga_e, **t) and torch.allclose(gV_p, gV_e, **t)
    u = torch.randn(P, 16, dtype=dtype, generator=gen).to(DEV)
    gg_p = torch.autograd.grad((gV_p * u).sum(), [a])[0]
    gg_e = torch.autograd.grad((gV_e * u).sum(), [a])[0]
    assert torch.allclose(gg_p, gg_e, **t)
    if dtype == torch.float64:
        a2 = torch.randn(B * n, 4, dtype=dtype, generator=gen).to(DEV).requires_grad_(True)
        V2 = torch.randn(P, 4, dtype=dtype, generator=gen).to(DEV).requires_grad_(True)
        assert torch.autograd.gradcheck(lambda x, v: ag2.SegPair.apply(x, v, plan), (a2, V2))
        assert torch.autograd.gradgradcheck(lambda x, v: ag2.SegPair.apply(x, v, plan), (a2, V2))
        d = torch.rand(plan.E, dtype=dtype, generator=gen).to(DEV).requires_grad_(True)
        assert torch.autograd.gradcheck(lambda x: ag2.PairSelect.apply(x, plan), (d,))
        assert torch.autograd.gradgradcheck(lambda x: ag2.PairSelect.apply(x, plan), (d,))


def test_tanh_operator_derivatives():
    """autograd.Tanh (derivatives as single kernels, mlcgb_tanh_grad) against torch.tanh: value, first, second and third
    derivative in float64 (gradcheck / gradgradcheck) and float32 values."""
    from mlcg_b200 import autograd as ag2
    gen = torch.Generator().manual_seed(21)
    x = (2 * torch.randn(37, 12, dtype=torch.float64, generator=gen)).to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(ag2.Tanh.apply, (x,))
    assert torch.autograd.gradgradcheck(ag2.Tanh.apply, (x,))
    w = torch.randn(37, 12, dtype=torch.float64, generator=gen).to(DEV)
    for fn in (ag2.Tanh.apply, torch.tanh):
        y = fn(x)
        (g1,) = torch.autograd.grad((y * w).sum(), x, create_graph=True)
        (g2,) = torch.autograd.grad((g1 * w).sum(), x, create_graph=True)
        (g3,) = torch.autograd.grad((g2 * w).sum(), x)
        if fn is torch.tanh:
            assert torch.allclose(ours[0], g1, rtol=1e-12, atol=1e-12) and torch.allclose(ours[1], g2, rtol=1e-12, atol=1e-12)
            assert torch.allclose(ours[2], g3, rtol=1e-11, atol=1e-11)
        else:
            ours = (g1.detach(), g2.detach(), g3.detach())
    x32 = (2 * torch.randn(1000, 128, generator=gen)).to(DEV).requires_grad_(True)       # the vectorised float32 kernels
    w32 = torch.randn(1000, 128, generator=gen).to(DEV)
    res = []
    for fn in (ag2.tanh, torch.tanh):
        (g1,) = torch.autograd.grad((fn(x32) * w32).sum(), x32, create_graph=True)
        (g2,) = torch.autograd.grad((g1 * w32).sum(), x32)
        res.append((g1.detach(), g2))
    assert torch.allclose(res[0][0], res[1][0], rtol=1e-5, atol=1e-6) and torch.allclose(res[0][1], res[1][1], rtol=1e-5, atol=1e-6)
