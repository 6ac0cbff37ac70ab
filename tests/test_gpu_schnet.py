"""The SchNet energy / force path on the GPU against the reference fixtures and the CPU oracle.

Tolerances are the ones the build targets for float32: energies 1e-5 relative, forces 1e-4 kcal/mol/A absolute."""
import numpy as np
import pytest
import torch

import mlcg_b200
from mlcg_b200 import nn as bnn
from oracle import radius_ref, schnet_ref

from helpers import (attentive_schnet_from_case, data_from_case, fullwidth_case, periodic_prior_cases, prior_setup, random_walk_chain, regularized_schnet_from_case,
                     schnet_from_case)

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
E_RTOL, F_ATOL = 1e-5, 1e-4
CASES = ["schnet_gaussian_f32", "schnet_expnormal_f32", "schnet_expnormal_trainable_f64"]


@pytest.mark.parametrize("name", CASES)
def test_golden_energy_forces(golden, name):
    c = golden[name]
    model = bnn.GradientsOut(schnet_from_case(c, device=DEV), "forces").eval()
    out = model(data_from_case(c, device=DEV))
    f64 = c["pos"].dtype == torch.float64
    assert torch.allclose(out.out["SchNet"]["energy"].cpu(), c["energy"], rtol=1e-10 if f64 else E_RTOL, atol=1e-10 if f64 else 1e-5)
    assert torch.allclose(out.out["SchNet"]["forces"].cpu(), c["forces"], rtol=0, atol=1e-9 if f64 else F_ATOL)


@pytest.mark.parametrize("name", CASES)
def test_golden_force_matching_gradients(golden, name):
    c = golden[name]
    net = schnet_from_case(c, device=DEV)
    out = bnn.GradientsOut(net, "forces").train()(data_from_case(c, device=DEV))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"].to(DEV))
    loss.backward()
    f64 = c["pos"].dtype == torch.float64
    assert torch.allclose(loss.detach().cpu(), c["loss"], rtol=1e-9 if f64 else 1e-5)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        tol_ = 1e-8 if f64 else 1e-4
        assert torch.allclose(grads[k].grad.cpu(), g, rtol=tol_, atol=tol_ * float(g.abs().max() + 1e-30)), k


@pytest.mark.parametrize("box", ["orthorhombic", "slab", "triclinic"])
def test_golden_priors_on_periodic_data(golden_priors_periodic, box):
    """The four priors on structures whose bonded terms and pairs cross a periodic box, against the reference."""
    c, cases = periodic_prior_cases(golden_priors_periodic, box, device=DEV)
    for k, p, data in cases:
        o = bnn.GradientsOut(p, "forces").eval()(data)
        assert torch.allclose(o.out[k]["energy"].cpu(), c["energy"][k], rtol=2e-5), k
        assert torch.allclose(o.out[k]["forces"].cpu(), c["forces"][k], rtol=1e-4, atol=1e-4 * float(c["forces"][k].abs().max())), k


FULLWIDTH_EVAL = ["chain100", "chain10", "chain268", "chain73"]


def _report(tag, e, f, c):
    """Prints the measured distances and checks the float32 bars against the reference: forces within 1e-4 kcal/mol/A of the
    reference's double-precision value and of its float32 value (up to that value's own rounding); energies within 1e-5 relative of
    the double-precision value, plus the largest distance of the reference's own float32 energies from it over the case (a
    structure whose energy nearly cancels cannot be met to 1e-5 of its own size by any float32 evaluation)."""
    e64, f64 = c["energy_f64"], c["forces_f64"]
    ours_e, ref_e = (e.double() - e64).abs(), (c["energy"].double() - e64).abs()
    ours_f, ref_f = float((f.double() - f64).abs().max()), float((c["forces"].double() - f64).abs().max())
    print(f"{tag}: |E| {float(e64.abs().min()):.3f}..{float(e64.abs().max()):.3f}, max |dE| vs f64 {float(ours_e.max()):.2e} (reference f32: {float(ref_e.max()):.2e}), "
          f"max |dE|/|E| {float((ours_e / e64.abs()).max()):.2e} (reference f32: {float((ref_e / e64.abs()).max()):.2e}); max |F| {float(f64.abs().max()):.2f}, "
          f"max |dF| vs f64 {ours_f:.2e} (reference f32: {ref_f:.2e}), vs reference f32 {float((f - c['forces']).abs().max()):.2e}")
    assert bool((ours_e <= E_RTOL * e64.abs() + float(ref_e.max())).all()), tag
    assert ours_f < F_ATOL, tag
    assert float((f - c["forces"]).abs().max()) < F_ATOL + ref_f, tag


@pytest.mark.parametrize("name", FULLWIDTH_EVAL)
def test_fullwidth_golden_fused_routes(golden_fullwidth, name):
    """The routes the benchmark times — the one-call evaluation (``mlcgb_schnet_eval``) and the fused tensor-core kernels launched
    one by one — against energies and forces produced by the reference's own modules at the same widths (hidden = filters = 128,
    128 exp-normal / 50 Gaussian functions): energies to 1e-5 relative, forces to 1e-4 kcal/mol/A."""
    from mlcg_b200.backend import KernelProfiler, get_backend
    c = fullwidth_case(golden_fullwidth, name)
    net = schnet_from_case(c, device=DEV)
    model = bnn.GradientsOut(net, "forces").eval()
    be = get_backend()
    assert c["B"] * c["n"] >= 128 and net.packed_weights() is not None and net._whole_model_setup(c["pos"].to(DEV)) is not None
    nl = mlcg_b200.atomic_data2neighbor_list(data_from_case(c, device=DEV), c["upper"])
    assert torch.equal(nl["index_mapping"].cpu(), c["edge_index"])                      # the reference's edge list, in its order
    out = model(data_from_case(c, device=DEV))                                           # one library call per evaluation
    e1, f1 = out.out["SchNet"]["energy"].cpu(), out.out["SchNet"]["forces"].cpu()
    be.profiler = KernelProfiler(time_kernels=False)                                     # per-kernel route: each launch is counted
    try:
        out = model(data_from_case(c, device=DEV))
        ran = set(be.profiler.stats)
    finally:
        be.profiler = None
    be.check_pending()
    assert {"filter_forward", "filter_backward", "seg_mul_sum", "gemm_tc"} <= ran and "gemm" not in ran and "rbf_expand" not in ran, ran
    e2, f2 = out.out["SchNet"]["energy"].cpu(), out.out["SchNet"]["forces"].cpu()
    for tag, e, f in ((f"{name} one-call", e1, f1), (f"{name} per-kernel", e2, f2)):
        _report(tag, e, f, c)


@pytest.mark.parametrize("name", ["chain100", "chain10", "chain73", "chain73_trainable"])
def test_fullwidth_golden_force_matching_step(golden_fullwidth, name):
    """Force-matching loss and its parameter gradients (second-order pass) at full width against the reference's."""
    from mlcg_b200.backend import KernelProfiler, get_backend
    c = fullwidth_case(golden_fullwidth, name)
    net = schnet_from_case(c, device=DEV)
    be = get_backend()
    be.profiler = KernelProfiler(time_kernels=False)
    try:
        out = bnn.GradientsOut(net, "forces").train()(data_from_case(c, device=DEV))
        _report(f"{name} training-mode forward", out.out["SchNet"]["energy"].detach().cpu(), out.out["SchNet"]["forces"].detach().cpu(), c)
        loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"].to(DEV))
        loss.backward()
        ran = set(be.profiler.stats)
    finally:
        be.profiler = None
    get_backend_check()
    # the basis runs on the kernels whether or not its parameters are trained; trained ones get their gradients from the
    # reduction kernel (the reference's default is ExpNormalBasis(trainable=True), exp_normal.py:52)
    assert {"rbf_expand", "rbf_contract"} <= ran, ran
    assert ("rbf_param_contract" in ran) == name.endswith("_trainable"), ran
    # the list is symmetric and loop-free: basis, filter network and their derivatives ran on one row per unordered pair
    assert "pair_mul" in ran and "edge_mul" not in ran, ran
    assert torch.allclose(loss.detach().cpu(), c["loss"], rtol=1e-5)
    grads = dict(net.named_parameters())
    worst = 0.0
    for k, g in c["param_grads"].items():
        assert grads[k].grad is not None, k
        err = float((grads[k].grad.cpu() - g).abs().max() / (g.abs().max() + 1e-30))
        worst = max(worst, err)
        assert err < 2e-4, (k, err)
    print(f"{name}: loss {float(loss):.6f} vs {float(c['loss']):.6f}; worst parameter-gradient error {worst:.2e} of the gradient's maximum")


def get_backend_check():
    from mlcg_b200.backend import get_backend
    get_backend().check_pending()


@pytest.mark.parametrize("name", ["shared", "independent"])
def test_golden_rbf_regularized_schnet(golden_regularized, name):
    """`RBFRegularizedSchNet` on the device against the reference's energies, forces and force-matching gradients."""
    c = golden_regularized[name]
    net = regularized_schnet_from_case(c, device=DEV)
    out = bnn.GradientsOut(net, "forces").eval()(data_from_case(c, device=DEV))
    assert torch.allclose(out.out["SchNet"]["energy"].cpu(), c["energy"], rtol=E_RTOL, atol=1e-5)
    assert torch.allclose(out.out["SchNet"]["forces"].cpu(), c["forces"], rtol=0, atol=F_ATOL)
    out = bnn.GradientsOut(net, "forces").train()(data_from_case(c, device=DEV))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"].to(DEV))
    loss.backward()
    assert torch.allclose(loss.detach().cpu(), c["loss"], rtol=1e-5)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        assert torch.allclose(grads[k].grad.cpu(), g, rtol=1e-4, atol=1e-4 * float(g.abs().max() + 1e-30)), k


@pytest.mark.parametrize("name", ["orthorhombic", "slab", "triclinic"])
def test_golden_periodic_structures(golden_periodic, name):
    """SchNet on periodic structures (graph over the periodic copies, distances with cell shifts) against the reference."""
    c = golden_periodic[name]
    cut = bnn.CosineCutoff(0.0, c["upper"])
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, c["R"], trainable=False), cut, [c["H"]], hidden_channels=c["H"], embedding_size=c["T"],
                             num_filters=c["H"], num_interactions=c["L"])
    net.load_state_dict(c["state_dict"])
    data = mlcg_b200.AtomicData(pos=c["pos"].to(DEV), atom_types=c["atom_types"].to(DEV), batch=c["batch"].to(DEV),
                                n_atoms=torch.full((c["B"],), c["n"]).to(DEV), cell=c["cells"].to(DEV), pbc=c["pbc"].to(DEV))
    out = bnn.GradientsOut(net.to(DEV), "forces").eval()(data)
    assert torch.allclose(out.out["SchNet"]["energy"].cpu(), c["energy"], rtol=E_RTOL, atol=1e-5)
    assert torch.allclose(out.out["SchNet"]["forces"].cpu(), c["forces"], rtol=0, atol=F_ATOL)


@pytest.mark.parametrize("name", ["normal_exact", "v2_favor", "normal_favor_single"])
def test_golden_attentive_schnet(golden_attentive, name):
    """`AttentiveSchNet` on the device against the reference's energies, forces and force-matching loss."""
    c = golden_attentive[name]
    net = attentive_schnet_from_case(c, device=DEV)
    out = bnn.GradientsOut(net, "forces").eval()(data_from_case(c, device=DEV))
    assert torch.allclose(out.out["SchNet"]["energy"].cpu(), c["energy"], rtol=E_RTOL, atol=2e-5)
    assert torch.allclose(out.out["SchNet"]["forces"].cpu(), c["forces"], rtol=0, atol=F_ATOL)
    out = bnn.GradientsOut(net, "forces").train()(data_from_case(c, device=DEV))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], c["target_forces"].to(DEV))
    loss.backward()
    assert torch.allclose(loss.detach().cpu(), c["loss"], rtol=2e-5)
    grads = dict(net.named_parameters())
    for k, g in c["param_grads"].items():
        assert torch.allclose(grads[k].grad.cpu(), g, rtol=2e-3, atol=2e-4 * float(g.abs().max() + 1e-30)), k


def _make(kind, B, n, n_types, upper, R, H, L, seed, min_dist=None, jitter=0.0):
    torch.manual_seed(seed)
    cut = bnn.CosineCutoff(0.0, upper)
    rbf = bnn.GaussianBasis(cut, R) if kind == "gaussian" else bnn.ExpNormalBasis(cut, R, trainable=False)
    model = bnn.StandardSchNet(rbf, cut, [H], hidden_channels=H, embedding_size=n_types, num_filters=H, num_interactions=L)
    gen = torch.Generator().manual_seed(seed)
    pos = torch.cat([random_walk_chain(n, gen, jitter=jitter, min_dist=min_dist) for _ in range(B)])
    types_ = torch.randint(0, n_types, (B * n,), generator=gen)
    return model, pos, types_, torch.arange(B).repeat_interleave(n)


def _oracle(model, kind, upper, L, pos, types_, batch, B, dtype=torch.float32):
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": upper}
    spec = {"kind": kind, "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": L}
    sd = {k: v.detach().cpu().to(dtype) if v.is_floating_point() else v.detach().cpu() for k, v in model.state_dict().items()}
    ei = torch.from_numpy(radius_ref.radius_graph_c(pos.numpy(), radius_ref.batch_to_ptr(batch.numpy(), B), upper, 1000, False, "cluster"))
    e, f, _ = schnet_ref.energy_and_forces(lambda p: schnet_ref.schnet_energy(sd, spec, p, types_, batch, ei, B), pos.to(dtype))
    return e, f, ei


@pytest.mark.parametrize("cfg", [
    dict(kind="gaussian", B=64, n=10, n_types=10, upper=30.0, R=50, H=128, L=2, jitter=0.3),            # the CPU-runnable configuration
    dict(kind="expnormal", B=24, n=100, n_types=20, upper=15.0, R=128, H=128, L=3, min_dist=4.0),       # 100-bead chains, 3 blocks
    dict(kind="expnormal", B=8, n=268, n_types=20, upper=12.0, R=128, H=128, L=3),                      # simulation-size chains
])
def test_full_shape_models_vs_oracle(cfg):
    kind, B, n, upper, L = cfg["kind"], cfg["B"], cfg["n"], cfg["upper"], cfg["L"]
    model, pos, types_, batch = _make(kind, B, n, cfg["n_types"], upper, cfg["R"], cfg["H"], L, 0, cfg.get("min_dist"), cfg.get("jitter", 0.0))
    e_ref, f_ref, ei = _oracle(model, kind, upper, L, pos, types_, batch, B)
    # the same float32 weights and positions evaluated in float64: the value both float32 evaluations round towards
    e_x, f_x, _ = _oracle(model, kind, upper, L, pos, types_, batch, B, torch.float64)
    data = mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((B,), n).to(DEV))
    out = bnn.GradientsOut(model.to(DEV), "forces").eval()(data)
    e, f = out.out["SchNet"]["energy"].detach().cpu(), out.out["SchNet"]["forces"].cpu()
    assert torch.allclose(e, e_ref, rtol=E_RTOL, atol=E_RTOL * float(e_ref.abs().max()))
    ref_err = float((f_ref.double() - f_x).abs().max())        # rounding of the float32 CPU reference path itself
    our_err = float((f.double() - f_x).abs().max())
    assert our_err < F_ATOL, (our_err, ref_err)                # forces within 1e-4 kcal/mol/A of the exact value
    assert float((f - f_ref).abs().max()) < F_ATOL + ref_err   # and of the float32 reference, up to that reference's own rounding


def test_gradcheck_on_device_float64():
    """First and second derivatives of the whole energy w.r.t. positions, CUDA kernels in float64."""
    model, pos, types_, batch = _make("expnormal", 2, 7, 4, 9.0, 6, 8, 2, 1, jitter=0.2)
    model = model.double().to(DEV)
    B, n = 2, 7

    def energy(p):
        data = mlcg_b200.AtomicData(pos=p, atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((B,), n).to(DEV))
        return model(data).out["SchNet"]["energy"]

    p = pos.double().to(DEV).requires_grad_(True)
    assert torch.autograd.gradcheck(energy, (p,), eps=1e-6, atol=1e-6, nondet_tol=1e-9)
    assert torch.autograd.gradgradcheck(energy, (p,), eps=1e-6, atol=1e-5, nondet_tol=1e-9)


def test_forces_are_reproducible_run_to_run():
    model, pos, types_, batch = _make("expnormal", 8, 100, 20, 15.0, 64, 64, 2, 3, min_dist=4.0)
    m = bnn.GradientsOut(model.to(DEV), "forces").eval()
    mk = lambda: mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((8,), 100).to(DEV))
    a, b = m(mk()), m(mk())
    assert torch.equal(a.out["SchNet"]["forces"], b.out["SchNet"]["forces"]) and torch.equal(a.out["SchNet"]["energy"], b.out["SchNet"]["energy"])


def test_sumout_of_schnet_and_four_priors_is_reproducible_and_matches_the_parts():
    """SumOut(SchNet + bonds + angles + dihedrals + repulsion) in eval mode: the priors are evaluated together in one launch with
    fixed-point sums.  Two evaluations give bit-identical energies and forces; every component equals what the same prior gives
    on its own (separate launches, floating-point atomics) to rounding; the totals are the sums of the components."""
    from mlcg_b200.nn.prior import evaluate_priors
    data, priors = prior_setup(60, 6, 4, torch.Generator().manual_seed(9))
    with torch.no_grad():      # sigma[a, b] = sigma[b, a], as physical tables are: the (i, j) and (j, i) terms are then equal
        priors["repulsion"].sigma.copy_(0.5 * (priors["repulsion"].sigma + priors["repulsion"].sigma.t()))
    torch.manual_seed(1)
    cut = bnn.CosineCutoff(0.0, 12.0)
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, 32, trainable=False), cut, [128], hidden_channels=128, embedding_size=4, num_filters=128,
                             num_interactions=2)
    models = {"SchNet": bnn.GradientsOut(net, "forces")}
    models.update({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})
    model = bnn.SumOut(torch.nn.ModuleDict(models)).eval().to(DEV)
    data = data.to(DEV)
    assert priors["repulsion"].to(DEV)._cached_list(data)[3] is True           # both (i, j) and (j, i) are listed: no scatter
    assert priors["bonds"].to(DEV)._cached_list(data)[3] is False
    lopsided = bnn.Repulsion({(a, b): {"sigma": 3.0 + a + 0.1 * b} for a in range(4) for b in range(4)}).to(DEV)
    assert lopsided._cached_list(data)[3] is False                              # sigma[a, b] != sigma[b, a]: every term scatters
    def run():
        data.out = {}
        out = model(data)
        return {k: (v["energy"].clone(), v["forces"].clone()) for k, v in out.out.items() if isinstance(v, dict)}, out.out["energy"].clone(), out.out["forces"].clone()
    parts_a, e_a, f_a = run()
    parts_b, e_b, f_b = run()
    assert torch.equal(e_a, e_b) and torch.equal(f_a, f_b)
    for k in parts_a:
        assert torch.equal(parts_a[k][0], parts_b[k][0]) and torch.equal(parts_a[k][1], parts_b[k][1]), k
    assert torch.allclose(e_a, sum(v[0] for v in parts_a.values()), rtol=1e-6)
    assert torch.allclose(f_a, sum(v[1] for v in parts_a.values()), rtol=1e-5, atol=1e-4)
    for k, p in priors.items():           # each prior alone: its own kernel launch, floating-point atomics
        data.out = {}
        alone = bnn.GradientsOut(p, "forces").eval()(data).out[k]
        assert torch.allclose(parts_a[k][0], alone["energy"], rtol=1e-5), k
        scale = float(alone["forces"].abs().max())
        assert float((parts_a[k][1] - alone["forces"]).abs().max()) < 1e-5 * scale + 1e-5, k
    bnn.set_prior_determinism(False)        # the same through floating-point atomics
    try:
        res = evaluate_priors(priors.values(), data)
        for k in priors:
            assert torch.allclose(res[k][0], parts_a[k][0], rtol=1e-5), k
            assert float((-res[k][1] - parts_a[k][1]).abs().max()) < 1e-5 * float(parts_a[k][1].abs().max()) + 1e-5, k
    finally:
        bnn.set_prior_determinism(True)


def test_truncated_neighbour_list_uses_general_plan():
    """max_num_neighbors below the real degree: the graph stops being symmetric and the general edge plan must agree with the oracle."""
    model, pos, types_, batch = _make("gaussian", 4, 40, 5, 12.0, 20, 32, 2, 4, jitter=0.2)
    model.max_num_neighbors = 6
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": 12.0}
    spec = {"kind": "gaussian", "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": 2}
    ei = torch.from_numpy(radius_ref.radius_graph_c(pos.numpy(), radius_ref.batch_to_ptr(batch.numpy(), 4), 12.0, 6, False, "cluster"))
    e_ref, f_ref, _ = schnet_ref.energy_and_forces(lambda p: schnet_ref.schnet_energy(sd, spec, p, types_, batch, ei, 4), pos)
    data = mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((4,), 40).to(DEV))
    out = bnn.GradientsOut(model.to(DEV), "forces").eval()(data)
    assert torch.allclose(out.out["SchNet"]["energy"].cpu(), e_ref, rtol=E_RTOL, atol=1e-5)
    assert float((out.out["SchNet"]["forces"].cpu() - f_ref).abs().max()) < F_ATOL


def test_priors_and_sumout_on_device(golden):
    c = golden["priors_f32"]
    data, priors = prior_setup(12, 2, c["tables"]["bonds"]["x_0"].shape[0], torch.Generator().manual_seed(0))
    for k, p in priors.items():
        p.load_state_dict(c["tables"][k])
    for mode in ("eval", "train"):
        for k, p in priors.items():
            d = mlcg_b200.AtomicData(pos=c["pos"].clone().to(DEV), atom_types=c["atom_types"].to(DEV), batch=c["batch"].to(DEV),
                                     n_atoms=torch.full((c["B"],), 12).to(DEV),
                                     neighbor_list={k: mlcg_b200.make_neighbor_list(k, c["mappings"][k].shape[0], c["mappings"][k].to(DEV), c["mapping_batch"][k].to(DEV))})
            m = bnn.GradientsOut(p.to(DEV), "forces")
            o = (m.eval() if mode == "eval" else m.train())(d)
            assert torch.allclose(o.out[k]["energy"].cpu(), c["energy"][k], rtol=2e-5), (mode, k)
            assert torch.allclose(o.out[k]["forces"].detach().cpu(), c["forces"][k], rtol=1e-4, atol=1e-4 * float(c["forces"][k].abs().max())), (mode, k)


def test_extension_is_the_compute_path():
    """The operators resolve to the CUDA back end of libmlcg_b200.so, not to a substitute."""
    from mlcg_b200 import _lib, backend
    be = backend.get_backend()
    assert be.name == "cuda" and be.lib is _lib.load()


def test_eval_mode_uses_the_fused_tensor_core_path_and_matches_the_composed_operators():
    """Same model, same inputs: eval mode (fused tcgen05 kernels) against training mode (composable operators)."""
    from mlcg_b200.backend import KernelProfiler, get_backend
    model, pos, types_, batch = _make("expnormal", 16, 100, 20, 15.0, 128, 128, 3, 5, min_dist=4.0)
    model = model.to(DEV)
    mk = lambda: mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((16,), 100).to(DEV))
    be = get_backend()
    be.profiler = KernelProfiler(time_kernels=False)
    fused = bnn.GradientsOut(model, "forces").eval()(mk())
    names = set(be.profiler.stats)
    be.profiler = None
    assert {"filter_forward", "filter_backward"} <= names and "gemm" not in names
    composed = bnn.GradientsOut(model, "forces").train()(mk())
    get_backend().check_pending()
    assert torch.allclose(fused.out["SchNet"]["energy"], composed.out["SchNet"]["energy"].detach(), rtol=E_RTOL, atol=1e-5)
    assert float((fused.out["SchNet"]["forces"] - composed.out["SchNet"]["forces"].detach()).abs().max()) < F_ATOL


def test_bf16_filter_mode_force_accuracy():
    """bf16 filter GEMMs: forces within 1e-2 relative RMS of the float32 reference."""
    model, pos, types_, batch = _make("expnormal", 16, 100, 20, 15.0, 128, 128, 3, 6, min_dist=4.0)
    e_ref, f_ref, _ = _oracle(model, "expnormal", 15.0, 3, pos, types_, batch, 16)
    bnn.set_filter_precision(model, "bf16")
    data = mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((16,), 100).to(DEV))
    out = bnn.GradientsOut(model.to(DEV), "forces").eval()(data)
    f = out.out["SchNet"]["forces"].cpu()
    rel_rms = float(((f - f_ref) ** 2).mean().sqrt() / (f_ref ** 2).mean().sqrt())
    assert rel_rms < 1e-2, rel_rms
    assert torch.allclose(out.out["SchNet"]["energy"].detach().cpu(), e_ref, rtol=2e-2, atol=2e-2 * float(e_ref.abs().max()))


def test_force_matching_gradients_full_width_vs_oracle():
    """Second-order pass at the real layer widths (128 filters, 128 RBF: the tensor-core GEMMs are on this path):
    gradient of the force-matching loss w.r.t. every parameter against the CPU oracle in float64."""
    model, pos, types_, batch = _make("expnormal", 6, 40, 8, 12.0, 128, 128, 2, 9, min_dist=4.0)
    B, n = 6, 40
    target = torch.randn(pos.shape, generator=torch.Generator().manual_seed(1))
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": 12.0}
    spec = {"kind": "expnormal", "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": 2}
    sd = {k: (v.detach().double().requires_grad_(True) if v.is_floating_point() else v) for k, v in model.state_dict().items()}
    ei = torch.from_numpy(radius_ref.radius_graph_c(pos.numpy(), radius_ref.batch_to_ptr(batch.numpy(), B), 12.0, 1000, False, "cluster"))
    _, f, _ = schnet_ref.energy_and_forces(lambda p: schnet_ref.schnet_energy(sd, spec, p, types_, batch, ei, B), pos.double(), create_graph=True)
    loss_ref = torch.nn.functional.mse_loss(f, target.double())
    loss_ref.backward()
    net = model.to(DEV)
    out = bnn.GradientsOut(net, "forces").train()(mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV),
                                                                        n_atoms=torch.full((B,), n).to(DEV)))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], target.to(DEV))
    loss.backward()
    from mlcg_b200.backend import get_backend
    get_backend().check_pending()
    assert abs(float(loss) - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    for k, p in net.named_parameters():
        if p.grad is None:
            continue
        g_ref = sd[k].grad
        assert g_ref is not None, k
        err = float((p.grad.cpu().double() - g_ref).abs().max())
        assert err < 2e-4 * float(g_ref.abs().max()) + 1e-7, (k, err, float(g_ref.abs().max()))


def test_ragged_batch_with_isolated_beads_and_no_edges():
    """Structures of different sizes, a single-bead structure, and a batch with no edge at all (cutoff below every distance)."""
    torch.manual_seed(0)
    sizes = [1, 17, 3, 60, 1, 128]
    gen = torch.Generator().manual_seed(2)
    pos = torch.cat([random_walk_chain(n, gen, jitter=0.2) for n in sizes])
    N, B = sum(sizes), len(sizes)
    types_ = torch.randint(0, 6, (N,), generator=gen)
    batch = torch.arange(B).repeat_interleave(torch.tensor(sizes))
    for upper in (9.0, 0.01):
        cut = bnn.CosineCutoff(0.0, upper)
        model = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, 128, trainable=False), cut, [128], hidden_channels=128, embedding_size=6,
                                   num_filters=128, num_interactions=2)
        e_ref, f_ref, ei = _oracle(model, "expnormal", upper, 2, pos, types_, batch, B)
        data = mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.tensor(sizes).to(DEV))
        out = bnn.GradientsOut(model.to(DEV), "forces").eval()(data)
        assert (upper < 1.0) == (ei.shape[1] == 0)   # the second pass has no edge at all
        assert torch.allclose(out.out["SchNet"]["energy"].detach().cpu(), e_ref, rtol=E_RTOL, atol=1e-5)
        assert float((out.out["SchNet"]["forces"].cpu() - f_ref).abs().max()) < F_ATOL
        tr = bnn.GradientsOut(model, "forces").train()(mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV),
                                                                             n_atoms=torch.tensor(sizes).to(DEV)))
        assert float((tr.out["SchNet"]["forces"].detach().cpu() - f_ref).abs().max()) < F_ATOL


def test_condensed_priors_on_the_device():
    """Merged Static priors (specialize_prior.py) through the CUDA prior kernel: same totals as the separate priors."""
    import itertools
    from mlcg_b200.data import collate
    from mlcg_b200.specialize_prior import condense_all_priors_for_simulation
    from helpers import random_walk_chain
    gen = torch.Generator().manual_seed(4)
    T, n, B = 3, 40, 6
    r = lambda: float(torch.rand(1, generator=gen))
    tab2 = lambda: {k: {"k": 50 + 100 * r(), "x_0": 3.5 + 0.6 * r()} for k in itertools.product(range(T), repeat=2)}
    def tab4(nd):
        return {k: {"v_0": r(), "k1s": {f"k1_{i}": r() - 0.5 for i in range(1, nd + 1)}, "k2s": {f"k2_{i}": r() - 0.5 for i in range(1, nd + 1)}}
                for k in itertools.product(range(T), repeat=4)}
    priors = {"bonds_even": bnn.HarmonicBonds(tab2()), "bonds_odd": bnn.HarmonicBonds(tab2()),
              "dih_short": bnn.Dihedral(tab4(2), n_degs=2, name="dih_short"), "dih_long": bnn.Dihedral(tab4(3), n_degs=3, name="dih_long")}
    for k, p in priors.items():
        p.name = k
    idx = torch.arange(n)
    bonds = torch.stack([idx[:-1], idx[1:]])
    dih = torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]])
    per = {"bonds_even": bonds[:, ::2], "bonds_odd": bonds[:, 1::2], "dih_short": dih[:, :10], "dih_long": dih[:, 10:]}
    data_list = [mlcg_b200.AtomicData(pos=random_walk_chain(n, gen, jitter=0.3), atom_types=torch.randint(0, T, (n,), generator=gen),
                                      neighbor_list={k: mlcg_b200.make_neighbor_list(k, m.shape[0], m.clone()) for k, m in per.items()})
                 for _ in range(B)]
    model = bnn.SumOut(torch.nn.ModuleDict({k: bnn.GradientsOut(p, "forces") for k, p in priors.items()})).eval().to(DEV)
    ref = model(collate(data_list).to(DEV))
    cmodel, cdata = condense_all_priors_for_simulation(model.cpu(), data_list)
    out = cmodel.eval().to(DEV)(collate(cdata).to(DEV))
    assert set(cmodel.models.keys()) == {"bonds", "dihedrals"}
    assert torch.allclose(out.out["energy"], ref.out["energy"], rtol=1e-5)
    assert torch.allclose(out.out["forces"], ref.out["forces"], rtol=1e-4, atol=1e-4 * float(ref.out["forces"].abs().max()))


def test_condensed_priors_equal_the_reference_s_on_the_device(golden_condensed_priors):
    """The merged model of the reference's own specialize_prior.py (fixture `reference_vectors_condensed_priors.pt`) against this
    package's merged model on the device: through the one-launch evaluation of all priors (eval mode, both summation modes)
    and through the per-prior kernel route (train mode)."""
    from helpers import condensed_prior_case
    from mlcg_b200.data import collate
    from mlcg_b200.specialize_prior import condense_all_priors_for_simulation
    g = golden_condensed_priors
    model, data_list = condensed_prior_case(g)
    cmodel, cdata = condense_all_priors_for_simulation(model, data_list)
    cmodel = cmodel.to(DEV)
    fscale = float(g["forces"].abs().max())
    runs = []
    for mode in (True, False):
        bnn.set_prior_determinism(mode)
        try:
            runs.append(cmodel.eval()(collate(cdata).to(DEV)))
        finally:
            bnn.set_prior_determinism(True)
    runs.append(cmodel.train()(collate(cdata).to(DEV)))
    for out in runs:
        assert torch.allclose(out.out["energy"].detach().cpu(), g["energy"], rtol=1e-5)
        assert float((out.out["forces"].detach().cpu() - g["forces"]).abs().max()) < 1e-4 * max(fscale, 1.0)
        for k, e in g["per_model_energy"].items():
            assert torch.allclose(out.out[k]["energy"].detach().cpu(), e, rtol=1e-5, atol=1e-4)


def test_whole_model_call_matches_the_individual_kernels():
    """`mlcgb_schnet_eval` (one library call per evaluation) issues the same edge kernels as the per-kernel path; only the
    output network differs in its arithmetic (fused tanh epilogue, fp32 dot product for the last layer), so the two agree to
    rounding.  With a profiler attached the package launches the kernels one by one."""
    from mlcg_b200.backend import KernelProfiler, get_backend
    model, pos, types_, batch = _make("expnormal", 8, 100, 20, 15.0, 128, 128, 3, 7, min_dist=4.0)
    model = bnn.GradientsOut(model.to(DEV), "forces").eval()
    mk = lambda: mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((8,), 100).to(DEV))
    be = get_backend()
    assert be.profiler is None
    assert model.model.packed_weights() is not None
    whole = model(mk())
    be.profiler = KernelProfiler(time_kernels=False)
    try:
        parts = model(mk())
        assert {"filter_forward", "filter_backward", "seg_mul_sum", "gemm_tc"} <= set(be.profiler.stats)
    finally:
        be.profiler = None
    be.check_pending()
    e_w, e_p = whole.out["SchNet"]["energy"], parts.out["SchNet"]["energy"]
    f_w, f_p = whole.out["SchNet"]["forces"], parts.out["SchNet"]["forces"]
    assert torch.allclose(e_w, e_p, rtol=2e-6, atol=2e-6 * float(e_p.abs().max()))
    assert float((f_w - f_p).abs().max()) < 2e-5
    # energies only (positions without requires_grad): no force pass, same energies
    with torch.no_grad():
        e_only = model.model(mk()).out["SchNet"]["energy"]
    assert torch.equal(e_only, e_w)
    # weights moved or changed in place are picked up
    with torch.no_grad():
        model.model.output_network.layers[2].weight.mul_(2.0)
    doubled = model(mk())
    assert torch.allclose(doubled.out["SchNet"]["energy"], 2.0 * e_w, rtol=1e-5, atol=1e-5 * float(e_w.abs().max()))
    assert torch.allclose(doubled.out["SchNet"]["forces"], 2.0 * f_w, rtol=1e-4, atol=2e-5)


def test_neighbour_list_is_rebuilt_for_every_evaluation():
    """A data object evaluated again after its positions moved gets a new radius graph (the list built on the fly is not kept
    in the data object, src/mlcg/nn/schnet.py:134-141), on the one-call route and on the per-kernel route."""
    from mlcg_b200.backend import KernelProfiler, get_backend
    model, pos, types_, batch = _make("expnormal", 4, 100, 20, 15.0, 128, 128, 2, 11, min_dist=4.0)
    model = bnn.GradientsOut(model.to(DEV), "forces").eval()
    mk = lambda p: mlcg_b200.AtomicData(pos=p.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((4,), 100).to(DEV))
    moved = pos.clone()
    moved[::7] += 6.0            # changes the edge set
    be = get_backend()
    for profiled in (False, True):
        be.profiler = KernelProfiler(time_kernels=False) if profiled else None
        try:
            data = mk(pos)
            first = model(data).out["SchNet"]["forces"].clone()
            assert "SchNet" not in data.neighbor_list
            data.pos = moved.to(DEV)
            data.out = {}
            second = model(data).out["SchNet"]["forces"]
            fresh = model(mk(moved)).out["SchNet"]["forces"]
        finally:
            be.profiler = None
        assert torch.equal(second, fresh)
        assert float((first - fresh).abs().max()) > 1e-3


def test_fixed_edge_capacity_evaluation():
    """With a fixed edge capacity the evaluation reads nothing on the host (`mlcgb_radius_graph_capacity`, `mlcgb_pair_plan`,
    `mlcgb_schnet_eval_counted`); energies and forces equal those of the route that reads the edge count, for capacities
    from exactly the edge count upwards.  A capacity that is too small is reported by the deferred status check."""
    from mlcg_b200.backend import get_backend
    from mlcg_b200.neighbor_list import edge_plan_for
    model, pos, types_, batch = _make("expnormal", 6, 100, 20, 15.0, 128, 128, 3, 5, min_dist=4.0)
    model = bnn.GradientsOut(model.to(DEV), "forces").eval()
    mk = lambda: mlcg_b200.AtomicData(pos=pos.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((6,), 100).to(DEV))
    be = get_backend()
    want = model(mk())
    be.check_pending()
    E = edge_plan_for(mk(), 15.0)[0].E
    for cap in (E, E + 2, E + 1000, 2 * E):
        bnn.set_edge_capacity(model, cap)
        for _ in range(2):                      # second call: the index buffers hold the previous list
            got = model(mk())
        be.check_pending()
        assert torch.equal(got.out["SchNet"]["energy"], want.out["SchNet"]["energy"])
        assert torch.equal(got.out["SchNet"]["forces"], want.out["SchNet"]["forces"])
    bnn.set_edge_capacity(model, E - 2)
    model(mk())
    with pytest.raises(RuntimeError, match="capacity"):
        be.check_pending()
    bnn.set_edge_capacity(model, None)
    again = model(mk())
    be.check_pending()
    assert torch.equal(again.out["SchNet"]["forces"], want.out["SchNet"]["forces"])


def test_evaluation_replayed_from_a_cuda_graph():
    """`GraphedForceField`: the evaluation recorded once (fixed edge capacity, no host read) and replayed for new positions
    gives what the plain call gives for those positions, graph rebuilt inside the replay."""
    from mlcg_b200.backend import get_backend
    from mlcg_b200.neighbor_list import edge_plan_for
    model, pos, types_, batch = _make("expnormal", 4, 100, 20, 15.0, 128, 128, 3, 21, min_dist=4.0)
    model = bnn.GradientsOut(model.to(DEV), "forces").eval()
    mk = lambda p: mlcg_b200.AtomicData(pos=p.to(DEV), atom_types=types_.to(DEV), batch=batch.to(DEV), n_atoms=torch.full((4,), 100).to(DEV))
    E = edge_plan_for(mk(pos), 15.0)[0].E
    moved = [pos, pos + 0.3 * torch.randn(pos.shape, generator=torch.Generator().manual_seed(1)), pos * 1.02]
    want = []
    for p in moved:
        o = model(mk(p))
        want.append((o.out["SchNet"]["energy"].clone(), o.out["SchNet"]["forces"].clone()))
    bnn.set_edge_capacity(model, int(1.3 * E))
    ff = mlcg_b200.GraphedForceField(model, mk(pos))
    for p, (e_w, f_w) in zip(moved, want):
        e, f = ff(p.to(DEV))
        assert torch.equal(e, e_w) and torch.equal(f, f_w)
    ff.check()
    bnn.set_edge_capacity(model, None)
