#!/usr/bin/env python
"""Benchmark of the coarse-grained SchNet hot path: energy + force evaluations per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at every N: 512 structures per GPU of a 100-bead C-alpha chain (3.8 A self-avoiding random
walk, 20 bead types), SchNet with 3 interaction blocks, hidden = filters = 128, 128 exp-normal radial
basis functions, 15 A cosine cutoff, float32; one step = radius graph + energy + forces for the batch.
Prints ONE JSON line (rank 0).

After the timed region the run checks itself: the first 64 structures of the timed batch are evaluated on the host
cores by the CPU arm and the run fails if the energies leave 1e-5 relative or the forces 1e-4 kcal/mol/A.  The
CPU arm is mlcg's own modules (``oracle/_ref/site``, installed by ``oracle/build_ref.py``; torch_geometric's and
torch_cluster's calls replaced by the stand-ins of ``oracle/mlcg_loader.py``) when they are there, else the
restatement in ``oracle/schnet_ref.py``; the same arm, timed, is the ``cpu_baseline`` and ``--impl reference``.
"""
import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "energy+force evaluations per second (structures/s), SchNet CG"
WORKLOAD = dict(workload="cfg2: 100-bead CA chains, 512 structures/GPU, SchNet 3x(H=128,F=128), 128 expnorm RBF, rc=15A, energy+forces",
                structures_per_gpu=512, beads=100, bead_types=20, hidden=128, filters=128, num_rbf=128, interactions=3,
                cutoff_A=15.0, l2="flushed between steps (256 MiB write); edge tensors (>= 500 MB) exceed L2 as well")
E_RTOL, F_ATOL = 1e-5, 1e-4          # float32 parity bars: energies relative, forces kcal/mol/A absolute
KCAL_BETA_300K = 1.0 / (0.0019872041 * 300)


# ----------------------------------------------------------------------------------------- workloads
def self_avoiding_chains(B, n, gen, step=3.8, min_dist=4.0):
    """B chains grown together: a bead is redrawn while it is closer than ``min_dist`` to any bead of its own
    chain except its predecessor; after 200 failed draws the chain steps back five beads."""
    pos = torch.zeros(B, n, 3)
    i = torch.ones(B, dtype=torch.long)
    fails = torch.zeros(B, dtype=torch.long)
    ar = torch.arange(n)
    while bool((i < n).any()):
        act = (i < n).nonzero().flatten()
        ia = i[act]
        v = torch.randn(len(act), 3, generator=gen)
        cand = pos[act, ia - 1] + step * v / v.norm(dim=1, keepdim=True)
        d = (pos[act] - cand[:, None, :]).norm(dim=2)
        considered = ar[None, :] < (ia - 1)[:, None]
        clash = ((d < min_dist) & considered).any(dim=1)
        ok = act[~clash]
        pos[ok, i[ok]] = cand[~clash]
        i[ok] += 1
        fails[ok] = 0
        bad = act[clash]
        fails[bad] += 1
        back = bad[fails[bad] > 200]
        i[back] = torch.clamp(i[back] - 5, min=1)
        fails[back] = 0
    return pos.reshape(B * n, 3)


def random_walks(B, n, gen, step=3.8, jitter=0.0):
    v = torch.randn(B, n, 3, generator=gen)
    pos = torch.cumsum(step * v / v.norm(dim=2, keepdim=True), dim=1)
    if jitter:
        pos = pos + jitter * torch.randn(B, n, 3, generator=gen)
    return pos.reshape(B * n, 3)


def make_inputs(B, n, n_types, seed):
    gen = torch.Generator().manual_seed(seed)
    pos = self_avoiding_chains(B, n, gen)
    types_ = torch.randint(0, n_types, (B * n,), generator=gen)
    batch = torch.arange(B).repeat_interleave(n)
    return pos, types_, batch


def make_model(ns=None, kind="expnormal", cutoff=None, num_rbf=None, interactions=None, n_types=None, seed=0):
    """StandardSchNet of the benchmark's widths from the classes of ``ns`` (this package's ``nn`` by default; the reference's
    namespace for the CPU arm: same constructor)."""
    if ns is None:
        from mlcg_b200 import nn as ns
    cutoff = WORKLOAD["cutoff_A"] if cutoff is None else cutoff
    num_rbf = WORKLOAD["num_rbf"] if num_rbf is None else num_rbf
    torch.manual_seed(seed)
    cut = ns.CosineCutoff(0.0, cutoff)
    rbf = ns.GaussianBasis(cut, num_rbf, trainable=False) if kind == "gaussian" else ns.ExpNormalBasis(cut, num_rbf, trainable=False)
    return ns.StandardSchNet(rbf, cut, [WORKLOAD["hidden"]], hidden_channels=WORKLOAD["hidden"],
                             embedding_size=WORKLOAD["bead_types"] if n_types is None else n_types, num_filters=WORKLOAD["filters"],
                             num_interactions=WORKLOAD["interactions"] if interactions is None else interactions)


# ----------------------------------------------------------------------------------------- CPU arm
class CpuArm:
    """The reference's CPU implementation of the path on the host cores.  ``kind`` "reference": mlcg's own modules from
    ``oracle/_ref/site`` (SchNet, CFConv, MLP, bases, cutoffs, priors, GradientsOut, SumOut unmodified; message passing,
    scatter and the radius graph through the stand-ins of ``oracle/mlcg_loader.py``); "port": the restatement in ``oracle/``."""

    def __init__(self):
        from oracle import mlcg_loader
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        self.kind = "reference" if mlcg_loader.available() else "port"
        self.ns = None
        if self.kind == "reference":
            mlcg_loader.install()
            self.ns = mlcg_loader.modules()

    def describe(self):
        if self.kind == "reference":
            return "mlcg's own modules on torch CPU float32 (torch_geometric propagate/scatter and torch_cluster.radius_graph replaced by stand-ins; radius graph by the C oracle)"
        return "restatement of mlcg's modules (oracle/schnet_ref.py) on torch CPU float32 + C radius oracle"

    def schnet_evaluator(self, state_dict, n, dtype=torch.float32, **arch):
        """``fn(pos, types, batch, B) -> (energy, forces)`` of a SchNet with this state_dict, radius graph rebuilt per call.
        ``dtype=torch.float64``: the same float32 weights and positions evaluated in double precision (the value every float32
        evaluation rounds towards)."""
        kind, cutoff = arch.get("kind", "expnormal"), arch.get("cutoff", WORKLOAD["cutoff_A"])
        L = arch.get("interactions", WORKLOAD["interactions"])
        from oracle import radius_ref, schnet_ref
        if self.kind == "reference":
            ns = self.ns
            model = make_model(ns, **arch)
            model.load_state_dict(state_dict)
            model = model.to(dtype)
            wrapped = ns.GradientsOut(model, "forces").eval()

            def fn(pos, types_, batch, B):
                # (in double precision the model rebuilds its graph from the same coordinates; a pair that changes sides within one
                # float32 rounding of the cutoff carries a filter of size ~1e-14, the cosine envelope vanishing there)
                data = ns.AtomicData(pos=pos.clone().to(dtype), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={})
                out = wrapped(data)
                return out.out["SchNet"]["energy"].detach(), out.out["SchNet"]["forces"].detach()

            return fn
        cut = {"cutoff": "cosine", "lower": 0.0, "upper": cutoff}
        spec = {"kind": kind, "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": L}
        sd = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in state_dict.items()}

        def fn(pos, types_, batch, B):
            ptr = radius_ref.batch_to_ptr(batch.numpy(), B)
            ei = torch.from_numpy(radius_ref.radius_graph_c(pos.numpy(), ptr, cutoff, 1000, False, "cluster"))
            e, f, _ = schnet_ref.energy_and_forces(lambda p: schnet_ref.schnet_energy(sd, spec, p, types_, batch, ei, B), pos.to(dtype))
            return e, f

        return fn


def timed_host(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(steps):
        out = fn()
    return (time.perf_counter() - t0) / steps, out


def parity(e, f, e32, f32, e64, f64):
    """Energies and forces of this package (``e``, ``f``) against the CPU arm in float32 (``e32``, ``f32``) and against the CPU
    arm's double-precision evaluation of the same float32 weights and positions (``e64``, ``f64``).  Bars: forces within 1e-4
    kcal/mol/A of the double-precision value, plus the distance of the reference's own float32 forces from it (on the 268-bead
    chains with priors forces reach 40-70 kcal/mol/A and the reference's float32 evaluation is itself 1.3e-4 away); energies
    within 1e-5 of the double-precision value, relative to the structure's own |E| or to the mean |E| of the sample, whichever
    is larger (an energy is a sum of per-bead terms of both signs: where they nearly cancel, no float32 evaluation, the
    reference's included, is accurate to 1e-5 of what is left)."""
    e, f, e32, f32 = e.double(), f.double(), e32.double(), f32.double()
    ours_e, cpu_e = (e - e64).abs(), (e32 - e64).abs()
    ours_f, cpu_f = float((f - f64).abs().max()), float((f32 - f64).abs().max())
    scale = torch.maximum(e64.abs(), e64.abs().mean())
    return dict(max_rel_dE=float((ours_e / scale).max()), cpu_f32_max_rel_dE=float((cpu_e / scale).max()),
                max_abs_dE_vs_f64=float(ours_e.max()), cpu_f32_max_abs_dE_vs_f64=float(cpu_e.max()), max_abs_dE_vs_cpu_f32=float((e - e32).abs().max()),
                min_abs_E=float(e64.abs().min()), mean_abs_E=float(e64.abs().mean()), max_abs_E=float(e64.abs().max()),
                max_abs_dF_vs_f64=ours_f, cpu_f32_max_abs_dF_vs_f64=cpu_f, max_abs_dF_vs_cpu_f32=float((f - f32).abs().max()),
                max_abs_F=float(f64.abs().max()), energy_rtol=E_RTOL, force_atol=F_ATOL,
                force_bar=F_ATOL + cpu_f,
                ok=bool((ours_e <= E_RTOL * scale).all() and ours_f <= F_ATOL + cpu_f))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm()
    sample_B, n = 128, WORKLOAD["beads"]
    sd = {k: v.detach() for k, v in make_model().state_dict().items()}
    pos, types_, batch = make_inputs(sample_B, n, WORKLOAD["bead_types"], seed=1000)
    fn = arm.schnet_evaluator(sd, n)
    sec, _ = timed_host(lambda: fn(pos, types_, batch, sample_B), max(args.steps, 1), max(args.warmup, 1))
    value = sample_B / sec
    sample = f"{sample_B} structures of the same workload per step (of {WORKLOAD['structures_per_gpu']}), radius graph rebuilt each step; {arm.describe()}"
    line = dict(metric=METRIC, value=value, unit="structures/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=sec * 1e3,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(WORKLOAD, sample_structures_per_step=sample_B),
                cpu_baseline=dict(value=value, unit="structures/s", cores=arm.cores, kind=arm.kind, sample=sample),
                e2e=dict(value=value, unit="structures/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0), gpu_launches=0)
    print(json.dumps(line))


# ----------------------------------------------------------------------------------------- clocks
class ClockSampler:
    FIELDS = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc = index, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100",
                                          "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        for ln in out.strip().splitlines():
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None, reasons=sorted(reasons), samples=len(sm))


def time_cuda(fn, iters=5, warm=2):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


# ----------------------------------------------------------------------------------------- the other configurations
def _uniform_tables(prior, T):
    """Give a prior built from one statistics entry the same parameters for all ``T`` bead types (its tables are indexed by the
    bead types of each term; their trailing ``order`` dimensions grow from 1 to T)."""
    order = prior.order
    for name, buf in list(prior.named_buffers()):
        lead = buf.dim() - order
        setattr(prior, name, buf.expand(*buf.shape[:lead], *([T] * order)).contiguous())
    return prior


def _chain_terms(n):
    idx = torch.arange(n)
    full = torch.cartesian_prod(idx, idx).t()
    return {"bonds": torch.stack([idx[:-1], idx[1:]]), "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
            "dihedrals": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]]), "repulsion": full[:, (full[0] - full[1]).abs() >= 3]}


def _prior_modules(ns, T):
    cos19 = float(torch.cos(torch.tensor(1.9)))
    pri = {"bonds": ns.HarmonicBonds({(0, 0): {"k": 100.0, "x_0": 3.8}}), "angles": ns.HarmonicAngles({(0, 0, 0): {"k": 50.0, "x_0": cos19}}),
           "dihedrals": ns.Dihedral({(0, 0, 0, 0): {"v_0": 0.0, "k1s": {"k1_1": 0.3, "k1_2": -0.2, "k1_3": 0.1}, "k2s": {"k2_1": 0.2, "k2_2": 0.1, "k2_3": -0.1}}}),
           "repulsion": ns.Repulsion({(0, 0): {"sigma": 4.0}})}
    return {k: _uniform_tables(p, T) for k, p in pri.items()}


def _batched_lists(terms, B, n, dev="cpu"):
    offs = torch.arange(B) * n
    out = {}
    for name, m in terms.items():
        M = m.shape[1] * B
        out[name] = ((m[:, None, :] + offs[None, :, None]).reshape(m.shape[0], M).contiguous().to(dev),
                     torch.arange(B).repeat_interleave(m.shape[1]).to(dev))
    return out


def _baoab_host(model_fn, pos, vel, forces, masses, beta_mass_ratio, noises, dt, friction):
    """The reference's BAOAB step on the host (src/mlcg/simulation/langevin.py:100-144), for the CPU leg of the simulation
    configuration: forces at t in, positions / velocities / forces at t+1 out, one model evaluation per step."""
    import math
    vscale = math.exp(-dt * friction)
    noisescale = math.sqrt(1 - vscale * vscale)
    pot = None
    for noise in noises:
        v = vel + 0.5 * dt * forces / masses[:, None]
        x = pos + v * dt * 0.5
        v = v * vscale + noisescale * beta_mass_ratio[:, None] * noise
        x = x + v * dt * 0.5
        pot, forces = model_fn(x)
        vel = v + 0.5 * dt * forces / masses[:, None]
        pos = x
    return pos, vel, pot, forces


def measure_small(dev, hbm_peak, arm, seed=0):
    """The CPU-runnable configuration: 64 structures x 10 beads, energy + forces, with the CPU arm beside it."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import get_backend
    from mlcg_b200.simulation import LangevinSimulation
    from oracle import radius_ref
    be = get_backend()
    out = {}
    gen = torch.Generator().manual_seed(seed)
    # ---- the CPU-runnable configuration: 64 structures x 10 beads, types 0..9, 50 Gaussians on 0-30 A, 2 blocks
    B1, n1 = 64, 10
    arch1 = dict(kind="gaussian", cutoff=30.0, num_rbf=50, interactions=2, n_types=10)
    net1 = make_model(**arch1)
    pos1 = random_walks(B1, n1, gen, jitter=0.3)
    types1, batch1 = torch.arange(n1).repeat(B1), torch.arange(B1).repeat_interleave(n1)
    m1 = bnn.GradientsOut(net1.to(dev), "forces").eval()
    d1 = dict(pos=pos1.to(dev), atom_types=types1.to(dev), batch=batch1.to(dev), n_atoms=torch.full((B1,), n1, device=dev))

    def eval1():
        o = m1(mlcg_b200.AtomicData(pos=d1["pos"].clone(), atom_types=d1["atom_types"], batch=d1["batch"], n_atoms=d1["n_atoms"]))
        return o.out["SchNet"]["energy"], o.out["SchNet"]["forces"]

    ms = time_cuda(eval1, iters=20, warm=5)
    e1, f1 = eval1()
    sd1 = {k: v.detach().cpu() for k, v in net1.state_dict().items()}
    fn1 = arm.schnet_evaluator(sd1, n1, **arch1)
    sec1, (e1r, f1r) = timed_host(lambda: fn1(pos1, types1, batch1, B1), 10, 2)
    e1x, f1x = arm.schnet_evaluator(sd1, n1, dtype=torch.float64, **arch1)(pos1, types1, batch1, B1)
    # the same evaluation with a fixed edge capacity (no host read of the edge count) recorded into a CUDA graph and replayed
    n_edges1 = int(be.radius_graph(d1["pos"], torch.arange(B1 + 1, device=dev) * n1, 30.0, 1000, False, 1)["edge_index"].shape[1])
    bnn.set_edge_capacity(m1, n_edges1 + (n_edges1 % 2) + 64)
    ff = mlcg_b200.GraphedForceField(m1, mlcg_b200.AtomicData(pos=d1["pos"].clone(), atom_types=d1["atom_types"], batch=d1["batch"], n_atoms=d1["n_atoms"]))
    ms_replay = time_cuda(lambda: ff(d1["pos"]), iters=20, warm=5)
    e1g, f1g = ff(d1["pos"])
    ff.check()
    if not (torch.allclose(e1g, e1, rtol=1e-6, atol=1e-6) and torch.allclose(f1g, f1, rtol=0, atol=1e-5)):
        raise RuntimeError("the replayed evaluation of 64 x 10 beads differs from the launched one")
    bnn.set_edge_capacity(m1, None)
    out["eval_64x10"] = dict(ms=ms, structures_per_s=B1 / (ms / 1e3), ms_graph_replay=ms_replay, structures_per_s_graph_replay=B1 / (ms_replay / 1e3),
                             cpu_ms=sec1 * 1e3, cpu_structures_per_s=B1 / sec1,
                             parity=parity(e1.cpu(), f1.cpu(), e1r, f1r, e1x, f1x),
                             note="64 structures x 10 beads, 2 blocks, 50 Gaussian functions on 0-30 A; radius graph + energy + forces per call; "
                                  "GPU time is the host's launch path at this size (`ms`), or the chain of small kernels when the call is "
                                  "replayed from a CUDA graph (`ms_graph_replay`); CPU: all 64 structures, 10 calls")
    del ff, m1, net1

    return out


def measure_radius(dev, hbm_peak, arm, radius_structures=256, seed=1):
    """The stand-alone radius graph: structures of 4000 points uniform in a 60 A cube, 10 A cutoff, no loops; the whole edge list
    is compared with the CPU oracle's."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import get_backend
    from mlcg_b200.simulation import LangevinSimulation
    from oracle import radius_ref
    be = get_backend()
    out = {}
    gen = torch.Generator().manual_seed(seed)
    # ---- stand-alone radius graph
    B, n = radius_structures, 4000
    pos_h = torch.rand(B * n, 3, generator=gen) * 60.0
    pos = pos_h.to(dev)
    ptr = torch.arange(B + 1, device=dev) * n
    res = be.radius_graph(pos, ptr, 10.0, 1000, False, 1, want_batch=False)
    E = int(res["edge_index"].shape[1])
    t0 = time.perf_counter()
    ei_cpu = radius_ref.radius_graph_c(pos_h.numpy(), (torch.arange(B + 1) * n).numpy(), 10.0, 1000, False, "cluster")
    cpu_s = time.perf_counter() - t0
    same = bool(torch.equal(res["edge_index"].cpu(), torch.from_numpy(ei_cpu)))
    del res, ei_cpu
    if not same:
        raise RuntimeError(f"radius graph of {B} x 4000 points differs from the CPU oracle's")
    ms = time_cuda(lambda: be.radius_graph(pos, ptr, 10.0, 1000, False, 1, want_batch=False), iters=5, warm=1)
    # the two library calls of that function on their own (CUDA events inside the library: no allocation, no host read between them)
    be.timeline_begin()
    for _ in range(5):
        be.radius_graph(pos, ptr, 10.0, 1000, False, 1, want_batch=False)
    tl = be.timeline_end()
    parts = {k: v["ms"] / v["calls"] for k, v in tl.items()}
    nbytes = 16 * E + 20 * B * n
    out[f"radius_graph_{B}x4000"] = dict(edges=E, ms=ms, edges_per_s=E / (ms / 1e3), algorithmic_GBps=nbytes / ms / 1e6,
                                        frac_of_hbm=nbytes / ms / 1e6 / hbm_peak, ms_library_calls=parts, ms_without_allocation_and_host_read=sum(parts.values()),
                                        frac_of_hbm_without_allocation_and_host_read=nbytes / sum(parts.values()) / 1e6 / hbm_peak if parts else None,
                                        bit_exact_vs_cpu_oracle=same, cpu_ms=cpu_s * 1e3,
                                        cpu_edges_per_s=E / cpu_s, cpu_cores=arm.cores,
                                        note="count + scan + host read of E + fill, allocation of the outputs included; algorithmic bytes = 16 B/edge "
                                             "written + 20 B/point read (the call also writes the two int32 index rows this package's kernels "
                                             "read, 8 B/edge more); CPU: the C oracle (all pairs of each structure, OpenMP over structures), "
                                             "every structure, one call; the two edge lists are compared whole")
    del pos

    return out


def measure_priors_and_dynamics(dev, hbm_peak, arm, seed=2, dynamics=True):
    """The prior terms and the Langevin dynamics of the simulation configuration (1024 replicas x 268 beads)."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import get_backend
    from mlcg_b200.simulation import LangevinSimulation
    from oracle import radius_ref
    be = get_backend()
    out = {}
    gen = torch.Generator().manual_seed(seed)
    # ---- priors of the simulation configuration
    Bp, npb, T = 1024, 268, 20
    terms = _chain_terms(npb)
    lists = _batched_lists(terms, Bp, npb, dev)
    ppos_h = self_avoiding_chains(Bp, npb, gen)
    ppos = ppos_h.to(dev)
    n_par = {"bonds": 2, "angles": 2, "dihedrals": 7, "repulsion": 1}
    for kind, name in enumerate(["bonds", "angles", "dihedrals", "repulsion"]):
        mapping, mb = lists[name]
        M = mapping.shape[1]
        params = torch.rand(n_par[name], M, device=dev) + (3.0 if name in ("bonds", "repulsion") else 0.0)
        ms = time_cuda(lambda: be.prior_terms(kind, ppos, mapping, mb, params, Bp), iters=5, warm=1)
        nbytes = M * (8 * mapping.shape[0] + 8 + 4 * n_par[name]) + 2 * ppos.numel() * 4
        out[f"prior_{name}_1024x268"] = dict(terms=M, ms=ms, terms_per_s=M / (ms / 1e3), algorithmic_GBps=nbytes / ms / 1e6,
                                             frac_of_hbm=nbytes / ms / 1e6 / hbm_peak)
        del params

    # ---- the four priors together, as SumOut evaluates them in eval mode: one launch, 32-bit indices, no scatter for the pair
    #      list that holds both directions, sums in fixed point (reproducible) or with floating-point atomics
    pri = {k: p.to(dev).eval() for k, p in _prior_modules(bnn, T).items()}
    nls = {name: mlcg_b200.make_neighbor_list(name, m.shape[0], m, mb) for name, (m, mb) in lists.items()}
    types5_h = torch.randint(0, T, (Bp * npb,), generator=gen)
    data = mlcg_b200.AtomicData(pos=ppos.clone(), atom_types=types5_h.to(dev), batch=torch.arange(Bp, device=dev).repeat_interleave(npb),
                                n_atoms=torch.full((Bp,), npb, device=dev), neighbor_list=nls)
    M_all = sum(int(m.shape[1]) for m, _ in lists.values())
    moved = sum(int(m.numel()) * 4 + int(m.shape[1]) * 4 * n_par[name] for name, (m, _) in lists.items()) + 2 * ppos.numel() * 4
    for mode, flag in (("fixed_point", True), ("float_atomics", False)):
        bnn.set_prior_determinism(flag)
        ms = time_cuda(lambda: bnn.evaluate_priors(list(pri.values()), data), iters=5, warm=2)
        out[f"priors_together_1024x268_{mode}"] = dict(terms=M_all, ms=ms, terms_per_s=M_all / (ms / 1e3), moved_GBps=moved / ms / 1e6,
                                                        frac_of_hbm=moved / ms / 1e6 / hbm_peak,
                                                        note="bonds + angles + dihedrals + repulsion in one launch; bytes moved: int32 indices, "
                                                             "float32 per-term parameters, positions in, gradients out")
    bnn.set_prior_determinism(True)
    if not dynamics:
        return out
    # ---- Langevin dynamics: 1024 replicas x 268 beads, SchNet (3 blocks, 12 A) + the four priors, BAOAB, graph rebuilt every step
    arch5 = dict(cutoff=12.0, n_types=T)
    net = make_model(**arch5)
    sd5 = {k: v.detach().clone() for k, v in net.state_dict().items()}
    models = {"SchNet": bnn.GradientsOut(net, "forces")}
    models.update({k: bnn.GradientsOut(p, "forces") for k, p in pri.items()})
    model = bnn.SumOut(torch.nn.ModuleDict(models)).eval().to(dev)
    mass = 12.0 / 418.39
    sim = LangevinSimulation(model, dt=0.002, friction=1.0, beta=KCAL_BETA_300K, rng=torch.Generator(device=dev).manual_seed(0))
    sim.attach(data, torch.full((Bp * npb,), mass, device=dev))
    pot, forces = sim.calculate_potential_and_forces(sim.data)
    e0, f0 = pot.cpu(), forces.cpu()               # energies and forces of the starting structures, for the check below
    for _ in range(2):
        _, pot, forces = sim.timestep(sim.data, forces)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    nsteps = 5
    a.record()
    for _ in range(nsteps):
        _, pot, forces = sim.timestep(sim.data, forces)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / nsteps
    be.check_pending()
    # CPU leg: 64 replicas x 5 BAOAB steps with the CPU arm's SchNet + four priors (reference modules when installed)
    Bc = 64
    cpu = None
    if arm.kind == "reference":
        ns = arm.ns
        clists = _batched_lists(terms, Bc, npb)
        ctypes_, cbatch = types5_h[: Bc * npb], torch.arange(Bc).repeat_interleave(npb)

        def cpu_model(dtype):
            cnet = make_model(ns, **arch5)
            cnet.load_state_dict(sd5)
            cmods = {"SchNet": ns.GradientsOut(cnet, "forces")}
            cmods.update({k: ns.GradientsOut(p, "forces") for k, p in _prior_modules(ns, T).items()})
            cmodel = ns.SumOut(torch.nn.ModuleDict(cmods)).eval().to(dtype)
            cnl = {name: dict(tag=name, order=m.shape[0], index_mapping=m, mapping_batch=mb, cell_shifts=None, rcut=None, self_interaction=False)
                   for name, (m, mb) in clists.items()}

            def model_fn(x):
                d = ns.AtomicData(pos=x.clone().to(dtype), atom_types=ctypes_, batch=cbatch, n_atoms=torch.full((Bc,), npb), neighbor_list=dict(cnl))
                o = cmodel(d)
                return o.out["energy"].detach(), o.out["forces"].detach()

            return model_fn

        model_fn = cpu_model(torch.float32)
        x0 = ppos_h[: Bc * npb].clone()
        ec, fc = model_fn(x0)
        ex, fx = cpu_model(torch.float64)(x0)
        chk = parity(e0[:Bc], f0[: Bc * npb], ec, fc, ex, fx)
        cgen = torch.Generator().manual_seed(1)
        masses_c = torch.full((Bc * npb,), mass)
        bmr = torch.sqrt(1.0 / (KCAL_BETA_300K * masses_c))
        noises = [torch.randn(Bc * npb, 3, generator=cgen) for _ in range(5)]
        t0 = time.perf_counter()
        _baoab_host(model_fn, x0, torch.zeros_like(x0), fc, masses_c, bmr, noises, 0.002, 1.0)
        cpu_s = (time.perf_counter() - t0) / len(noises)
        cpu = dict(ms_per_md_step_64_replicas=cpu_s * 1e3, replica_steps_per_s=Bc / cpu_s, parity_first_evaluation=chk,
                   sample="64 of the 1024 replicas, 5 BAOAB steps (mlcg's SchNet, priors, GradientsOut and SumOut; the step loop restates "
                          "langevin.py:100-144), scaled per replica-step")
        if not chk["ok"]:
            raise RuntimeError(f"SchNet + priors on 64 x 268 beads differ from the CPU arm: {chk}")
    out["langevin_1024x268"] = dict(ms_per_md_step=ms, md_steps_per_s=1e3 / ms, replica_steps_per_s=Bp * 1e3 / ms, finite=bool(torch.isfinite(pot).all()),
                                    cpu=cpu, cpu_cores=arm.cores,
                                    note="SchNet (3 blocks, 128 expnorm RBF, 12 A) + bonds/angles/dihedrals/repulsion(|i-j|>=3), BAOAB dt=2 fs, "
                                         "radius graph rebuilt every step, 1024 replicas on one GPU")
    return out


def extra_measurements(dev, hbm_peak, arm):
    """The other configurations on one GPU: the small CPU-runnable system (64 x 10 beads), the stand-alone radius graph (256 x 4000
    points, 60 A cube, 10 A cutoff, compared bit for bit with the CPU oracle on all 256 structures), the prior terms and the
    Langevin dynamics of the simulation configuration (1024 x 268 beads).  Device time by CUDA events; inputs far larger than L2
    except where the configuration itself is small.  Each GPU figure has the CPU arm's figure beside it (bounded samples)."""
    out = {}
    out.update(measure_small(dev, hbm_peak, arm))
    out.update(measure_radius(dev, hbm_peak, arm))
    torch.cuda.empty_cache()
    out.update(measure_priors_and_dynamics(dev, hbm_peak, arm))
    return out


# ----------------------------------------------------------------------------------------- force-matching training step
def training_step_measurement(dev, world, steps=10, warmup=3):
    """Force-matching training step of the training configuration on every rank: 256 structures x 73 beads per GPU (3.8 A random
    walk, 20 types), SchNet 3 blocks / 128 / 128 exp-normal functions / 10 A, ``model.train()`` so that the force pass keeps its graph,
    MSE on forces against N(0,1) targets, gradient all-reduce over the ranks (NCCL; mean), AdamW(lr 1e-4, weight decay 0) — the step
    of src/mlcg/pl/model.py:113-131 under examples/input_yamls/slurm_example/train.yaml:9.  Returns this rank's
    (ms per step, ms in the all-reduce per step, last loss)."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.distributed import allreduce_gradients
    rank = int(os.environ.get("RANK", "0"))
    B, n, T = 256, 73, 20
    net = make_model(cutoff=10.0, n_types=T).to(dev)        # the same initial weights on every rank
    model = bnn.GradientsOut(net, "forces").train()
    gen = torch.Generator().manual_seed(4000 + rank)         # every rank its own structures and targets
    pos = random_walks(B, n, gen).to(dev)
    types_ = torch.randint(0, T, (B * n,), generator=gen).to(dev)
    batch = torch.arange(B).repeat_interleave(n).to(dev)
    target = torch.randn(B * n, 3, generator=gen).to(dev)
    n_atoms = torch.full((B,), n, device=dev)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, weight_decay=0)
    params = list(net.parameters())
    ar_events = []

    def step(timed):
        opt.zero_grad(set_to_none=True)
        out = model(mlcg_b200.AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=n_atoms))
        loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], target)
        loss.backward()
        if world > 1:
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            allreduce_gradients(params)
            b.record()
            if timed:
                ar_events.append((a, b))
        opt.step()
        return loss

    for _ in range(warmup):
        step(False)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step(True)
    b.record()
    torch.cuda.synchronize()
    from mlcg_b200.backend import get_backend
    get_backend().check_pending()
    ar_ms = sum(x.elapsed_time(y) for x, y in ar_events) / steps if ar_events else 0.0
    return a.elapsed_time(b) / steps, ar_ms, float(loss.detach()), B, sum(p.numel() for p in params)


def training_cpu_leg(arm, steps=2):
    """The same step on the host cores with the CPU arm's modules, 64 structures (a quarter of one GPU's batch)."""
    if arm.kind != "reference":
        return None
    ns = arm.ns
    B, n, T = 64, 73, 20
    net = make_model(ns, cutoff=10.0, n_types=T)
    model = ns.GradientsOut(net, "forces").train()
    gen = torch.Generator().manual_seed(4000)
    pos, types_ = random_walks(B, n, gen), torch.randint(0, T, (B * n,), generator=gen)
    batch, target = torch.arange(B).repeat_interleave(n), torch.randn(B * n, 3, generator=gen)
    opt = torch.optim.AdamW(net.parameters(), lr=1e-4, weight_decay=0)

    def step():
        opt.zero_grad(set_to_none=True)
        out = model(ns.AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={}))
        loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], target)
        loss.backward()
        opt.step()
        return loss

    # the first step's loss and parameter gradients (before any update), for the check against the GPU arm below
    opt.zero_grad(set_to_none=True)
    out = model(ns.AtomicData(pos=pos.clone(), atom_types=types_, batch=batch, n_atoms=torch.full((B,), n), neighbor_list={}))
    loss0 = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], target)
    loss0.backward()
    grads0 = {k: p.grad.detach().clone() for k, p in net.named_parameters() if p.grad is not None}
    sec, _ = timed_host(step, steps, 1)
    return dict(ms_per_step_64_structures=sec * 1e3, structures_per_s=B / sec, cores=arm.cores, kind=arm.kind,
                sample=f"64 structures x 73 beads per step, {steps} steps after 1 warm-up; {arm.describe()}"), float(loss0.detach()), grads0


def training_parity(dev, loss_cpu, grads_cpu):
    """The GPU arm's first training step on the CPU leg's 64 structures (same seeds, same initial weights): loss within 1e-5
    relative, every parameter gradient within 2e-4 of its tensor's largest entry (the bars of the test-suite's force-matching
    cases); raises otherwise."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    B, n, T = 64, 73, 20
    net = make_model(cutoff=10.0, n_types=T).to(dev)
    model = bnn.GradientsOut(net, "forces").train()
    gen = torch.Generator().manual_seed(4000)
    pos, types_ = random_walks(B, n, gen), torch.randint(0, T, (B * n,), generator=gen)
    batch, target = torch.arange(B).repeat_interleave(n), torch.randn(B * n, 3, generator=gen)
    out = model(mlcg_b200.AtomicData(pos=pos.to(dev), atom_types=types_.to(dev), batch=batch.to(dev), n_atoms=torch.full((B,), n, device=dev)))
    loss = torch.nn.functional.mse_loss(out.out["SchNet"]["forces"], target.to(dev))
    loss.backward()
    worst, worst_name = 0.0, None
    for k, p in net.named_parameters():
        if k in grads_cpu and p.grad is not None:
            err = float((p.grad.cpu() - grads_cpu[k]).abs().max() / (grads_cpu[k].abs().max() + 1e-30))
            if err > worst:
                worst, worst_name = err, k
    rel_loss = abs(float(loss.detach()) - loss_cpu) / abs(loss_cpu)
    res = dict(loss=float(loss.detach()), cpu_loss=loss_cpu, rel_loss_difference=rel_loss, worst_gradient_error=worst, worst_gradient=worst_name,
               loss_rtol=1e-5, gradient_bar=2e-4, ok=bool(rel_loss <= 1e-5 and worst <= 2e-4))
    if not res["ok"]:
        raise RuntimeError(f"first training step on 64 x 73 beads differs from the CPU arm: {res}")
    return res


# ----------------------------------------------------------------------------------------- GPU arm
def kernel_work(name, E, P, N, F, R):
    """Algorithmic (bytes, flops) of one call of a library entry point at the benchmark's sizes: E directed edges, P = E/2
    unordered pairs, N beads, F filters, R radial functions.  Index arrays at their stored width (int32 rows, int64 pointers)."""
    if name == "filter_forward":        # d in, one filter row and one hidden row per pair out; 2(RF + F^2) flop per directed edge
        return P * (8 * F + 4), 2 * E * F * (R + F)
    if name == "filter_backward":       # d, two index rows, the saved hidden row, gd; node rows x'[row0], g[row1] from L2; 2(F^2 + RF) flop per edge
        return 16 * E + P * 4 * F + 2 * N * F * 4, 2 * E * F * (R + F)
    if name == "seg_mul_sum":           # one filter row per pair, neighbour index and pair index per edge, node rows in and out
        return P * F * 4 + 8 * E + 2 * N * F * 4 + 8 * N, 2 * E * F
    if name.startswith("gemm_tc"):      # node-sized Linear layers, 128 wide
        return (2 * N * F + F * F) * 4, 2 * N * F * F
    if name == "radius_graph_capacity":
        return 24 * N + 8 * E, 0
    if name == "pair_plan":
        return 28 * E + 20 * N, 0
    if name == "edge_distance":
        return 12 * E + 12 * N, 0
    if name == "edge_distance_backward":
        return 2 * E * 24 + 24 * N, 0
    return 0, 0


def run_ours(args):
    import torch.distributed as dist
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import get_backend

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        # (a rank that fails must not keep the others waiting for NCCL's default ten minutes)
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    B, n = WORKLOAD["structures_per_gpu"], WORKLOAD["beads"]
    pos_h, types_h, batch_h = make_inputs(B, n, WORKLOAD["bead_types"], seed=1000 + rank)   # every rank its own replicas
    net = make_model()
    state_dict_h = {k: v.detach().clone() for k, v in net.state_dict().items()}
    model = bnn.GradientsOut(net.to(dev), "forces").eval()
    be = get_backend()
    n_atoms = torch.full((B,), n, device=dev)
    pos_d, types_d, batch_d = pos_h.to(dev), types_h.to(dev), batch_h.to(dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step_resident():
        data = mlcg_b200.AtomicData(pos=pos_d.clone(), atom_types=types_d, batch=batch_d, n_atoms=n_atoms)
        out = model(data)
        return out.out["SchNet"]["energy"], out.out["SchNet"]["forces"]

    pin = lambda t: t.pin_memory()
    pos_p, types_p, batch_p = pin(pos_h), pin(types_h), pin(batch_h)

    # results come back into two pinned slots used in turn: the host waits for a slot's copies only when it needs the slot
    # again, so it prepares and launches step k+1 while the device still works on step k (every step's inputs are copied
    # in and every step's energies and forces are on the host when the clock stops)
    slots = [dict(e=torch.empty(B, dtype=torch.float32).pin_memory(), f=torch.empty((B * n, 3), dtype=torch.float32).pin_memory(),
                  done=torch.cuda.Event()) for _ in range(2)]

    def step_e2e(k):
        slot = slots[k % 2]
        slot["done"].synchronize()
        data = mlcg_b200.AtomicData(pos=pos_p.to(dev, non_blocking=True), atom_types=types_p.to(dev, non_blocking=True),
                                    batch=batch_p.to(dev, non_blocking=True), n_atoms=n_atoms)
        out = model(data)
        slot["e"].copy_(out.out["SchNet"]["energy"], non_blocking=True)
        slot["f"].copy_(out.out["SchNet"]["forces"], non_blocking=True)
        slot["done"].record()
        return slot

    group = {"alive": world > 1}      # cleared once the ranks have parted: rank 0 then works on alone

    def barrier():
        if group["alive"]:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    torch.cuda.synchronize()
    n_edges = int(be.radius_graph(pos_d, torch.arange(B + 1, device=dev) * n, WORKLOAD["cutoff_A"], 1000, False, 1)["edge_index"].shape[1])
    # Edge buffers sized once, for 1.1 x the edge count of these structures: the radius graph is still rebuilt in every step,
    # but its edge count stays on the device (no host read inside a step; an overflow would be reported by check_pending below)
    bnn.set_edge_capacity(model, int(1.1 * n_edges))
    for _ in range(3):
        step_resident()
    be.check_pending()

    # ---- timed region: K steps, device time per step (L2 flushed outside the event pair)
    def timed_steps():
        pairs = []
        for _ in range(args.steps):
            flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            step_resident()
            b.record()
            pairs.append((a, b))
        barrier()
        return [a.elapsed_time(b) for a, b in pairs]

    clocks = ClockSampler(local)
    clocks.start()
    barrier()
    step_ms = timed_steps()
    ms_total = sum(step_ms)
    be.check_pending()          # status words of the timed steps (edge capacity, tensor-core waits): raises if any is set
    # ---- the same K steps once more, on the same route (one library call per evaluation), with the library's timeline on: a
    # CUDA-event pair around every kernel-launching entry point, recorded inside the library call (the per-kernel durations
    # behind `roofline` and `kernels`).  Kept out of the region above because a recorded launch cannot start its set-up under
    # the tail of the launch before it.
    be.timeline_begin()
    ms_recorded = sum(timed_steps())
    timeline = be.timeline_end()
    clk = clocks.stop()

    # ---- end to end through the public API: pinned host inputs in, energies and forces back to the host
    step_e2e(0)
    step_e2e(1)
    barrier()
    t0 = time.perf_counter()
    for k in range(args.steps):
        step_e2e(k)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    be.check_pending()
    e_res, f_res = step_resident()
    last = slots[(args.steps - 1) % 2]
    if not (torch.equal(last["e"], e_res.cpu()) and torch.equal(last["f"], f_res.cpu())):
        raise RuntimeError("end-to-end results differ from the device-resident evaluation of the same structures")
    e_timed, f_timed = e_res.cpu(), f_res.cpu()
    barrier()

    # ---- the same evaluation recorded once into a CUDA graph and replayed: the step without the host's launch path (what the
    # maximum over the ranks' host processes adds at N > 1 shows as the difference to `ms_per_step`)
    ff = mlcg_b200.GraphedForceField(model, mlcg_b200.AtomicData(pos=pos_d.clone(), atom_types=types_d, batch=batch_d, n_atoms=n_atoms))
    e_g, f_g = ff(pos_d)
    if not (torch.equal(e_g, e_res) and torch.equal(f_g, f_res)):
        raise RuntimeError("the replayed evaluation differs from the launched one")
    pairs = []
    barrier()
    for _ in range(args.steps):
        flush.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        ff(pos_d)
        b.record()
        pairs.append((a, b))
    barrier()
    replay_ms = sum(a.elapsed_time(b) for a, b in pairs)
    ff.check()
    del ff

    t = torch.tensor([ms_total, e2e_s * 1e3, ms_recorded, replay_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, ms_recorded, replay_ms = float(t[0]), float(t[1]), float(t[2]), float(t[3])

    # ---- the training configuration's step, on every rank, with the gradient all-reduce when there are several
    training = None
    if not args.no_extras:
        del flush
        torch.cuda.empty_cache()
        bnn.set_edge_capacity(model, None)
        tr_ms, ar_ms, tr_loss, tr_B, n_params = training_step_measurement(dev, world)
        tt = torch.tensor([tr_ms, ar_ms], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        training = dict(ms_per_step=float(tt[0]), structures_per_s=world * tr_B / (float(tt[0]) / 1e3), allreduce_ms_per_step=float(tt[1]),
                        allreduce_bytes=4 * n_params, structures_per_gpu=tr_B, n_gpus=world, loss=tr_loss,
                        note="256 structures x 73 beads per GPU, SchNet 3 blocks / 128 / 128 expnorm / 10 A, train mode (second-order pass), "
                             "MSE on forces, gradient all-reduce (mean) over the ranks, AdamW(1e-4); 10 steps after 3 warm-ups, CUDA events, "
                             "maximum over ranks")
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        bnn.set_edge_capacity(model, int(1.1 * n_edges))
    # the ranks part here: everything below is rank 0's own reporting (no collective may follow)
    if world > 1:
        dist.barrier()
        group["alive"] = False
        dist.destroy_process_group()
    if rank != 0:
        return

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    tf_peak = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_src = "measured" if peaks else "fallback"
    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the Nsight Compute captures summarised under
    # profiles/: one record per kernel with the row count of the captured launch, scaled here to this run's rows
    try:
        traffic_table = json.load(open(os.path.join(ROOT, "profiles", "traffic.json")))
    except OSError:
        traffic_table = {}
    F, R, N, P = WORKLOAD["filters"], WORKLOAD["num_rbf"], B * n, n_edges // 2

    def traffic_of(name):
        rec = traffic_table.get(name)
        if not rec:
            return None, None
        rows_now = {"pairs": P, "edges": n_edges, "nodes": N}[rec["rows_are"]]
        return rec["dram_bytes_per_launch"] * rows_now / rec["rows"], rec["source"]

    kernels = {}
    for name, rec in sorted(timeline.items(), key=lambda kv: -kv[1]["ms"]):
        nbytes, flops = kernel_work(name, n_edges, P, N, F, R)
        per_launch = rec["ms"] / rec["calls"]
        kernels[name] = dict(calls_per_step=rec["calls"] / args.steps, ms_per_step=rec["ms"] / args.steps, ms_per_launch=per_launch,
                             GBps=(nbytes / per_launch / 1e6 if nbytes else None), TFLOPs=(flops / per_launch / 1e9 if flops else None))
    tensor_kernels = {"filter_forward": "filter_fwd_pipe_kernel (tcgen05: RBF prologue, 2 GEMMs, tanh, cutoff, hidden layer kept; one row per unordered pair)",
                      "filter_backward": "filter_bwd_saved_kernel (tcgen05: gather of gW, 2 GEMMs per row on the forward's hidden layer; one row per unordered pair)"}
    name = next(iter(kernels))
    k = kernels[name]
    tr, tr_src = traffic_of(name)
    if name in tensor_kernels:
        roof = dict(kernel=tensor_kernels[name], bound="tensor", achieved=k["TFLOPs"], peak=tf_peak, unit="TFLOP/s", frac=k["TFLOPs"] / tf_peak,
                    traffic=tr, traffic_source=tr_src, peak_source=f"{peak_src} bf16 sustained", avg_launch_ms=k["ms_per_launch"],
                    share_of_recorded_step=k["ms_per_step"] / (ms_recorded / args.steps),
                    executed_TFLOPs=k["TFLOPs"] / 2, tensor_pipe_TFLOPs=1.5 * k["TFLOPs"],
                    note="algorithmic flops: 2*F*(R+F) per directed edge and pass (forward: R*F + F*F multiply-adds; backward to the input the "
                         "same), times the E edges of the launch.  The kernels evaluate one row per unordered pair (E/2 rows: a pair's two "
                         "edges share their filter), so the executed products are half of that (`executed_TFLOPs`); the fp32-equivalent mode "
                         "issues three fp16 products per executed product (`tensor_pipe_TFLOPs`).  Duration from CUDA events recorded inside "
                         "the library call on the timed route")
    else:
        roof = dict(kernel=name, bound="hbm", achieved=k["GBps"], peak=hbm_peak, unit="GB/s", frac=(k["GBps"] or 0) / hbm_peak, traffic=tr,
                    traffic_source=tr_src, peak_source=f"{peak_src} copy bandwidth", avg_launch_ms=k["ms_per_launch"],
                    share_of_recorded_step=k["ms_per_step"] / (ms_recorded / args.steps))
    cfconv = None
    seg = timeline.get("seg_mul_sum")
    if seg and seg["ms"] > 0:
        # two figures.  `reference_algorithm_*`: the bytes the reference's formulation of the aggregation moves per edge (a filter
        # row per directed edge, [2,E] int64 indices, node tensors once) at this kernel's edge rate: can exceed the peak, because
        # this kernel reads one filter row per unordered pair and int32 indices.  `achieved` / `frac`: the bytes this kernel has to
        # move (kernel_work) over its duration: its position on the HBM roofline.
        per_edge = 4 * F + 16 + 8 * F * N / n_edges
        per_launch = seg["ms"] / seg["calls"]
        moved, _ = kernel_work("seg_mul_sum", n_edges, P, N, F, R)
        s_tr, s_src = traffic_of("seg_mul_sum")
        cfconv = dict(kernel="seg_mul_sum_async_kernel (CFConv gather * filter, segmented sum; filters stored once per pair, rows through a cp.async ring)", bound="hbm",
                      achieved=moved / per_launch / 1e6, peak=hbm_peak, unit="GB/s", frac=moved / per_launch / 1e6 / hbm_peak,
                      edges_per_s=n_edges / (per_launch / 1e3), reference_algorithm_bytes_per_edge=per_edge,
                      reference_algorithm_GBps=per_edge * n_edges / per_launch / 1e6, reference_algorithm_frac=per_edge * n_edges / per_launch / 1e6 / hbm_peak,
                      traffic=s_tr, traffic_source=s_src, avg_launch_ms=per_launch)

    # ---- parity of what was timed + the CPU baseline: the first 64 structures of the timed batch on the host cores
    cpu = check = None
    arm = None
    if not args.no_cpu and world == 1:        # the CPU leg is timed at N = 1 only (other ranks would share the host cores)
        arm = CpuArm()
        sample_B = min(64, B)
        fn = arm.schnet_evaluator(state_dict_h, n)
        sl = slice(0, sample_B * n)
        sec, (e_cpu, f_cpu) = timed_host(lambda: fn(pos_h[sl], types_h[sl], batch_h[sl], sample_B), 12, 1)
        e_64, f_64 = arm.schnet_evaluator(state_dict_h, n, dtype=torch.float64)(pos_h[sl], types_h[sl], batch_h[sl], sample_B)
        check = parity(e_timed[:sample_B], f_timed[sl], e_cpu, f_cpu, e_64, f_64)
        cpu = dict(value=sample_B / sec, unit="structures/s", cores=arm.cores, kind=arm.kind,
                   sample=f"the first {sample_B} structures of the timed batch per step, 12 steps after 1 warm-up, radius graph rebuilt each step; {arm.describe()}")
        if not check["ok"]:
            raise RuntimeError(f"timed batch differs from the CPU arm beyond the parity bars: {check}")

    extras = None
    if not args.no_extras and world == 1:      # side measurements of other kernels and configurations: single-GPU runs only
        try:
            # the same step with the filter-network GEMMs on bf16 operands (forces within 1e-2 relative RMS of the fp32 mode)
            bnn.set_filter_precision(model, "bf16")
            for _ in range(3):
                step_resident()
            bf16_ms = timed_steps()
            e_b, f_b = step_resident()
            bnn.set_filter_precision(model, "fp32")
            rel_rms = float(((f_b.cpu() - f_timed).pow(2).mean() / f_timed.pow(2).mean()).sqrt())
            del flush
            torch.cuda.empty_cache()
            arm = arm or CpuArm()
            extras = extra_measurements(dev, hbm_peak, arm)
            extras["bf16_filter_mode"] = dict(ms_per_step=sum(bf16_ms) / len(bf16_ms), structures_per_s=B / (sum(bf16_ms) / len(bf16_ms) / 1e3),
                                              force_rel_rms_vs_fp32_mode=rel_rms,
                                              note="same workload, filter-network GEMMs with bf16 operands (one product, tanh.approx)")
            if training is not None:
                leg = training_cpu_leg(arm)
                if leg is not None:
                    training["cpu"], loss_cpu, grads_cpu = leg
                    training["parity_first_step"] = training_parity(dev, loss_cpu, grads_cpu)
        except Exception as exc:   # the headline line is still printed
            extras = {"error": repr(exc)}
    if training is not None:
        extras = dict(extras or {}, training_step_256x73=training)

    # kernels of the library per evaluation on the route the timed region takes (one library call for the model): radius graph 11
    # (cells, work-item scan, count by the block kernel and by the warp kernel, three scan kernels, clamp to the capacity, fill by
    # the expanding kernel, the testing block kernel and the warp kernel), reverse-edge map / pair selection / pair index 5 (count
    # of upper edges, three scan kernels, plan), distances 1, embedding 1, four per block forward (lin1, filter network,
    # aggregation, the two chained layers), output network 3 (layer + tanh, dot product, per-structure sum), its derivative 1,
    # four per block backward (chained layers, aggregation, lin1 with the residual, filter network; two for the first block,
    # whose input gradient nobody needs; the distance gradients of the blocks are added up by the filter kernels), distance
    # backward 1
    L = WORKLOAD["interactions"]
    launches_timed = args.steps * (11 + 5 + 1 + 1 + 4 * L + 3 + 1 + 4 * (L - 1) + 2 + 1)
    value = world * B * args.steps / (ms_total / 1e3)
    h2d = pos_h.numel() * 4 + types_h.numel() * 8 + batch_h.numel() * 8
    d2h = B * 4 + pos_h.numel() * 4
    line = dict(metric=METRIC, value=value, unit="structures/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_total / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(WORKLOAD, edges_per_gpu=n_edges, edge_capacity=int(1.1 * n_edges) + int(1.1 * n_edges) % 2, global_structures=world * B, parallelism=f"replicas x{world}, no collective",
                            kernel_timing="second pass over the same K steps on the same route (one library call per evaluation) with the "
                                          "library's timeline on: a CUDA-event pair around every kernel-launching entry point"),
                e2e=dict(value=world * B * args.steps / (e2e_ms / 1e3), unit="structures/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
                gpu_launches=launches_timed, ms_per_step_median=sorted(step_ms)[len(step_ms) // 2], ms_per_step_min=min(step_ms),
                ms_per_step_with_kernel_events=ms_recorded / args.steps,
                graph_replay=dict(ms_per_step=replay_ms / args.steps, structures_per_s=world * B / (replay_ms / args.steps / 1e3),
                                  note="the same evaluation recorded into a CUDA graph and replayed K times (positions copied in, radius graph rebuilt "
                                       "in every replay); maximum over ranks"),
                roofline=roof, cfconv_roofline=cfconv, parity_of_timed_batch=check,
                other_kernels=extras, cpu_baseline=cpu, clocks=clk, kernels=kernels,
                edges_per_s=world * n_edges * args.steps / (ms_total / 1e3))
    print(json.dumps(line))


def run_only(args):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    try:
        hbm_peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))).get("hbm_gbs", 6650.0)
    except OSError:
        hbm_peak = 6650.0
    arm = CpuArm()
    if args.only == "small":
        rec = measure_small(dev, hbm_peak, arm)
    elif args.only == "radius":
        rec = measure_radius(dev, hbm_peak, arm, radius_structures=args.radius_structures)
    elif args.only in ("priors", "dynamics"):
        rec = measure_priors_and_dynamics(dev, hbm_peak, arm, dynamics=args.only == "dynamics")
    else:
        ms, ar, loss, B, n_params = training_step_measurement(dev, 1, steps=max(args.steps, 1) if args.steps != 50 else 10, warmup=max(args.warmup, 1) if args.warmup != 10 else 3)
        rec = {"training_step_256x73": dict(ms_per_step=ms, structures_per_s=B / (ms / 1e3), loss=loss, parameters=n_params)}
    print(json.dumps(rec))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--structures", type=int, default=None, help="structures per GPU (default 512; smaller values are for profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the other configurations (radius graph, priors, dynamics, training step)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU arm: no baseline and no parity check of the timed batch (profiler captures)")
    ap.add_argument("--only", default=None, choices=["small", "radius", "priors", "dynamics", "training"],
                    help="run one of the other configurations alone on one GPU and print its record (profiler captures)")
    ap.add_argument("--radius-structures", type=int, default=256, help="structures of 4000 points for --only radius")
    args = ap.parse_args()
    if args.structures:
        WORKLOAD["structures_per_gpu"] = args.structures
        WORKLOAD["workload"] += f" [REDUCED to {args.structures} structures/GPU: not the benchmark configuration]"
    if args.only:
        run_only(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
