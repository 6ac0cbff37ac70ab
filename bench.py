#!/usr/bin/env python
"""Benchmark of the coarse-grained SchNet hot path: energy + force evaluations per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload at every N: 512 structures per GPU of a 100-bead C-alpha chain (3.8 A self-avoiding random
walk, 20 bead types), SchNet with 3 interaction blocks, hidden = filters = 128, 128 exp-normal radial
basis functions, 15 A cosine cutoff, float32; one step = radius graph + energy + forces for the batch.
Prints ONE JSON line (rank 0).  ``--impl reference`` times the CPU restatement of mlcg's own PyTorch
path (``oracle/``) on the host cores, on a bounded sample of the same workload.
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
WORKLOAD = dict(workload="cfg1: 100-bead CA chains, 512 structures/GPU, SchNet 3x(H=128,F=128), 128 expnorm RBF, rc=15A, energy+forces",
                structures_per_gpu=512, beads=100, bead_types=20, hidden=128, filters=128, num_rbf=128, interactions=3,
                cutoff_A=15.0, l2="flushed between steps (256 MiB write); edge tensors (>= 500 MB) exceed L2 as well")


# ----------------------------------------------------------------------------------------- workload
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


def make_inputs(B, n, n_types, seed):
    gen = torch.Generator().manual_seed(seed)
    pos = self_avoiding_chains(B, n, gen)
    types_ = torch.randint(0, n_types, (B * n,), generator=gen)
    batch = torch.arange(B).repeat_interleave(n)
    return pos, types_, batch


def make_model():
    from mlcg_b200 import nn as bnn
    torch.manual_seed(0)
    cut = bnn.CosineCutoff(0.0, WORKLOAD["cutoff_A"])
    rbf = bnn.ExpNormalBasis(cut, WORKLOAD["num_rbf"], trainable=False)
    return bnn.StandardSchNet(rbf, cut, [WORKLOAD["hidden"]], hidden_channels=WORKLOAD["hidden"], embedding_size=WORKLOAD["bead_types"],
                              num_filters=WORKLOAD["filters"], num_interactions=WORKLOAD["interactions"])


# ----------------------------------------------------------------------------------------- CPU legs
def oracle_step_fn(model_sd, pos, types_, batch, B):
    """One energy+force evaluation with the CPU oracle (radius graph included), returns (E, F)."""
    from oracle import radius_ref, schnet_ref
    cut = {"cutoff": "cosine", "lower": 0.0, "upper": WORKLOAD["cutoff_A"]}
    spec = {"kind": "expnormal", "rbf_cutoff": cut, "cutoff": cut, "activation": "tanh", "num_interactions": WORKLOAD["interactions"]}
    ptr = radius_ref.batch_to_ptr(batch.numpy(), B)

    def step():
        ei = torch.from_numpy(radius_ref.radius_graph_c(pos.numpy(), ptr, WORKLOAD["cutoff_A"], 1000, False, "cluster"))
        e, f, _ = schnet_ref.energy_and_forces(lambda p: schnet_ref.schnet_energy(model_sd, spec, p, types_, batch, ei, B), pos)
        return e, f

    return step


def cpu_leg(sample_B, steps, warmup):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    model = make_model()
    sd = {k: v.detach() for k, v in model.state_dict().items()}
    pos, types_, batch = make_inputs(sample_B, WORKLOAD["beads"], WORKLOAD["bead_types"], seed=0)
    step = oracle_step_fn(sd, pos, types_, batch, sample_B)
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(steps):
        step()
    dt = time.perf_counter() - t0
    return sample_B * steps / dt, dt / steps * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample_B = 128
    value, ms, cores = cpu_leg(sample_B, max(args.steps, 1), max(args.warmup, 1))
    sample = f"{sample_B} structures of the same workload per step (of 512), torch CPU float32, radius graph rebuilt each step"
    line = dict(metric=METRIC, value=value, unit="structures/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup, ms_per_step=ms,
                higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic", impl="reference",
                config=dict(WORKLOAD, sample_structures_per_step=sample_B),
                cpu_baseline=dict(value=value, unit="structures/s", cores=cores, kind="port", sample=sample),
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



# ----------------------------------------------------------------------------------------- other kernel families
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


def extra_measurements(dev, hbm_peak):
    """Kernel families that the headline step exercises only lightly, at the sizes of the other configurations:
    the stand-alone radius graph (256 x 4000 points, 60 A cube, 10 A cutoff) and the prior terms of the simulation
    configuration (1024 x 268 beads).  Device time, CUDA events; inputs are far larger than L2."""
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import get_backend
    be = get_backend()
    out = {}
    gen = torch.Generator().manual_seed(0)
    B, n = 256, 4000
    pos = (torch.rand(B * n, 3, generator=gen) * 60.0).to(dev)
    ptr = torch.arange(B + 1, device=dev) * n
    res = be.radius_graph(pos, ptr, 10.0, 1000, False, 1)
    E = int(res["edge_index"].shape[1])
    del res
    ms = time_cuda(lambda: be.radius_graph(pos, ptr, 10.0, 1000, False, 1), iters=5, warm=1)
    nbytes = 16 * E + 20 * B * n
    out["radius_graph_256x4000"] = dict(edges=E, ms=ms, edges_per_s=E / (ms / 1e3), algorithmic_GBps=nbytes / ms / 1e6,
                                        frac_of_hbm=nbytes / ms / 1e6 / hbm_peak,
                                        note="count + scan + host read of E + fill, allocation of the outputs included; "
                                             "algorithmic bytes = 16 B/edge written + 20 B/point read")
    del pos
    # priors of the simulation configuration
    Bp, npb = 1024, 268
    idx = torch.arange(npb, device=dev)
    full = torch.cartesian_prod(idx, idx).t()
    lists = {"bonds": torch.stack([idx[:-1], idx[1:]]), "angles": torch.stack([idx[:-2], idx[1:-1], idx[2:]]),
             "dihedrals": torch.stack([idx[:-3], idx[1:-2], idx[2:-1], idx[3:]]), "repulsion": full[:, (full[0] - full[1]).abs() >= 3]}
    ppos = self_avoiding_chains(Bp, npb, gen).to(dev)    # 3.8 A walk, no two beads closer than 4 A
    offs = (torch.arange(Bp, device=dev) * npb)
    n_par = {"bonds": 2, "angles": 2, "dihedrals": 7, "repulsion": 1}
    for kind, name in enumerate(["bonds", "angles", "dihedrals", "repulsion"]):
        m = lists[name]
        M = m.shape[1] * Bp
        mapping = (m[:, None, :] + offs[None, :, None]).reshape(m.shape[0], M).contiguous()
        mb = torch.arange(Bp, device=dev).repeat_interleave(m.shape[1])
        params = torch.rand(n_par[name], M, device=dev) + (3.0 if name in ("bonds", "repulsion") else 0.0)
        ms = time_cuda(lambda: be.prior_terms(kind, ppos, mapping, mb, params, Bp), iters=5, warm=1)
        nbytes = M * (8 * m.shape[0] + 8 + 4 * n_par[name]) + 2 * ppos.numel() * 4
        out[f"prior_{name}_1024x268"] = dict(terms=M, ms=ms, terms_per_s=M / (ms / 1e3), algorithmic_GBps=nbytes / ms / 1e6,
                                             frac_of_hbm=nbytes / ms / 1e6 / hbm_peak)
        del mapping, mb, params
    # Langevin dynamics of the simulation configuration: 1024 replicas x 268 beads, SchNet (3 blocks, 12 A) + the four
    # priors, BAOAB, graph rebuilt every step
    from mlcg_b200.simulation import LangevinSimulation
    import itertools
    T = 20
    torch.manual_seed(0)
    cut = bnn.CosineCutoff(0.0, 12.0)
    net = bnn.StandardSchNet(bnn.ExpNormalBasis(cut, 128, trainable=False), cut, [128], hidden_channels=128, embedding_size=T,
                             num_filters=128, num_interactions=3)
    stats2 = lambda d: {k: d for k in itertools.product(range(1), repeat=2)}
    pri = {"bonds": bnn.HarmonicBonds({(0, 0): {"k": 100.0, "x_0": 3.8}}), "angles": bnn.HarmonicAngles({(0, 0, 0): {"k": 50.0, "x_0": float(torch.cos(torch.tensor(1.9)))}}),
           "dihedrals": bnn.Dihedral({(0, 0, 0, 0): {"v_0": 0.0, "k1s": {"k1_1": 0.3, "k1_2": -0.2, "k1_3": 0.1}, "k2s": {"k2_1": 0.2, "k2_2": 0.1, "k2_3": -0.1}}}),
           "repulsion": bnn.Repulsion({(0, 0): {"sigma": 4.0}})}
    models = {"SchNet": bnn.GradientsOut(net, "forces")}
    models.update({k: bnn.GradientsOut(p, "forces") for k, p in pri.items()})
    model = bnn.SumOut(torch.nn.ModuleDict(models)).eval().to(dev)
    nls = {}
    for name in ["bonds", "angles", "dihedrals", "repulsion"]:
        m = lists[name]
        M = m.shape[1] * Bp
        nls[name] = mlcg_b200.make_neighbor_list(name, m.shape[0], (m[:, None, :] + offs[None, :, None]).reshape(m.shape[0], M).contiguous(),
                                                 torch.arange(Bp, device=dev).repeat_interleave(m.shape[1]))
    class _Data(mlcg_b200.AtomicData):
        pass
    data = _Data(pos=ppos.clone(), atom_types=torch.randint(0, T, (Bp * npb,), generator=gen).to(dev), batch=torch.arange(Bp, device=dev).repeat_interleave(npb),
                 n_atoms=torch.full((Bp,), npb, device=dev), neighbor_list=nls)
    # priors use bead type 0 tables: give them a type vector of zeros through their cached parameters
    zero_types = torch.zeros(Bp * npb, dtype=torch.long, device=dev)
    real_types = data.atom_types
    data.atom_types = zero_types
    for name, p in pri.items():
        p._cached_params(data)
    data.atom_types = real_types
    sim = LangevinSimulation(model, dt=0.002, friction=1.0, beta=1.0 / (0.0019872041 * 300), rng=torch.Generator(device=dev).manual_seed(0))
    sim.attach(data, torch.full((Bp * npb,), 12.0 / 418.39, device=dev))
    pot, forces = sim.calculate_potential_and_forces(sim.data)
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
    out["langevin_1024x268"] = dict(ms_per_md_step=ms, md_steps_per_s=1e3 / ms, replica_steps_per_s=Bp * 1e3 / ms, finite=bool(torch.isfinite(pot).all()),
                                    note="SchNet (3 blocks, 128 expnorm RBF, 12 A) + bonds/angles/dihedrals/repulsion(|i-j|>=3), BAOAB dt=2 fs, "
                                         "radius graph rebuilt every step, 1024 replicas on one GPU")
    return out

# ----------------------------------------------------------------------------------------- GPU arm
def run_ours(args):
    import torch.distributed as dist
    import mlcg_b200
    from mlcg_b200 import nn as bnn
    from mlcg_b200.backend import KernelProfiler, get_backend

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
    model = bnn.GradientsOut(make_model().to(dev), "forces").eval()
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
    # ---- the same K steps once more with a CUDA-event pair around every launch of the library (the per-kernel
    # durations behind `roofline` and `kernels`); kept out of the region above because ~170 event records per step
    # cost the host about as much as the launches themselves
    prof = KernelProfiler()
    be.profiler = prof
    ms_profiled = sum(timed_steps())
    stats = prof.summary()
    be.profiler = None
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
    barrier()

    t = torch.tensor([ms_total, e2e_s * 1e3, ms_profiled], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, e2e_ms, ms_profiled = float(t[0]), float(t[1]), float(t[2])
    # the ranks part here: everything below is rank 0's own reporting (no collective may follow)
    if world > 1:
        dist.barrier()
        group["alive"] = False
        dist.destroy_process_group()
    if rank != 0:
        return

    # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels on this workload, from the
    # Nsight Compute capture summarised under profiles/ (full-size launches; scaled by the row count for other sizes)
    ncu_traffic = {"filter_backward": 75.1e6, "filter_forward": 230.5e6, "seg_mul_sum": 343.3e6, "gemm_tc": 39.0e6}
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = peaks.get("hbm_gbs", 6650.0)
    tf_peak = peaks.get("bf16_tflops_sustained", 1400.0)
    peak_src = "measured" if peaks else "fallback"
    top = max(stats.items(), key=lambda kv: kv[1]["ms"])
    name, st = top
    per_launch_ms = st["ms"] / max(st["calls"], 1)
    tensor_kernels = {"gemm": "gemm_kernel<float> (filter-network GEMMs, fp32 FMA)",
                      "filter_forward": "filter_fwd_pipe_kernel (tcgen05: RBF prologue, 2 GEMMs, tanh, cutoff; one row per unordered pair)",
                      "filter_backward": "filter_bwd_pipe_kernel (tcgen05: recompute + 4 GEMMs per tile, gather of gW; one row per unordered pair)"}
    if name in tensor_kernels:
        achieved = st["flops"] / max(st["ms"], 1e-9) / 1e9            # TFLOP/s of algorithmic (fp32-equivalent) flops
        roof = dict(kernel=tensor_kernels[name], bound="tensor", achieved=achieved, peak=tf_peak, unit="TFLOP/s", frac=achieved / tf_peak,
                    traffic=ncu_traffic.get(name, 0) * B / 512 or None, peak_source=f"{peak_src} bf16 sustained", avg_launch_ms=per_launch_ms,
                    note="algorithmic flops 2*F*(R+F) per evaluated row and GEMM pair (rows = E/2 on a symmetric edge list); the fp32-equivalent "
                         "mode issues three fp16 products per algorithmic product, so tensor-pipe work is 3x this figure")
    else:
        achieved = st["bytes"] / max(st["ms"], 1e-9) / 1e6            # GB/s
        roof = dict(kernel=name, bound="hbm", achieved=achieved, peak=hbm_peak, unit="GB/s", frac=achieved / hbm_peak,
                    traffic=ncu_traffic.get(name, 0) * B / 512 or None,
                    peak_source=f"{peak_src} copy bandwidth", avg_launch_ms=per_launch_ms)
    seg = stats.get("seg_mul_sum")
    cfconv = None
    if seg and seg["ms"] > 0:
        # algorithmic bytes of the CFConv aggregation per edge: the filter row (4F), the [2,E] int64 indices (16) and the node
        # tensors read and written once (8F N/E); what the kernel really moves is less, because it reads one filter row per
        # unordered pair and int32 indices (`unique_GBps`)
        F, n_nodes = WORKLOAD["filters"], B * n
        per_edge = 4 * F + 16 + 8 * F * n_nodes / n_edges
        edges_per_s = seg["calls"] * n_edges / (seg["ms"] / 1e3)
        gbs = per_edge * edges_per_s / 1e9
        cfconv = dict(kernel="seg_mul_sum_kernel<float,32,true,true> (CFConv gather * filter, segmented sum; filters stored once per pair)", bound="hbm", achieved=gbs,
                      peak=hbm_peak, unit="GB/s", frac=gbs / hbm_peak, edges_per_s=edges_per_s, bytes_per_edge=per_edge,
                      unique_GBps=seg["bytes"] / seg["ms"] / 1e6, traffic=ncu_traffic["seg_mul_sum"] * B / 512, avg_launch_ms=seg["ms"] / seg["calls"])
    kernels = {k: dict(calls=v["calls"], ms_per_step=v["ms"] / args.steps,
                       GBps=(v["bytes"] / v["ms"] / 1e6 if v["ms"] > 0 else None),
                       TFLOPs=(v["flops"] / v["ms"] / 1e9 if v["ms"] > 0 and v["flops"] else None)) for k, v in sorted(stats.items(), key=lambda kv: -kv[1]["ms"])}

    cpu = None
    if not args.no_cpu and world == 1:        # the CPU leg is timed at N = 1 only (other ranks would share the host cores)
        sample_B = 128
        v, ms, cores = cpu_leg(sample_B, 16, 1)     # about 10 s of host work
        cpu = dict(value=v, unit="structures/s", cores=cores, kind="port",
                   sample=f"{sample_B} structures of the same workload per step, 16 steps after 1 warm-up, torch CPU float32 + C radius oracle")

    extras = None
    if not args.no_extras and world == 1:      # side measurements of other kernels and configurations: single-GPU runs only
        try:
            # the same step with the filter-network GEMMs on bf16 operands (forces within 1e-2 relative RMS of the fp32 mode)
            bnn.set_filter_precision(model, "bf16")
            for _ in range(3):
                step_resident()
            bf16_ms = timed_steps()
            bnn.set_filter_precision(model, "fp32")
            del flush
            torch.cuda.empty_cache()
            extras = extra_measurements(dev, hbm_peak)
            extras["bf16_filter_mode"] = dict(ms_per_step=sum(bf16_ms) / len(bf16_ms), structures_per_s=B / (sum(bf16_ms) / len(bf16_ms) / 1e3),
                                              note="same workload, filter-network GEMMs with bf16 operands (one product, tanh.approx)")
        except Exception as exc:   # the headline line is still printed
            extras = {"error": repr(exc)}

    # kernels of the library per evaluation on the route the timed region takes (one library call for the model): radius graph 7
    # (cells, count, three scan kernels, clamp to the capacity, fill), reverse-edge map / pair selection / pair index 5 (count of
    # upper edges, three scan kernels, plan), distances 1, embedding 1, five per block
    # forward, output network 3 (layer + tanh, dot product, per-structure sum), its derivative 1, five per block backward
    # (three for the first block, whose input gradient nobody needs; the distance gradients of the blocks are added up by
    # the filter kernels), distance backward 1
    L = WORKLOAD["interactions"]
    launches_timed = args.steps * (7 + 5 + 1 + 1 + 5 * L + 3 + 1 + 5 * (L - 1) + 3 + 1)
    value = world * B * args.steps / (ms_total / 1e3)
    h2d = pos_h.numel() * 4 + types_h.numel() * 8 + batch_h.numel() * 8
    d2h = B * 4 + pos_h.numel() * 4
    line = dict(metric=METRIC, value=value, unit="structures/s", n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                ms_per_step=ms_total / args.steps, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(WORKLOAD, edges_per_gpu=n_edges, edge_capacity=int(1.1 * n_edges) + int(1.1 * n_edges) % 2, global_structures=world * B, parallelism=f"replicas x{world}, no collective",
                            kernel_timing="second pass over the same K steps with a CUDA-event pair around every library launch "
                                          "(the package then issues its kernels one by one instead of one library call per evaluation)"),
                e2e=dict(value=world * B * args.steps / (e2e_ms / 1e3), unit="structures/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h),
                gpu_launches=launches_timed, gpu_launches_kernel_timing_pass=prof.total_launches, ms_per_step_median=sorted(step_ms)[len(step_ms) // 2], ms_per_step_min=min(step_ms),
                ms_per_step_with_kernel_events=ms_profiled / args.steps, roofline=roof, cfconv_roofline=cfconv, other_kernels=extras, cpu_baseline=cpu, clocks=clk, kernels=kernels,
                edges_per_s=world * n_edges * args.steps / (ms_total / 1e3))
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--structures", type=int, default=None, help="structures per GPU (default 512; smaller values are for profiler captures)")
    ap.add_argument("--no-extras", action="store_true", help="skip the stand-alone radius-graph and prior-kernel measurements")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiler captures)")
    args = ap.parse_args()
    if args.structures:
        WORKLOAD["structures_per_gpu"] = args.structures
        WORKLOAD["workload"] += f" [REDUCED to {args.structures} structures/GPU: not the benchmark configuration]"
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
