"""TEST INFRASTRUCTURE — run the reference's own native extension (``oracle/_ref/radius_kernel.so``, built by
``oracle/build_ref.py``) on a list of jobs, in a process of its own.

    python oracle/ref_runner.py <jobs.pt> <results.pt>

``jobs.pt`` is a ``torch.save``d list of dictionaries:

* ``{"op": "radius_cuda", "x", "ptr_x" | None, "r", "max_num_neighbors", "ignore_same_index",
  "exclude_pair_xs" | None, "ptr_exclude_pair_xs" | None}`` — tensors on the CPU; they are moved to ``cuda:0``, the
  extension's ``radius_cuda`` is called with exactly these seven arguments (its signature at
  ``src/opt_radius/mlcg_opt_radius/radius.cu:197-203``) and ``(edge_index [2,E] contiguous, distance [E])`` come back on the CPU;
* ``{"op": "exclusion_pair_to_ptr", "pairs" [2,P] int64, "num_nodes"}`` — runs on the CPU
  (``exclusion_pairs.cpp:7-62``) and returns ``(pair_xs, y_ptr)``;
* ``{"op": "schemas"}`` — the schema strings under which the extension registered ``mlcg::radius_cuda`` and
  ``mlcg::exclusion_pair_to_ptr`` (``radius.cu:313-314``, ``exclusion_pairs.cpp:64-65``).

A separate process because the extension registers ``mlcg::radius_cuda`` and ``mlcg::exclusion_pair_to_ptr`` with torch's
dispatcher, which a process can do only once per name.
"""
import importlib.util
import os
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "_ref", "radius_kernel.so")


def available() -> bool:
    return os.path.exists(SO)


def _load():
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    spec = importlib.util.spec_from_file_location("radius_kernel", SO)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _main(jobs_path, results_path):
    import torch
    mod = _load()
    jobs = torch.load(jobs_path, weights_only=False)
    results = []
    for job in jobs:
        if job["op"] == "exclusion_pair_to_ptr":
            xs, ptr = mod.exclusion_pair_to_ptr(job["pairs"], int(job["num_nodes"]))
            results.append((xs.clone(), ptr.clone()))
        elif job["op"] == "radius_cuda":
            dev = torch.device("cuda:0")
            on = lambda t: None if t is None else t.to(dev)
            ei, dist = mod.radius_cuda(on(job["x"]).contiguous(), on(job["ptr_x"]), float(job["r"]), int(job["max_num_neighbors"]),
                                       bool(job["ignore_same_index"]), on(job["exclude_pair_xs"]), on(job["ptr_exclude_pair_xs"]))
            torch.cuda.synchronize()
            results.append((ei.contiguous().cpu(), dist.cpu()))
        elif job["op"] == "schemas":
            results.append((str(torch.ops.mlcg.radius_cuda.default._schema), str(torch.ops.mlcg.exclusion_pair_to_ptr.default._schema)))
        else:
            raise ValueError(job["op"])
    torch.save(results, results_path)


def run(jobs, timeout=600):
    """Run ``jobs`` in a child process and return the list of results (used by the tests)."""
    import torch
    if not available():
        raise FileNotFoundError(SO)
    with tempfile.TemporaryDirectory() as tmp:
        a, b = os.path.join(tmp, "jobs.pt"), os.path.join(tmp, "results.pt")
        torch.save(jobs, a)
        proc = subprocess.run([sys.executable, os.path.abspath(__file__), a, b], capture_output=True, text=True, timeout=timeout)
        if proc.returncode != 0:
            raise RuntimeError(f"reference extension failed (exit {proc.returncode}):\n{proc.stdout[-2000:]}\n{proc.stderr[-4000:]}")
        return torch.load(b, weights_only=False)


if __name__ == "__main__":
    _main(sys.argv[1], sys.argv[2])
