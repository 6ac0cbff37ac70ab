"""TEST INFRASTRUCTURE — build the reference itself as a comparator and as the timed CPU baseline.

    python oracle/build_ref.py /path/to/mlcg [--force]

Two products, both under ``oracle/_ref/`` (kept out of version control; they travel to a GPU machine with the working tree):

1. ``radius_kernel.so`` — the reference's native radius-graph extension (below);
2. ``site/mlcg`` — the reference's Python package, installed by pip (``--no-deps``: its dependencies are not available, and
   ``oracle/mlcg_loader.py`` loads the hot-path modules without them).  ``bench.py --impl reference`` and the bench's
   CPU-baseline legs time these modules.

Compiles ``src/opt_radius/mlcg_opt_radius/{binding.cpp, radius.cu, exclusion_pairs.cpp}`` of a checkout of
ClementiGroup/mlcg, from where they lie, the way the reference's own just-in-time recipe does
(``src/opt_radius/mlcg_opt_radius/radius.py:24-34``: ``torch.utils.cpp_extension.load`` with ``-O3`` for
both compilers), for sm_100a, into ``oracle/_ref/radius_kernel.so``.  Nothing of the reference is copied
into this repository: ``oracle/_ref/`` holds build products only and is kept out of version control.

The product never loads this file.  ``oracle/ref_runner.py`` loads it in a process of its own (it registers
``mlcg::radius_cuda`` and ``mlcg::exclusion_pair_to_ptr`` with torch's dispatcher, the names the product
registers too), and only the tests start that process.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
SO = os.path.join(OUT, "radius_kernel.so")
SOURCES = ["binding.cpp", "radius.cu", "exclusion_pairs.cpp"]


def source_dir(ref_root: str) -> str:
    return os.path.join(ref_root, "src", "opt_radius", "mlcg_opt_radius")


def up_to_date(ref_root: str) -> bool:
    if not os.path.exists(SO):
        return False
    srcs = [os.path.join(source_dir(ref_root), s) for s in SOURCES]
    return all(os.path.exists(s) and os.path.getmtime(SO) >= os.path.getmtime(s) for s in srcs)


def build(ref_root: str, force: bool = False, verbose: bool = False) -> str:
    """Returns the path of the built extension (several minutes on first use: torch's headers are heavy)."""
    if not force and up_to_date(ref_root):
        return SO
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")       # no GPU is needed to compile
    from torch.utils.cpp_extension import load
    load(name="radius_kernel", sources=[os.path.join(source_dir(ref_root), s) for s in SOURCES], extra_cflags=["-O3"],
         extra_cuda_cflags=["-O3"], build_directory=OUT, verbose=verbose)
    for leftover in ("build.ninja", ".ninja_deps", ".ninja_log"):
        p = os.path.join(OUT, leftover)
        if os.path.exists(p):
            os.remove(p)
    return SO


def install_python(ref_root: str, force: bool = False) -> str:
    """``pip install --no-deps --target oracle/_ref/site`` of the reference checkout (from a temporary copy, because the
    build writes into the source tree and a checkout may be read-only).  Returns the installed package directory."""
    import shutil
    import subprocess
    import tempfile
    site = os.path.join(OUT, "site")
    pkg = os.path.join(site, "mlcg")
    if os.path.isdir(pkg) and not force:
        return pkg
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory() as tmp:
        copy = os.path.join(tmp, "mlcg_src")
        shutil.copytree(ref_root, copy, ignore=shutil.ignore_patterns(".git", "docs", "examples", "tests"))
        if os.path.isdir(site):
            shutil.rmtree(site)
        subprocess.check_call([sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
                               "--target", site, copy])
    return pkg


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python oracle/build_ref.py <path to a checkout of ClementiGroup/mlcg> [--force]")
    print(install_python(sys.argv[1], force="--force" in sys.argv))
    print(build(sys.argv[1], force="--force" in sys.argv, verbose=True))
