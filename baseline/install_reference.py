"""Puts the unmodified reference where `bench.py --impl reference` looks for it: baseline/_ref.

    python baseline/install_reference.py [path of the reference checkout]

First the documented way, an offline `pip install --target baseline/_ref <reference>`; the
reference has neither setup.py nor pyproject.toml at its root, so pip refuses it, and what
runs unmodified is its own PyTorch benchmark on the NCCL backend. The fallback is therefore a
plain copy of the reference's `dev_root/benchmarks/` directory to baseline/_ref/benchmarks/.
The reference is looked for in the path given, in $SWITCHML_REFERENCE_ROOT, or in a directory
called `reference` next to this repository. Nothing is changed in the reference itself.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
TARGET = os.path.join(HERE, "_ref")
SCRIPT = os.path.join(TARGET, "benchmarks", "allreduce_pytorch_benchmark", "allreduce_pytorch_benchmark.py")


def find_reference(argv):
    candidates = list(argv) + [os.environ.get("SWITCHML_REFERENCE_ROOT", ""),
                               os.path.join(os.path.dirname(REPO), "reference")]
    for c in candidates:
        if c and os.path.isdir(os.path.join(c, "dev_root", "benchmarks")):
            return c
    return None


def install(reference, try_pip=True, quiet=False):
    """Returns "pip", "copy" or None (nothing to install from)."""
    if reference is None:
        return None
    os.makedirs(TARGET, exist_ok=True)
    if try_pip:
        cmd = [sys.executable, "-m", "pip", "install", "--no-index", "--no-build-isolation"]
        if os.environ.get("SWITCHML_WHEELHOUSE"):  # directory of wheels for an offline install
            cmd += ["--find-links", os.environ["SWITCHML_WHEELHOUSE"]]
        cmd += ["--target", TARGET, reference]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode == 0:
            return "pip"
        if not quiet:
            print("pip cannot install the reference: %s" % (r.stderr.strip().splitlines() or ["?"])[-1])
    dst = os.path.join(TARGET, "benchmarks")
    if os.path.isdir(dst):
        shutil.rmtree(dst)
    shutil.copytree(os.path.join(reference, "dev_root", "benchmarks"), dst)
    return "copy"


def ensure(quiet=True):
    """Install only if the benchmark script is not there yet (used by the build entry point)."""
    if os.path.exists(SCRIPT):
        return "present"
    return install(find_reference([]), try_pip=False, quiet=quiet)


if __name__ == "__main__":
    how = install(find_reference(sys.argv[1:]))
    if how is None:
        sys.exit("no reference checkout found (argument, $SWITCHML_REFERENCE_ROOT or ../reference)")
    print("reference available under baseline/_ref (%s)" % how)
