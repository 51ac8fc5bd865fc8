"""Build recipe for the CPU oracle (test infrastructure; never imported by the product package).

`python oracle/build.py` compiles oracle/qc_oracle.c into oracle/_build/libqc_oracle.so with gcc.
Floating-point contraction and fast-math are disabled so every fp32 operation is a single
correctly-rounded IEEE operation, which the bit-exact comparisons rely on.

`python oracle/build.py --ref [PATH]` additionally installs the UNMODIFIED reference project
(vkuzo/quant_cast_bench, a pure-Python package) from a checkout into oracle/_ref/ with an offline
`pip install --no-deps --target` (from a temporary copy, so the checkout itself is never written to).
oracle/_ref/ is kept out of version control; it exists so that the benchmark's comparison legs can run the
reference's own gold recipes on the host CPU and its own Triton kernels on the GPU next to this backend
(see oracle/ref_gold.py).  PATH defaults to $QCC_REFERENCE_ROOT, else a checkout named `reference`
beside this repository.  Nothing of the reference is copied into tracked files.
"""
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "qc_oracle.c")
OUT_DIR = os.path.join(HERE, "_build")
OUT = os.path.join(OUT_DIR, "libqc_oracle.so")


def build(force: bool = False) -> str:
    os.makedirs(OUT_DIR, exist_ok=True)
    if not force and os.path.exists(OUT) and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    cmd = [
        "gcc", "-O2", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-fno-unsafe-math-optimizations",
        "-shared", "-fPIC", "-o", OUT, SRC, "-lm",
    ]
    subprocess.run(cmd, check=True)
    return OUT


REF_DIR = os.path.join(HERE, "_ref")


def find_reference(path=None):
    """The reference checkout to install from, or None."""
    cands = [path, os.environ.get("QCC_REFERENCE_ROOT"), os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "quant_cast_bench", "quant_cast_gold", "recipes.py")):
            return c
    return None


def build_ref(path=None, force: bool = False):
    """Install the reference package into oracle/_ref/ (returns that directory, or None when no checkout is found)."""
    marker = os.path.join(REF_DIR, "quant_cast_bench", "quant_cast_gold", "recipes.py")
    if os.path.exists(marker) and not force:
        return REF_DIR
    src = find_reference(path)
    if src is None:
        return None
    with tempfile.TemporaryDirectory() as tmp:
        work = os.path.join(tmp, "src")
        shutil.copytree(src, work, ignore=shutil.ignore_patterns(".git", "*.egg-info", "__pycache__"))
        if os.path.isdir(REF_DIR):
            shutil.rmtree(REF_DIR)
        cmd = [sys.executable, "-m", "pip", "install", "--quiet", "--no-index", "--no-build-isolation", "--no-deps",
               "--target", REF_DIR, work]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0 or not os.path.exists(marker):
            # pip could not build it here: the package is pure Python, so its directory is the install
            os.makedirs(REF_DIR, exist_ok=True)
            shutil.copytree(os.path.join(work, "quant_cast_bench"), os.path.join(REF_DIR, "quant_cast_bench"), dirs_exist_ok=True)
    return REF_DIR if os.path.exists(marker) else None


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        i = sys.argv.index("--ref")
        arg = sys.argv[i + 1] if i + 1 < len(sys.argv) and not sys.argv[i + 1].startswith("-") else None
        print(build_ref(arg, force="--force" in sys.argv))
