"""Build recipe for the CPU oracle (test infrastructure, never part of the product path).

Two artefacts:

* ``oracle/libsru_oracle.so`` -- the plain-C restatement in ``sru_oracle.c``
  (gcc, OpenMP over columns).  Always built.
* ``oracle/_ref/libsru_cpu_ref.so`` -- the reference's OWN forward-only CPU scan,
  compiled from its single source file ``sru/csrc/sru_cpu_impl.cpp`` where it lies
  in the reference checkout (g++ against the installed libtorch; no source is
  copied).  Built only where the reference checkout is present; the built file is
  git-ignored and is used to cross-check the restatement and as a timed baseline.
  It registers ``torch.ops.sru_cpu.cpu_forward`` / ``cpu_bi_forward``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
# the reference checkout: $SRU_REFERENCE_ROOT, or a directory "reference" beside this repository
REF_ROOT = os.environ.get("SRU_REFERENCE_ROOT",
                          os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
ORACLE_SO = os.path.join(HERE, "libsru_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libsru_cpu_ref.so")


def _newer(target, *sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force=False):
    src = os.path.join(HERE, "sru_oracle.c")
    inc = os.path.join(HERE, "sru_oracle_body.inc")
    if not force and _newer(ORACLE_SO, src, inc):
        return ORACLE_SO
    cmd = ["gcc", "-O2", "-fno-fast-math", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           "-o", ORACLE_SO, src, "-lm"]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference_cpu(force=False):
    """Compile the reference's sru_cpu_impl.cpp in place.  Returns the .so path or None."""
    src = os.path.join(REF_ROOT, "sru", "csrc", "sru_cpu_impl.cpp")
    if not os.path.exists(src):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, src):
        return REF_SO
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(REF_DIR, exist_ok=True)
    incs = []
    for p in ce.include_paths():
        incs += ["-isystem", p]
    libdir = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O3", "-std=c++17", "-shared", "-fPIC", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + incs + [
           src, "-o", REF_SO, "-L" + libdir, "-Wl,-rpath," + libdir,
           "-ltorch", "-ltorch_cpu", "-lc10"]
    subprocess.check_call(cmd)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    print(build_reference_cpu(force="--force" in sys.argv))
