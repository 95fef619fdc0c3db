"""In-tree build of the native libraries (sm_100a only).

* ``sru_b200/lib/libsru_b200.so``        -- CUDA kernels + the C ABI of include/sru_b200.h
  (nvcc, no torch dependency).
* ``sru_b200/lib/libsru_b200_torch.so``  -- the torch operator binding that registers the
  reference's ``sru_cuda::*`` operator names on top of the C ABI (g++ against libtorch).

Run ``python -m sru_b200.build`` (add ``--force`` to rebuild everything).
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(HERE, "_obj")
CAPI_SO = os.path.join(LIBDIR, "libsru_b200.so")
TORCH_SO = os.path.join(LIBDIR, "libsru_b200_torch.so")
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
NVCC = os.path.join(CUDA_HOME, "bin", "nvcc")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC", "-Xcompiler", "-Wno-unused-variable",
]


def _deps(src):
    hdrs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    hdrs.append(os.path.join(HERE, "..", "include", "sru_b200.h"))
    return [src] + hdrs


def _stale(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _compile_cu(src, force, verbose):
    obj = os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")
    if not force and not _stale(obj, _deps(src)):
        return obj
    cmd = [NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed on " + src)
    return obj


def build_capi(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    os.makedirs(OBJDIR, exist_ok=True)
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile_cu(s, force, verbose), srcs))
    if force or _stale(CAPI_SO, objs):
        cmd = [NVCC, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", CAPI_SO] + objs + ["-lcudart", "-lcuda"]
        subprocess.check_call(cmd)
    return CAPI_SO


def build_torch_binding(force=False):
    src = os.path.join(CSRC, "torch_binding.cpp")
    if not os.path.exists(src):
        return None
    build_capi()
    if not force and not _stale(TORCH_SO, [src, CAPI_SO, os.path.join(HERE, "..", "include", "sru_b200.h")]):
        return TORCH_SO
    import torch
    from torch.utils import cpp_extension as ce
    incs = []
    for p in ce.include_paths():
        incs += ["-isystem", p]
    incs += ["-isystem", os.path.join(CUDA_HOME, "include")]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + incs + [
           src, "-o", TORCH_SO, "-L" + LIBDIR, "-lsru_b200", "-Wl,-rpath,$ORIGIN",
           "-L" + tlib, "-Wl,-rpath," + tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda", "-lc10_cuda",
           "-L" + os.path.join(CUDA_HOME, "lib64"), "-lcudart"]
    subprocess.check_call(cmd)
    return TORCH_SO


TS_HOST = os.path.join(LIBDIR, "sru_b200_ts_host")


def build_ts_host(force=False):
    """The C++ host of tests/cpp/ts_host.cpp: a libtorch program linked against the operator binding the way a C++
    application of the reference links libsru_cuda (sru/csrc/CMakeLists.txt:38-44: --no-as-needed, so that the
    registrations run at load time).  Test infrastructure; returns the path of the executable."""
    src = os.path.join(HERE, "..", "tests", "cpp", "ts_host.cpp")
    if not os.path.exists(src):
        return None
    build_torch_binding()
    if not force and not _stale(TS_HOST, [src, TORCH_SO]):
        return TS_HOST
    import torch
    from torch.utils import cpp_extension as ce
    incs = []
    for p in ce.include_paths():
        incs += ["-isystem", p]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O1", "-std=c++17", "-w",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + incs + [
           src, "-o", TS_HOST, "-L" + LIBDIR, "-Wl,--no-as-needed", "-lsru_b200_torch", "-lsru_b200",
           "-Wl,-rpath,$ORIGIN", "-L" + tlib, "-Wl,-rpath," + tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-ltorch_cuda",
           "-lc10_cuda", "-Wl,--as-needed", "-lpthread"]
    subprocess.check_call(cmd)
    return TS_HOST


def build_all(force=False, verbose=False):
    return build_capi(force, verbose), build_torch_binding(force)


if __name__ == "__main__":
    print(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv))
