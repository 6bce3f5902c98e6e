"""Build the native parts in-tree: lib/libb200q.so (CUDA kernels + C ABI, sm_100a only) and
lib/b200_hpu_ops_ext.so (the C++ torch extension that registers the hpu::* operators).

Usage: python build.py [--force] [--verbose-ptxas]
Objects are rebuilt only when a source or header is newer.
"""
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "lib")
OBJ = os.path.join(HERE, "build")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _newer(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _run(cmd, quiet=True):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0 or not quiet:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd[:3]))
    return r.stdout + r.stderr


def build_kernels(force=False, ptxas_verbose=False):
    os.makedirs(LIB, exist_ok=True)
    os.makedirs(OBJ, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(ROOT, "include", "*.h"))
    objs = []
    log = ""
    for src in sorted(glob.glob(os.path.join(CSRC, "*.cu"))):
        obj = os.path.join(OBJ, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        if force or _newer(obj, [src] + headers):
            cmd = [NVCC, *ARCH, "-O3", "-lineinfo", "-std=c++17", "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
                   "-I", os.path.join(ROOT, "include"), "-I", CSRC, "-c", src, "-o", obj]
            if ptxas_verbose:
                cmd[1:1] = ["-Xptxas", "-v"]
            log += _run(cmd)
    so = os.path.join(LIB, "libb200q.so")
    if force or _newer(so, objs):
        _run([NVCC, *ARCH, "-shared", "-o", so, *objs])
    return so, log


def build_torch_ext(force=False):
    import torch
    from torch.utils import cpp_extension as ce

    src = os.path.join(CSRC, "torch_ext", "hpu_ops.cpp")
    so = os.path.join(LIB, "b200_hpu_ops_ext.so")
    deps = [src, os.path.join(ROOT, "include", "b200q.h"), os.path.join(LIB, "libb200q.so")]
    if not (force or _newer(so, deps)):
        return so
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    inc = []
    for p in ce.include_paths():
        inc += ["-isystem", p]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI),
           "-DTORCH_API_INCLUDE_EXTENSION_H", *inc, "-isystem", "/usr/local/cuda/include",
           "-I", os.path.join(ROOT, "include"), src, "-o", so,
           "-L", LIB, "-lb200q", "-Wl,-rpath,$ORIGIN", "-L", tlib, "-ltorch", "-ltorch_cpu", "-lc10", "-lc10_cuda",
           "-ltorch_cuda", "-Wl,-rpath," + tlib]
    _run(cmd)
    return so


def build_all(force=False, ptxas_verbose=False):
    so, log = build_kernels(force, ptxas_verbose)
    ext = build_torch_ext(force)
    return so, ext, log


if __name__ == "__main__":
    so, ext, log = build_all("--force" in sys.argv, "--verbose-ptxas" in sys.argv)
    if "--verbose-ptxas" in sys.argv:
        print(log)
    print(so)
    print(ext)
