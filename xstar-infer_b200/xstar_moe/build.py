"""Builds the native pieces in-tree: libxs_moe.so (CUDA kernels + C ABI, sm_100a) and the `xstar_cpp`
pybind11 module (host C++ mirror of the reference's op interface)."""
import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
HOST = os.path.join(PKG, "host")
LIB = os.path.join(PKG, "libxs_moe.so")
PYMOD_DIR = os.path.join(PKG, "xstar_cpp_py")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17"]


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(d, exts):
    out = []
    for r, _, fs in os.walk(d):
        out += [os.path.join(r, f) for f in fs if f.endswith(exts)]
    return out


def build_cuda(force=False, verbose=False):
    srcs = _sources(CSRC, (".cu", ".cuh", ".inl", ".h")) + _sources(os.path.join(ROOT, "include"), (".h",))
    if not (force or _newer(LIB, srcs)):
        return LIB
    cmd = ["nvcc", *NVCC_FLAGS, "-shared", "-Xcompiler", "-fPIC", "-I" + os.path.join(ROOT, "include"), "-o", LIB,
           os.path.join(CSRC, "xs_moe_api.cu"), "-ldl"]
    if verbose:
        cmd.insert(1, "-Xptxas=-v")
    subprocess.run(cmd, check=True)
    return LIB


def build_host(force=False):
    """g++-only: the host side never includes a CUDA header; it reaches the device through the C ABI."""
    if not os.path.isdir(HOST):
        return None
    import pybind11

    ext = sysconfig.get_config_var("EXT_SUFFIX")
    os.makedirs(PYMOD_DIR, exist_ok=True)
    target = os.path.join(PYMOD_DIR, "xstar_cpp" + ext)
    srcs = _sources(HOST, (".cpp", ".h")) + _sources(os.path.join(ROOT, "include"), (".h",))
    if not (force or _newer(target, srcs) or _newer(target, [LIB])):
        return target
    cpps = [s for s in srcs if s.endswith(".cpp")]
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-fvisibility=hidden", "-I" + os.path.join(HOST, "include"),
           "-I" + os.path.join(ROOT, "include"), "-I" + pybind11.get_include(), "-I" + sysconfig.get_paths()["include"],
           "-o", target, *cpps, "-L" + PKG, "-lxs_moe", "-Wl,-rpath,$ORIGIN/..", "-lpthread"]
    subprocess.run(cmd, check=True)
    return target


def build_all(force=False):
    build_cuda(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("built", LIB)
