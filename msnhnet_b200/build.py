"""Builds the native libraries in-tree.

  libmsnh_b200.so      CUDA kernels + plan compiler behind the C ABI of include/msnh_b200.h (nvcc, sm_100a only)
  libmsnhnet_host.so   the C++ host side: .msnhnet parser, NetBuilder mirror, the reference's 13 C entry points

Run as `python -m msnhnet_b200.build` or through `__graft_entry__.build()`.
"""
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
HOST = os.path.join(HERE, "host")
KERNEL_LIB = os.path.join(HERE, "libmsnh_b200.so")
HOST_LIB = os.path.join(HERE, "libmsnhnet_host.so")


def _newer(target, sources):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources)


def _sources(folder, exts):
    out = []
    for name in sorted(os.listdir(folder)):
        if name.endswith(exts):
            out.append(os.path.join(folder, name))
    return out


def _host_cxx():
    # the first g++ on PATH in some images is a wrapper that cannot link OpenMP; prefer the distro one
    return "/usr/bin/g++" if os.access("/usr/bin/g++", os.X_OK) else (shutil.which("g++") or "g++")


def build_kernels(force=False, verbose=False):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    deps = _sources(CSRC, (".cu", ".cuh", ".h")) + [os.path.join(ROOT, "include", "msnh_b200.h")]
    if not force and not _newer(KERNEL_LIB, deps):
        return KERNEL_LIB
    cmd = [nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "--threads", "0",
           "-Xcompiler", "-fPIC", "-shared", "-ccbin", _host_cxx(),
           "-o", KERNEL_LIB] + _sources(CSRC, (".cu",))
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return KERNEL_LIB


def build_host(force=False):
    deps = _sources(HOST, (".cpp", ".h")) + [os.path.join(ROOT, "include", "msnh_b200.h"),
                                             os.path.join(ROOT, "include", "msnhnet_capi.h")]
    deps = [d for d in deps if os.path.exists(d)]
    if not force and not _newer(HOST_LIB, deps):
        return HOST_LIB
    cmd = [_host_cxx(), "-O2", "-std=c++17", "-fPIC", "-shared", "-Wall", "-I", os.path.join(ROOT, "include"),
           "-o", HOST_LIB] + _sources(HOST, (".cpp",)) + ["-L", HERE, "-lmsnh_b200", "-Wl,-rpath,$ORIGIN", "-lpthread"]
    subprocess.run(cmd, check=True)
    return HOST_LIB


def build_all(force=False, verbose=False):
    build_kernels(force, verbose)
    if os.path.isdir(HOST) and _sources(HOST, (".cpp",)):
        build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built", KERNEL_LIB)
