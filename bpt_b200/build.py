"""Builds libbpt_b200.so (the C-ABI CUDA library) in-tree with nvcc for sm_100a.

Usage: python -m bpt_b200.build [--force] [--verbose]
"""
import glob
import os
import subprocess
import sys

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG_DIR, "csrc")
OBJ_DIR = os.path.join(CSRC, "_obj")
LIB_PATH = os.path.join(PKG_DIR, "libbpt_b200.so")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "--expt-extended-lambda", "-Xcompiler", "-fPIC",
    "-diag-suppress", "20012",
]


def _nvcc():
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    raise RuntimeError("nvcc not found")


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _deps():
    return sorted(glob.glob(os.path.join(CSRC, "*.cuh"))) + \
        [os.path.join(os.path.dirname(PKG_DIR), "include", "bpt_b200.h"), os.path.abspath(__file__)]


def build(force=False, verbose=False):
    """Compile every csrc/*.cu to an object and link them into libbpt_b200.so.
    Objects are rebuilt only when their source or a header is newer."""
    os.makedirs(OBJ_DIR, exist_ok=True)
    nvcc = _nvcc()
    dep_mtime = max(os.path.getmtime(p) for p in _deps())
    objs, procs = [], []
    for src in sources():
        obj = os.path.join(OBJ_DIR, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        stale = force or not os.path.exists(obj) or \
            os.path.getmtime(obj) < max(os.path.getmtime(src), dep_mtime)
        if stale:
            cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
            procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT)))
    failed = False
    for src, p in procs:
        out = p.communicate()[0].decode()
        if p.returncode != 0 or verbose:
            sys.stderr.write("== %s\n%s\n" % (os.path.basename(src), out))
        failed = failed or p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    if procs or not os.path.exists(LIB_PATH):
        tmp = LIB_PATH + ".tmp%d" % os.getpid()
        subprocess.check_call([nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", tmp] + objs + ["-lcudart", "-lcublas"])
        os.replace(tmp, LIB_PATH)
    return LIB_PATH


EXT_SRC = os.path.join(PKG_DIR, "csrc_torch", "graphop_ext.cpp")
EXT_NAME = "_graphop_ext"


def ext_path():
    import sysconfig
    return os.path.join(PKG_DIR, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build_torch_ext(force=False):
    """Compile the thin torch C++ extension (csrc_torch/graphop_ext.cpp) in-tree with g++ against the
    installed torch and link it to libbpt_b200.so (found through $ORIGIN at run time)."""
    import sysconfig
    import torch
    from torch.utils import cpp_extension
    out = ext_path()
    deps = [EXT_SRC, os.path.join(os.path.dirname(PKG_DIR), "include", "bpt_b200.h"), os.path.abspath(__file__)]
    if not force and os.path.exists(out) and os.path.getmtime(out) >= max(os.path.getmtime(p) for p in deps):
        return out
    build()  # the library the extension links to
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-w", EXT_SRC,
           "-DTORCH_EXTENSION_NAME=" + EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    for inc in cpp_extension.include_paths() + [sysconfig.get_paths()["include"], "/usr/local/cuda/include"]:
        cmd += ["-I", inc]
    cmd += ["-L", torch_lib, "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
            "-L", PKG_DIR, "-l:libbpt_b200.so", "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + torch_lib]
    tmp = out + ".tmp%d" % os.getpid()
    subprocess.check_call(cmd + ["-o", tmp])
    os.replace(tmp, out)
    return out


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    if "--no-torch-ext" not in sys.argv:
        print(build_torch_ext(force="--force" in sys.argv))
