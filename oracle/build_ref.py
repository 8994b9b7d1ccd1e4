"""Compile the reference's own graph builder into oracle/_ref/ (test infrastructure only).

The reference implementation of the binary-partition graph is a single Cython file,
graph_builder/builder.pyx, built by graph_builder/setup.py:7-16 as an extension called
`graphbuilder`.  This recipe cythonises that file *where it lies* in a read-only checkout
of the reference, keeps all intermediates in a temporary directory, and writes only the
resulting shared object to oracle/_ref/.  No reference source is copied into this
repository.  The result is used (a) to validate oracle/bpt_oracle.c, (b) to generate the
golden digests under tests/golden/, and (c) as the timed CPU baseline for graph
construction.  Nothing in the shipped package may import it.

Usage:  python oracle/build_ref.py [--ref /path/to/reference/checkout]
"""
import argparse
import glob
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")


def ref_so_path():
    """Path of the built reference builder, or None when it has not been built."""
    hits = sorted(glob.glob(os.path.join(OUT, "graphbuilder*.so")))
    return hits[0] if hits else None


def build(ref_root, quiet=True):
    pyx = os.path.join(ref_root, "graph_builder", "builder.pyx")
    if not os.path.isfile(pyx):
        raise FileNotFoundError(pyx)
    import numpy as np
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="bpt_ref_build_") as tmp:
        cpp = os.path.join(tmp, "graphbuilder.cpp")
        # --module-name makes the init symbol PyInit_graphbuilder, as graph_builder/setup.py:9 does.
        subprocess.check_call(
            [sys.executable, "-m", "cython", "--cplus", "--module-name", "graphbuilder",
             pyx, "-o", cpp],
            stdout=subprocess.DEVNULL if quiet else None,
            stderr=subprocess.DEVNULL if quiet else None)
        ext = sysconfig.get_config_var("EXT_SUFFIX")
        so = os.path.join(tmp, "graphbuilder" + ext)
        subprocess.check_call(
            ["g++", "-O3", "-shared", "-fPIC", "-w", "-std=c++17",
             "-I" + sysconfig.get_paths()["include"], "-I" + np.get_include(),
             cpp, "-o", so])
        shutil.copy2(so, os.path.join(OUT, os.path.basename(so)))
    return ref_so_path()


def load():
    """Import the built reference builder under the alias `_ref_graphbuilder`."""
    import importlib.machinery
    import importlib.util
    path = ref_so_path()
    if path is None:
        return None
    loader = importlib.machinery.ExtensionFileLoader("graphbuilder", path)
    spec = importlib.util.spec_from_loader("graphbuilder", loader, origin=path)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BPT_REFERENCE_ROOT", "/root/reference"))
    args = ap.parse_args()
    print(build(args.ref, quiet=False))
