"""Compile the reference's own CUDA operators and attention block into oracle/_ref/ (test
infrastructure only).

Two artefacts, both built from the reference's files *where they lie* in a read-only checkout,
with every intermediate in a temporary directory and only shared objects written to oracle/_ref/:

  graphop<ext>.so          graph_kernel/graphop.cpp + graph_kernel/graphop_kernel.cu, unmodified,
                           as graph_kernel/setup.py:5-16 builds them, for sm_100a.  The only help
                           they get is oracle/shim/THC/THC.h on the include path (the header the
                           file includes at graphop_kernel.cu:4 left PyTorch years ago).
  bpt_ref_modules/         modules/op.py and modules/attention.py, unmodified, compiled with Cython
      op<ext>.so           into extension modules of a package of their own (the reference's
      attention<ext>.so    modules/__init__.py also imports its DGL-bound model and beam code and
                           is not used), so that the reference's BPTBlock.forward can be run where
                           the checkout itself is not mounted.

They pin the floating-point side of the parity tests to the reference's own kernels, prove that the
reference's attention block runs unchanged on this library's `graphop`, and serve as the "reference
kernels on the same GPU" leg of the benchmark.  Nothing in the shipped package may import them.

Usage:  python oracle/build_ref_graphop.py [--ref /path/to/reference/checkout]
"""
import argparse
import atexit
import glob
import importlib.machinery
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import types

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
MODULES_PKG = "bpt_ref_modules"


def graphop_so_path():
    hits = sorted(glob.glob(os.path.join(OUT, "graphop*.so")))
    return hits[0] if hits else None


MODULE_NAMES = ("op", "attention", "embedding", "model")  # modules/*.py, in import order


def modules_so_paths():
    """{'op': path, 'attention': path, 'embedding': path, 'model': path} of the compiled reference modules,
    or None when one is missing."""
    out = {}
    for name in MODULE_NAMES:
        hits = sorted(glob.glob(os.path.join(OUT, MODULES_PKG, name + "*.so")))
        if not hits:
            return None
        out[name] = hits[0]
    return out


def _torch_paths():
    import torch
    root = os.path.dirname(torch.__file__)
    inc = [os.path.join(root, "include"), os.path.join(root, "include", "torch", "csrc", "api", "include")]
    return inc, os.path.join(root, "lib"), int(torch._C._GLIBCXX_USE_CXX11_ABI)


def build_graphop(ref_root, quiet=True):
    cu = os.path.join(ref_root, "graph_kernel", "graphop_kernel.cu")
    cpp = os.path.join(ref_root, "graph_kernel", "graphop.cpp")
    for f in (cu, cpp):
        if not os.path.isfile(f):
            raise FileNotFoundError(f)
    inc, libdir, abi = _torch_paths()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    incs = ["-I" + os.path.join(HERE, "shim")] + ["-I" + p for p in inc] + \
           ["-I" + sysconfig.get_paths()["include"], "-I" + os.path.join(cuda, "include")]
    defs = ["-DTORCH_EXTENSION_NAME=graphop", "-D_GLIBCXX_USE_CXX11_ABI=%d" % abi, "-DTORCH_API_INCLUDE_EXTENSION_H"]
    sink = dict(stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) if quiet else {}
    os.makedirs(OUT, exist_ok=True)
    with tempfile.TemporaryDirectory(prefix="bpt_ref_graphop_") as tmp:
        o_cu, o_cpp = os.path.join(tmp, "graphop_kernel.o"), os.path.join(tmp, "graphop.o")
        subprocess.check_call([os.path.join(cuda, "bin", "nvcc"), "-c", cu, "-o", o_cu] + incs + defs +
                              ["-gencode", "arch=compute_100a,code=sm_100a", "-std=c++17", "-O2", "-w",
                               "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC"], **sink)
        subprocess.check_call(["g++", "-c", cpp, "-o", o_cpp] + incs + defs + ["-std=c++17", "-O2", "-fPIC", "-w"],
                              **sink)
        so = os.path.join(tmp, "graphop" + sysconfig.get_config_var("EXT_SUFFIX"))
        subprocess.check_call(["g++", "-shared", o_cpp, o_cu, "-o", so, "-L" + libdir,
                               "-L" + os.path.join(cuda, "lib64"), "-lc10", "-lc10_cuda", "-ltorch_cpu",
                               "-ltorch_cuda", "-ltorch", "-ltorch_python", "-lcudart"], **sink)
        shutil.copy2(so, os.path.join(OUT, os.path.basename(so)))
    return graphop_so_path()


def build_modules(ref_root, quiet=True):
    pkg_out = os.path.join(OUT, MODULES_PKG)
    os.makedirs(pkg_out, exist_ok=True)
    sink = dict(stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL) if quiet else {}
    ext = sysconfig.get_config_var("EXT_SUFFIX")
    with tempfile.TemporaryDirectory(prefix="bpt_ref_modules_") as tmp:
        for name in MODULE_NAMES:
            py = os.path.join(ref_root, "modules", name + ".py")
            if not os.path.isfile(py):
                raise FileNotFoundError(py)
            c = os.path.join(tmp, name + ".c")
            subprocess.check_call([sys.executable, "-m", "cython", "-3", "--module-name",
                                   MODULES_PKG + "." + name, py, "-o", c], **sink)
            so = os.path.join(tmp, name + ext)
            subprocess.check_call(["gcc", "-O1", "-shared", "-fPIC", "-w", "-I" + sysconfig.get_paths()["include"],
                                   c, "-o", so], **sink)
            shutil.copy2(so, os.path.join(pkg_out, os.path.basename(so)))
    return modules_so_paths()


def build(ref_root, quiet=True):
    return build_graphop(ref_root, quiet), build_modules(ref_root, quiet)


def load_graphop():
    """The reference's own `graphop` extension as a module object (not registered in sys.modules)."""
    path = graphop_so_path()
    if path is None:
        return None
    import torch  # noqa: F401  (the extension links against libtorch)
    loader = importlib.machinery.ExtensionFileLoader("graphop", path)
    spec = importlib.util.spec_from_loader("graphop", loader, origin=path)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


class FakeGraph:
    """What the reference's blocks and models touch of a DGLGraph: dict-like node and edge frames
    (modules/attention.py:55-57,62-64,81), `g.nodes[ids].data[key]` read and assignment over a subset of the
    nodes (modules/model.py:249-262,275; rows never assigned are zero, as in a DGL frame), local_var() and
    number_of_nodes() (modules/model.py:89-93, modules/attention.py:163-164)."""

    def __init__(self, ndata=None, edata=None, n_nodes=None):
        self.ndata = dict(ndata or {})
        self.edata = dict(edata or {})
        self.n_nodes = n_nodes
        self.nodes = _NodeIndexer(self)

    def local_var(self):
        return self

    def number_of_nodes(self):
        return self.n_nodes


class _NodeIndexer:
    def __init__(self, graph):
        self.graph = graph

    def __getitem__(self, ids):
        return _NodeSubset(self.graph, ids)


class _NodeSubset:
    def __init__(self, graph, ids):
        self.data = _NodeSubsetData(graph, ids)


class _NodeSubsetData:
    def __init__(self, graph, ids):
        self.graph, self.ids = graph, ids

    def __getitem__(self, key):
        return self.graph.ndata[key][self.ids]

    def __setitem__(self, key, value):
        import torch
        g = self.graph
        old = g.ndata.get(key)
        if old is None or old.shape[1:] != value.shape[1:] or old.dtype != value.dtype:
            old = torch.zeros((g.n_nodes,) + tuple(value.shape[1:]), dtype=value.dtype, device=value.device)
        new = old.clone()          # out of place: autograd keeps the previous version
        new[self.ids] = value
        g.ndata[key] = new


def _stub_dgl():
    """modules/attention.py:3,5 imports dgl.function and dgl.nn.pytorch.softmax.edge_softmax at module
    level; only its DGL decoding path (BPTMemBlock.infer) uses them.  Empty stand-ins let it import."""
    made = []
    for name in ("dgl", "dgl.function", "dgl.nn", "dgl.nn.pytorch", "dgl.nn.pytorch.softmax"):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__path__ = []
            sys.modules[name] = m
            made.append(name)
    sys.modules["dgl.nn.pytorch.softmax"].edge_softmax = None
    sys.modules["dgl"].function = sys.modules["dgl.function"]
    return made


_TEMP_DIRS = []


@atexit.register
def _remove_temp_dirs():
    for d in _TEMP_DIRS:
        shutil.rmtree(d, ignore_errors=True)


def load_modules(graphop_module, ref_root=None):
    """The reference's modules/op.py, attention.py, embedding.py and model.py bound to `graphop_module`
    (what `from graphop import *`, modules/op.py:2, resolves to).  Taken from the checkout's .py files
    when ref_root holds them, else from the compiled copies in oracle/_ref/.  Returns
    (op, attention, embedding, model) module objects, or None when neither source is available.
    sys.modules is left as found."""
    src = None
    if ref_root and os.path.isfile(os.path.join(ref_root, "modules", "attention.py")):
        src = {n: os.path.join(ref_root, "modules", n + ".py") for n in MODULE_NAMES}
    else:
        src = modules_so_paths()
        if src is not None:
            # An extension module file is initialised once per process; every call here must yield modules
            # of its own (bound to its own `graphop`), so each call loads private copies of the two files.
            tmp = tempfile.mkdtemp(prefix="bpt_ref_modules_")
            _TEMP_DIRS.append(tmp)
            src = {n: shutil.copy2(path, os.path.join(tmp, os.path.basename(path))) for n, path in src.items()}
    if src is None:
        return None
    saved = {k: sys.modules.get(k) for k in ("graphop", MODULES_PKG) + tuple(MODULES_PKG + "." + n for n in MODULE_NAMES)}
    stubs = _stub_dgl()
    try:
        sys.modules["graphop"] = graphop_module
        pkg = types.ModuleType(MODULES_PKG)
        pkg.__path__ = []
        sys.modules[MODULES_PKG] = pkg
        mods = []
        for name in MODULE_NAMES:
            full = MODULES_PKG + "." + name
            if src[name].endswith(".py"):
                spec = importlib.util.spec_from_file_location(full, src[name])
            else:
                loader = importlib.machinery.ExtensionFileLoader(full, src[name])
                spec = importlib.util.spec_from_loader(full, loader, origin=src[name])
            mod = importlib.util.module_from_spec(spec)
            sys.modules[full] = mod
            spec.loader.exec_module(mod)
            setattr(pkg, name, mod)
            mods.append(mod)
        return tuple(mods)
    finally:
        for k, v in saved.items():
            if v is None:
                sys.modules.pop(k, None)
            else:
                sys.modules[k] = v
        for name in stubs:
            sys.modules.pop(name, None)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("BPT_REFERENCE_ROOT", "/root/reference"))
    args = ap.parse_args()
    print(build(args.ref, quiet=False))
