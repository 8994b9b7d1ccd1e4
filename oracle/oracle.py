"""ctypes front end of the CPU oracle (oracle/bpt_oracle.c).  TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg import this module; the
shipped package never does.  Every function names the reference code it restates.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
BUILD_DIR = os.path.join(HERE, "_build")
LIB_PATH = os.path.join(BUILD_DIR, "libbpt_oracle.so")
_SOURCES = [os.path.join(HERE, "bpt_oracle.c"), os.path.join(HERE, "bpt_oracle_attn.inc")]

_lib = None


def build_lib(force=False):
    """gcc -O3 -fopenmp build of the C restatement into oracle/_build/."""
    os.makedirs(BUILD_DIR, exist_ok=True)
    if not force and os.path.exists(LIB_PATH):
        if all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(s) for s in _SOURCES):
            return LIB_PATH
    tmp = LIB_PATH + ".tmp%d" % os.getpid()
    subprocess.check_call(["gcc", "-O3", "-fopenmp", "-shared", "-fPIC", "-std=c11",
                           _SOURCES[0], "-o", tmp, "-lm"])
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build_lib()
        L = ctypes.CDLL(LIB_PATH)
        L.bpto_levels.restype = ctypes.c_int
        L.bpto_build.restype = ctypes.c_int64
        L.bpto_partition_csr.restype = ctypes.c_int64
        L.bpto_fully_connected.restype = ctypes.c_int64
        L.bpto_openai_sparse.restype = ctypes.c_int64
        L.bpto_num_threads.restype = ctypes.c_int
        _lib = L
    return _lib


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def num_threads():
    return lib().bpto_num_threads()


def set_num_threads(n):
    lib().bpto_set_num_threads(ctypes.c_int(int(n)))


# ----------------------------------------------------------------------------- builder

def levels(length):
    """Level sizes and first node id per level (graph_builder/builder.pyx:41-56)."""
    nn = np.zeros(64, np.uint32)
    sh = np.zeros(64, np.uint32)
    tot = ctypes.c_int64(0)
    n_lvl = lib().bpto_levels(ctypes.c_int64(length), _p(nn), _p(sh), ctypes.byref(tot))
    return nn[:n_lvl].copy(), sh[:n_lvl].copy(), int(tot.value)


def binary_partition(length, triu=False, step=1, clip_dist=10):
    """BinaryPartition(length, triu, step, clip_dist) of graph_builder/builder.pyx:23-116.

    Returns a dict with src/dst/etype (int64, as get_edges() gives them, builder.pyx:137-140),
    pos (int64, builder.pyx:134-135), n_nodes, n_levels, n_nodes_arr.
    """
    L = lib()
    nn, sh, tot = levels(length)
    e = L.bpto_build(ctypes.c_int64(length), ctypes.c_int(bool(triu)), ctypes.c_int(step),
                     ctypes.c_int(clip_dist), None, None, None)
    src = np.empty(e, np.uint32)
    dst = np.empty(e, np.uint32)
    et = np.empty(e, np.uint32)
    L.bpto_build(ctypes.c_int64(length), ctypes.c_int(bool(triu)), ctypes.c_int(step),
                 ctypes.c_int(clip_dist), _p(src), _p(dst), _p(et))
    pos = np.empty(tot, np.uint32)
    L.bpto_pos(ctypes.c_int64(length), _p(pos))
    return dict(src=src.astype(np.int64), dst=dst.astype(np.int64), etype=et.astype(np.int64),
                pos=pos.astype(np.int64), n_nodes=tot, n_levels=len(nn), n_nodes_arr=nn,
                shift=sh, n_edges=int(e))


def _baseline(fn, length, *args):
    e = fn(ctypes.c_int64(length), *args, None, None, None, None)
    src, dst, et = [np.empty(e, np.uint32) for _ in range(3)]
    pos = np.empty(length + 1, np.uint32)
    fn(ctypes.c_int64(length), *args, _p(src), _p(dst), _p(et), _p(pos))
    return dict(src=src.astype(np.int64), dst=dst.astype(np.int64), etype=et.astype(np.int64),
                pos=pos.astype(np.int64), n_nodes=length + 1, n_edges=int(e))


def fully_connected(length, triu=False, window=8192):
    """FullyConnected(length, triu, window) of graph_builder/builder.pyx:228-274."""
    return _baseline(lib().bpto_fully_connected, length, ctypes.c_int(bool(triu)), ctypes.c_int64(window))


def openai_sparse(length, stride, c):
    """OpenAISparse(length, stride, c, triu=True) of graph_builder/builder.pyx:154-196."""
    return _baseline(lib().bpto_openai_sparse, length, ctypes.c_int64(stride), ctypes.c_int64(c))


def inter_graph(src_ranges, dst_ranges):
    """Sentence-aligned cross graph of graph/mt.py:318-321: for every pair of id ranges
    (first, count), np.repeat(source ids, n_dst) against np.tile(destination ids, n_src),
    concatenated in order.  Returns (src, dst) int64."""
    rows, cols = [np.zeros(0, np.int64)], [np.zeros(0, np.int64)]
    for (s0, ns), (d0, nd) in zip(src_ranges, dst_ranges):
        rows.append(np.repeat(np.arange(s0, s0 + ns, dtype=np.int64), nd))
        cols.append(np.tile(np.arange(d0, d0 + nd, dtype=np.int64), ns))
    return np.concatenate(rows), np.concatenate(cols)


def partition_csr(indptr, chunk_size=32):
    """partition_csr(indptr, chunk_size) of graph_builder/builder.pyx:305-321."""
    indptr = np.ascontiguousarray(indptr, np.int64)
    n_rows = len(indptr) - 1
    L = lib()
    c = L.bpto_partition_csr(_p(indptr), ctypes.c_int64(n_rows), ctypes.c_int(chunk_size), None, None)
    row = np.empty(c, np.int64)
    ip = np.empty(c + 1, np.int64)
    L.bpto_partition_csr(_p(indptr), ctypes.c_int64(n_rows), ctypes.c_int(chunk_size), _p(row), _p(ip))
    return row, ip


def coo_to_csr(key, other, n_rows):
    """Rows = key, columns = other, data = edge id, ascending edge id inside a row."""
    key = np.ascontiguousarray(key, np.int64)
    other = np.ascontiguousarray(other, np.int64)
    e = len(key)
    indptr = np.empty(n_rows + 1, np.int64)
    indices = np.empty(e, np.int64)
    eid = np.empty(e, np.int64)
    lib().bpto_coo_to_csr(_p(key), _p(other), ctypes.c_int64(e), ctypes.c_int64(n_rows),
                          _p(indptr), _p(indices), _p(eid))
    return indptr, indices, eid


def get_csrs(src, dst, n_nodes):
    """get_csrs(g) of graph/base.py:71-86 on a COO edge list:
    (out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C), each csr = (indptr, indices, eid)."""
    out_csr = coo_to_csr(src, dst, n_nodes)
    in_csr = coo_to_csr(dst, src, n_nodes)
    ROW, INDPTR_R = partition_csr(out_csr[0])
    COL, INDPTR_C = partition_csr(in_csr[0])
    return out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C


def batch_graphs(graphs):
    """Block-diagonal batching rule of graph/lm.py:59-98: concatenate each sequence's
    get_edges(v_shift) in order, v_shift advancing by number_of_nodes; edge id = position."""
    srcs, dsts, ets, poss = [], [], [], []
    v = 0
    for g in graphs:
        srcs.append(g["src"] + v)
        dsts.append(g["dst"] + v)
        ets.append(g["etype"])
        poss.append(g["pos"])
        v += g["n_nodes"]
    return dict(src=np.concatenate(srcs), dst=np.concatenate(dsts), etype=np.concatenate(ets),
                pos=np.concatenate(poss), n_nodes=v, n_edges=int(sum(len(s) for s in srcs)))


# ----------------------------------------------------------------------------- attention

def _real(precision):
    return (np.float64, "f64") if precision == "f64" else (np.float32, "f32")


def attn_fwd(in_csr, etype, q, k, v, ak, scale, precision="f64", want_p=True):
    """Fused-chain forward (modules/attention.py:189-209 / :66-77).  q,k,v: (N,H,D) float32
    arrays; ak: (T,D) float32 or None; etype: (E,) by edge id.  Returns (o, lse, p)."""
    dt, suf = _real(precision)
    indptr, indices, eid = [np.ascontiguousarray(a, np.int64) for a in in_csr]
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    N, H, D = q.shape
    E = len(indices)
    et = None if etype is None else np.ascontiguousarray(etype, np.int32)
    akc = None if ak is None else np.ascontiguousarray(ak, np.float32)
    o = np.empty((N, H, D), dt)
    lse = np.empty((N, H), dt)
    p = np.empty((E, H), dt) if want_p else None
    fn = getattr(lib(), "bpto_attn_fwd_" + suf)
    fn(ctypes.c_int64(N), ctypes.c_int(H), ctypes.c_int(D), ctypes.c_int64(E),
       _p(indptr), _p(indices), _p(eid), _p(et), _p(q), _p(k), _p(v), _p(akc),
       ctypes.c_double(scale), _p(o), _p(lse), _p(p))
    return o, lse, p


def attn_bwd(in_csr, out_csr, etype, q, k, v, ak, scale, o, p, d_o, precision="f64"):
    """Analytic gradients of attn_fwd.  Returns (dq, dk, dv, dak or None).  k, v may have a
    different number of rows than q (out_csr then has that many rows)."""
    dt, suf = _real(precision)
    indptr, indices, eid = [np.ascontiguousarray(a, np.int64) for a in in_csr]
    indptr_o, indices_o, eid_o = [np.ascontiguousarray(a, np.int64) for a in out_csr]
    q = np.ascontiguousarray(q, np.float32)
    k = np.ascontiguousarray(k, np.float32)
    v = np.ascontiguousarray(v, np.float32)
    d_o = np.ascontiguousarray(d_o, np.float32)
    o = np.ascontiguousarray(o, dt)
    p = np.ascontiguousarray(p, dt)
    N, H, D = q.shape
    N_src = k.shape[0]
    E = len(indices)
    et = None if etype is None else np.ascontiguousarray(etype, np.int32)
    akc = None if ak is None else np.ascontiguousarray(ak, np.float32)
    T = 0 if akc is None else akc.shape[0]
    ds = np.empty((E, H), dt)
    dq = np.empty((N, H, D), dt)
    dk = np.empty((N_src, H, D), dt)
    dv = np.empty((N_src, H, D), dt)
    dak = None if akc is None else np.empty((T, D), dt)
    fn = getattr(lib(), "bpto_attn_bwd_" + suf)
    fn(ctypes.c_int64(N), ctypes.c_int64(N_src), ctypes.c_int(H), ctypes.c_int(D), ctypes.c_int64(E), ctypes.c_int(T),
       _p(indptr), _p(indices), _p(eid), _p(indptr_o), _p(indices_o), _p(eid_o), _p(et),
       _p(q), _p(k), _p(v), _p(akc), ctypes.c_double(scale), _p(o), _p(p), _p(d_o),
       _p(ds), _p(dq), _p(dk), _p(dv), _p(dak))
    return dq, dk, dv, dak
