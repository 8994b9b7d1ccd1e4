"""Generates tests/golden/builder_golden.json from the reference's own graph builder.

Run in a container where the reference checkout is mounted:
    python oracle/build_ref.py          # compiles graph_builder/builder.pyx into oracle/_ref/
    python tests/golden/make_golden.py

For each (length, triu, step, clip_dist) the file records node/edge/level counts and the
SHA-256 of the int64 little-endian bytes of src | dst | etype (get_edges(), builder.pyx:137-140)
| pos (get_pos(), :134-135) concatenated in that order; small cases also carry the arrays themselves.  It also
records partition_csr (builder.pyx:305-321) outputs for a few seeded indptr arrays.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", "..", "oracle"))
import build_ref  # noqa: E402


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a, dtype="<i8").tobytes()).hexdigest()


def grid():
    cases = []
    for n in list(range(1, 25)) + [31, 32, 33, 63, 64, 65, 100, 127, 128, 129, 255, 256, 257, 511, 512, 513, 1000]:
        for step in (1, 2, 3, 4, 8):
            for triu in (False, True):
                for clip in ((10,) if n > 12 else (0, 2, 10)):
                    cases.append((n, triu, step, clip))
    for n in (1023, 1024, 2500, 4096, 8192):
        for step in (1, 4, 8, 64):
            for triu in (False, True):
                cases.append((n, triu, step, 10))
    cases += [(8192, True, 4, 6), (8192, True, 64, 6), (2500, True, 4, 5), (1800, False, 4, 3),
              (16384, False, 4, 10), (32768, False, 4, 10), (65536, False, 4, 10), (65536, False, 8, 10),
              (65536, True, 4, 10), (65536, False, 1, 10), (65536, False, 2, 10)]
    return cases


def main():
    ref = build_ref.load()
    if ref is None:
        raise SystemExit("build the reference first: python oracle/build_ref.py")
    out = {"source": "graph_builder/builder.pyx compiled unmodified (oracle/build_ref.py)", "cases": [],
           "partition_csr": []}
    for (n, triu, step, clip) in grid():
        g = ref.BinaryPartition(n, triu, step, clip)
        s, d, t = g.get_edges()
        p = g.get_pos()
        rec = dict(length=n, triu=bool(triu), step=step, clip_dist=clip, n_nodes=int(g.number_of_nodes),
                   n_edges=int(g.number_of_edges), n_levels=int(g.number_of_levels),
                   sha256=digest(np.concatenate([s, d, t, p])))
        if n <= 9 and step <= 2 and clip == 10:
            rec["arrays"] = dict(src=s.tolist(), dst=d.tolist(), etype=t.tolist(), pos=p.tolist())
        out["cases"].append(rec)
    out["baselines"] = []
    for (n, triu, window) in [(1, False, 8192), (2, True, 1), (7, False, 3), (30, False, 8192), (30, True, 8192),
                              (100, False, 8), (100, True, 0), (513, False, 64), (2000, True, 128)]:
        g = ref.FullyConnected(n, triu, window)
        s, d, t = g.get_edges()
        out["baselines"].append(dict(kind="fc", length=n, triu=triu, window=window, n_edges=int(g.number_of_edges),
                                     sha256=digest(np.concatenate([s, d, t, g.get_pos()]))))
    for (n, stride, c) in [(1, 4, 2), (9, 4, 2), (64, 8, 3), (100, 16, 16), (100, 4, 6), (1000, 32, 8), (4096, 128, 32)]:
        g = ref.OpenAISparse(n, stride, c)
        s, d, t = g.get_edges()
        out["baselines"].append(dict(kind="oas", length=n, stride=stride, c=c, n_edges=int(g.number_of_edges),
                                     sha256=digest(np.concatenate([s, d, t, g.get_pos()]))))
    rng = np.random.default_rng(7)
    for n_rows, hi, chunk in ((1, 5, 32), (17, 100, 32), (64, 40, 4), (200, 300, 32), (50, 3, 1)):
        deg = rng.integers(0, hi, n_rows)
        indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
        row, ip = ref.partition_csr(indptr, chunk)
        out["partition_csr"].append(dict(indptr=indptr.tolist(), chunk_size=chunk, row=row.tolist(),
                                         indptr_out=ip.tolist()))
    path = os.path.join(HERE, "builder_golden.json")
    with open(path, "w") as f:
        json.dump(out, f, separators=(",", ":"))
    print(path, len(out["cases"]), "cases", os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
