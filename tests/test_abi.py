"""The C-ABI library loads on a machine without a GPU and exports every symbol that
include/bpt_b200.h declares; the ctypes signature table covers the same set."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "bpt_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(bpt_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built_lib():
    from bpt_b200 import build
    return build.build()


def test_library_exports_every_declared_symbol(built_lib):
    L = ctypes.CDLL(built_lib)
    names = declared_symbols()
    assert len(names) >= 19
    for name in names:
        assert hasattr(L, name), name


def test_signature_table_matches_header(built_lib):
    from bpt_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_symbols()
    assert _lib.lib().bpt_version() >= 1


def test_argument_errors_need_no_gpu(built_lib):
    from bpt_b200 import _lib
    L = _lib.lib()
    rc = L.bpt_bp_levels(0, None, None, None, None)
    assert rc == 1 and b"length" in L.bpt_last_error()
    with pytest.raises(RuntimeError, match="length"):
        _lib.check(rc)
    assert L.bpt_bp_fill(8, 0, 1, 10, None, 0, 4, None, None, None, None, None) == 1


def test_host_level_table(built_lib):
    from bpt_b200 import graphbuilder
    nn, sh, total = graphbuilder.levels(5)
    assert nn == [5, 3, 2, 1] and sh == [0, 5, 8, 10] and total == 11
    nn, sh, total = graphbuilder.levels(8192)
    assert total == 16383 and len(nn) == 14
    assert graphbuilder.levels(1) == ([1], [0], 1)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "bpt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower() or f == "build.py", os.path.join(dirpath, f)


def test_tile_kernel_shared_memory_query():
    """bpt_attn_tc_smem_bytes is host-only: the headline plan fits twice per SM, a plan with
    ~900 edge types (step = 64) does not fit a block at all, bad arguments give 0."""
    from bpt_b200 import _lib
    L = _lib.lib()
    assert 0 < L.bpt_attn_tc_smem_bytes(384, 72, 1) <= 113 * 1024
    assert L.bpt_attn_tc_smem_bytes(384, 904, 2) > 227 * 1024
    assert L.bpt_attn_tc_smem_bytes(384, 72, 3) == 0 and L.bpt_attn_tc_smem_bytes(-64, 72, 1) == 0


def test_torch_extension_exports_the_reference_module_surface():
    """bpt_b200._graphop_ext (csrc_torch/graphop_ext.cpp) carries the eight names the reference's module
    exports at graph_kernel/graphop.cpp:216-225 and refuses CPU tensors with a RuntimeError, as CHECK_INPUT
    does (graphop.cpp:4-6).  No kernel is launched."""
    import torch
    import bpt_b200
    import bpt_b200.graphop
    from bpt_b200 import build as lib_build
    lib_build.build_torch_ext()
    ext = bpt_b200.graphop_extension()
    names = ["maskedmm_csr_forward", "maskedmm_csr_backward", "node_mul_edge_forward", "node_mul_edge_backward",
             "sparse_softmax_forward", "sparse_softmax_backward", "vector_spmm_forward", "vector_spmm_backward"]
    assert sorted(n for n in dir(ext) if not n.startswith("_")) == sorted(names)
    assert sorted(names) == sorted(bpt_b200.graphop.__all__)
    idx = torch.zeros(2, dtype=torch.long)
    with pytest.raises(RuntimeError):
        ext.sparse_softmax_forward(idx, idx, idx, torch.zeros(2))
    installed = bpt_b200.install_dropin("extension")[0]
    import graphop
    assert graphop is installed is ext
    assert bpt_b200.install_dropin("ctypes")[0] is bpt_b200.graphop


def test_tile_kernel_shared_memory_keeps_two_blocks_per_sm_where_it_can():
    """bpt_attn_tc_smem_bytes (host arithmetic only): the per-warp score tables take the odd-word row stride
    (t_max + 10 entries) unless exactly those 512 bytes would push a block past (228 KB - 2 KB) / 2, the most
    that lets two blocks share an SM -- the case of plans whose widest tile has 192 columns."""
    from bpt_b200 import _lib
    L = _lib.lib()
    other = lambda cols, t: 8 * 8192 + 2 * cols * 4 + 2 * 16 * (cols + 8) + t * 128
    two_blocks = (228 * 1024 - 2 * 1024) // 2
    assert L.bpt_attn_tc_smem_bytes(128, 104, 1) == other(128, 104) + 128 * 114 * 2 <= two_blocks
    assert L.bpt_attn_tc_smem_bytes(192, 104, 1) == other(192, 104) + 128 * 112 * 2 <= two_blocks
    assert other(192, 104) + 128 * 114 * 2 > two_blocks
    assert L.bpt_attn_tc_smem_bytes(384, 104, 1) == other(384, 104) + 128 * 114 * 2 > two_blocks
    assert L.bpt_attn_tc_smem_bytes(128, 0, 1) == other(128, 0) + 128 * 10 * 2
