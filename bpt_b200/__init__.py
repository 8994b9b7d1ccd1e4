"""bpt_b200: BP-Transformer's binary-partition graph attention for NVIDIA B200 (sm_100a).

Host side in Python over a C-ABI CUDA library (libbpt_b200.so, include/bpt_b200.h).
`graphop` and `graphbuilder` mirror the reference's extension modules of the same names.
"""
import sys

__all__ = ["install_dropin"]


def install_dropin():
    """Registers this package's `graphop` and `graphbuilder` under the top-level module
    names the reference imports (`from graphop import *`, modules/op.py:2;
    `from graphbuilder import ...`, graph/base.py:1,69)."""
    from . import graphbuilder, graphop
    sys.modules["graphop"] = graphop
    sys.modules["graphbuilder"] = graphbuilder
    return graphop, graphbuilder
