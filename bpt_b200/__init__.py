"""bpt_b200: BP-Transformer's binary-partition graph attention for NVIDIA B200 (sm_100a).

Host side in Python over a C-ABI CUDA library (libbpt_b200.so, include/bpt_b200.h).
`graphop` and `graphbuilder` mirror the reference's extension modules of the same names.
"""
import sys

__all__ = ["install_dropin"]


def graphop_extension():
    """The thin torch C++ extension (csrc_torch/graphop_ext.cpp, built by `python -m bpt_b200.build`):
    the reference's `graphop` module as compiled code over libbpt_b200.so.  Raises ImportError with the
    build command when it has not been built."""
    try:
        from . import _graphop_ext
    except ImportError as e:
        raise ImportError("bpt_b200._graphop_ext is not built (%s); run `python -m bpt_b200.build`" % e)
    return _graphop_ext


def install_dropin(binding=None):
    """Registers this package's `graphop` and `graphbuilder` under the top-level module
    names the reference imports (`from graphop import *`, modules/op.py:2;
    `from graphbuilder import ...`, graph/base.py:1,69).
    binding: "extension" = the torch C++ extension (what the reference's setup.py builds, here over the
    C-ABI library), "ctypes" = the Python module bpt_b200.graphop (same functions through ctypes).
    Default: BPT_GRAPHOP_BINDING, else the extension when it has been built, else ctypes."""
    import os
    from . import graphbuilder, graphop
    binding = binding or os.environ.get("BPT_GRAPHOP_BINDING")
    if binding is None:
        try:
            graphop_extension()
            binding = "extension"
        except ImportError:
            binding = "ctypes"
    if binding not in ("extension", "ctypes"):
        raise ValueError("install_dropin: binding must be 'extension' or 'ctypes'")
    module = graphop_extension() if binding == "extension" else graphop
    sys.modules["graphop"] = module
    sys.modules["graphbuilder"] = graphbuilder
    return module, graphbuilder
