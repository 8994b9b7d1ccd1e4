"""State dicts of the reference's models load into the re-hosted ones with strict=True (relative-position
configurations, dim_embed == dim_model).  The reference's modules/model.py is instantiated on CPU from the
mounted checkout (with stand-ins for `dgl` and `graphop`, which its constructors do not touch); skipped
where the checkout is not mounted."""
import importlib.util
import os
import sys
import types

import pytest
import torch

REF_ROOT = os.environ.get("BPT_REFERENCE_ROOT", "/root/reference")


@pytest.fixture(scope="module")
def ref_model_module():
    if not os.path.isfile(os.path.join(REF_ROOT, "modules", "model.py")):
        pytest.skip("reference checkout not mounted")
    names = ["dgl", "dgl.function", "dgl.nn", "dgl.nn.pytorch", "dgl.nn.pytorch.softmax", "graphop", "refmods"]
    saved = {n: sys.modules.get(n) for n in names}
    try:
        for n in names[:-2]:
            m = types.ModuleType(n)
            m.__path__ = []
            sys.modules[n] = m
        sys.modules["dgl.nn.pytorch.softmax"].edge_softmax = None
        sys.modules["dgl"].function = sys.modules["dgl.function"]
        sys.modules["graphop"] = types.ModuleType("graphop")
        pkg = types.ModuleType("refmods")
        pkg.__path__ = [os.path.join(REF_ROOT, "modules")]
        sys.modules["refmods"] = pkg
        mods = {}
        for name in ("op", "embedding", "attention", "model"):
            spec = importlib.util.spec_from_file_location("refmods." + name, os.path.join(REF_ROOT, "modules", name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules["refmods." + name] = mod
            spec.loader.exec_module(mod)
            mods[name] = mod
        yield mods["model"]
    finally:
        for n in list(sys.modules):
            if n.startswith("refmods"):
                sys.modules.pop(n)
        for n, v in saved.items():
            if v is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = v


def test_reference_state_dicts_load_strictly(ref_model_module):
    from bpt_b200.model import BPTClassifier, BPTEncoderDecoder, BPTLanguageModel
    ref = ref_model_module
    torch.manual_seed(0)
    # character LM: BinaryPartitionTransformer(vocab, dim_embed, dim_model, dim_ff, h, n_classes, n_layers, rel_pos=True)
    theirs = ref.BinaryPartitionTransformer(256, 64, 64, 128, 4, 256, 2, rel_pos=True)
    mine = BPTLanguageModel(256, 64, 128, 4, 2, dropout=0.1, dropout_a=0.1)
    assert mine.load_state_dict(theirs.state_dict(), strict=True)
    assert torch.equal(mine.layers[1].embed_ak.weight, theirs.layers[1].embed_ak.weight)
    assert torch.equal(mine.embed.lut.weight, theirs.embed.lut.weight)
    # classifier: same class, n_classes = 2
    theirs = ref.BinaryPartitionTransformer(1000, 48, 48, 96, 6, 2, 3, rel_pos=True)
    mine = BPTClassifier(1000, 48, 96, 6, 3, 2)
    assert mine.load_state_dict(theirs.state_dict(), strict=True)
    # encoder-decoder
    theirs = ref.BinaryPartitionEncoderDecoder([300, 400], 64, 128, 4, 2, 2, rel_pos=True)
    mine = BPTEncoderDecoder([300, 400], 64, 128, 4, 2, 2)
    assert mine.load_state_dict(theirs.state_dict(), strict=True)
    assert torch.equal(mine.dec_layers[0].proj_q[1].weight, theirs.dec_layers[0].proj_q[1].weight)
