"""bpt_attn_forward_static: the forward entry point for callers that cannot allocate device
memory at call time (a fixed memory plan, a thread that may not enter the framework's
allocator).  It must give what bpt_attn_forward gives, call after call, although every call
reuses the same built-in scratch array without clearing it.  Kept in a file that sorts last
so that a run stopping at the first failure has already exercised everything else."""
import numpy as np
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


def _case(oracle_lib, n, seed):
    from bpt_b200.attention import AttentionPlan
    g = oracle_lib.binary_partition(n, True, 8, 6)  # causal, k = 8: the root row has n incoming edges
    N, T = g["n_nodes"], int(g["etype"].max()) + 1
    dev = "cuda"
    plan = AttentionPlan(torch.from_numpy(g["src"]).to(dev), torch.from_numpy(g["dst"]).to(dev),
                         torch.from_numpy(g["etype"]).to(dev), N, n_etypes=T)
    gen = torch.Generator().manual_seed(seed)
    q, k, v = [(torch.randn(N, 8, 64, generator=gen) * 0.125).to(dev) for _ in range(3)]
    ak = (torch.randn(T, 64, generator=gen) * 0.125).to(dev)
    return plan, q, k, v, ak


def test_static_scratch_forward_matches_workspace_forward_twice(oracle_lib):
    from bpt_b200.attention import attention_forward, attention_forward_static
    # two different graphs back to back: the second call finds the first call's partials in the scratch
    for n, seed in ((3000, 0), (1700, 1)):
        plan, q, k, v, ak = _case(oracle_lib, n, seed)
        assert plan.counts[1] > 0, "the case must have split rows, or no scratch is used"
        o_ref, lse_ref = attention_forward(plan, q, k, v, ak, 0.125)
        out = torch.empty_like(q)
        lse_out = torch.empty(plan.n_nodes, 8, dtype=torch.float32, device="cuda")
        count = lambda: torch.cuda.memory_stats()["allocation.all.allocated"]  # cumulative allocations
        before = count()
        o, lse = attention_forward_static(plan, q, k, v, ak, 0.125, out=out, lse_out=lse_out)
        torch.cuda.synchronize()
        assert count() == before, "the call went through the caching allocator"
        assert o.data_ptr() == out.data_ptr()
        assert rel_err(o.cpu(), o_ref.cpu()) < 1e-5
        assert rel_err(lse.cpu(), lse_ref.cpu()) < 1e-5
        # and once more on the same inputs
        o2, lse2 = attention_forward_static(plan, q, k, v, ak, 0.125)
        assert rel_err(o2.cpu(), o_ref.cpu()) < 1e-5 and rel_err(lse2.cpu(), lse_ref.cpu()) < 1e-5


def test_static_scratch_rejects_graphs_beyond_its_size():
    from bpt_b200 import graphbuilder
    from bpt_b200.attention import AttentionPlan, attention_forward_static
    g = graphbuilder.BinaryPartition(65536, False, 4, 10)
    src, dst, etype = g.edges_device()
    plan = AttentionPlan(src, dst, etype, g.number_of_nodes)
    q = torch.zeros(g.number_of_nodes, 8, 64, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError, match="built-in scratch"):
        attention_forward_static(plan, q, q, q, None, 0.125)


def test_static_scratch_checks_caller_buffers(oracle_lib):
    """out and lse_out reach the library as raw pointers: a wrong shape or dtype must raise first."""
    from bpt_b200.attention import attention_forward_static
    plan, q, k, v, ak = _case(oracle_lib, 200, 2)
    with pytest.raises(RuntimeError, match="lse_out"):
        attention_forward_static(plan, q, k, v, ak, 0.125,
                                 lse_out=torch.empty(plan.n_nodes, 8, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(RuntimeError, match="out must"):
        attention_forward_static(plan, q, k, v, ak, 0.125, out=torch.empty_like(q)[:-1])
    with pytest.raises(RuntimeError, match="embed_ak"):
        attention_forward_static(plan, q, k, v, ak.double(), 0.125)
