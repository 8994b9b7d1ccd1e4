"""Destination-node sharding of one sequence, checked on CPU with two gloo ranks: the index
logic of bpt_b200/shard.py (ownership, gathered-space renumbering, all-gather layout,
reduce-scatter of the K/V gradients) with the CPU oracle doing the arithmetic each rank's GPU
kernel would do."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n, k, out):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    from bpt_b200 import shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = oracle.binary_partition(n, False, k, 10)
    N, H, D, T = g["n_nodes"], 2, 8, int(g["etype"].max()) + 1
    gen = torch.Generator().manual_seed(0)
    q, kk, v, d_o = [torch.randn(N, H, D, generator=gen) * 0.5 for _ in range(4)]
    ak = torch.randn(T, D, generator=gen) * 0.5
    s = sh.SequenceShard(torch.from_numpy(g["src"]), torch.from_numpy(g["dst"]), torch.from_numpy(g["etype"]),
                         g["n_nodes_arr"], g["shift"], rank, world)
    own = s.owned
    k_g = sh.all_gather_rows(s, kk[own])
    v_g = sh.all_gather_rows(s, v[own])
    # local problem: n_owned destinations, n_gathered sources
    src_g, dst_l, et_l = s.src_g.numpy().astype(np.int64), s.dst_l.numpy().astype(np.int64), s.etype_l.numpy()
    in_csr = oracle.coo_to_csr(dst_l, src_g, s.n_owned)
    out_csr = oracle.coo_to_csr(src_g, dst_l, s.n_gathered)
    o, lse, p = oracle.attn_fwd(in_csr, et_l, q[own].numpy(), k_g.numpy(), v_g.numpy(), ak.numpy(), 0.3)
    dq, dk_g, dv_g, dak = oracle.attn_bwd(in_csr, out_csr, et_l, q[own].numpy(), k_g.numpy(), v_g.numpy(), ak.numpy(),
                                          0.3, o, p, d_o[own].numpy())
    dk = sh.reduce_scatter_rows(s, torch.from_numpy(dk_g))
    dv = sh.reduce_scatter_rows(s, torch.from_numpy(dv_g))
    dak_t = torch.from_numpy(dak)
    dist.all_reduce(dak_t)
    # reference: the unsharded problem
    csr = oracle.get_csrs(g["src"], g["dst"], N)
    o_ref, _, p_ref = oracle.attn_fwd(csr[1], g["etype"], q.numpy(), kk.numpy(), v.numpy(), ak.numpy(), 0.3)
    ref = oracle.attn_bwd(csr[1], csr[0], g["etype"], q.numpy(), kk.numpy(), v.numpy(), ak.numpy(), 0.3, o_ref, p_ref,
                          d_o.numpy())
    own_np = own.numpy()
    errs = [np.abs(o - o_ref[own_np]).max(), np.abs(dq - ref[0][own_np]).max(), np.abs(dk.numpy() - ref[1][own_np]).max(),
            np.abs(dv.numpy() - ref[2][own_np]).max(), np.abs(dak_t.numpy() - ref[3]).max()]
    # the halo exchange: only the rows this rank's edges name travel
    s.build_halo(torch.from_numpy(g["src"]), torch.from_numpy(g["dst"]))
    k_h, v_h = sh.halo_exchange(s, kk[own]), sh.halo_exchange(s, v[own])
    src_h = s.src_h.numpy().astype(np.int64)
    in_h = oracle.coo_to_csr(dst_l, src_h, s.n_owned)
    out_h = oracle.coo_to_csr(src_h, dst_l, s.n_ext)
    o_h, _, p_h = oracle.attn_fwd(in_h, et_l, q[own].numpy(), k_h.numpy(), v_h.numpy(), ak.numpy(), 0.3)
    dq_h, dk_e, dv_e, _ = oracle.attn_bwd(in_h, out_h, et_l, q[own].numpy(), k_h.numpy(), v_h.numpy(), ak.numpy(), 0.3,
                                          o_h, p_h, d_o[own].numpy())
    dk_h = sh.halo_return(s, torch.from_numpy(dk_e))
    dv_h = sh.halo_return(s, torch.from_numpy(dv_e))
    errs += [np.abs(o_h - o_ref[own_np]).max(), np.abs(dq_h - ref[0][own_np]).max(),
             np.abs(dk_h.numpy() - ref[1][own_np]).max(), np.abs(dv_h.numpy() - ref[2][own_np]).max()]
    assert s.n_halo < s.n_owned and sum(s.recv_counts) == s.n_halo
    counts = torch.tensor([s.n_owned, int(s.eid.numel())])
    gathered = [torch.zeros(2, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, counts)
    if rank == 0:
        out.put((float(max(errs)), [t.tolist() for t in gathered], N, g["n_edges"]))
    dist.destroy_process_group()


@pytest.mark.parametrize("n,k", [(64, 2), (100, 4)])
def test_two_rank_sequence_sharding_matches_unsharded(n, k):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + (os.getpid() % 1000) + n
    procs = [ctx.Process(target=_worker, args=(r, 2, port, n, k, out)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    err, gathered, N, E = out.get(timeout=10)
    assert err < 1e-12
    assert sum(g[0] for g in gathered) == N      # every node has exactly one owner
    assert sum(g[1] for g in gathered) == E      # every edge is computed by exactly one rank


def test_ownership_partitions_every_level():
    sys.path.insert(0, ROOT)
    from bpt_b200 import shard as sh
    nn, shift = [100, 50, 25, 13, 7, 4, 2, 1], [0, 100, 150, 175, 188, 195, 199, 201]
    for world in (1, 2, 4, 8):
        ids = torch.cat([sh.owned_nodes(nn, shift, r, world) for r in range(world)])
        assert sorted(ids.tolist()) == list(range(202))
        sizes = [sh.owned_nodes(nn, shift, r, world).numel() for r in range(world)]
        assert max(sizes) - min(sizes) <= len(nn)


def _straddle_worker(rank, world, port, n, k, out):
    """halo_attention with split straddlers on CPU ranks: the real autograd function (index
    logic, partial merges, collectives) with the oracle standing in for the two GPU kernels."""
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import types
    import oracle
    from bpt_b200 import shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = oracle.binary_partition(n, False, k, 10)
    N, H, D, T = g["n_nodes"], 2, 8, int(g["etype"].max()) + 1
    gen = torch.Generator().manual_seed(0)
    q, kk, v, d_o = [torch.randn(N, H, D, generator=gen) * 0.5 for _ in range(4)]
    ak = torch.randn(T, D, generator=gen) * 0.5
    src, dst, et = [torch.from_numpy(g[x]) for x in ("src", "dst", "etype")]
    s = sh.SequenceShard(src, dst, et, g["n_nodes_arr"], g["shift"], rank, world)
    s.build_halo(src, dst, split_straddlers=True)
    src_h, dst_l, et_l = s.src_h.numpy().astype(np.int64), s.dst_l.numpy().astype(np.int64), s.etype_l.numpy()
    plan = types.SimpleNamespace(in_csr=oracle.coo_to_csr(dst_l, src_h, s.n_dst_local),
                                 out_csr=oracle.coo_to_csr(src_h, dst_l, s.n_ext), etype=et_l)

    def fwd(plan, q_, k_, v_, ak_, scale):
        o, lse, _ = oracle.attn_fwd(plan.in_csr, plan.etype, q_.numpy(), k_.numpy(), v_.numpy(), ak_.numpy(), scale)
        return torch.from_numpy(o).float(), torch.from_numpy(lse).float()

    def bwd(plan, q_, k_, v_, ak_, scale, lse, d_o_, o=None):
        _, lse_loc, p = oracle.attn_fwd(plan.in_csr, plan.etype, q_.numpy(), k_.numpy(), v_.numpy(), ak_.numpy(), scale)
        # probabilities against the merged (global) lse of each destination row
        shift = np.exp(np.nan_to_num(lse_loc - lse.double().numpy(), neginf=0.0))
        row_of = np.repeat(np.arange(len(plan.in_csr[0]) - 1), np.diff(plan.in_csr[0]))
        p_glob = np.empty_like(p)
        p_glob[plan.in_csr[2]] = p[plan.in_csr[2]] * shift[row_of]
        r = oracle.attn_bwd(plan.in_csr, plan.out_csr, plan.etype, q_.numpy(), k_.numpy(), v_.numpy(), ak_.numpy(),
                            scale, o.double().numpy(), p_glob, d_o_.numpy())
        return tuple(torch.from_numpy(x).float() for x in r)

    sh._KERNELS = (fwd, bwd)
    own = s.owned
    ql, kl, vl = [x[own].clone().requires_grad_(True) for x in (q, kk, v)]
    akl = ak.clone().requires_grad_(True)
    o = sh.halo_attention(s, plan, ql, kl, vl, akl, 0.3)
    o.backward(d_o[own])
    dak = akl.grad.clone()
    dist.all_reduce(dak)
    csr = oracle.get_csrs(g["src"], g["dst"], N)
    o_ref, _, p_ref = oracle.attn_fwd(csr[1], g["etype"], q.numpy(), kk.numpy(), v.numpy(), ak.numpy(), 0.3)
    ref = oracle.attn_bwd(csr[1], csr[0], g["etype"], q.numpy(), kk.numpy(), v.numpy(), ak.numpy(), 0.3, o_ref, p_ref,
                          d_o.numpy())
    own_np = own.numpy()
    errs = [np.abs(o.detach().numpy() - o_ref[own_np]).max(), np.abs(ql.grad.numpy() - ref[0][own_np]).max(),
            np.abs(kl.grad.numpy() - ref[1][own_np]).max(), np.abs(vl.grad.numpy() - ref[2][own_np]).max(),
            np.abs(dak.numpy() - ref[3]).max()]
    # the same step through the fixed schedule with packed exchanges (HaloRunner), twice on its static buffers
    runner = sh.HaloRunner(s, plan, H, D, torch.float32, torch.device("cpu"), 0.3, T)
    for _ in range(2):
        o_r = runner.own_rows(runner.forward(q[own], kk[own], v[own], ak))
        dq_l, dq_s, dk_r, dv_r, dak_r = runner.backward(d_o[own])
        dq_r, dk_r, dv_r, dak_r = runner.own_rows(dq_l, dq_s), dk_r.clone(), dv_r.clone(), dak_r.clone()
    dist.all_reduce(dak_r)
    errs += [np.abs(o_r.numpy() - o_ref[own_np]).max(), np.abs(dq_r.numpy() - ref[0][own_np]).max(),
             np.abs(dk_r.numpy() - ref[1][own_np]).max(), np.abs(dv_r.numpy() - ref[2][own_np]).max(),
             np.abs(dak_r.numpy() - ref[3]).max()]
    info = torch.tensor([s.n_strad, s.n_halo, int(s.eid.numel())])
    gathered = [torch.zeros(3, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(gathered, info)
    if rank == 0:
        out.put((float(max(errs)), [t.tolist() for t in gathered], g["n_edges"]))
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n,k", [(2, 128, 2), (4, 256, 4), (8, 512, 4)])
def test_split_straddlers_match_unsharded(world, n, k):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29300 + (os.getpid() % 500) + world
    procs = [ctx.Process(target=_straddle_worker, args=(r, world, port, n, k, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=180)
        assert p.exitcode == 0
    err, gathered, E = out.get(timeout=10)
    assert err < 2e-5                                    # the stand-in kernels return fp32
    assert all(g[0] == world - 1 for g in gathered)      # world-1 span nodes straddle the ranks' leaf ranges
    assert sum(g[2] for g in gathered) == E              # every edge is computed by exactly one rank
    assert max(g[1] for g in gathered) < 2 * n // world  # the halo stays below a shard's own node count
