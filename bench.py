#!/usr/bin/env python
"""Benchmark of the fused binary-partition graph attention layer (forward + backward).

One "step" is one pass of the hot path over one batch: a block-diagonal batch of `--seqs`
independent sequences of `--seq-len` tokens with `--step` neighbours per side per level, 8 heads x 64,
forward and backward.  The metric is attention edges per second (edges of the batch graph
divided by the step time), quoted at n = 8192, k = 4.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

With N > 1 it is launched by torch.distributed.run, one rank per GPU; every rank processes
its own batch (independent graphs shard by graph, no collective on the data path) and the
reported value is all ranks' edges over the slowest rank's device time.  The default line also
carries sub-records measured in the same run: `single_seq` (one sequence of n = 8192, k = 4),
`fp32` (the headline workload in fp32), `lm` (12-layer language-model forward, tokens/s, weak
scaling) and `seqshard` (one 65,536-token sequence with its destination nodes split over the
ranks, strong scaling).
`--impl reference` times the CPU restatement of the reference's math on the host cores.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, D = 8, 64
MAX_ETYPE = 1000  # rows of the reference's embed_ak table (modules/attention.py:23,42)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp32"])
    ap.add_argument("--seqs", type=int, default=8)
    ap.add_argument("--seq-len", dest="n", type=int, default=8192)
    ap.add_argument("--step", dest="k", type=int, default=4)
    ap.add_argument("--causal", action="store_true")
    ap.add_argument("--mode", default="graphs", choices=["graphs", "seqshard"],
                    help="graphs: independent sequences per rank (weak scaling); seqshard: ONE sequence of "
                         "--seq-len tokens, destination nodes split over the ranks, K/V all-gathered (strong scaling)")
    ap.add_argument("--exchange", default="halo", choices=["halo", "allgather"],
                    help="seqshard mode: send only the remote K/V rows a shard reads (halo) or all-gather K/V")
    ap.add_argument("--no-step-graphs", action="store_true",
                    help="seqshard mode with the halo exchange: issue the pieces between collectives eagerly instead "
                         "of replaying them from CUDA graphs (collectives are never captured)")
    ap.add_argument("--workload", default="attention", choices=["attention", "lm", "mt", "cls", "chain", "sweep"],
                    help="attention: the fused layer forward+backward (headline); lm: 12-layer character LM "
                         "forward, batch 8 x 8192 tokens per rank, tokens/s; mt: 6+6-layer encoder-decoder "
                         "forward over 16 documents of 64 sentences per rank, target tokens/s; cls: 5-layer fp32 "
                         "classifier (d_model 300, 6 x 50) over 32 variable-length sequences per rank, forward + "
                         "backward with the graph, CSRs and plans rebuilt every step, sequences/s; chain: the same "
                         "layer as `attention` through the reference's four separate operators (modules/op.py), "
                         "forward + backward; sweep: one sequence per rank for n in {8192..65536} x k in {1, 2, 4, 8}")
    ap.add_argument("--attn-dropout", type=float, default=0.0,
                    help="dropout rate on the attention weights inside the fused call (attention workload; the "
                         "reference's training configurations use 0.1-0.3, the headline measures 0)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="attention workload: only the headline line, without the single_seq / fp32 / lm / seqshard "
                         "sub-records")
    return ap.parse_args()


def workload_name(a):
    return "bpt_attention_fwd_bwd %dx(n=%d,k=%d,%s) h=%dx%d %s" % (
        a.seqs, a.n, a.k, "causal" if a.causal else "bidirectional", H, D, a.dtype)


def attention_config(a, seqs, n, k, dtype_name, causal, n_nodes, n_edges):
    """The `config` of an attention line; both arms (ours and --impl reference) print the same dict."""
    elem = 2 if dtype_name == "bf16" else 4
    per_step_mb = 8 * n_nodes * H * D * elem / 1e6
    return {"workload": "bpt_attention_fwd_bwd %dx(n=%d,k=%d,%s) h=%dx%d %s" % (
                seqs, n, k, "causal" if causal else "bidirectional", H, D, dtype_name),
            "nodes_per_gpu": n_nodes, "edges_per_gpu": n_edges,
            "sharding": "independent graphs per rank, no data-path collective",
            "l2": ("inputs+outputs %.0f MB per step exceed the 126 MB L2" if per_step_mb > 126
                   else "inputs+outputs %.0f MB per step fit the 126 MB L2: not flushed between steps") % per_step_mb}


def algorithmic_bytes(n_nodes, n_edges, elem_bytes):
    """Bytes a perfect kernel must move: unique Q/K/V/O (and gradient) bytes plus the int32
    CSR (indptr, indices, etype).  Forward reads Q,K,V and writes O; backward reads Q,K,V,dO
    and lse/delta-sized rows and writes dQ,dK,dV, walking the CSR and its transpose."""
    csr = 4 * (n_nodes + 1) + 8 * n_edges
    fwd = 4 * n_nodes * H * D * elem_bytes + csr
    bwd = 8 * n_nodes * H * D * elem_bytes + 2 * n_nodes * H * 4 + 2 * csr
    return fwd, bwd


# ----------------------------------------------------------------------------- CPU side

def cpu_reference_run(a, steps, warmup, min_seconds=0.0):
    """fp32 CPU restatement of the reference math (oracle/bpt_oracle.c) on ONE sequence of the
    workload, all host threads: forward + backward per step.  Returns (edges/s, info)."""
    import numpy as np
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle
    oracle.build_lib()
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm is meant to use the cores this process may run on
    oracle.set_num_threads(len(os.sched_getaffinity(0)))
    g = oracle.binary_partition(a.n, a.causal, a.k, 10)
    N, E = g["n_nodes"], g["n_edges"]
    csr = oracle.get_csrs(g["src"], g["dst"], N)
    rng = np.random.default_rng(2)
    q, k, v = [(rng.standard_normal((N, H, D)) * 0.125).astype(np.float32) for _ in range(3)]
    ak = (rng.standard_normal((MAX_ETYPE, D)) * 0.125).astype(np.float32)
    d_o = rng.standard_normal((N, H, D)).astype(np.float32)
    scale = 1.0 / math.sqrt(D)

    def step():
        o, lse, p = oracle.attn_fwd(csr[1], g["etype"], q, k, v, ak, scale, precision="f32")
        oracle.attn_bwd(csr[1], csr[0], g["etype"], q, k, v, ak, scale, o, p, d_o, precision="f32")

    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    done = 0
    while done < steps or (time.perf_counter() - t0) < min_seconds:
        step()
        done += 1
    dt = time.perf_counter() - t0
    info = dict(cores=oracle.num_threads(), steps=done, seconds=dt, edges_per_step=E, nodes=N,
                sample="1 of %d sequences (n=%d,k=%d), fp32, forward+backward, %d repetitions" %
                       (a.seqs, a.n, a.k, done))
    return E * done / dt, info


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(a.steps, 60))   # each step is one sequence of the batch, forward + backward, on the host cores
    value, info = cpu_reference_run(a, steps, a.warmup)
    line = {
        "impl": "reference", "metric": "bpt_attention_edges_per_sec", "value": value, "unit": "edges/s",
        "n_gpus": a.gpus, "steps": info["steps"], "warmup": a.warmup,
        "ms_per_step": 1e3 * info["seconds"] / info["steps"], "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "timed_on": "host CPU, fp32, one sequence of the batch per step",
        "config": attention_config(a, a.seqs, a.n, a.k, a.dtype, a.causal, a.seqs * info["nodes"],
                                   a.seqs * info["edges_per_step"]),
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": info["cores"], "kind": "port",
                         "sample": info["sample"]},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clock and throttle reasons of this process's GPU with nvidia-smi while the
    timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid, self.proc, self.lines = uuid, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", self.uuid, "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax = float(parts[1])
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": smax,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------- GPU side

_CTX = None


def dist_context():
    """(world, rank, device) of this process; the NCCL process group is created once and shared by every
    measurement of the run."""
    global _CTX
    if _CTX is None:
        import datetime
        import torch
        import torch.distributed as dist
        world = int(os.environ.get("WORLD_SIZE", "1"))
        rank = int(os.environ.get("RANK", "0"))
        local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device: the attention path has no CPU fallback")
        torch.cuda.set_device(local_rank)
        dev = torch.device("cuda", local_rank)
        if world > 1:
            dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
        _CTX = (world, rank, dev)
    return _CTX


def barrier():
    import torch
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(values, dev):
    """Element-wise maximum of a list of floats over the ranks."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        return list(values)
    t = torch.tensor(list(values), device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.tolist()


def timed_blocks(run_step, steps, dev, min_seconds=1.0, max_blocks=50):
    """Times blocks of exactly `steps` steps with CUDA events (barrier + synchronize on both sides of
    every block), repeating blocks until about `min_seconds` have been measured.  Returns (median ms
    per step over the blocks after the maximum over ranks, number of blocks)."""
    import torch
    per_step = []
    total = 0.0
    while True:
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for _ in range(steps):
            run_step()
        stop.record()
        barrier()
        ms = max_over_ranks([start.elapsed_time(stop)], dev)[0]
        per_step.append(ms / steps)
        total += ms
        if total >= 1e3 * min_seconds or len(per_step) >= max_blocks:
            break
    per_step.sort()
    return per_step[len(per_step) // 2], len(per_step)


def measure_seqshard(a, n, k, steps, warmup, min_seconds=1.0):
    """One long sequence of n tokens, destination nodes sharded over the ranks (bpt_b200/shard.py):
    forward + backward of one attention layer, K/V rows exchanged over NCCL.  Strong scaling: the
    work is fixed, the ranks split it.  Returns the record (rank 0) or None."""
    import torch
    from bpt_b200 import graphbuilder, shard as sh
    from bpt_b200.attention import AttentionPlan, attention_backward, attention_forward

    world, rank, dev = dist_context()
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    halo = a.exchange == "halo" and dtype == torch.bfloat16
    g = graphbuilder.BinaryPartition(n, a.causal, k, 10)
    src, dst, et = g.edges_device()
    s = sh.SequenceShard(src, dst, et, g.n_nodes_arr, g.shift, rank, world)
    if halo:
        s.build_halo(src, dst, split_straddlers=True)
        plan = AttentionPlan(s.src_h, s.dst_l, s.etype_l, s.n_dst_local, n_etypes=MAX_ETYPE, n_src=s.n_ext)
    else:
        plan = AttentionPlan(s.src_g, s.dst_l, s.etype_l, s.n_owned, n_etypes=MAX_ETYPE, n_src=s.n_gathered)
    E = g.number_of_edges
    gen = torch.Generator().manual_seed(2 + rank)
    q, k_, v, d_o = [(torch.randn(s.n_owned, H, D, generator=gen) * sg).to(dtype).to(dev)
                     for sg in (0.125, 0.125, 0.125, 1.0)]
    ak = (torch.randn(MAX_ETYPE, D, generator=torch.Generator().manual_seed(1)) * 0.125).to(dtype).to(dev)
    scale = 1.0 / math.sqrt(D)
    runner = None
    if halo:
        # fixed schedule on static buffers: two packed all-to-alls, one all-gather and one all-reduce per step, the
        # pieces between them replayed from CUDA graphs (the collectives themselves are issued eagerly)
        runner = sh.HaloRunner(s, plan, H, D, dtype, dev, scale, MAX_ETYPE, graphs=not a.no_step_graphs)
        for buf, x in ((runner.q_in, q), (runner.k_in, k_), (runner.v_in, v), (runner.do_in, d_o), (runner.ak_in, ak)):
            buf.copy_(x)

    def step():
        if halo:
            runner.forward()          # the inputs sit in the runner's buffers, as a layer's projections would
            runner.backward()
            return
        if world > 1:
            k_g, v_g = sh.all_gather_rows(s, k_), sh.all_gather_rows(s, v)
        else:
            k_g, v_g = s.pad_rows(k_), s.pad_rows(v)
        o, lse = attention_forward(plan, q, k_g, v_g, ak, scale)
        dq, dk_g, dv_g, dak = attention_backward(plan, q, k_g, v_g, ak, scale, lse, d_o, o=o)
        if world > 1:
            sh.reduce_scatter_rows(s, dk_g), sh.reduce_scatter_rows(s, dv_g)

    for _ in range(max(warmup, 3)):
        step()
    run_step = step
    graph_note = ("pieces between collectives replayed from CUDA graphs" if halo and runner.graphs
                  else "eager")
    ms, blocks = timed_blocks(run_step, steps, dev, min_seconds)
    if rank != 0:
        return None
    return {
        "metric": "bpt_attention_edges_per_sec", "value": E / (ms * 1e-3), "unit": "edges/s", "n_gpus": world,
        "steps": steps, "blocks": blocks, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": a.dtype, "data": "synthetic", "cuda_graph": graph_note,
        "config": {"workload": "bpt_attention_fwd_bwd 1x(n=%d,k=%d) destination-sharded, %s over NCCL" % (
                       n, k, "halo all-to-all of K/V rows and of their gradients, straddling span nodes merged across ranks"
                       if halo else "K/V all-gather + dK/dV reduce-scatter"),
                   "edges": E, "nodes": g.number_of_nodes, "owned_nodes_rank0": s.n_owned,
                   "kv_bytes_received_rank0": 2 * (s.n_halo if halo else s.n_gathered) * H * D * q.element_size(),
                   "collectives_per_step": (4 if world > 1 else 0) if halo else (4 if world > 1 else 0)}}


def run_seqshard(a):
    rec = measure_seqshard(a, a.n, a.k, a.steps, a.warmup)
    if rec is not None:
        print(json.dumps(rec), flush=True)


def measure_lm(a, steps, warmup, min_seconds=1.0):
    """12-layer causal BPT character LM forward (d_model 512, 8 x 64, FFN 2048 GELU in its tanh form, vocab 256,
    bf16 activations, fp32 softmax), batch of 8 sequences of 8192 tokens per rank, Zipf(1.1) bytes (seed 1),
    weights N(0, 0.02).  tokens/s = tokens of all ranks / slowest rank's time (the quantity the reference
    logs at lm.py:158-163).  Every step copies its tokens from pinned host memory."""
    import numpy as np
    import torch
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTLanguageModel

    world, rank, dev = dist_context()
    seqs, n, k = 8, 8192, 4
    g = graphbuilder.BinaryPartition(n, True, k, 10)
    batch = csrmod.batch_graphs([g] * seqs)
    plan = AttentionPlan.from_batch(batch, n_etypes=MAX_ETYPE)
    leaf_ids = batch.leaf_ids()
    torch.manual_seed(0)
    model = BPTLanguageModel(256, 512, 2048, 8, 12, dropout=0.0, activation="gelu_tanh")
    for p_ in model.parameters():
        torch.nn.init.normal_(p_, 0.0, 0.02)
    model = model.to(dev).to(torch.bfloat16).eval()
    rng = np.random.default_rng(1 + rank)
    w = 1.0 / np.arange(1, 257) ** 1.1
    host_tokens = torch.from_numpy(rng.choice(256, size=seqs * n, p=w / w.sum())).pin_memory()
    out = [None]

    def step():
        tokens = host_tokens.to(dev, non_blocking=True)
        with torch.no_grad():
            out[0] = model(tokens, leaf_ids, plan)

    for _ in range(max(warmup, 3)):
        step()
    ms, blocks = timed_blocks(step, steps, dev, min_seconds)
    finite = bool(torch.isfinite(out[0].float()).all().item())
    del model
    if rank != 0:
        return None
    return {
        "metric": "lm_tokens_per_sec", "value": world * seqs * n / (ms * 1e-3), "unit": "tokens/s",
        "n_gpus": world, "steps": steps, "blocks": blocks, "warmup": max(warmup, 3), "ms_per_step": ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "bpt_lm_forward 12 layers d512 8x64 ffn2048 gelu(tanh) vocab256, %dx(n=%d,k=%d,causal) "
                               "per rank" % (seqs, n, k),
                   "nodes_per_gpu": batch.n_nodes, "edges_per_gpu_per_layer": batch.n_edges, "finite": finite}}


def run_lm(a):
    rec = measure_lm(a, a.steps, a.warmup)
    if rec is not None:
        print(json.dumps(rec), flush=True)


def run_mt(a):
    """Document-level translation forward (encoder-decoder, 6 + 6 layers, d_model 512, 8 x 64, FFN 2048,
    bf16): per rank 16 documents of 64 sentences, sentence lengths Poisson(28) clipped to [3, 100] on both
    sides (numpy default_rng(4 + rank)); encoder graphs bidirectional, decoder graphs causal, step 4,
    clip 3; cross-attention over sentence-aligned dense blocks.  tokens/s = target tokens of all ranks /
    slowest rank's time."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from bpt_b200 import csr as csrmod
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTEncoderDecoder

    world, rank, dev = dist_context()
    rng = np.random.default_rng(4 + rank)
    docs, sents, vocab = 16, 64, 8000
    src_len = np.clip(rng.poisson(28, (docs, sents)), 3, 100)
    trg_len = np.clip(rng.poisson(28, (docs, sents)), 3, 100)
    enc_cache = csrmod.GraphCache(triu=False, step=4, clip_dist=3)
    dec_cache = csrmod.GraphCache(triu=True, step=4, clip_dist=3)
    enc = csrmod.batch_graphs([enc_cache.get(int(n)) for n in src_len.sum(1)])
    dec = csrmod.batch_graphs([dec_cache.get(int(n)) for n in trg_len.sum(1)])
    src_ranges, dst_ranges = [], []
    for d_ in range(docs):  # graph/mt.py:289-321: leaves of sentence i on one side see those on the other
        s0, t0 = enc.node_offsets[d_], dec.node_offsets[d_]
        for i in range(sents):
            src_ranges.append((s0, int(src_len[d_, i])))
            dst_ranges.append((t0, int(trg_len[d_, i])))
            s0 += int(src_len[d_, i])
            t0 += int(trg_len[d_, i])
    isrc, idst = csrmod.inter_graph(src_ranges, dst_ranges)
    enc_plan = AttentionPlan.from_batch(enc, n_etypes=MAX_ETYPE)
    dec_plan = AttentionPlan.from_batch(dec, n_etypes=MAX_ETYPE)
    inter_plan = AttentionPlan(isrc, idst, None, dec.n_nodes, n_src=enc.n_nodes)
    enc_leaves, dec_leaves = enc.leaf_ids(), dec.leaf_ids()
    torch.manual_seed(0)
    model = BPTEncoderDecoder([vocab, vocab], 512, 2048, 8, 6, 6, dropout=0.0)
    for p in model.parameters():
        torch.nn.init.normal_(p, 0.0, 0.02)
    model = model.to(dev).to(torch.bfloat16).eval()
    n_src_tok, n_trg_tok = int(src_len.sum()), int(trg_len.sum())
    host_enc = torch.from_numpy(rng.integers(0, vocab, n_src_tok)).pin_memory()
    host_dec = torch.from_numpy(rng.integers(0, vocab, n_trg_tok)).pin_memory()

    def step():
        e_tok, d_tok = host_enc.to(dev, non_blocking=True), host_dec.to(dev, non_blocking=True)
        with torch.no_grad():
            return model(e_tok, enc_leaves, enc_plan, d_tok, dec_leaves, dec_plan, inter_plan, dec_leaves)

    for _ in range(max(a.warmup, 3)):
        step()
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(a.steps):
        out = step()
    stop.record()
    barrier()
    ms = start.elapsed_time(stop) / a.steps
    tokens = torch.tensor([float(n_trg_tok)], device=dev, dtype=torch.float64)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(tokens)
        ms = t.item()
    if rank == 0:
        print(json.dumps({
            "metric": "mt_target_tokens_per_sec", "value": tokens.item() / (ms * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "bpt_encoder_decoder_forward 6+6 layers d512 8x64 ffn2048, 16 documents x 64 "
                                   "sentences per rank, k=4, clip 3",
                       "encoder_nodes": enc.n_nodes, "encoder_edges": enc.n_edges, "decoder_nodes": dec.n_nodes,
                       "decoder_edges": dec.n_edges, "cross_edges": int(isrc.numel()),
                       "source_tokens": n_src_tok, "target_tokens": n_trg_tok,
                       "finite": bool(torch.isfinite(out.float()).all().item())}}), flush=True)


def run_cls(a):
    """Variable-length classification step (5 layers, d_model 300, 6 heads x 50, FFN 600, fp32, causal
    k = 4 graphs with clip 5 as configs/imdb-4.yml): 32 sequences per rank and step with lengths
    clip(round(lognormal(5.3, 0.6)), 10, 2500) drawn anew every step (numpy default_rng(3 + rank)), so the
    timed step includes batching the graphs and building the attention plan, then forward, loss and
    backward.  Mean-pooled leaves feed a 2-way head.  sequences/s = sequences of all ranks / slowest rank."""
    import numpy as np
    import torch
    import torch.distributed as dist
    from bpt_b200 import csr as csrmod
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTClassifier

    world, rank, dev = dist_context()
    rng = np.random.default_rng(3 + rank)
    batch_size, vocab = 32, 50000
    cache = csrmod.GraphCache(triu=True, step=4, clip_dist=5)
    torch.manual_seed(0)
    model = BPTClassifier(vocab, 300, 600, 6, 5, 2, dropout=0.0, readout="mean").to(dev)
    n_steps = max(a.warmup, 3) + a.steps
    all_lengths = np.clip(np.round(rng.lognormal(5.3, 0.6, (n_steps, batch_size))), 10, 2500).astype(np.int64)
    for n in np.unique(all_lengths):       # a training run meets every length again and again: graphs are cached
        cache.get(int(n))
    labels = torch.from_numpy(rng.integers(0, 2, (n_steps, batch_size))).to(dev)
    tokens_host = [torch.from_numpy(rng.integers(0, vocab, int(l.sum()))).pin_memory() for l in all_lengths]
    stats = {"tokens": 0, "edges": 0}

    def step(i):
        lengths = all_lengths[i]
        batch = csrmod.batch_graphs([cache.get(int(n)) for n in lengths])      # graph/text_classification.py:36-67
        plan = AttentionPlan.from_batch(batch, n_etypes=MAX_ETYPE)
        tokens = tokens_host[i].to(dev, non_blocking=True)
        logp = model(tokens, batch.leaf_ids(), plan, batch.root_ids(), torch.from_numpy(lengths).to(dev))
        loss = torch.nn.functional.nll_loss(logp, labels[i])
        model.zero_grad(set_to_none=True)
        loss.backward()
        stats["tokens"] += int(lengths.sum())
        stats["edges"] += batch.n_edges
        return loss

    w = max(a.warmup, 3)
    # The largest batch of the run first: it sizes the caching allocator's blocks the way the first epoch of a
    # training run does, so that no timed step pays a cudaMalloc (tens of ms each when a new maximum is met).
    step(int(np.argmax(all_lengths.sum(axis=1))))
    for i in range(w):
        step(i)
    barrier()
    stats = {"tokens": 0, "edges": 0}
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for i in range(w, n_steps):
        loss = step(i)
    stop.record()
    barrier()
    ms = start.elapsed_time(stop) / a.steps
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    if rank == 0:
        print(json.dumps({
            "metric": "cls_sequences_per_sec", "value": world * batch_size / (ms * 1e-3), "unit": "sequences/s",
            "n_gpus": world, "steps": a.steps, "warmup": w, "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "fp32", "data": "synthetic",
            "config": {"workload": "bpt_classifier_train_step 5 layers d300 6x50 ffn600 fp32, 32 variable-length "
                                   "sequences per rank (lognormal 5.3/0.6 in [10, 2500]), k=4 causal, graph batch and "
                                   "plan rebuilt every step",
                       "tokens_per_step_rank0": stats["tokens"] // a.steps,
                       "edges_per_step_rank0": stats["edges"] // a.steps,
                       "finite_loss": bool(torch.isfinite(loss).item())}}), flush=True)


def run_chain(a):
    """The layer of the headline workload spelled as the reference spells it (modules/attention.py:56-77):
    embed_ak(etype) gathered to (E, d), masked_mm + node_mul_edge, sparse_softmax, vec_spmm, and autograd
    through them -- on this library's deterministic operator kernels.  One GPU; edges/s."""
    import torch
    from bpt_b200 import csr as csrmod, graphbuilder, op

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    dtype = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    g = graphbuilder.BinaryPartition(a.n, a.causal, a.k, 10)
    batch = csrmod.batch_graphs([g] * a.seqs)
    N, E = batch.n_nodes, batch.n_edges
    out_csr, in_csr, ROW, INDPTR_R, COL, INDPTR_C = csrmod.get_csrs(batch.src, batch.dst, N)
    gen = torch.Generator(device="cpu").manual_seed(2)
    q, k, v = [(torch.randn(N, H, D, generator=gen) * 0.125).to(dtype).to(dev).requires_grad_(True) for _ in range(3)]
    d_o = torch.randn(N, H, D, generator=gen).to(dtype).to(dev)
    table = (torch.randn(MAX_ETYPE, D, generator=gen) * 0.125).to(dtype).to(dev).requires_grad_(True)
    etype = batch.etype.long()
    scale = 1.0 / math.sqrt(D)

    def step():
        for t_ in (q, k, v, table):
            t_.grad = None
        ak = torch.nn.functional.embedding(etype, table)                       # attention.py:56-57
        e = op.masked_mm(ROW, INDPTR_R, out_csr[2], out_csr[1], COL, INDPTR_C, in_csr[2], in_csr[1], k, q)
        e_rel = op.node_mul_edge(COL, INDPTR_C, in_csr[2], q, ak)
        p_ = op.sparse_softmax(COL, INDPTR_C, in_csr[2], (e_rel + e) * scale)
        o = op.vec_spmm(COL, INDPTR_C, in_csr[2], in_csr[1], ROW, INDPTR_R, out_csr[2], out_csr[1], p_, v)
        o.backward(d_o)
        return o

    for _ in range(max(a.warmup, 3)):
        step()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(a.steps):
        step()
    stop.record()
    torch.cuda.synchronize()
    ms = start.elapsed_time(stop) / a.steps
    print(json.dumps({
        "metric": "bpt_attention_edges_per_sec", "value": E / (ms * 1e-3), "unit": "edges/s", "n_gpus": 1,
        "steps": a.steps, "warmup": max(a.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": a.dtype, "data": "synthetic",
        "config": {"workload": "operator chain (masked_mm, node_mul_edge, sparse_softmax, vec_spmm) fwd+bwd, "
                               + workload_name(a), "nodes": N, "edges": E}}), flush=True)


# dram__bytes_read + dram__bytes_write of the forward kernel from ncu captures of 2 sequences of n = 8192, k = 4
# (bidirectional, bf16): bytes per edge, keyed by the kernel that was captured.  A kernel without an entry
# (or another shape) reports traffic = null rather than a stale figure.
FORWARD_TRAFFIC_PER_EDGE = {
    "attn_forward_tile_kernel": {"bytes_per_edge": (123.61e6 + 18.83e6) / 1491572,
                                 "source": "ncu dram__bytes, 2 x (n=8192,k=4), profiles/attn_tile_kernels_bf16_n8192_k4.md"},
    "attn_forward_tc5_kernel": {"bytes_per_edge": (112.53e6 + 20.41e6) / 1491572,
                                "source": "ncu dram__bytes, 2 x (n=8192,k=4), profiles/attn_forward_tc5_bf16_n8192_k4.md"},
}


def measure_attention(a, seqs, n, k, dtype_name, causal, steps, warmup, with_e2e, with_clocks, min_seconds=1.0):
    """Fused attention forward + backward over a block-diagonal batch of `seqs` sequences per rank.
    Returns (record, state) on rank 0 and (None, state) elsewhere."""
    import torch
    from bpt_b200 import attention as att, csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan, attention_backward, attention_forward

    world, rank, dev = dist_context()
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    g = graphbuilder.BinaryPartition(n, causal, k, 10)
    batch = csrmod.batch_graphs([g] * seqs)
    plan = AttentionPlan.from_batch(batch, n_etypes=MAX_ETYPE)
    N, E = batch.n_nodes, batch.n_edges
    gen = torch.Generator(device="cpu").manual_seed(2 + rank)
    host = {}
    for name, sigma in (("q", 0.125), ("k", 0.125), ("v", 0.125), ("d_o", 1.0)):
        host[name] = (torch.randn(N, H, D, generator=gen) * sigma).to(dtype)
        if with_e2e:
            host[name] = host[name].pin_memory()
    ak = (torch.randn(MAX_ETYPE, D, generator=gen) * 0.125).to(dtype).to(dev)
    q, k_, v, d_o = [host[n_].to(dev) for n_ in ("q", "k", "v", "d_o")]
    scale = 1.0 / math.sqrt(D)

    if dtype == torch.bfloat16:
        tc5 = att.FORWARD_IMPL == "tc5" and att.tc5_eligible(q, ak, plan)
        tp = plan.tile_plan5() if tc5 else plan.tile_plan()
        launches_fwd = 1 + (tp.n_split > 0) + (tp.n_row_items > 0)
        fwd_kernel = "attn_forward_tc5_kernel" if tc5 else "attn_forward_tile_kernel"
        tpd, tpt = plan.tile_plan(), plan.tile_plan_t()
        # destination-side tiles, per-row type table, source-side tiles (+ merges); the two GEMMs of
        # the relative-position gradients are cuBLAS launches and not counted
        launches_bwd = 3 + (tpd.n_split > 0) + (tpt.n_split > 0)
        bwd_kernels = "attn_backward_dq_tile_kernel + build_type_table_kernel + 2 cuBLAS GEMMs + attn_backward_dkv_tile_kernel"
    else:
        tc32 = dtype == torch.float32 and att.FP32_FORWARD == "tc32" and att.tc32_eligible(q, ak, plan)
        launches_fwd = 1 + ((plan.tile_plan().n_split > 0) if tc32 else (plan.counts[2] > 0))
        fwd_kernel = "attn_forward_tile32_kernel" if tc32 else "attn_forward_kernel"
        if tc32 and att.FP32_BACKWARD == "tc32":
            # destination-side tiles, relative-position part of dQ, source-side tiles (or the CUDA-core
            # kernel), d embed_ak (+ merges)
            tiles_t = att.FP32_BACKWARD_SOURCE_SIDE == "tc32"
            tpd = plan.tile_plan()
            n_split_src = plan.tile_plan_t().n_split if tiles_t else plan.counts[5]
            dkv_name = "attn_backward_dkv_tile32_kernel" if tiles_t else "attn_backward_dkv_kernel"
            if 0 < tpd.t_max <= 256 and 4 * H * tpd.t_max * 4 <= 48 * 1024:
                # per-row type table; its two fp32 GEMMs are cuBLAS launches and not counted
                launches_bwd = 3 + (tpd.n_split > 0) + (n_split_src > 0)
                bwd_kernels = ("attn_backward_dq_tile32_kernel + build_type_table_kernel + 2 cuBLAS fp32 GEMMs + " +
                               dkv_name)
            else:
                launches_bwd = 4 + (tpd.n_split > 0) + (n_split_src > 0) + (plan.counts[8] > 0)
                bwd_kernels = ("attn_backward_dq_tile32_kernel + attn_backward_dq_ak_kernel + " + dkv_name +
                               " + attn_backward_dak_kernel")
        else:
            launches_bwd = 3 + (plan.counts[2] > 0) + (plan.counts[5] > 0) + (plan.counts[8] > 0)
            bwd_kernels = "attn_backward_{dq,dkv,dak}_kernel"

    drop = (float(a.attn_dropout), 20240607) if getattr(a, "attn_dropout", 0.0) > 0.0 else None

    def step():
        o, lse = attention_forward(plan, q, k_, v, ak, scale, dropout=drop)
        return o, attention_backward(plan, q, k_, v, ak, scale, lse, d_o, o=o, dropout=drop)

    for _ in range(max(warmup, 3)):
        step()
    barrier()

    sampler = None
    if with_clocks and rank == 0:
        sampler = ClockSampler("GPU-" + str(torch.cuda.get_device_properties(dev).uuid))
        sampler.start()
    # blocks of exactly `steps` steps, forward and backward also timed apart by events on the launching stream
    blocks, total_s = [], 0.0
    while True:
        ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(steps)]
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(steps):
            ev[i][0].record()
            o, lse = attention_forward(plan, q, k_, v, ak, scale, dropout=drop)
            ev[i][1].record()
            attention_backward(plan, q, k_, v, ak, scale, lse, d_o, o=o, dropout=drop)
            ev[i][2].record()
        stop.record()
        barrier()
        t = [start.elapsed_time(stop) / steps, sum(e[0].elapsed_time(e[1]) for e in ev) / steps,
             sum(e[1].elapsed_time(e[2]) for e in ev) / steps]
        blocks.append(max_over_ranks(t, dev))
        total_s += blocks[-1][0] * steps * 1e-3
        if total_s >= min_seconds or len(blocks) >= 50:
            break
    clocks = sampler.stop() if sampler else None
    blocks.sort()
    ms_per_step, fwd_ms, bwd_ms = blocks[len(blocks) // 2]
    if dtype == torch.bfloat16 and att.FORWARD_IMPL == "tc5" and att.tc5_status(plan, H) != 0:
        raise RuntimeError("bench: a bounded wait of the tcgen05 forward ran out; its results are invalid")

    # end to end: host buffers in, host buffers out, through the public call.  Every step copies
    # its q, k, v, dO from pinned host memory and copies o, dq, dk, dv back; copies and kernels of
    # consecutive steps overlap on three streams (two sets of device buffers), as a caller
    # feeding the layer from host memory would arrange it.
    e2e = None
    if with_e2e:
        names = ("q", "k", "v", "d_o")
        e2e_steps = max(4, min(steps, 12))
        n_buf = 2
        dev_in = [[torch.empty((N, H, D), dtype=dtype, device=dev) for _ in names] for _ in range(n_buf)]
        host_out = [[torch.empty((N, H, D), dtype=dtype).pin_memory() for _ in range(4)] for _ in range(n_buf)]
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        s_main = torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(n_buf)]
        ev_done = [torch.cuda.Event() for _ in range(n_buf)]
        ev_out = [torch.cuda.Event() for _ in range(n_buf)]
        results = [None] * n_buf

        def e2e_run(count):
            for i in range(count):
                b = i % n_buf
                with torch.cuda.stream(s_in):
                    s_in.wait_event(ev_done[b])      # the kernels that read this input set are done
                    for t_dev, name in zip(dev_in[b], names):
                        t_dev.copy_(host[name], non_blocking=True)
                    ev_in[b].record(s_in)
                s_main.wait_event(ev_in[b])
                s_main.wait_event(ev_out[b])         # the previous results of this set have left the device
                q_, kk_, v_, do_ = dev_in[b]
                o, lse = attention_forward(plan, q_, kk_, v_, ak, scale, dropout=drop)
                grads = attention_backward(plan, q_, kk_, v_, ak, scale, lse, do_, o=o, dropout=drop)
                results[b] = (o, grads[0], grads[1], grads[2])
                ev_done[b].record(s_main)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_done[b])
                    for t_host, t_dev in zip(host_out[b], results[b]):
                        t_host.copy_(t_dev, non_blocking=True)
                        t_dev.record_stream(s_out)
                    ev_out[b].record(s_out)

        e2e_run(n_buf)
        barrier()
        s2, t2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s2.record()
        e2e_run(e2e_steps)
        s_main.wait_stream(s_in)
        s_main.wait_stream(s_out)
        t2.record()
        barrier()
        e2e_ms = max_over_ranks([s2.elapsed_time(t2) / e2e_steps], dev)[0]
        nbytes = N * H * D * q.element_size()
        e2e = {"value": world * E / (e2e_ms * 1e-3), "unit": "edges/s", "h2d_bytes_per_step": 4 * nbytes,
               "d2h_bytes_per_step": 4 * nbytes, "ms_per_step": e2e_ms, "steps": e2e_steps,
               "overlap": "H2D, kernels and D2H of consecutive steps on three streams"}

    if rank != 0:
        return None
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        peak, peak_src = json.load(open(peaks_path))["hbm_gbs"], "measured"
    else:
        peak, peak_src = 6650.0, "fallback"
    fwd_bytes, bwd_bytes = algorithmic_bytes(N, E, q.element_size())
    fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    traffic, traffic_src = None, None
    known = FORWARD_TRAFFIC_PER_EDGE.get(fwd_kernel)
    if known and dtype_name == "bf16" and n == 8192 and k == 4 and not causal:
        traffic, traffic_src = known["bytes_per_edge"] * E, known["source"]
    line = {
        "metric": "bpt_attention_edges_per_sec", "value": world * E / (ms_per_step * 1e-3),
        "unit": "edges/s", "n_gpus": world, "steps": steps, "blocks": len(blocks), "warmup": max(warmup, 3),
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": dtype_name, "data": "synthetic",
        "config": dict(attention_config(a, seqs, n, k, dtype_name, causal, N, E),
                       **({"attention_dropout": drop[0]} if drop else {})),
        "gpu_launches": steps * len(blocks) * (launches_fwd + launches_bwd),
        "forward": {"ms": fwd_ms, "edges_per_sec": world * E / (fwd_ms * 1e-3)},
        "backward": {"ms": bwd_ms, "edges_per_sec": world * E / (bwd_ms * 1e-3)},
        "roofline": {"kernel": fwd_kernel, "bound": "hbm", "achieved": fwd_gbs, "peak": peak,
                     "peak_source": peak_src, "unit": "GB/s", "frac": fwd_gbs / peak,
                     "algorithmic_bytes": fwd_bytes, "traffic": traffic, "traffic_source": traffic_src},
        "roofline_backward": {"kernels": bwd_kernels, "bound": "hbm",
                              "achieved": bwd_gbs, "peak": peak, "unit": "GB/s", "frac": bwd_gbs / peak,
                              "algorithmic_bytes": bwd_bytes},
    }
    if clocks is not None:
        line["clocks"] = clocks
    if e2e:
        line["e2e"] = e2e
    return line


def brief(rec, keys=("metric", "value", "unit", "n_gpus", "steps", "blocks", "ms_per_step", "scaling", "dtype", "config",
                     "forward", "backward", "roofline", "roofline_backward")):
    return None if rec is None else {k_: rec[k_] for k_ in keys if k_ in rec}


def run_ours(a):
    """The headline line, then -- in the same process group -- the other parts of the metric as sub-records:
    the exact single-sequence cell, the same workload in fp32, the language-model forward (tokens/s, weak
    scaling) and the destination-sharded 65,536-token sequence (strong scaling)."""
    world, rank, dev = dist_context()
    line = measure_attention(a, a.seqs, a.n, a.k, a.dtype, a.causal, a.steps, a.warmup, not a.no_e2e, True)
    extras = {}
    if not a.no_extras:
        sub_steps = max(5, min(a.steps, 20))
        subs = (
            ("single_seq", lambda: measure_attention(a, 1, 8192, 4, "bf16", False, sub_steps, 3, False, False, 0.3)),
            ("fp32", lambda: measure_attention(a, a.seqs, a.n, a.k, "fp32", a.causal, max(3, sub_steps // 4), 3,
                                               False, False, 0.3)),
            ("lm", lambda: measure_lm(a, max(3, sub_steps // 4), 3, 0.5)),
            ("seqshard", lambda: measure_seqshard(a, 65536, 4, sub_steps, 3, 0.5)),
        )
        for name, fn in subs:
            # a sub-record that fails (on every rank alike: they run the same code on the same shapes) is
            # reported as such and does not take the headline line with it
            try:
                extras[name] = brief(fn())
            except Exception as exc:  # noqa: BLE001
                extras[name] = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:300])}
                print("bench: sub-record %s failed: %s" % (name, exc), file=sys.stderr)
    if rank == 0:
        line.update(extras)
        if world == 1 and not a.no_cpu_baseline:
            value, info = cpu_reference_run(a, 1, 1, min_seconds=10.0)
            line["cpu_baseline"] = {"value": value, "unit": "edges/s", "cores": info["cores"], "kind": "port",
                                    "sample": info["sample"]}
        print(json.dumps(line), flush=True)


def run_sweep(a):
    """One attention layer forward + backward on ONE sequence per rank for n in {8192, 16384, 32768, 65536}
    and k in {1, 2, 4, 8} (8 x 64, bf16 unless --dtype says otherwise): one JSON line with a cell per (n, k)."""
    world, rank, dev = dist_context()
    cells = []
    for n in (8192, 16384, 32768, 65536):
        for k in (1, 2, 4, 8):
            rec = measure_attention(a, 1, n, k, a.dtype, a.causal, max(5, min(a.steps, 20)), 3, False, False, 0.25)
            if rank == 0:
                cells.append({"n": n, "k": k, "nodes": rec["config"]["nodes_per_gpu"], "edges": rec["config"]["edges_per_gpu"],
                              "ms_per_step": rec["ms_per_step"], "forward_ms": rec["forward"]["ms"],
                              "backward_ms": rec["backward"]["ms"], "edges_per_sec": rec["value"] / world,
                              "forward_kernel": rec["roofline"]["kernel"], "forward_frac": rec["roofline"]["frac"],
                              "backward_frac": rec["roofline_backward"]["frac"]})
    if rank == 0:
        print(json.dumps({"metric": "bpt_attention_edges_per_sec", "unit": "edges/s", "n_gpus": world, "dtype": a.dtype,
                          "data": "synthetic", "config": {"workload": "sweep: 1 x (n, k) per rank, h=8x64, fwd+bwd"},
                          "cells": cells}), flush=True)


def main():
    a = parse()
    if a.impl == "reference":
        run_reference(a)
        return
    try:
        dispatch(a)
    finally:
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()


def dispatch(a):
    if a.workload == "lm":
        run_lm(a)
    elif a.workload == "mt":
        run_mt(a)
    elif a.workload == "cls":
        run_cls(a)
    elif a.workload == "chain":
        run_chain(a)
    elif a.workload == "sweep":
        run_sweep(a)
    elif a.mode == "seqshard":
        run_seqshard(a)
    else:
        run_ours(a)


if __name__ == "__main__":
    main()
