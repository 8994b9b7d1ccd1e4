"""Incremental decoding (bpt_b200/decode.py) against the full forward of the encoder-decoder:
a causal binary-partition graph lets the nodes of position t be computed from positions <= t, so
feeding the target tokens step by step must give the log-probabilities of the one-shot forward
(fp32, CUDA-core kernels, 1e-4), and greedy decoding must be a fixed point of the full forward."""
import pytest
import torch

from helpers import rel_err

pytestmark = pytest.mark.gpu


def _setup(dim=64, heads=4, dtype=torch.float32):
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.model import BPTEncoderDecoder
    torch.manual_seed(7)
    enc_len, dec_len = [23, 40], [17, 9]
    enc = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, False, 2, 3) for n in enc_len])
    dec = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, True, 2, 3) for n in dec_len])
    src_ranges = [(enc.node_offsets[i], enc_len[i]) for i in range(2)]
    dst_ranges = [(dec.node_offsets[i], dec_len[i]) for i in range(2)]
    isrc, idst = csrmod.inter_graph(src_ranges, dst_ranges)
    model = BPTEncoderDecoder([50, 60], dim, 2 * dim, heads, 2, 2).cuda().to(dtype).eval()
    enc_plan = AttentionPlan.from_batch(enc, n_etypes=1000)
    dec_plan = AttentionPlan.from_batch(dec, n_etypes=1000)
    inter_plan = AttentionPlan(isrc, idst, None, dec.n_nodes, n_src=enc.n_nodes)
    enc_tok = torch.randint(0, 50, (sum(enc_len),), device="cuda")
    return model, enc, dec, isrc, idst, enc_plan, dec_plan, inter_plan, enc_tok, dec_len


def test_teacher_forced_steps_equal_full_forward():
    from bpt_b200.decode import DecodeSchedule, teacher_forced
    model, enc, dec, isrc, idst, enc_plan, dec_plan, inter_plan, enc_tok, dec_len = _setup()
    dec_tok = torch.randint(0, 60, (sum(dec_len),), device="cuda")
    with torch.no_grad():
        want = model(enc_tok, enc.leaf_ids(), enc_plan, dec_tok, dec.leaf_ids(), dec_plan, inter_plan, dec.leaf_ids())
    sched = DecodeSchedule(dec, isrc, idst, enc.n_nodes)
    assert sched.n_steps == max(dec_len) and sum(r.numel() for r in sched.rows) == dec.n_nodes
    per_seq = list(torch.split(dec_tok, dec_len))
    got = teacher_forced(model, sched, enc_tok, enc.leaf_ids(), enc_plan, per_seq)
    assert got.shape == want.shape
    assert rel_err(got.cpu(), want.cpu()) < 1e-4


def test_teacher_forced_steps_equal_full_forward_bf16_tile_kernels():
    """The same in bf16 with head dim 64: the full forward and every per-step plan run on the tensor-core
    tile kernels; both are compared with the fp32 full forward of the same (bf16-rounded) weights at the
    bf16 bar of 2e-2 on the log-probabilities."""
    from bpt_b200.decode import DecodeSchedule, teacher_forced
    model, enc, dec, isrc, idst, enc_plan, dec_plan, inter_plan, enc_tok, dec_len = _setup(256, 4, torch.bfloat16)
    dec_tok = torch.randint(0, 60, (sum(dec_len),), device="cuda")
    sched = DecodeSchedule(dec, isrc, idst, enc.n_nodes)
    per_seq = list(torch.split(dec_tok, dec_len))
    with torch.no_grad():
        full = model(enc_tok, enc.leaf_ids(), enc_plan, dec_tok, dec.leaf_ids(), dec_plan, inter_plan, dec.leaf_ids())
        got = teacher_forced(model, sched, enc_tok, enc.leaf_ids(), enc_plan, per_seq)
        assert dec_plan.tiles is not None and sched.self_plans[-1].tiles is not None, "not on the tile kernels"
        want = model.float()(enc_tok, enc.leaf_ids(), enc_plan, dec_tok, dec.leaf_ids(), dec_plan, inter_plan,
                             dec.leaf_ids())
    assert rel_err(full.float().cpu(), want.cpu()) < 2e-2
    assert rel_err(got.float().cpu(), want.cpu()) < 2e-2


def test_greedy_decoding_is_a_fixed_point_of_the_full_forward():
    from bpt_b200.decode import DecodeSchedule, greedy
    model, enc, dec, isrc, idst, enc_plan, dec_plan, inter_plan, enc_tok, dec_len = _setup()
    sched = DecodeSchedule(dec, isrc, idst, enc.n_nodes)
    first = torch.tensor([1, 2], device="cuda")
    out = greedy(model, sched, enc_tok, enc.leaf_ids(), enc_plan, first)         # (n_steps, n_seq)
    assert out.shape == (max(dec_len), 2)
    for b, n in enumerate(dec_len):
        assert bool((out[:n, b] >= 0).all()) and bool((out[n:, b] == -1).all())
    # the decoder inputs of greedy decoding: the first token, then each step's arg-max
    inputs = torch.cat([torch.cat([first[b:b + 1], out[:n - 1, b]]) for b, n in enumerate(dec_len)])
    with torch.no_grad():
        logp = model(enc_tok, enc.leaf_ids(), enc_plan, inputs, dec.leaf_ids(), dec_plan, inter_plan, dec.leaf_ids())
    want = torch.cat([out[:n, b] for b, n in enumerate(dec_len)])
    top2 = logp.topk(2, -1).values
    clear = (top2[:, 0] - top2[:, 1]) > 1e-3      # positions where the arg-max is not a near tie
    assert bool((logp.argmax(-1)[clear] == want[clear]).all())


def test_beam_search_hypotheses_rescore_and_beam_one_is_greedy():
    """beam_search keeps beam_size hypotheses per sequence on the fused call (modules/beam.py:64-173): with
    beam 1 it is greedy decoding; with beam 3 its hypotheses come best first, the best is at least as good
    as the greedy one, and every returned score equals the summed log-probability the full forward gives
    for that hypothesis' tokens (which checks the cache rows a hypothesis inherits)."""
    from bpt_b200 import csr as csrmod, graphbuilder
    from bpt_b200.attention import AttentionPlan
    from bpt_b200.decode import DecodeSchedule, beam_search, greedy
    from bpt_b200.model import BPTEncoderDecoder
    torch.manual_seed(11)
    enc_len, dec_len, beam = [23, 40], [9, 14], 3
    enc = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, False, 2, 3) for n in enc_len])
    model = BPTEncoderDecoder([50, 20], 64, 128, 4, 2, 2).cuda().eval()
    enc_plan = AttentionPlan.from_batch(enc, n_etypes=1000)
    enc_tok = torch.randint(0, 50, (sum(enc_len),), device="cuda")
    first = torch.tensor([1, 2], device="cuda")

    def schedule(copies):
        lens = [n for n in dec_len for _ in range(copies)]
        dec = csrmod.batch_graphs([graphbuilder.BinaryPartition(n, True, 2, 3) for n in lens])
        src_ranges = [(enc.node_offsets[i // copies], enc_len[i // copies]) for i in range(len(lens))]
        dst_ranges = [(dec.node_offsets[i], lens[i]) for i in range(len(lens))]
        isrc, idst = csrmod.inter_graph(src_ranges, dst_ranges)
        return dec, isrc, idst, DecodeSchedule(dec, isrc, idst, enc.n_nodes)

    dec1, isrc1, idst1, sched1 = schedule(1)
    g_tokens = greedy(model, sched1, enc_tok, enc.leaf_ids(), enc_plan, first)            # (n_steps, 2)
    b1_tokens, b1_scores = beam_search(model, sched1, 1, enc_tok, enc.leaf_ids(), enc_plan, first)
    assert torch.equal(b1_tokens[:, :, 0], g_tokens)
    _, _, _, sched3 = schedule(beam)
    tokens, scores = beam_search(model, sched3, beam, enc_tok, enc.leaf_ids(), enc_plan, first)
    assert tokens.shape == (max(dec_len), 2, beam) and scores.shape == (2, beam)
    assert bool((scores[:, :-1] >= scores[:, 1:]).all())
    assert bool((scores[:, 0] >= b1_scores[:, 0] - 1e-4).all())
    # rescore every hypothesis with the one-shot forward over the single-copy decoder batch
    dec_plan = AttentionPlan.from_batch(dec1, n_etypes=1000)
    inter_plan = AttentionPlan(isrc1, idst1, None, dec1.n_nodes, n_src=enc.n_nodes)
    for j in range(beam):
        inputs = torch.cat([torch.cat([first[b:b + 1], tokens[:n - 1, b, j]]) for b, n in enumerate(dec_len)])
        with torch.no_grad():
            logp = model(enc_tok, enc.leaf_ids(), enc_plan, inputs, dec1.leaf_ids(), dec_plan, inter_plan, dec1.leaf_ids())
        off = 0
        for b, n in enumerate(dec_len):
            want = logp[off:off + n].gather(1, tokens[:n, b, j].unsqueeze(1)).sum().item()
            assert abs(want - scores[b, j].item()) < 1e-3 * max(1.0, abs(want)), (b, j, want, scores[b, j].item())
            off += n
