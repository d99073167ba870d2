"""The hybrid decoder family (pipelinerl_b200/hybrid.py and its kernels) against oracle/hybrid_oracle.py: each mixer
alone, whole prompts against token-by-token decoding, portions down to two tokens, unequal batches against each request
alone, pages and slots that are given back and taken again, far keys and page borders, the first tokens, long decoding,
awkward sizes, greedy generation through the engine's scheduler, and the trace runner's command line."""
import json
import subprocess
import sys

import pytest
import torch

from tests import hybrid_cases as hc

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4      # fp32 kernels against the float64 oracle (measured ~1e-5)
BF16_TOL = 8e-2     # bf16 operands / cache: rounding of activations dominates


def _weights(config, seed=0):
    from oracle import hybrid_oracle as ho
    return ho.random_weights(config, seed)


# ---- each mechanism alone ---------------------------------------------------------------------------------------
MECHANISMS = {
    "gla": hc.model([hc.gla_layer()]),
    "gla_strong_decay": hc.model([hc.gla_layer(heads=2, dim=17, vdim=33, tau=1.0, rank=3)]),
    "attention": hc.model([hc.par_layer(left_scale=1.0, right_scale=0.0)]),
    "attention_mha_full_rotary": hc.model([hc.par_layer(heads=3, kv_heads=3, dim=16, vdim=16, rot=16, left_scale=1.0, right_scale=0.0)]),
    "attention_mqa_no_rotary": hc.model([hc.par_layer(heads=4, kv_heads=1, dim=20, vdim=70, rot=0, left_scale=1.0, right_scale=0.0)]),
    "state_space": hc.model([hc.par_layer(left_scale=0.0, right_scale=1.0)]),
    "state_space_one_group_taps5": hc.model([hc.par_layer(left_scale=0.0, right_scale=1.0, s_heads=3, s_vdim=20, state=9, groups=1,
                                                          conv=5, norm_groups=1)]),
    "state_space_taps1": hc.model([hc.par_layer(left_scale=0.0, right_scale=1.0, conv=1, norm_groups=4, groups=4)]),
    # one norm group of 5632 channels: wider than what the gate-and-norm kernel keeps in shared memory between its passes
    "state_space_wide_norm_group": hc.model([hc.par_layer(left_scale=0.0, right_scale=1.0, s_heads=44, s_vdim=128, state=8,
                                                          groups=1, norm_groups=1)]),
    "feed_forward": hc.model([hc.gla_layer(mlp=hc.dense())]),
    "parallel_both": hc.model([hc.par_layer(mlp=hc.dense(ff=40, limit=0.5))]),
}


@pytest.mark.parametrize("name", sorted(MECHANISMS))
def test_each_mechanism_matches_the_oracle_fp32(cuda_device, name):
    config = MECHANISMS[name]
    wt = _weights(config, seed=len(name))
    toks = hc.tokens_for(config, 150)
    ref = hc.oracle_logits(config, wt, toks)
    eng = hc.build_engine(config, wt, torch.float32, cuda_device)
    whole = hc.stream_logits(eng, toks, [150])
    assert hc.rel_err(whole, ref) < F32_TOL
    pieces = hc.stream_logits(eng, toks, [2, 3, 61, 2, 7, 64, 2])          # then one by one
    assert hc.rel_err(pieces, ref) < F32_TOL
    # per-layer residual stream of a whole prompt
    from oracle import hybrid_oracle as ho
    res = []
    ho.forward(config, wt, toks[:20], res)
    s = eng.open_stream()
    s.prompt_ids.extend(toks[:20])
    s.pages += eng._alloc_pages(1)
    eng.block_table[s.slot, :1].copy_(torch.tensor(s.pages, dtype=torch.int32))
    got = []
    eng._forward_rows([(s, 0, 20)], [], trace=got)
    eng.close_stream(s)
    for a, b in zip(got, res):
        assert (a.double().cpu() - b).abs().max().item() < 1e-4 * max(1.0, b.abs().max().item())


FULL = hc.model([hc.gla_layer(mlp=hc.dense()), hc.par_layer(mlp=hc.dense(ff=48)), hc.shared(hc.gla_layer(mlp=hc.dense()), 0),
                 hc.par_layer(heads=2, kv_heads=1, dim=12, vdim=8, rot=4, conv=2, groups=1, norm_groups=1, s_heads=2, s_vdim=16,
                              state=20), hc.shared(hc.par_layer(mlp=hc.dense(ff=48)), 1)], vocab=80, width=64)


def test_prefill_against_token_by_token_decoding(cuda_device):
    wt = _weights(FULL, 3)
    toks = hc.tokens_for(FULL, 140, seed=5)
    ref = hc.oracle_logits(FULL, wt, toks)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device)
    whole = hc.stream_logits(eng, toks, [140])
    single = hc.stream_logits(eng, toks, [])                                 # every token alone, through the cache / state
    assert hc.rel_err(whole, ref) < F32_TOL and hc.rel_err(single, ref) < F32_TOL
    # fp32: a token's logits do not depend on how the prompt was cut (fixed summation orders)
    assert hc.rel_err(whole, single) < 2e-5


@pytest.mark.parametrize("portions", [[2] * 40, [63, 2, 63, 2], [64, 64], [1, 65, 1, 2, 59], [129, 2]])
def test_portions_of_several_sizes(cuda_device, portions):
    wt = _weights(FULL, 4)
    toks = hc.tokens_for(FULL, 140, seed=6)
    ref = hc.oracle_logits(FULL, wt, toks)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device, prefill_chunk=96)   # 129 is cut by the engine too
    assert hc.rel_err(hc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_wanted_rows_come_back_in_the_order_asked_for(cuda_device):
    """A portion that the engine cuts (96-row batches) with wanted places out of order, beside a second stream."""
    wt = _weights(FULL, 4)
    toks, other = hc.tokens_for(FULL, 140, seed=6), hc.tokens_for(FULL, 9, seed=8)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device, prefill_chunk=96)
    every = hc.stream_logits(eng, toks, [140])
    alone = hc.stream_logits(eng, other, [9])
    a, b = eng.open_stream(), eng.open_stream()
    asked = [139, 0, 97, 95, 96, 3]
    got = eng.feed([(a, toks, asked), (b, other, [8, 2])]).double().cpu()
    eng.close_stream(a), eng.close_stream(b)
    assert got.shape[0] == 8
    assert hc.rel_err(got[:6], every[asked]) < F32_TOL and hc.rel_err(got[6:], alone[[8, 2]]) < F32_TOL


def test_unequal_batches_equal_each_request_alone(cuda_device):
    wt = _weights(FULL, 7)
    seqs = [hc.tokens_for(FULL, n, seed=10 + n) for n in (1, 37, 130, 66)]
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device)
    alone = [hc.stream_logits(eng, s, [len(s)]) for s in seqs]
    # together: every step brings a different mix of portion sizes; request 0 joins late, request 2 skips a step
    streams = [eng.open_stream() for _ in seqs]
    got = [[] for _ in seqs]
    at = [0] * len(seqs)
    plan = [{1: 5, 2: 64}, {0: 1, 1: 1, 2: 2, 3: 30}, {1: 31, 3: 36}, {2: 64, 3: 0}]
    for step in plan:
        entries, who = [], []
        for i, k in step.items():
            if k:
                entries.append((streams[i], seqs[i][at[i]:at[i] + k], list(range(k))))
                who.append((i, k))
                at[i] += k
        lg = eng.feed(entries).double().cpu()
        r = 0
        for i, k in who:
            got[i].append(lg[r:r + k])
            r += k
    assert at == [len(s) for s in seqs]
    for i, s in enumerate(streams):
        eng.close_stream(s)
        assert torch.equal(torch.cat(got[i]), alone[i]), f"request {i} depends on its batch"
    ref = hc.oracle_logits(FULL, wt, seqs[2])
    assert hc.rel_err(alone[2], ref) < F32_TOL


def test_pages_and_slots_are_reused(cuda_device):
    """Two slots and five pages for eight sequences: every later sequence runs in a slot whose state another one left
    and on pages that held other keys."""
    wt = _weights(FULL, 8)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=192, n_pages=1 + 5)
    lens = [100, 70, 5, 128, 64, 1, 150, 65]
    for k, n in enumerate(lens):
        toks = hc.tokens_for(FULL, n, seed=40 + k)
        ref = hc.oracle_logits(FULL, wt, toks)
        held = eng.open_stream()
        eng.feed([(held, hc.tokens_for(FULL, 60 + k, seed=k), [])])          # a neighbour that dirties the other slot
        got = hc.stream_logits(eng, toks, [max(1, n // 2), 2])
        eng.close_stream(held)
        assert hc.rel_err(got, ref) < F32_TOL, f"sequence {k}"
        assert len(eng.free_pages) == 5 and len(eng.free_slots) == 2
    with pytest.raises(RuntimeError):                                         # the pool really is that small
        s = eng.open_stream()
        try:
            eng.feed([(s, hc.tokens_for(FULL, 190), [])])
            t = eng.open_stream()
            eng.feed([(t, hc.tokens_for(FULL, 190), [])])
        finally:
            eng.close_stream(s)


def test_far_keys_and_page_borders_with_a_peaked_softmax(cuda_device):
    """A large score scale makes every query put nearly all its weight on ONE earlier key, somewhere among up to 330:
    a key that is dropped, shifted by one or read from the wrong page changes that query's logits by O(1).  330 tokens
    span five page borders; prompts, portions that end on / next to a border, and single decoded tokens."""
    config = hc.model([hc.par_layer(heads=4, kv_heads=2, dim=24, vdim=40, rot=8, scale=6.0, left_scale=1.0, right_scale=0.0)])
    wt = _weights(config, 9)
    toks = hc.tokens_for(config, 330, seed=3)
    ref = hc.oracle_logits(config, wt, toks)
    from oracle import hybrid_oracle as ho
    eng = hc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([330], [63, 1, 1, 63, 2, 126], [64, 64, 64, 64], [200]):
        assert hc.rel_err(hc.stream_logits(eng, toks, portions), ref) < F32_TOL
    # losing the oldest page of keys must be visible far away at this scale (the sharpness of the test itself; rotary
    # angles are relative, so cutting the front changes nothing else)
    shifted = ho.forward(config, wt, toks[64:])
    assert hc.rel_err(shifted[150:], ref[214:]) > 50 * F32_TOL


def test_long_memory_of_the_recurrent_states(cuda_device):
    """Decay close to 1 (a large positive decay bias, small step sizes): the state at token 300 still holds the first
    tokens, so a state that is lost, reset or not carried across portions shows at every later position."""
    config = hc.model([hc.gla_layer(tau=8.0), hc.par_layer(left_scale=0.0, right_scale=1.0)])
    wt = _weights(config, 11)
    wt["l0.mix.a2.b"] += 4.0
    wt["l1.mix.right.dt_bias"] -= 3.0
    toks = hc.tokens_for(config, 300, seed=4)
    ref = hc.oracle_logits(config, wt, toks)
    from oracle import hybrid_oracle as ho
    assert hc.rel_err(ho.forward(config, wt, toks[1:])[250:], ref[251:]) > 50 * F32_TOL   # token 0 still matters at 250+
    eng = hc.build_engine(config, wt, torch.float32, cuda_device)
    assert hc.rel_err(hc.stream_logits(eng, toks, [300]), ref) < F32_TOL
    assert hc.rel_err(hc.stream_logits(eng, toks, [7, 2, 120, 2, 9]), ref) < F32_TOL      # then 160 single tokens


@pytest.mark.parametrize("piece", [16, 64])
def test_long_portions_as_side_by_side_pieces(cuda_device, piece):
    """The recurrences of a long portion cut into pieces that are scanned from a zero state, chained, and corrected by
    the incoming state's share (prl_gla_scan_split / prl_ssd_scan_split), in fp32 against the oracle: pieces that end
    inside a portion, a ragged last piece, portions below the threshold walking token by token from the state the
    pieces left (and the other way round), several long segments in one batch, and decays close to 1 so that the
    first tokens still matter hundreds of tokens and many pieces later."""
    config = hc.model([hc.gla_layer(tau=8.0, mlp=hc.dense()), hc.par_layer(mlp=hc.dense(ff=48)),
                       hc.shared(hc.gla_layer(tau=8.0, mlp=hc.dense()), 0),
                       hc.par_layer(heads=2, kv_heads=1, dim=12, vdim=8, rot=4, conv=2, groups=1, norm_groups=1, s_heads=2,
                                    s_vdim=16, state=20)], vocab=80, width=64)
    wt = _weights(config, 21)
    wt["l0.mix.a2.b"] += 4.0
    wt["l1.mix.right.dt_bias"] -= 3.0
    toks = hc.tokens_for(config, 300, seed=9)
    ref = hc.oracle_logits(config, wt, toks)
    from oracle import hybrid_oracle as ho
    assert hc.rel_err(ho.forward(config, wt, toks[1:])[250:], ref[251:]) > 50 * F32_TOL   # token 0 still matters at 250+
    eng = hc.build_engine(config, wt, torch.float32, cuda_device, prefill_chunk=256)
    eng.split_scan, eng.split_min_rows, eng.piece_tokens = True, 40, piece
    for portions in ([300], [41, 2, 130, 3, 100], [1, 255, 39, 2]):
        assert hc.rel_err(hc.stream_logits(eng, toks, portions), ref) < F32_TOL
    assert eng._rows.n_sub == 0                       # the last batches were single tokens: no pieces
    a, b, c = eng.open_stream(), eng.open_stream(), eng.open_stream()
    other = hc.tokens_for(config, 75, seed=10)
    eng.feed([(c, toks[:5], [])])
    got = eng.feed([(a, toks[:100], list(range(100))), (c, toks[5:6], [0]), (b, other, list(range(75)))]).double().cpu()
    assert eng._rows.n_sub == -(-100 // piece) + 1 + -(-75 // piece)
    assert hc.rel_err(got[:100], ref[:100]) < F32_TOL and hc.rel_err(got[100:101], ref[5:6]) < F32_TOL
    assert hc.rel_err(got[101:], hc.oracle_logits(config, wt, other)) < F32_TOL
    got = eng.feed([(a, toks[100:190], list(range(90))), (b, toks[:1], [])]).double().cpu()      # pieces continue a state
    assert hc.rel_err(got, ref[100:190]) < F32_TOL
    for s in (a, b, c):
        eng.close_stream(s)


def test_first_tokens_and_one_token_sequences(cuda_device):
    wt = _weights(FULL, 12)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device)
    for n in (1, 2, 3, 4):
        toks = hc.tokens_for(FULL, n, seed=70 + n)
        ref = hc.oracle_logits(FULL, wt, toks)
        assert hc.rel_err(hc.stream_logits(eng, toks, [n]), ref) < F32_TOL
        assert hc.rel_err(hc.stream_logits(eng, toks, []), ref) < F32_TOL


@pytest.mark.parametrize("plain_gemm", [False, True])
def test_bf16_serving_mode(cuda_device, plain_gemm):
    """bf16 operands and cache with the tcgen05 GEMMs (and with the CUDA-core GEMM) against the float64 oracle."""
    config = hc.model([hc.gla_layer(heads=4, dim=16, vdim=32, rank=8, mlp=hc.dense(ff=136)), hc.par_layer(mlp=hc.dense(ff=72))],
                      vocab=200, width=128)
    wt = _weights(config, 13)
    toks = hc.tokens_for(config, 200, seed=8)
    ref = hc.oracle_logits(config, wt, toks)
    eng = hc.build_engine(config, wt, torch.bfloat16, cuda_device)
    eng.force_plain_gemm = plain_gemm
    assert hc.rel_err(hc.stream_logits(eng, toks, [200]), ref) < BF16_TOL      # > 128 rows: the CTA-pair GEMM
    assert hc.rel_err(hc.stream_logits(eng, toks, [100, 2, 30]), ref) < BF16_TOL


def test_greedy_generation_through_the_scheduler(cuda_device):
    """DecodeEngine-style entry point: add_request / run_prefill / CUDA-graph token steps / harvest, five prompts on two
    slots (slots and pages are reused), greedy ids against the oracle wherever its top-2 margin is not a rounding matter."""
    from pipelinerl_b200.engine import SamplingParams
    wt = _weights(FULL, 14)
    eng = hc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=256, use_cuda_graph=True,
                          prefill_chunk=64)
    prompts = [hc.tokens_for(FULL, n, seed=90 + n) for n in (1, 5, 70, 130, 64)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, greedy=True, ignore_eos=True))
    assert len(eng.free_slots) == 2 and len(eng.free_pages) == eng.n_pages - 1
    for p, r in zip(prompts, outs):
        assert len(r.output_ids) == 6 and r.finish_reason == "length"
        seq = list(p)
        for tok, lp in zip(r.output_ids, r.output_logprobs):
            lg = hc.oracle_logits(FULL, wt, seq)[-1]
            top = torch.topk(lg, 2)
            if (top.values[0] - top.values[1]).item() > 1e-3:
                assert tok == top.indices[0].item()
            assert abs(lp - torch.log_softmax(lg, -1)[tok].item()) < 1e-3
            seq.append(tok)


def test_trace_runner_command_line(cuda_device, tmp_path):
    """bin/trace_run on a checkpoint folder: registry, safetensors loader, streams, output files, in both dtypes."""
    config = hc.model([hc.gla_layer(mlp=hc.dense()), hc.par_layer()], vocab=64, width=40)
    wt = _weights(config, 15)
    hc.write_checkpoint(tmp_path, config, wt)
    a, b = hc.tokens_for(config, 90, seed=1), hc.tokens_for(config, 20, seed=2)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:50], want=[0, 49])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[50:52], want=[]), dict(id="b", tokens=b[:19], want=[3])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=b[19:], want=[0]), dict(id="a", tokens=a[52:], want=[37])], end=["a", "b"]),
        dict(step=3, entries=[dict(id="c", tokens=b, want=[19])], end=["c"]),
    ]
    ra, rb = hc.oracle_logits(config, wt, a), hc.oracle_logits(config, wt, b)
    expect = {0: torch.stack([ra[0], ra[49]]), 1: rb[3:4], 2: torch.stack([rb[19], ra[89]]), 3: rb[19:20]}
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    for dtype, tol in (("float32", F32_TOL), ("bfloat16", BF16_TOL)):
        out = tmp_path / dtype
        p = subprocess.run([sys.executable, str(root / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", dtype,
                            "--out", str(out), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0, p.stderr[-2000:]
        assert [l for l in p.stdout.split("\n") if l.startswith("done")] == [f"done {i}" for i in range(4)]
        import numpy as np
        for i, ref in expect.items():
            got = torch.from_numpy(np.fromfile(out / f"{i}.f32", dtype="<f4")).view(-1, config["vocab"])
            assert got.shape == ref.shape and hc.rel_err(got, ref) < tol


def test_head_size_128_runs_the_tcgen05_attention_kernels(cuda_device):
    """bf16 with key = value size 128: the layer takes the chunked-prefill (tcgen05) and paged-decode kernels of the
    Qwen2 engine, with its own score scale; against the oracle, against the any-geometry kernel, and through generation."""
    from pipelinerl_b200.engine import SamplingParams
    config = hc.model([hc.par_layer(heads=4, kv_heads=2, dim=128, vdim=128, rot=32, scale=0.11, mlp=hc.dense(ff=128)),
                       hc.gla_layer(heads=2, dim=32, vdim=64, rank=8)], vocab=160, width=256)
    wt = _weights(config, 21)
    toks = hc.tokens_for(config, 300, seed=9)
    ref = hc.oracle_logits(config, wt, toks)
    eng = hc.build_engine(config, wt, torch.bfloat16, cuda_device, use_cuda_graph=True, max_seq_len=512)
    assert eng.tc_attn[0]
    fast = hc.stream_logits(eng, toks, [200, 2, 63, 1, 1])
    assert hc.rel_err(fast, ref) < BF16_TOL
    eng.force_plain_attn = True
    plain = hc.stream_logits(eng, toks, [200, 2, 63, 1, 1])
    eng.force_plain_attn = False
    assert hc.rel_err(plain, ref) < BF16_TOL and hc.rel_err(fast, plain) < BF16_TOL
    # ff = 128: the clamped gate runs in the gate_up GEMM's epilogue (both the 200-row and the few-row kernel); against
    # the separate activation kernel on the fp32 GEMM output
    eng.unfused_glu = True
    unfused = hc.stream_logits(eng, toks, [200, 2, 63, 1, 1])
    eng.unfused_glu = False
    assert hc.rel_err(unfused, ref) < BF16_TOL and hc.rel_err(fast, unfused) < 0.25 * BF16_TOL
    # two requests in one batch (a portion beside a single token, then the reverse) against each alone
    a, b = toks[:150], toks[150:260]
    alone_a, alone_b = hc.stream_logits(eng, a, [len(a)]), hc.stream_logits(eng, b, [len(b)])
    sa, sb = eng.open_stream(), eng.open_stream()
    l1 = eng.feed([(sa, a[:149], list(range(149))), (sb, b[:1], [0])]).double().cpu()
    l2 = eng.feed([(sb, b[1:], list(range(109))), (sa, a[149:], [0])]).double().cpu()
    eng.close_stream(sa), eng.close_stream(sb)
    assert hc.rel_err(torch.cat([l1[:149], l2[109:]]), alone_a) < 0.25 * BF16_TOL
    assert hc.rel_err(torch.cat([l1[149:], l2[:109]]), alone_b) < 0.25 * BF16_TOL
    # decode steps through the CUDA graph: the paged-decode kernel reads what the prefill kernel's front end cached
    prompts = [toks[:130], toks[:3]]
    outs = eng.generate(prompts, SamplingParams(max_tokens=5, greedy=True, ignore_eos=True))
    for p, r in zip(prompts, outs):
        seq = list(p)
        for tok, lp in zip(r.output_ids, r.output_logprobs):
            lg = hc.oracle_logits(config, wt, seq)[-1]
            assert abs(lp - torch.log_softmax(lg, -1)[tok].item()) < 0.15
            seq.append(tok)


def test_rollouts_through_the_plugin_interface(cuda_device):
    """The family behind the framework's serving thread and LLM handle (serving.EngineServer, llm.TrainableLLM,
    actor.schedule_rollouts with the synthetic rollout plugin): temperature-1 sampling by the engine's own sampler, more
    rollouts than slots, and every returned logprob equal to the oracle's log-softmax at the sampled token."""
    import asyncio
    from pipelinerl_b200.actor import schedule_rollouts
    from pipelinerl_b200.domains.synthetic import load_problems
    from pipelinerl_b200.llm import SyntheticTokenizer, TrainableLLM
    from pipelinerl_b200.serving import EngineServer
    config = hc.model([hc.gla_layer(mlp=hc.dense()), hc.par_layer(mlp=hc.dense(ff=48))], vocab=96, width=64)
    wt = _weights(config, 31)
    eng = hc.build_engine(config, wt, torch.float32, cuda_device, max_batch=3, max_seq_len=128, max_new_tokens=16,
                          use_cuda_graph=True, eos_id=2)
    server = EngineServer("hybrid-sampler", eng).start()
    try:
        llm = TrainableLLM(server.base_url, "tiny-hybrid", parameters={"max_tokens": 7, "temperature": 1.0},
                           tokenizer=SyntheticTokenizer(vocab_size=config["vocab"]))
        problems = load_problems(["train"], n_problems=3, prompt_tokens=21, vocab_limit=config["vocab"])
        groups = []
        stats = asyncio.run(schedule_rollouts(None, 3, problems, [llm],
                                              "pipelinerl_b200.domains.synthetic.generate_synthetic_rollout", groups.append,
                                              get_model_version=lambda: 0))
        assert stats["groups"] == 3 and stats["finished"] == 9
    finally:
        server.stop()
    checked = 0
    for group in groups:
        for result in group:
            text = result.training_texts[0]
            ids, lps = list(text.input_ids), list(text.logprobs)
            n_prompt = len(ids) - len(lps)
            assert n_prompt == 21 and 1 <= len(lps) <= 7
            ref = torch.log_softmax(hc.oracle_logits(config, wt, ids[:-1]), -1)
            for k, lp in enumerate(lps):
                assert abs(lp - ref[n_prompt - 1 + k, ids[n_prompt + k]].item()) < 2e-3
                checked += 1
    assert checked >= 9
