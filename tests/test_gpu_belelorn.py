"""The Belelorn decoders on the hybrid engine (pipelinerl_b200/hybrid.py and its kernels) against
oracle/belelorn_oracle.py: each mechanism alone, whole prompts against token-by-token decoding, portions down to two
tokens, unequal batches against each request alone, pages and slots that are given back and taken again, keys far
away, at page borders and just inside / outside the window and the kept first tokens (prompts and decoding), the first
tokens, long decoding, awkward sizes, greedy generation through the engine's scheduler, and the trace runner."""
import copy
import json
import subprocess
import sys

import pytest
import torch

from tests import belelorn_cases as bc

pytestmark = pytest.mark.gpu

F32_TOL = 2e-4      # fp32 kernels against the float64 oracle
BF16_TOL = 8e-2     # bf16 operands / cache: rounding of activations dominates


def _weights(config, seed=0):
    from oracle import belelorn_oracle as bo
    return bo.random_weights(config, seed)


def _only(wt, side):
    """Silence one branch of every parallel mixer (its width gain to zero): the other branch alone reaches the stream."""
    for name in wt:
        if name.endswith(f"mix.{side}.out"):
            wt[name] = torch.zeros_like(wt[name])
    return wt


# ---- each mechanism alone ---------------------------------------------------------------------------------------
def _mechanisms():
    a = bc.attn
    return {
        "attention_window_sinks": (bc.model([bc.par_layer()]), "right"),
        "attention_no_sinks_one_kv_head": (bc.model([bc.par_layer(left=a(heads=3, kv_heads=1, dim=20, size=17, keep_first=0))]), "right"),
        "attention_window_longer_than_prompt": (bc.model([bc.par_layer(left=a(heads=2, kv_heads=2, dim=7, size=400, keep_first=5))]), "right"),
        "attention_hard_cap": (bc.model([bc.par_layer(left=a(scale=3.0, softcap=2.0, size=33, keep_first=1))]), "right"),
        "lightning": (bc.model([bc.par_layer()]), "left"),
        "lightning_slow_and_fast_decay": (bc.model([bc.par_layer(right=bc.lightning(heads=2, dim=17, vdim=33, decay=[0.9995, 0.05]))]), "left"),
        "both_branches": (bc.model([bc.par_layer()]), None),
        "mlstm": (bc.model([bc.mlstm_layer()]), None),
        "mlstm_one_head_tight_cap": (bc.model([bc.mlstm_layer(heads=1, dim=33, vdim=7, gate_cap=2.0)]), None),
        "squared_relu": (bc.model([bc.mlstm_layer(mlp=bc.dense())]), None),
        "routed_top2_shared": (bc.model([bc.mlstm_layer(mlp=bc.moe())]), None),
        "routed_top1_no_shared": (bc.model([bc.mlstm_layer(mlp=bc.moe(experts=7, top=1, ff=10, shared_ff=0))]), None),
        "routed_all_experts": (bc.model([bc.par_layer(mlp=bc.moe(experts=3, top=3, ff=9, limit=0.4, shared_ff=16))]), None),
        "repeated_block": (bc.model([bc.mlstm_layer(mlp=bc.dense()), bc.par_layer(mlp=bc.dense(ff=40))], loop=(0, 2, 3)), None),
        "repeated_block_inside": (bc.model([bc.par_layer(), bc.mlstm_layer(mlp=bc.dense()), bc.par_layer(mlp=bc.moe())],
                                           loop=(1, 2, 2)), None),
    }


@pytest.mark.parametrize("name", sorted(_mechanisms()))
def test_each_mechanism_matches_the_oracle_fp32(cuda_device, name):
    config, silence = _mechanisms()[name]
    wt = _weights(config, seed=len(name))
    if silence:
        _only(wt, silence)
    toks = bc.tokens_for(config, 150)
    ref = bc.oracle_logits(config, wt, toks)
    eng = bc.build_engine(config, wt, torch.float32, cuda_device)
    assert bc.rel_err(bc.stream_logits(eng, toks, [150]), ref) < F32_TOL
    assert bc.rel_err(bc.stream_logits(eng, toks, [2, 3, 61, 2, 7, 64, 2]), ref) < F32_TOL     # then one by one
    # the residual stream after every layer run of a whole prompt
    from oracle import belelorn_oracle as bo
    res = []
    bo.forward(config, wt, toks[:20], res)
    s = eng.open_stream()
    s.prompt_ids.extend(toks[:20])
    s.pages += eng._alloc_pages(1)
    eng.block_table[s.slot, :1].copy_(torch.tensor(s.pages, dtype=torch.int32))
    got = []
    eng._forward_rows([(s, 0, 20)], [], trace=got)
    eng.close_stream(s)
    assert len(got) == len(res)
    for a, b in zip(got, res):
        assert (a.double().cpu() - b).abs().max().item() < 1e-4 * max(1.0, b.abs().max().item())


FULL = bc.model([bc.par_layer(mlp=bc.dense()), bc.mlstm_layer(mlp=bc.moe()), bc.par_layer(left=bc.attn(heads=2, kv_heads=1, dim=16, size=70, keep_first=2),
                                                                                           right=bc.lightning(heads=2, dim=8, vdim=24), mlp=None),
                 bc.mlstm_layer(heads=2, dim=16, vdim=12, mlp=bc.dense(ff=48))], vocab=80, width=64, loop=(1, 3, 2))


def test_prefill_against_token_by_token_decoding(cuda_device):
    wt = _weights(FULL, 3)
    toks = bc.tokens_for(FULL, 140, seed=5)
    ref = bc.oracle_logits(FULL, wt, toks)
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device)
    whole = bc.stream_logits(eng, toks, [140])
    single = bc.stream_logits(eng, toks, [])                                 # every token alone, through the cache / state
    assert bc.rel_err(whole, ref) < F32_TOL and bc.rel_err(single, ref) < F32_TOL
    assert bc.rel_err(whole, single) < 2e-5


@pytest.mark.parametrize("portions", [[2] * 40, [63, 2, 63, 2], [64, 64], [1, 65, 1, 2, 59], [129, 2]])
def test_portions_of_several_sizes(cuda_device, portions):
    wt = _weights(FULL, 4)
    toks = bc.tokens_for(FULL, 140, seed=6)
    ref = bc.oracle_logits(FULL, wt, toks)
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device, prefill_chunk=96)   # 129 is cut by the engine too
    assert bc.rel_err(bc.stream_logits(eng, toks, portions), ref) < F32_TOL


def test_unequal_batches_equal_each_request_alone(cuda_device):
    wt = _weights(FULL, 7)
    seqs = [bc.tokens_for(FULL, n, seed=10 + n) for n in (1, 37, 130, 66)]
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device)
    alone = [bc.stream_logits(eng, s, [len(s)]) for s in seqs]
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
        assert bc.rel_err(torch.cat(got[i]), alone[i]) < 2e-5, f"request {i} depends on its batch"
    assert bc.rel_err(alone[2], bc.oracle_logits(FULL, wt, seqs[2])) < F32_TOL


def test_pages_and_slots_are_reused(cuda_device):
    """Two slots and five pages for eight sequences: every later sequence runs in a slot whose states (matrix memories,
    the gates' running maximum) another one left, and on pages that held other keys."""
    wt = _weights(FULL, 8)
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=192, n_pages=1 + 5)
    lens = [100, 70, 5, 128, 64, 1, 150, 65]
    for k, n in enumerate(lens):
        toks = bc.tokens_for(FULL, n, seed=40 + k)
        ref = bc.oracle_logits(FULL, wt, toks)
        held = eng.open_stream()
        eng.feed([(held, bc.tokens_for(FULL, 60 + k, seed=k), [])])          # a neighbour that dirties the other slot
        got = bc.stream_logits(eng, toks, [max(1, n // 2), 2])
        eng.close_stream(held)
        assert bc.rel_err(got, ref) < F32_TOL, f"sequence {k}"
        assert len(eng.free_pages) == 5 and len(eng.free_slots) == 2


def _peaked(window, keep_first, heads=2, kv_heads=1, dim=16):
    """One attention layer (the other branch silenced) whose softmax is nearly one-hot: score scale 2.5 on unit-RMS
    vectors and a cap far above the scores, so each query puts almost all its weight on a single visible key."""
    return bc.model([bc.par_layer(left=bc.attn(heads=heads, kv_heads=kv_heads, dim=dim, scale=2.5, softcap=500.0, size=window,
                                               keep_first=keep_first))], width=48, vocab=64)


@pytest.mark.parametrize("window,keep_first", [(64, 4), (37, 1), (129, 70)])
def test_window_edges_kept_tokens_and_page_borders(cuda_device, window, keep_first):
    """330 tokens span five page borders.  With a peaked softmax a key that is dropped, shifted by one, wrongly kept or
    read from the wrong page changes the logits by O(1): the oracle with the window one longer or shorter, or one kept
    token more or fewer, is far outside the tolerance (checked first: that is the sharpness of this test).  Prompts,
    portions that end on and next to page borders and window edges, and single decoded tokens."""
    config = _peaked(window, keep_first)
    wt = _only(_weights(config, 9), "right")
    toks = bc.tokens_for(config, 330, seed=3)
    ref = bc.oracle_logits(config, wt, toks)
    for dw, dk in ((1, 0), (-1, 0), (0, 1), (0, -1)):
        other = copy.deepcopy(config)
        other["layers"][0]["mixer"]["left"]["mask"] = dict(size=window + dw, keep_first=keep_first + dk)
        assert bc.rel_err(bc.oracle_logits(other, wt, toks)[window + keep_first:], ref[window + keep_first:]) > 25 * F32_TOL
    eng = bc.build_engine(config, wt, torch.float32, cuda_device)
    for portions in ([330], [63, 1, 1, 63, 2, 126], [64, 64, 64, 64], [window - 1, 2, window, 1, keep_first + 1], [200]):
        assert bc.rel_err(bc.stream_logits(eng, toks, portions), ref) < F32_TOL
    assert bc.rel_err(bc.stream_logits(eng, toks[:200], [3]), ref[:200]) < F32_TOL        # 197 decoded tokens pass the window


def test_far_tokens_in_the_recurrent_states(cuda_device):
    """Decays close to 1 and forget gates close to open: the states at token 300 still hold the first tokens, so a state
    that is lost, reset or not carried across portions shows at every later position."""
    config = bc.model([bc.par_layer(right=bc.lightning(heads=2, dim=12, vdim=20, decay=[0.999, 0.9999])), bc.mlstm_layer()])
    wt = _only(_weights(config, 11), "left")
    wt["l1.mix.f.b"] += 6.0
    toks = bc.tokens_for(config, 300, seed=4)
    ref = bc.oracle_logits(config, wt, toks)
    other = [(toks[0] + 1) % config["vocab"]] + toks[1:]
    assert bc.rel_err(bc.oracle_logits(config, wt, other)[250:], ref[250:]) > 50 * F32_TOL     # token 0 still matters at 250+
    eng = bc.build_engine(config, wt, torch.float32, cuda_device)
    assert bc.rel_err(bc.stream_logits(eng, toks, [300]), ref) < F32_TOL
    assert bc.rel_err(bc.stream_logits(eng, toks, [7, 2, 120, 2, 9]), ref) < F32_TOL      # then 160 single tokens


def test_strong_input_gates_need_the_stabiliser(cuda_device):
    """Input-gate pre-activations pushed up to the cap (exp(12) unstabilised) and, in a second model, forget gates
    pushed shut: the running maximum keeps everything in range and the normaliser's floor exp(-m) takes part."""
    for shift_i, shift_f in ((30.0, 0.0), (-30.0, -30.0)):
        config = bc.model([bc.mlstm_layer(heads=2, dim=8, vdim=12, gate_cap=12.0)])
        wt = _weights(config, 5)
        wt["l0.mix.i.b"] += shift_i
        wt["l0.mix.f.b"] += shift_f
        toks = bc.tokens_for(config, 90, seed=2)
        ref = bc.oracle_logits(config, wt, toks)
        eng = bc.build_engine(config, wt, torch.float32, cuda_device)
        assert bc.rel_err(bc.stream_logits(eng, toks, [50, 2]), ref) < F32_TOL


@pytest.mark.parametrize("piece", [16, 64])
def test_long_portions_as_side_by_side_pieces(cuda_device, piece):
    """The matrix-state recurrences of a long portion cut into pieces that are scanned from a zero state, chained, and
    corrected by the incoming state's share (prl_decay_scan_split), in fp32 against the oracle."""
    config = bc.model([bc.par_layer(right=bc.lightning(heads=2, dim=12, vdim=20, decay=[0.999, 0.97]), mlp=bc.dense()),
                       bc.mlstm_layer(mlp=bc.moe())], vocab=80, width=64, loop=(0, 2, 2))
    wt = _weights(config, 21)
    wt["l1.mix.f.b"] += 5.0
    toks = bc.tokens_for(config, 300, seed=9)
    ref = bc.oracle_logits(config, wt, toks)
    eng = bc.build_engine(config, wt, torch.float32, cuda_device, prefill_chunk=256)
    eng.split_scan, eng.split_min_rows, eng.piece_tokens = True, 40, piece
    for portions in ([300], [41, 2, 130, 3, 100], [1, 255, 39, 2]):
        assert bc.rel_err(bc.stream_logits(eng, toks, portions), ref) < F32_TOL
    a, b = eng.open_stream(), eng.open_stream()
    other = bc.tokens_for(config, 75, seed=10)
    got = eng.feed([(a, toks[:100], list(range(100))), (b, other, list(range(75)))]).double().cpu()
    assert eng._rows.n_sub == -(-100 // piece) + -(-75 // piece)
    assert bc.rel_err(got[:100], ref[:100]) < F32_TOL
    assert bc.rel_err(got[100:], bc.oracle_logits(config, wt, other)) < F32_TOL
    eng.close_stream(a), eng.close_stream(b)


def test_first_tokens_and_one_token_sequences(cuda_device):
    wt = _weights(FULL, 12)
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device)
    for n in (1, 2, 3, 4):
        toks = bc.tokens_for(FULL, n, seed=70 + n)
        ref = bc.oracle_logits(FULL, wt, toks)
        assert bc.rel_err(bc.stream_logits(eng, toks, [n]), ref) < F32_TOL
        assert bc.rel_err(bc.stream_logits(eng, toks, []), ref) < F32_TOL


def test_routing_follows_the_scores(cuda_device):
    """Router rows scaled so that the choice is never a close call, eleven experts of which three are taken: a wrong
    expert, a renormalised weight or a weight applied after the expert instead of before its clamps shows at once."""
    config = bc.model([bc.mlstm_layer(mlp=bc.moe(experts=11, top=3, ff=12, limit=0.3, shared_ff=0))], width=40)
    wt = _weights(config, 17)
    wt["l0.mlp.router"] = (wt["l0.mlp.router"] * 3.0).to(torch.bfloat16).double()
    toks = bc.tokens_for(config, 120, seed=4)
    ref = bc.oracle_logits(config, wt, toks)
    eng = bc.build_engine(config, wt, torch.float32, cuda_device)
    assert bc.rel_err(bc.stream_logits(eng, toks, [100, 2]), ref) < F32_TOL


@pytest.mark.parametrize("plain_gemm", [False, True])
def test_bf16_serving_mode(cuda_device, plain_gemm):
    """bf16 operands and cache with the tcgen05 GEMMs (and with the CUDA-core GEMM) against the float64 oracle.  The
    routed feed-forward sits in the last layer run, so a token whose two best-but-one router logits are closer than bf16
    rounding can tell apart (the oracle reports the gaps) touches only its own logits; those positions are left out."""
    from oracle import belelorn_oracle as bo
    config = bc.model([bc.par_layer(left=bc.attn(heads=4, kv_heads=2, dim=32, size=48, keep_first=2), right=bc.lightning(heads=2, dim=32, vdim=64),
                                    mlp=bc.dense(ff=136)),
                       bc.mlstm_layer(heads=2, dim=16, vdim=32, mlp=bc.moe(experts=6, top=2, ff=64, shared_ff=128))],
                      vocab=200, width=128, loop=(0, 1, 2))
    wt = _weights(config, 13)
    toks = bc.tokens_for(config, 300, seed=8)
    gaps = []
    ref = bo.forward(config, wt, toks, margins=gaps)
    clear = torch.tensor(gaps[-1]) > 0.1
    assert len(gaps) == 1 and clear.float().mean().item() > 0.8
    eng = bc.build_engine(config, wt, torch.bfloat16, cuda_device)
    eng.force_plain_gemm = plain_gemm
    whole = bc.stream_logits(eng, toks, [300])                                 # pieces side by side, the CTA-pair GEMM
    assert bc.rel_err(whole[clear], ref[clear]) < BF16_TOL
    assert bc.rel_err(bc.stream_logits(eng, toks, [100, 2, 30])[clear], ref[clear]) < BF16_TOL


@pytest.mark.parametrize("dim,window,keep_first", [(64, 37, 1), (128, 64, 4), (32, 129, 70), (64, 0, 0)])
def test_tensor_core_attention_for_prompt_portions(cuda_device, dim, window, keep_first):
    """bf16 with head sizes 32 / 64 / 128: portions of 16 rows and more take the mma.sync attention kernel.  Peaked softmax,
    330 tokens over five page borders, two query heads per key head; against the CUDA-core kernel on the same cache
    (they differ only by the bf16 rounding of the softmax weights) and against the oracle."""
    from pipelinerl_b200 import _lib
    config = _peaked(window or 1000, keep_first, heads=4, kv_heads=2, dim=dim)
    config["width"] = 64
    wt = _only(_weights(config, 9), "right")
    toks = bc.tokens_for(config, 330, seed=3)
    ref = bc.oracle_logits(config, wt, toks)
    eng = bc.build_engine(config, wt, torch.bfloat16, cuda_device)
    lib = _lib.load()
    try:
        fast = [bc.stream_logits(eng, toks, portions) for portions in ([330], [63, 17, 16, 130, 65, 20])]
        lib.prl_attn_any_tensor_cores(0)
        plain = [bc.stream_logits(eng, toks, portions) for portions in ([330], [63, 17, 16, 130, 65, 20])]
    finally:
        lib.prl_attn_any_tensor_cores(1)
    for f, p in zip(fast, plain):
        assert bc.rel_err(f, p) < 0.25 * BF16_TOL
        assert bc.rel_err(f, ref) < 2 * BF16_TOL and bc.rel_err(p, ref) < 2 * BF16_TOL


def test_greedy_generation_through_the_scheduler(cuda_device):
    """add_request / run_prefill / CUDA-graph token steps / harvest, five prompts on two slots (slots and pages are
    reused), greedy ids against the oracle wherever its top-2 margin is not a rounding matter."""
    from pipelinerl_b200.engine import SamplingParams
    wt = _weights(FULL, 14)
    eng = bc.build_engine(FULL, wt, torch.float32, cuda_device, max_batch=2, max_seq_len=256, use_cuda_graph=True,
                          prefill_chunk=64)
    prompts = [bc.tokens_for(FULL, n, seed=90 + n) for n in (1, 5, 70, 130, 64)]
    outs = eng.generate(prompts, SamplingParams(max_tokens=6, greedy=True, ignore_eos=True))
    assert len(eng.free_slots) == 2 and len(eng.free_pages) == eng.n_pages - 1
    for p, r in zip(prompts, outs):
        assert len(r.output_ids) == 6 and r.finish_reason == "length"
        seq = list(p)
        for tok, lp in zip(r.output_ids, r.output_logprobs):
            lg = bc.oracle_logits(FULL, wt, seq)[-1]
            top = torch.topk(lg, 2)
            if (top.values[0] - top.values[1]).item() > 1e-3:
                assert tok == top.indices[0].item()
            assert abs(lp - torch.log_softmax(lg, -1)[tok].item()) < 1e-3
            seq.append(tok)


def test_trace_runner_command_line(cuda_device, tmp_path):
    """bin/trace_run on a checkpoint folder: registry, safetensors loader, streams, output files, in both dtypes."""
    config = bc.model([bc.par_layer(mlp=bc.moe(experts=4, top=1, ff=8, shared_ff=0)), bc.mlstm_layer(mlp=bc.dense(ff=24))],
                      vocab=64, width=40, loop=(0, 1, 2))
    wt = _weights(config, 15)
    bc.write_checkpoint(tmp_path, config, wt)
    a, b = bc.tokens_for(config, 90, seed=1), bc.tokens_for(config, 20, seed=2)
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=a[:50], want=[0, 49])], end=[]),
        dict(step=1, entries=[dict(id="a", tokens=a[50:52], want=[]), dict(id="b", tokens=b[:19], want=[3])], end=[]),
        dict(step=2, entries=[dict(id="b", tokens=b[19:], want=[0]), dict(id="a", tokens=a[52:], want=[37])], end=["a", "b"]),
        dict(step=3, entries=[dict(id="c", tokens=b, want=[19])], end=["c"]),
    ]
    ra, rb = bc.oracle_logits(config, wt, a), bc.oracle_logits(config, wt, b)
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
            assert got.shape == ref.shape and bc.rel_err(got, ref) < tol
