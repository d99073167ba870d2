"""Host side of the hybrid decoder family, no GPU: configuration parsing, the fused arena layout and its checkpoint
names, the safetensors reader, the model registry, the page pool / slot states, and the trace runner's refusal."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from tests import hybrid_cases as hc

ROOT = Path(__file__).resolve().parent.parent
CONFIG = hc.model([hc.gla_layer(mlp=hc.dense()), hc.par_layer(), hc.shared(hc.gla_layer(mlp=hc.dense()), 0),
                   hc.shared(hc.par_layer(), 1)])


def test_config_reads_every_size_and_constant():
    from pipelinerl_b200.hybrid import HybridConfig
    cfg = HybridConfig.from_povurax(CONFIG)
    assert (cfg.vocab_size, cfg.width, cfg.eps, cfg.embed_scale) == (96, 72, 1e-5, 3.0)
    g, p = cfg.layers[0], cfg.layers[1]
    assert (g.kind, g.gla.heads, g.gla.dim, g.gla.vdim, g.gla.tau, g.gla.rank, g.mlp.ff, g.mlp.limit) == ("gla", 3, 10, 24, 5.0, 5, 56, 1.25)
    assert (p.attn.heads, p.attn.kv_heads, p.attn.dim, p.attn.vdim, p.attn.rot_dims, p.attn.rot_base, p.attn.scale) == (4, 2, 24, 40, 8, 100.0, 0.3)
    assert (p.ssd.heads, p.ssd.vdim, p.ssd.state, p.ssd.groups, p.ssd.conv, p.ssd.norm_groups) == (4, 12, 12, 2, 3, 2)
    assert (p.left_scale, p.right_scale, p.mlp) == (0.7, 1.3, None)
    assert [L.weights_of for L in cfg.layers] == [0, 1, 0, 1]
    assert p.ssd.in_rows == 2 * 48 + 2 * 2 * 12 + 4 and p.ssd.conv_channels == 48 + 48


def test_config_rejects_what_the_design_does_not_have():
    from pipelinerl_b200.hybrid import HybridConfig
    bad = hc.model([hc.gla_layer()])
    bad["layers"][0]["type"] = "window"
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)
    bad = hc.model([hc.gla_layer(mlp=dict(kind="experts", ff=8, limit=1.0))])
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)
    bad = hc.model([hc.gla_layer(), hc.shared(hc.gla_layer(), 2), hc.shared(hc.gla_layer(), 1)])    # a circle
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)
    bad = hc.model([hc.gla_layer(), hc.shared(hc.par_layer(), 0)])                                 # another kind of mixer
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)
    bad = hc.model([hc.gla_layer(), hc.shared(hc.gla_layer(), 7)])
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)
    chain = HybridConfig.from_povurax(hc.model([hc.gla_layer(), hc.shared(hc.gla_layer(), 0), hc.shared(hc.gla_layer(), 1),
                                                hc.shared(hc.gla_layer(), 4), hc.gla_layer()]))
    assert [L.weights_of for L in chain.layers] == [0, 0, 0, 4, 4]       # chains and forward references resolve to the owner
    bad = hc.model([hc.par_layer(heads=3, kv_heads=2)])
    with pytest.raises(ValueError):
        HybridConfig.from_povurax(bad)


def test_checkpoint_names_tile_the_fused_tensors_exactly():
    from oracle import hybrid_oracle as ho
    from pipelinerl_b200.hybrid import HybridConfig
    from pipelinerl_b200.model import ParamArena
    cfg = HybridConfig.from_povurax(CONFIG)
    wt = ho.random_weights(CONFIG, 1)
    slices, shapes = cfg.checkpoint_slices(), dict(cfg.fused_shapes())
    assert set(slices) == set(wt), "checkpoint names and the oracle's tensors differ"
    covered = {}
    for name, (fused, r0, rn) in slices.items():
        assert wt[name].shape[0] == rn and tuple(wt[name].shape[1:]) == tuple(shapes[fused][1:])
        covered.setdefault(fused, []).append((r0, r0 + rn))
    for fused, spans in covered.items():
        spans.sort()
        assert spans[0][0] == 0 and spans[-1][1] == shapes[fused][0]
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert set(covered) == set(shapes)
    for dtype in (torch.bfloat16, torch.float32):                           # the arena on the CPU: layout only
        arena = ParamArena(cfg, "cpu", dtype=dtype)
        arena.load_hf_state_dict(wt)
        assert torch.equal(arena.view("l1.mix.in")[4 * 24:4 * 24 + 2 * 24].float(), wt["l1.mix.left.k"])
        assert torch.equal(arena.view("l0.mlp.gate_up")[56:].float(), wt["l0.mlp.up"])
    with pytest.raises(KeyError):
        ParamArena(cfg, "cpu").load_hf_state_dict({k: v for k, v in wt.items() if k != "l1.mix.right.D"})


def test_safetensors_reader_and_registry(tmp_path):
    from oracle import hybrid_oracle as ho
    from pipelinerl_b200 import registry
    wt = ho.random_weights(CONFIG, 2)
    hc.write_checkpoint(tmp_path, CONFIG, wt)
    back = registry.read_safetensors(tmp_path / "model.safetensors")
    assert set(back) == set(wt) and all(torch.equal(back[k].float(), wt[k]) for k in wt)
    fam, cfg = registry.load_config(tmp_path)                                # the rank comes from the a1 tensor's shape
    assert fam.name == "Povurax" and cfg.layers[0].gla.rank == 5 and torch.float32 in fam.dtypes
    assert registry.family_of({"architectures": ["Qwen2ForCausalLM"]}).name == "Qwen2ForCausalLM"
    with pytest.raises(KeyError):
        registry.family_of({"architecture": "Nothing"})


def test_trace_runner_refuses_a_dtype_the_family_lacks(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps(dict(
        architectures=["Qwen2ForCausalLM"], vocab_size=64, hidden_size=256, intermediate_size=128, num_hidden_layers=1,
        num_attention_heads=2, num_key_value_heads=1)))
    p = subprocess.run([sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(tmp_path), "--dtype", "float32",
                        "--out", str(tmp_path / "o"), "--max-tokens", "64"], input="", capture_output=True, text=True)
    assert p.returncode == 3


def test_page_pool_and_slot_states():
    from pipelinerl_b200.cache import PagePool, SlotStates
    pool = PagePool(5)
    a = pool.alloc(3)
    assert 0 not in a and pool.available() == 1
    pool.retain(a[0])
    pool.release(a)
    assert pool.available() == 3                  # a[0] is still held once
    pool.release([a[0]])
    assert pool.available() == 4 and sorted(pool.free) == [1, 2, 3, 4]
    with pytest.raises(RuntimeError):
        pool.alloc(5)
    with pytest.raises(RuntimeError):
        pool.release([a[1]])
    st = SlotStates(3, "cpu")
    s = st.add("m", (2, 2))
    s.fill_(1.0)
    st.reset(1)
    assert s[1].abs().sum() == 0 and s[0].sum() == 4 and st.nbytes() == 3 * 4 * 4
    with pytest.raises(KeyError):
        st.add("m", (1,))


def test_oracle_recurrences_agree_with_their_closed_forms():
    """The oracle's own loops against an independent formulation: linear attention with decay as a masked product."""
    from oracle import hybrid_oracle as ho
    config = hc.model([hc.gla_layer(heads=1, dim=4, vdim=3, rank=2)])
    wt = {k: v.double() for k, v in ho.random_weights(config, 3).items()}
    h = torch.randn(9, config["width"], dtype=torch.float64)
    got = ho.gated_linear_attention(h, wt, "l0.mix.", config["layers"][0]["mixer"], 1e-5)
    q = (h @ wt["l0.mix.q"].T) * 4 ** -0.5
    k, v = h @ wt["l0.mix.k"].T, h @ wt["l0.mix.v"].T
    la = torch.log(torch.sigmoid((h @ wt["l0.mix.a1"].T) @ wt["l0.mix.a2"].T + wt["l0.mix.a2.b"])) / 5.0
    cum = la.cumsum(0)
    o = torch.zeros(9, 3, dtype=torch.float64)
    for t in range(9):
        for s in range(t + 1):
            o[t] += (q[t] * torch.exp(cum[t] - cum[s]) * k[s]).sum() * v[s]
    o = ho.rms_unit(o, 1e-5) * wt["l0.mix.norm"]
    want = (o * ho.silu(h @ wt["l0.mix.g"].T)) @ wt["l0.mix.o"].T
    assert (got - want).abs().max() < 1e-9
