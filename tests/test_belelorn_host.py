"""Host-side checks of the Belelorn reading of a config (no GPU): layer runs of a repeated block, the fused arena layout
against the checkpoint names, and the oracle's recurrences against closed forms."""
import math

import pytest
import torch

from oracle import belelorn_oracle as bo
from pipelinerl_b200.hybrid import HybridConfig
from tests import belelorn_cases as bc


def test_repeated_block_is_unrolled_into_runs():
    config = bc.model([bc.par_layer(), bc.mlstm_layer(mlp=bc.dense()), bc.par_layer(mlp=bc.moe()), bc.mlstm_layer()], loop=(1, 3, 3))
    cfg = HybridConfig.from_belelorn(config)
    assert [(L.weights_of, L.opens_pass) for L in cfg.layers] == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2),
                                                                  (2, None), (3, None)]
    assert [(i, p) for i, p in bo.layer_runs(config)] == [(L.weights_of, L.opens_pass) for L in cfg.layers]
    assert cfg.loop_times == 3 and cfg.norm_offset == 1.0 and cfg.positions == "sinusoid"
    plain = HybridConfig.from_belelorn(bc.model([bc.mlstm_layer()]))
    assert plain.loop_times == 0 and "loop.in" not in dict(plain.fused_shapes())


def test_every_checkpoint_tensor_has_its_rows_in_the_arena():
    config = bc.model([bc.par_layer(mlp=bc.moe(experts=3, top=2, shared_ff=0)), bc.mlstm_layer(mlp=bc.moe()),
                       bc.par_layer(mlp=bc.dense()), bc.mlstm_layer(mlp=None)], loop=(0, 2, 2))
    cfg = HybridConfig.from_belelorn(config)
    shapes, fused = bo.tensor_shapes(config), dict(cfg.fused_shapes())
    slices = cfg.checkpoint_slices()
    assert set(slices) == set(shapes)
    rows = {}
    for name, (dst, r0, n) in slices.items():
        assert shapes[name][0] == n and tuple(shapes[name][1:]) == tuple(fused[dst][1:]), name
        rows.setdefault(dst, []).append((r0, n))
    for dst, shape in fused.items():
        at = 0
        for r0, n in sorted(rows[dst]):
            assert r0 == at, dst
            at += n
        assert at == shape[0], dst


def test_bad_configs_are_refused():
    with pytest.raises(ValueError):
        HybridConfig.from_belelorn(bc.model([dict(type="conv", mixer={}, mlp=None)]))
    with pytest.raises(ValueError):
        HybridConfig.from_belelorn(bc.model([bc.mlstm_layer()], loop=(0, 2, 2)))
    with pytest.raises(ValueError):
        HybridConfig.from_belelorn(bc.model([bc.par_layer(right=bc.lightning(heads=3, decay=[0.5, 0.6]))]))
    with pytest.raises(ValueError):
        HybridConfig.from_belelorn(bc.model([bc.mlstm_layer(mlp=bc.moe(experts=2, top=3))]))


def test_oracle_lightning_equals_the_decayed_sum():
    r = bc.lightning(heads=2, dim=5, vdim=6, decay=[0.8, 0.3])
    g = torch.Generator().manual_seed(0)
    W, T = 12, 9
    wt = {"q": torch.randn(10, W, generator=g, dtype=torch.float64), "k": torch.randn(10, W, generator=g, dtype=torch.float64),
          "v": torch.randn(12, W, generator=g, dtype=torch.float64), "g": torch.randn(12, W, generator=g, dtype=torch.float64),
          "o": torch.eye(12, dtype=torch.float64), "norm": torch.ones(12, dtype=torch.float64)}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = bo.lightning_attention(h, wt, "", r, 1e-6)
    q, k, v = (bo.silu(h @ wt[n].T) for n in "qkv")
    raw = torch.zeros(T, 12, dtype=torch.float64)
    for head in range(2):
        for t in range(T):
            for s in range(t + 1):
                raw[t, head * 6:(head + 1) * 6] += r["decay"][head] ** (t - s) * (q[t, head * 5:(head + 1) * 5] @ k[s, head * 5:(head + 1) * 5]) * v[s, head * 6:(head + 1) * 6]
    want = bo.rms_unit(raw, 1e-6) * torch.sigmoid(h @ wt["g"].T)
    assert (got - want).abs().max().item() < 1e-12


def test_oracle_mlstm_equals_the_unstabilised_cell_where_that_is_representable():
    """With small gates the cell can be written without its running maximum: C_t = F_t C_(t-1) + I_t k v^T with
    F = sigmoid-like exp(f), I = exp(i); its read-out o = C^T q / (max(|n . q|, 1) + 1e-6 exp(m)) ... the stabilised
    form differs from it only through the 1e-6 term, which is scaled by exp(-m); compared with that term tracked."""
    m = dict(heads=1, dim=4, vdim=3, gate_cap=15.0)
    g = torch.Generator().manual_seed(1)
    W, T = 8, 12
    wt = {n: torch.randn(s, W, generator=g, dtype=torch.float64) * 0.5 for n, s in (("q", 4), ("k", 4), ("v", 3), ("g", 3), ("i", 1), ("f", 1))}
    wt.update({"i.b": torch.zeros(1, dtype=torch.float64), "f.b": torch.ones(1, dtype=torch.float64), "o": torch.eye(3, dtype=torch.float64),
               "norm": torch.ones(3, dtype=torch.float64)})
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    got = bo.mlstm(h, wt, "", m, 1e-6)
    q, k, v = (h @ wt["q"].T) * 0.5, h @ wt["k"].T, h @ wt["v"].T
    gi = 15.0 * torch.tanh((h @ wt["i"].T + wt["i.b"]) / 15.0)
    gf = torch.nn.functional.logsigmoid(15.0 * torch.tanh((h @ wt["f"].T + wt["f.b"]) / 15.0))
    C, n, run, rows = torch.zeros(4, 3, dtype=torch.float64), torch.zeros(4, dtype=torch.float64), 0.0, []
    for t in range(T):
        C = math.exp(gf[t, 0]) * C + math.exp(gi[t, 0]) * torch.outer(k[t], v[t])
        n = math.exp(gf[t, 0]) * n + math.exp(gi[t, 0]) * k[t]
        run = max(float(gf[t, 0]) + run, float(gi[t, 0]))
        rows.append((C.T @ q[t]) / (max(abs(float(n @ q[t])), 1.0) + 1e-6 * math.exp(run)))
    want = bo.rms_unit(torch.stack(rows), 1e-6) * torch.sigmoid(h @ wt["g"].T)
    assert (got - want).abs().max().item() < 1e-10


def test_oracle_window_keeps_the_first_tokens():
    a = bc.attn(heads=1, kv_heads=1, dim=4, scale=1.0, softcap=0.0, size=3, keep_first=2)
    g = torch.Generator().manual_seed(2)
    W, T = 6, 9
    wt = {"q": torch.randn(4, W, generator=g, dtype=torch.float64), "k": torch.randn(4, W, generator=g, dtype=torch.float64),
          "q.b": torch.zeros(4, dtype=torch.float64), "k.b": torch.randn(4, generator=g, dtype=torch.float64),
          "o": torch.eye(4, dtype=torch.float64)}
    h = torch.randn(T, W, generator=g, dtype=torch.float64)
    full = bo.windowed_attention(h, wt, "", a, 1e-6)
    # position 8 sees 0, 1 (kept) and 6, 7, 8 (window of three): changing token 4 or 5 changes nothing there, token 1 does
    for changed, moves in ((4, False), (5, False), (1, True), (6, True)):
        h2 = h.clone()
        h2[changed] += 1.0
        diff = (bo.windowed_attention(h2, wt, "", a, 1e-6)[8] - full[8]).abs().max().item()
        assert (diff > 1e-6) == moves, (changed, diff)
