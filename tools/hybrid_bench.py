#!/usr/bin/env python
"""Prefill and decode throughput of the hybrid decoder family beside the Qwen2 engine at equal width / depth / ff /
heads (random weights), and the new kernels alone against their rooflines.  One JSON line.

    python tools/hybrid_bench.py [--sizes w2048,w4096] [--prompt 4096] [--context 2048] [--batch 32] [--steps 20]

End to end: `prefill` = one prompt through EngineCore.run_prefill (chunks of 1024 rows), `decode` = token steps of
`batch` sequences that hold `context` tokens each (CUDA graph + sampler + state advance), both timed with CUDA events.
Kernels: each launched alone on the engine's buffers at the same shapes, L2 flushed between timed launches; the
memory-bound ones against the measured copy bandwidth, the sequential scans against the fp32 FMA rate of the SMs.
"""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

SIZES = {
    # width, layers, ff, heads, kv_heads, vocab
    "w1024": dict(width=1024, layers=8, ff=4096, heads=8, kv=2, vocab=32768),
    "w2048": dict(width=2048, layers=8, ff=8192, heads=16, kv=4, vocab=32768),
    "w4096": dict(width=4096, layers=8, ff=14336, heads=32, kv=8, vocab=32768),
}


def hybrid_config(s):
    """Alternating GLA / (attention + state-space) layers, every one with a feed-forward: the same width, depth, ff,
    attention heads (size 128) and vocabulary as the Qwen2 model it is compared with."""
    W = s["width"]
    gla = dict(type="gla", mixer=dict(heads=W // 256, dim=128, vdim=256, tau=16.0, rank=64),
               mlp=dict(kind="dense", ff=s["ff"], limit=7.0))
    par = dict(type="parallel",
               mixer=dict(left=dict(heads=s["heads"], kv_heads=s["kv"], dim=128, vdim=128, rot=dict(dims=64, base=1e6), scale=128 ** -0.5),
                          right=dict(heads=W // 64, vdim=64, state=128, groups=1, conv=4, norm_groups=1),
                          left_scale=1.0, right_scale=1.0),
               mlp=dict(kind="dense", ff=s["ff"], limit=7.0))
    return dict(architecture="Povurax", vocab=s["vocab"], width=W, norm=dict(eps=1e-5), embedding=dict(scale=1.0),
                layers=[gla if i % 2 == 0 else par for i in range(s["layers"])])


def peaks():
    try:
        p = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:  # noqa: BLE001
        return 6650.0, 1590.0, "fallback"


class Timer:
    def __init__(self):
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")

    def events(self, fn, iters=10, warm=3, flush=True):
        for _ in range(warm):
            fn()
        total = 0.0
        for _ in range(iters):
            if flush:
                self.flush.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            total += a.elapsed_time(b)
        return total / iters


def end_to_end(eng, vocab, prompt, context, batch, steps, warm):
    from pipelinerl_b200.engine import SamplingParams
    g = torch.Generator().manual_seed(1)
    rnd = lambda n: torch.randint(8, vocab - 8, (n,), generator=g).tolist()  # noqa: E731
    sp = SamplingParams(max_tokens=2, greedy=True, ignore_eos=True)

    def drain():
        while eng.slot_req:
            eng.step()
            eng.harvest()
    eng.add_request(rnd(1100), sp)                      # warm-up: buffers, kernel attributes
    eng.run_prefill()
    drain()
    ms = []
    for _ in range(2):
        eng.add_request(rnd(prompt), sp)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        eng.run_prefill()
        b.record()
        torch.cuda.synchronize()
        ms.append(a.elapsed_time(b))
        drain()
    prefill_ms = min(ms)
    spd = SamplingParams(max_tokens=warm + steps + 4, greedy=False, temperature=1.0, ignore_eos=True)
    for _ in range(batch):
        eng.add_request(rnd(context), spd)
    eng.run_prefill()
    for _ in range(warm):
        eng.step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        eng.step()
    b.record()
    torch.cuda.synchronize()
    step_ms = a.elapsed_time(b) / steps
    drain()
    return {"prefill_ms": round(prefill_ms, 2), "prefill_tokens_per_s": round((prompt - 1) / prefill_ms * 1e3),
            "decode_ms_per_step": round(step_ms, 3), "decode_tokens_per_s": round(batch / step_ms * 1e3)}


def kernel_table(eng, s, batch, chunk, timer):
    """The new kernels alone, at the decode shape (`batch` one-token segments) and the prefill shape (one segment of
    `chunk` rows), with the Qwen2 engine's closest row kernels on the same row counts."""
    import ctypes as C  # noqa: F401
    from pipelinerl_b200 import _lib
    from pipelinerl_b200.hybrid import _Rows
    lib, cfg = eng.lib, eng.cfg
    hbm, _, how = peaks()
    fma_tflops = 148 * 128 * 2 * 1.965e9 / 1e12          # fp32 FMA rate of the SMs at the maximum clock (nominal)
    W = cfg.width
    g = next(L.gla for L in cfg.layers if L.kind == "gla")
    par = next(L for L in cfg.layers if L.kind == "parallel")
    a, ss = par.attn, par.ssd
    gi = next(i for i, L in enumerate(cfg.layers) if L.kind == "gla")
    pi = next(i for i, L in enumerate(cfg.layers) if L.kind == "parallel")
    st = _lib.stream_ptr()
    out = {}
    i32 = dict(dtype=torch.int32, device=eng.dev)
    for shape, n, ns in (("decode", batch, batch), ("prefill", chunk, 1)):
        R = _Rows(eng, n, pieces=shape == "prefill")
        R.P.normal_(0, 0.5)
        R.aux.uniform_(0.9, 1.0)                           # decays (GLA) / convolved inputs (state-space)
        if shape == "decode":
            R.seg.copy_(torch.stack([torch.arange(n, **i32), torch.ones(n, **i32), torch.full((n,), 64, **i32), torch.arange(n, **i32)]))
            R.row_slot.copy_(torch.arange(n, **i32)); R.row_pos.fill_(64); R.row_back.zero_()
        else:
            R.seg[:, :1].copy_(torch.tensor([[0], [n], [0], [0]], **i32))
            R.row_slot.zero_(); R.row_pos.copy_(torch.arange(n, **i32)); R.row_back.copy_(torch.arange(n, **i32))
            step = eng.piece_tokens                            # the one segment as side-by-side pieces
            n_sub = (n + step - 1) // step
            R.sub[0, :n_sub].copy_(torch.arange(0, n, step, **i32))
            R.sub[1, :n_sub].copy_(torch.tensor([min(step, n - c) for c in range(0, n, step)], **i32))
            R.seg_sub[:, :1].copy_(torch.tensor([[0], [n_sub]], **i32))
            pieces = (R.seg_sub[0].data_ptr(), R.seg_sub[1].data_ptr(), R.sub[0].data_ptr(), R.sub[1].data_ptr(), n_sub,
                      R.scratch.data_ptr(), R.cdec.data_ptr())
        seg = [R.seg[k].data_ptr() for k in range(4)]
        vec = eng.vec
        nq, nv = g.heads * g.dim, g.heads * g.vdim
        ldg = 2 * nq + 2 * nv + g.rank
        w = f"l{cfg.layers[gi].weights_of}."

        def gla():
            _lib.check(lib.prl_gla_scan(R.P.data_ptr(), ldg, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                        g.vdim, seg[0], seg[1], seg[3], ns, eng.gla_state[gi].data_ptr(), R.o.data_ptr(), nv, st))
        ms = timer.events(gla)
        state_b = 2 * ns * g.heads * g.dim * g.vdim * 4
        io_b = n * (3 * nq + 2 * nv) * 4
        flops = 5.0 * n * g.heads * g.dim * g.vdim
        out[f"gla_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                        fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))
        if shape == "prefill":
            def gla_split():
                _lib.check(lib.prl_gla_scan_split(R.P.data_ptr(), ldg, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads,
                                                  g.dim, g.vdim, seg[3], ns, *pieces, eng.gla_state[gi].data_ptr(),
                                                  R.o.data_ptr(), nv, st))
            ms = timer.events(gla_split)
            out["gla_scan_split/prefill"] = dict(ms=round(ms, 4), hbm_frac=round((state_b * (1 + 2 * n_sub) + io_b) / ms / 1e6 / hbm, 3),
                                                 fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))
        wp = f"l{par.weights_of}."
        left = a.heads * a.dim + a.kv_heads * (a.dim + a.vdim) + a.heads * a.vdim
        ldp, inner, ch = left + ss.in_rows, ss.inner, ss.conv_channels

        def ssd():
            _lib.check(lib.prl_ssd_scan(R.P.data_ptr(), ldp, left + inner + ch, R.aux.data_ptr(), ch,
                                        vec[wp + "mix.right.dt_bias"].data_ptr(), vec[wp + "mix.right.A_log"].data_ptr(),
                                        vec[wp + "mix.right.D"].data_ptr(), ss.heads, ss.groups, ss.state, ss.vdim, seg[0], seg[1],
                                        seg[3], ns, eng.ssd_state[pi].data_ptr(), R.o2.data_ptr(), inner, st))
        ms = timer.events(ssd)
        state_b = 2 * ns * ss.heads * ss.state * ss.vdim * 4
        io_b = n * (2 * inner + 2 * ss.groups * ss.state) * 4
        flops = 5.0 * n * ss.heads * ss.state * ss.vdim
        out[f"ssd_scan/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round((state_b + io_b) / ms / 1e6 / hbm, 3),
                                        fp32_fma_frac=round(flops / ms / 1e9 / fma_tflops, 3))

        if shape == "prefill":
            def ssd_split():
                _lib.check(lib.prl_ssd_scan_split(R.P.data_ptr(), ldp, left + inner + ch, R.aux.data_ptr(), ch,
                                                  vec[wp + "mix.right.dt_bias"].data_ptr(), vec[wp + "mix.right.A_log"].data_ptr(),
                                                  vec[wp + "mix.right.D"].data_ptr(), ss.heads, ss.groups, ss.state, ss.vdim,
                                                  seg[3], ns, *pieces, eng.ssd_state[pi].data_ptr(), R.o2.data_ptr(), inner, st))
            ms = timer.events(ssd_split)
            out["ssd_scan_split/prefill"] = dict(ms=round(ms, 4), hbm_frac=round((state_b * (1 + 2 * n_sub) + io_b) / ms / 1e6 / hbm, 3),
                                                 fp32_fma_frac=round(1.4 * flops / ms / 1e9 / fma_tflops, 3))

        def conv():
            _lib.check(lib.prl_conv_silu(R.P.data_ptr(), ldp, left + inner, n, ch, ss.conv, vec[wp + "mix.right.conv"].data_ptr(),
                                         vec[wp + "mix.right.conv.b"].data_ptr(), R.row_slot.data_ptr(), R.row_back.data_ptr(),
                                         eng.conv_state[pi].data_ptr(), R.aux.data_ptr(), st))
        ms = timer.events(conv)
        out[f"conv_silu/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * ch * 8 / ms / 1e6 / hbm, 3))

        def post():
            _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, 1, R.y1.data_ptr(), W, 1.0, 1, vec[wp + "norm1"].data_ptr(),
                                                 cfg.eps, n, W, R.x.data_ptr(), R.xa.data_ptr(), 0, st))
        ms = timer.events(post)
        out[f"postnorm_residual/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (4 * 4 + 2) / ms / 1e6 / hbm, 3))

        def gate():
            _lib.check(lib.prl_gate_norm(R.o2.data_ptr(), 1, inner, R.P.data_ptr() + 4 * left, ldp, vec[wp + "mix.right.norm"].data_ptr(),
                                         inner, inner // ss.norm_groups, n, inner, 0, 1, 1, cfg.eps, R.yb.data_ptr(), 0, st))
        ms = timer.events(gate)
        out[f"gate_norm/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * inner * (4 + 4 + 2) / ms / 1e6 / hbm, 3))
        F = par.mlp.ff

        def glu():
            _lib.check(lib.prl_glu_clamped(R.P.data_ptr(), 2 * F, n, F, par.mlp.limit, par.mlp.beta, R.act.data_ptr(), 0, st))
        if 2 * F <= R.P.numel() // n:
            ms = timer.events(glu)
            out[f"glu_clamped/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (8 + 2) / ms / 1e6 / hbm, 3))
        # the Qwen2 engine's row kernels on the same rows (their bytes: fp32 partial in, fp32 residual in/out, bf16 out)
        h = torch.zeros(n, W, dtype=torch.float32, device=eng.dev)
        xb = torch.zeros(n, W, dtype=torch.bfloat16, device=eng.dev)
        gam = torch.ones(W, dtype=torch.bfloat16, device=eng.dev)
        part = torch.randn(n, 2 * F, dtype=torch.float32, device=eng.dev)
        actb = torch.zeros(n, F, dtype=torch.bfloat16, device=eng.dev)

        def qres():
            _lib.check(lib.prl_residual_rmsnorm(part.data_ptr(), 1, n, W, gam.data_ptr(), 1e-6, h.data_ptr(), xb.data_ptr(), None, 0, st))
        ms = timer.events(qres)
        out[f"qwen2.residual_rmsnorm/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * W * (3 * 4 + 2) / ms / 1e6 / hbm, 3))

        def qsilu():
            _lib.check(lib.prl_silu_mul(part.data_ptr(), 1, n, F, actb.data_ptr(), None, 0, st))
        ms = timer.events(qsilu)
        out[f"qwen2.silu_mul/{shape}"] = dict(ms=round(ms, 4), hbm_frac=round(n * F * (8 + 2) / ms / 1e6 / hbm, 3))
        del R
    out["_denominators"] = {"hbm_gbs": hbm, "hbm": how, "fp32_fma_tflops_nominal": round(fma_tflops, 1)}
    return out


def run(sizes, prompt, context, batch, steps, warm, kernels=True, e2e=True):
    from pipelinerl_b200.engine import DecodeEngine
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ModelConfig, ParamArena
    dev = torch.device("cuda:0")
    timer = Timer()
    res = {}
    for name in sizes:
        s = SIZES[name]
        kw = dict(max_batch=batch, max_seq_len=max(prompt, context) + 256, max_new_tokens=warm + steps + 8, device=dev,
                  prefill_chunk=1024)
        qcfg = ModelConfig(vocab_size=s["vocab"], hidden_size=s["width"], intermediate_size=s["ff"], num_layers=s["layers"],
                           num_q_heads=s["heads"], num_kv_heads=s["kv"])
        hcfg = HybridConfig.from_povurax(hybrid_config(s))
        entry = {}
        if e2e:
            eng = DecodeEngine(qcfg, ParamArena(qcfg, dev).init_random(seed=1), **kw)
            q = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            q["params_M"] = round(qcfg.num_params() / 1e6)
            del eng
            torch.cuda.empty_cache()
        eng = HybridEngine(hcfg, ParamArena(hcfg, dev).init_random(seed=1), **kw)
        if e2e:
            h = end_to_end(eng, s["vocab"], prompt, context, batch, steps, warm)
            h["params_M"] = round(hcfg.num_params() / 1e6)
            entry = {"qwen2": q, "hybrid": h,
                     "hybrid_over_qwen2": {"prefill": round(h["prefill_tokens_per_s"] / q["prefill_tokens_per_s"], 3),
                                           "decode": round(h["decode_tokens_per_s"] / q["decode_tokens_per_s"], 3)}}
        if kernels:
            entry["kernels"] = kernel_table(eng, s, batch, 1024, timer)
        res[name] = entry
        del eng
        torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sizes", default="w2048,w4096")
    ap.add_argument("--prompt", type=int, default=4096)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=32)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-kernels", action="store_true")
    ap.add_argument("--only-kernels", action="store_true", help="skip the end-to-end runs (a small case for a profiler)")
    a = ap.parse_args()
    from pipelinerl_b200 import _lib
    before = _lib.launch_count()
    res = run(a.sizes.split(","), a.prompt, a.context, a.batch, a.steps, a.warmup, kernels=not a.no_kernels, e2e=not a.only_kernels)
    print(json.dumps({"bench": "hybrid_vs_qwen2", "dtype": "bf16", "data": "synthetic", "prompt": a.prompt,
                      "context": a.context, "batch": a.batch, "steps": a.steps, "warmup": a.warmup,
                      "gpu_launches": _lib.launch_count() - before, "sizes": res}), flush=True)


if __name__ == "__main__":
    main()
