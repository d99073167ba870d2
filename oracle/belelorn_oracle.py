"""Oracle for the "Belelorn" decoders (pipelinerl_b200/hybrid.py, `HybridConfig.from_belelorn`): a plain, slow,
whole-sequence implementation.

TEST INFRASTRUCTURE (see oracle/__init__.py).  Torch float64 on CPU, one function per mechanism, every recurrence an
explicit loop over time, no cache, no chunks, no batching, nothing shared with the product path.  The reference has no
model code of its own (it serves through vLLM, pipelinerl/launch.py:191-247), so these functions restate the design's
equations and are the yardstick for the CUDA kernels.

Notation: T tokens, W the model width, h [T, W] a sublayer's input, weights stored [out, in] and applied as h @ M.T.
`wt` maps a checkpoint tensor name to a float64 tensor, `p` is the prefix of a sublayer's tensors, `cfg` the dict of
config.json.  `round_in`, when given, is applied to both operands of every matrix product (tests use it to measure the
least error a bf16 product can have).
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def _mm(a, w, round_in=None):
    if round_in is not None:
        a, w = round_in(a), round_in(w)
    return a @ w.T


def rms_unit(x, eps):
    """x over its root mean square along the last axis (eps under the root)."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def norm_zero_centred(x, w, eps):
    """RMS norm whose stored weight is an offset from one."""
    return rms_unit(x, eps) * (1.0 + w)


def silu(x):
    return x * torch.sigmoid(x)


def sinusoid_positions(T, W):
    """[T, W]: channel 2i carries sin(p * 10000^(-2i/W)), channel 2i+1 the cosine of the same angle."""
    out = torch.zeros(T, W, dtype=F64)
    for c in range(W):
        i = c // 2
        ang = torch.arange(T, dtype=F64) * 10000.0 ** (-2.0 * i / W)
        out[:, c] = torch.sin(ang) if c % 2 == 0 else torch.cos(ang)
    return out


def embed(tokens, wt):
    W = wt["embed"].shape[1]
    return wt["embed"][torch.tensor(tokens)] + sinusoid_positions(len(tokens), W)


# ---- mixers ---------------------------------------------------------------------------------------------------------
def mlstm(h, wt, p, m, eps, round_in=None):
    """Matrix-memory LSTM cell with exponential gating and a running stabiliser that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (_mm(h, wt[p + "q"], round_in) * d ** -0.5).view(T, H, d)
    k = _mm(h, wt[p + "k"], round_in).view(T, H, d)
    v = _mm(h, wt[p + "v"], round_in).view(T, H, dv)
    gi = cap * torch.tanh((_mm(h, wt[p + "i"], round_in) + wt[p + "i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((_mm(h, wt[p + "f"], round_in) + wt[p + "f.b"]) / cap))
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        n = torch.zeros(d, dtype=F64)
        run = 0.0
        for t in range(T):
            new = max(float(gf[t, head]) + run, float(gi[t, head]))
            keep, take = math.exp(float(gf[t, head]) + run - new), math.exp(float(gi[t, head]) - new)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            run = new
            den = max(abs(float(n @ q[t, head])), math.exp(-run)) + 1e-6
            out[t, head] = (S.T @ q[t, head]) / den
    y = rms_unit(out, eps).reshape(T, H * dv) * wt[p + "norm"]
    y = y * torch.sigmoid(_mm(h, wt[p + "g"], round_in))
    return _mm(y, wt[p + "o"], round_in)


def windowed_attention(h, wt, p, a, eps, round_in=None):
    """Softmax attention whose values are its (un-normed) keys: unit-RMS q and k per head, tanh-capped scores, a
    sliding window that also keeps the first tokens of the sequence; positions do not enter the scores."""
    T = h.shape[0]
    H, G, d = a["heads"], a["kv_heads"], a["dim"]
    win, first = a["mask"]["size"], a["mask"]["keep_first"]
    q = (_mm(h, wt[p + "q"], round_in) + wt[p + "q.b"]).view(T, H, d)
    kv = (_mm(h, wt[p + "k"], round_in) + wt[p + "k.b"]).view(T, G, d)
    qn, kn = rms_unit(q, eps), rms_unit(kv, eps)
    out = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        seen = torch.tensor([j for j in range(t + 1) if t - j < win or j < first])
        for head in range(H):
            g = head // (H // G)
            s = (kn[seen, g] @ qn[t, head]) * a["scale"]
            if a.get("softcap"):
                s = a["softcap"] * torch.tanh(s / a["softcap"])
            out[t, head] = torch.softmax(s, dim=0) @ kv[seen, g]
    return _mm(out.reshape(T, H * d), wt[p + "o"], round_in)


def lightning_attention(h, wt, p, r, eps, round_in=None):
    """Linear attention with one fixed decay per head: S <- decay S + k v^T, o = S^T q, SiLU on q, k and v."""
    T = h.shape[0]
    H, d, dv = r["heads"], r["dim"], r["vdim"]
    q = silu(_mm(h, wt[p + "q"], round_in)).view(T, H, d)
    k = silu(_mm(h, wt[p + "k"], round_in)).view(T, H, d)
    v = silu(_mm(h, wt[p + "v"], round_in)).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = float(r["decay"][head]) * S + torch.outer(k[t, head], v[t, head])
            out[t, head] = S.T @ q[t, head]
    y = rms_unit(out.reshape(T, H * dv), eps) * wt[p + "norm"]
    y = y * torch.sigmoid(_mm(h, wt[p + "g"], round_in))
    return _mm(y, wt[p + "o"], round_in)


def parallel_mixer(h, wt, p, m, eps, round_in=None):
    left = windowed_attention(h, wt, p + "left.", m["left"], eps, round_in)
    right = lightning_attention(h, wt, p + "right.", m["right"], eps, round_in)
    return 0.5 * (rms_unit(left, eps) * wt[p + "left.out"] + rms_unit(right, eps) * wt[p + "right.out"])


# ---- feed-forward ---------------------------------------------------------------------------------------------------
def relu2_ff(h, wt, p, round_in=None):
    return _mm(torch.relu(_mm(h, wt[p + "up"], round_in)) ** 2, wt[p + "down"], round_in)


def clamped_expert(h, wt, p, limit, round_in=None):
    g = torch.clamp(_mm(h, wt[p + "gate"], round_in), max=limit)
    u = torch.clamp(_mm(h, wt[p + "up"], round_in), -limit, limit)
    return _mm(g * torch.sigmoid(1.702 * g) * (u + 1.0), wt[p + "down"], round_in)


def routed_ff(h, wt, p, mlp, round_in=None, margins=None):
    """Sigmoid router; each token's `top` best experts get the token SCALED by their score (scores not renormalised);
    a shared expert sees every token unscaled.  `margins` (a list) receives, per token, the gap between the router
    logits of the last expert taken and the first one left out."""
    T, W = h.shape
    logit = _mm(h, wt[p + "router"], round_in)
    score = torch.sigmoid(logit)
    out = torch.zeros(T, W, dtype=F64)
    n_exp, top = mlp["router"]["experts"], mlp["router"]["top"]
    for t in range(T):
        order = sorted(range(n_exp), key=lambda e: -float(score[t, e]))
        if margins is not None:
            margins.append(float(logit[t, order[top - 1]] - logit[t, order[top]]) if top < n_exp else math.inf)
        for e in order[:mlp["router"]["top"]]:
            out[t] += clamped_expert((score[t, e] * h[t])[None], wt, f"{p}e{e}.", mlp["expert"]["limit"], round_in)[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, wt, p + "shared.", mlp["shared"]["limit"], round_in)
    return out


# ---- the model --------------------------------------------------------------------------------------------------------
def layer_runs(cfg):
    """[(layer index, pass number or None)]: pass number t on the run that opens pass t of the repeated block."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, wt, tokens, residuals=None, round_in=None, margins=None):
    """Logits [T, vocab] of a whole sequence; `residuals` collects the stream after every layer run, `margins` the
    router margins of every routed feed-forward run (one list of T gaps per run)."""
    eps = cfg["norm"]["eps"]
    x0 = embed(tokens, wt)
    x = x0
    for i, opens in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if opens is not None:
            x = _mm(torch.cat([x, x0], dim=1), wt["loop.in"], round_in) + wt["loop.step"][opens]
        hin = norm_zero_centred(x, wt[p + "norm1"], eps)
        if L["type"] == "mlstm":
            y = mlstm(hin, wt, p + "mix.", L["mixer"], eps, round_in)
        elif L["type"] == "parallel":
            y = parallel_mixer(hin, wt, p + "mix.", L["mixer"], eps, round_in)
        else:
            raise ValueError(L["type"])
        x = x + norm_zero_centred(y, wt[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            hin = norm_zero_centred(x, wt[p + "norm2"], eps)
            if L["mlp"]["kind"] == "dense":
                y = relu2_ff(hin, wt, p + "mlp.", round_in)
            else:
                gaps = [] if margins is not None else None
                y = routed_ff(hin, wt, p + "mlp.", L["mlp"], round_in, gaps)
                if margins is not None:
                    margins.append(gaps)
            x = x + norm_zero_centred(y, wt[p + "norm2b"], eps)
        if residuals is not None:
            residuals.append(x.clone())
    return _mm(norm_zero_centred(x, wt["final.norm"], eps), wt["head"], round_in) * cfg["logit_scale"]


def tensor_shapes(cfg):
    """Checkpoint tensor names and shapes of a config."""
    W, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    if cfg.get("loop"):
        out["loop.in"] = (W, 2 * W)
        out["loop.step"] = (cfg["loop"]["times"], W)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for nm in ("norm1", "norm1b"):
            out[p + nm] = (W,)
        if L["type"] == "mlstm":
            nq, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            out.update({p + "mix.q": (nq, W), p + "mix.k": (nq, W), p + "mix.v": (nv, W), p + "mix.g": (nv, W),
                        p + "mix.o": (W, nv), p + "mix.norm": (nv,), p + "mix.i": (m["heads"], W),
                        p + "mix.i.b": (m["heads"],), p + "mix.f": (m["heads"], W), p + "mix.f.b": (m["heads"],)})
        else:
            a, r = m["left"], m["right"]
            nq, nk = a["heads"] * a["dim"], a["kv_heads"] * a["dim"]
            rq, rv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            out.update({p + "mix.left.q": (nq, W), p + "mix.left.q.b": (nq,), p + "mix.left.k": (nk, W),
                        p + "mix.left.k.b": (nk,), p + "mix.left.o": (W, nq), p + "mix.right.q": (rq, W),
                        p + "mix.right.k": (rq, W), p + "mix.right.v": (rv, W), p + "mix.right.g": (rv, W),
                        p + "mix.right.o": (W, rv), p + "mix.right.norm": (rv,), p + "mix.left.out": (W,),
                        p + "mix.right.out": (W,)})
        mlp = L.get("mlp")
        if mlp is None:
            continue
        for nm in ("norm2", "norm2b"):
            out[p + nm] = (W,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            F = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared") is not None:
                Fs = mlp["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (Fs, W), p + "mlp.shared.up": (Fs, W), p + "mlp.shared.down": (W, Fs)})
    return out


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Random tensors, rounded to `dtype` so that the engine and the oracle see the same numbers.  Matrices have unit
    row gain (std 1/sqrt(fan_in)), gains are spread around their neutral value, gate biases favour remembering."""
    g = torch.Generator().manual_seed(seed)
    wt = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if name == "embed":
            t = torch.randn(shape, generator=g)
        elif leaf in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            t = torch.randn(shape, generator=g) * 0.2                       # offsets from one
        elif leaf in ("norm", "out"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif name.endswith("f.b"):
            t = 2.0 + torch.randn(shape, generator=g)
        elif leaf == "b":
            t = torch.randn(shape, generator=g) * 0.5
        elif name == "loop.step":
            t = torch.randn(shape, generator=g) * 0.3
        elif leaf == "router":
            t = torch.randn(shape, generator=g) * 4.0 / math.sqrt(shape[-1])   # well separated scores
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[-1])
        wt[name] = t.to(dtype).to(F64)
    return wt
