"""Oracle for the hybrid decoder family (pipelinerl_b200/hybrid.py): a plain, slow, whole-sequence implementation.

TEST INFRASTRUCTURE (see oracle/__init__.py).  Torch float64 on CPU, one function per mechanism, every recurrence
written as the explicit loop over time of its defining equation; no cache, no chunks, no batching, nothing shared
with the product path.  The reference has no model code of its own (it serves through vLLM, pipelinerl/launch.py:191-247),
so these functions restate the architecture's published equations and are the only yardstick for the CUDA kernels.

Notation: T tokens, h [T, W] the sublayer input, weights stored [out, in] and applied as h @ W.T.  `wt` maps a
checkpoint tensor name to a float64 tensor; `p` is the prefix of the mixer's tensors.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, n_rot: int, base: float) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i+1), i < n_rot/2, turn by the angle position * base^(-2i/n_rot)."""
    out = x.clone()
    for i in range(n_rot // 2):
        ang = positions.to(F64) * base ** (-2.0 * i / n_rot)
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - v * s
        out[..., 2 * i + 1] = v * c + u * s
    return out


def softmax_attention(h, wt, p, spec, eps):
    """Causal GQA attention with whole-projection q / k norms, partial interleaved rotary, a free scale, separate key
    and value sizes and a sigmoid output gate.  spec: heads, kv_heads, dim, vdim, rot_dims, rot_base, scale."""
    T = h.shape[0]
    H, G, d, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    q = rms_unit(h @ wt[p + "q"].T, eps) * wt[p + "q.norm"]          # norm over ALL heads' channels at once
    k = rms_unit(h @ wt[p + "k"].T, eps) * wt[p + "k.norm"]
    v = (h @ wt[p + "v"].T).view(T, G, dv)
    pos = torch.arange(T)
    q = rotate_pairs(q.view(T, H, d), pos, spec["rot_dims"], spec["rot_base"])
    k = rotate_pairs(k.view(T, G, d), pos, spec["rot_dims"], spec["rot_base"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        for head in range(H):
            g = head // (H // G)
            score = (k[:t + 1, g] @ q[t, head]) * spec["scale"]
            w = torch.softmax(score, dim=0)
            out[t, head] = w @ v[:t + 1, g]
    gate = torch.sigmoid(h @ wt[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ wt[p + "o"].T


def state_space(h, wt, p, spec, eps):
    """Mamba-2 form.  spec: heads, vdim, state, groups, conv, norm_groups."""
    T = h.shape[0]
    Hh, dv, N, G, taps, parts = spec["heads"], spec["vdim"], spec["state"], spec["groups"], spec["conv"], spec["norm_groups"]
    inner = Hh * dv
    proj = h @ wt[p + "in"].T
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt_raw = proj[:, 2 * inner + 2 * G * N:]
    # causal depthwise convolution, zeros before the sequence, the last tap on the current token
    C = xbc.shape[1]
    conv = torch.zeros(T, C, dtype=F64)
    for t in range(T):
        acc = wt[p + "conv.b"].clone()
        for j in range(taps):
            src = t - (taps - 1) + j
            if src >= 0:
                acc = acc + wt[p + "conv"][:, j] * xbc[src]
        conv[t] = silu(acc)
    x = conv[:, :inner].view(T, Hh, dv)
    Bm = conv[:, inner:inner + G * N].view(T, G, N)
    Cm = conv[:, inner + G * N:].view(T, G, N)
    dt = torch.nn.functional.softplus(dt_raw + wt[p + "dt_bias"])
    rate = torch.exp(wt[p + "A_log"])
    y = torch.zeros(T, Hh, dv, dtype=F64)
    for head in range(Hh):
        g = head // (Hh // G)
        S = torch.zeros(N, dv, dtype=F64)
        for t in range(T):
            S = math.exp(-rate[head].item() * dt[t, head].item()) * S + dt[t, head] * torch.outer(Bm[t, g], x[t, head])
            y[t, head] = S.T @ Cm[t, g] + wt[p + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)                                     # gate first ...
    y = rms_unit(y.view(T, parts, inner // parts), eps).reshape(T, inner)  # ... then the norm, part by part
    return (y * wt[p + "norm"]) @ wt[p + "o"].T


def gated_linear_attention(h, wt, p, spec, eps):
    """spec: heads, dim, vdim, tau.  Decay per key channel from a low-rank projection."""
    T = h.shape[0]
    H, d, dv, tau = spec["heads"], spec["dim"], spec["vdim"], spec["tau"]
    q = ((h @ wt[p + "q"].T) * d ** -0.5).view(T, H, d)
    k = (h @ wt[p + "k"].T).view(T, H, d)
    v = (h @ wt[p + "v"].T).view(T, H, dv)
    z = (h @ wt[p + "a1"].T) @ wt[p + "a2"].T + wt[p + "a2.b"]
    decay = torch.sigmoid(z).pow(1.0 / tau).view(T, H, d)
    o = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, head][:, None] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_unit(o, eps) * wt[p + "norm"]                                  # per head, one gain vector for all heads
    return (o.reshape(T, H * dv) * silu(h @ wt[p + "g"].T)) @ wt[p + "o"].T


def clamped_glu(h, wt, p, spec):
    lim = spec["limit"]
    g = torch.clamp(h @ wt[p + "gate"].T, max=lim)
    u = torch.clamp(h @ wt[p + "up"].T, min=-lim, max=lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ wt[p + "down"].T


def forward(config: dict, wt: dict, tokens, residuals: list | None = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence under a Povurax-style config dict; `residuals` collects the stream after
    every layer run."""
    wt = {k: v.to(F64) for k, v in wt.items()}
    eps = config["norm"]["eps"]
    x = wt["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        m = layer["mixer"]
        if layer["type"] == "gla":
            mixed = gated_linear_attention(x, wt, p + "mix.", m, eps)
        elif layer["type"] == "parallel":
            left = dict(m["left"], rot_dims=m["left"]["rot"]["dims"], rot_base=m["left"]["rot"]["base"])
            mixed = m["left_scale"] * softmax_attention(x, wt, p + "mix.left.", left, eps) \
                + m["right_scale"] * state_space(x, wt, p + "mix.right.", m["right"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_unit(mixed, eps) * wt[p + "norm1"]
        if layer.get("mlp") is not None:
            x = x + rms_unit(clamped_glu(x, wt, p + "mlp.", layer["mlp"]), eps) * wt[p + "norm2"]
        if residuals is not None:
            residuals.append(x.clone())
    return (rms_unit(x, eps) * wt["final.norm"]) @ wt["head"].T


def random_weights(config: dict, seed: int = 0, dtype=torch.bfloat16) -> dict:
    """Checkpoint-named random tensors for a config dict (values exactly representable in `dtype`)."""
    g = torch.Generator().manual_seed(seed)
    W = config["width"]

    def mat(rows, cols, std=None):
        std = cols ** -0.5 if std is None else std
        return (torch.randn(rows, cols, generator=g) * std).to(dtype).float()

    def vec(n, mean=0.0, std=0.1):
        return (mean + torch.randn(n, generator=g) * std).to(dtype).float()
    wt = {"embed": mat(config["vocab"], W, 0.5), "final.norm": vec(W, 1.0), "head": mat(config["vocab"], W)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        wt[p + "norm1"] = vec(W, 1.0)
        if layer["type"] == "gla":
            nq, nv, r = m["heads"] * m["dim"], m["heads"] * m["vdim"], m["rank"]
            wt.update({p + "mix.q": mat(nq, W), p + "mix.k": mat(nq, W), p + "mix.v": mat(nv, W), p + "mix.g": mat(nv, W),
                       p + "mix.o": mat(W, nv), p + "mix.norm": vec(m["vdim"], 1.0), p + "mix.a1": mat(r, W),
                       p + "mix.a2": mat(nq, r), p + "mix.a2.b": vec(nq, 2.0, 1.0)})
        else:
            a, s = m["left"], m["right"]
            nq, nk, nv = a["heads"] * a["dim"], a["kv_heads"] * a["dim"], a["kv_heads"] * a["vdim"]
            ng = a["heads"] * a["vdim"]
            inner = s["heads"] * s["vdim"]
            ch = inner + 2 * s["groups"] * s["state"]
            q = p + "mix.left."
            wt.update({q + "q": mat(nq, W), q + "k": mat(nk, W), q + "v": mat(nv, W), q + "g": mat(ng, W),
                       q + "o": mat(W, ng), q + "q.norm": vec(nq, 1.0), q + "k.norm": vec(nk, 1.0)})
            r = p + "mix.right."
            wt.update({r + "in": mat(2 * inner + 2 * s["groups"] * s["state"] + s["heads"], W),
                       r + "conv": mat(ch, s["conv"], 0.5), r + "conv.b": vec(ch), r + "dt_bias": vec(s["heads"], 0.0, 0.5),
                       r + "A_log": vec(s["heads"], 0.0, 0.5), r + "D": vec(s["heads"], 1.0, 0.3),
                       r + "norm": vec(inner, 1.0), r + "o": mat(W, inner)})
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            wt.update({p + "mlp.gate": mat(F, W), p + "mlp.up": mat(F, W), p + "mlp.down": mat(W, F), p + "norm2": vec(W, 1.0)})
    return wt
