"""Small Belelorn configurations and helpers for the tests (random weights, sizes chosen to be awkward)."""
import copy
import json
import struct

import torch

from oracle import belelorn_oracle as bo


def attn(heads=4, kv_heads=2, dim=12, scale=0.5, softcap=20.0, size=24, keep_first=3):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, softcap=softcap,
                mask=dict(size=size, keep_first=keep_first))


def lightning(heads=3, dim=10, vdim=14, decay=None):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=decay or [0.5 + 0.49 * (h + 1) / heads for h in range(heads)])


def par_layer(left=None, right=None, mlp=None):
    return dict(type="parallel", mixer=dict(left=left or attn(), right=right or lightning()), mlp=mlp)


def mlstm_layer(heads=3, dim=9, vdim=20, gate_cap=12.0, mlp=None):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=gate_cap), mlp=mlp)


def dense(ff=56):
    return dict(kind="dense", ff=ff)


def moe(experts=5, top=2, ff=24, limit=1.5, shared_ff=40, shared_limit=1.25):
    out = dict(kind="moe", router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=limit))
    if shared_ff:
        out["shared"] = dict(ff=shared_ff, limit=shared_limit)
    return out


def model(layers, vocab=96, width=72, eps=1e-5, loop=None, logit_scale=1.5):
    cfg = dict(architecture="Belelorn", vocab=vocab, width=width, norm=dict(eps=eps), logit_scale=logit_scale,
               layers=copy.deepcopy(layers))
    if loop is not None:
        cfg["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return cfg


def build_engine(config, wt, dtype, device, **kw):
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ParamArena
    cfg = HybridConfig.from_belelorn(config)
    arena = ParamArena(cfg, device, dtype=dtype)
    arena.load_hf_state_dict(wt)
    args = dict(max_batch=4, max_seq_len=512, max_new_tokens=32, prefill_chunk=256, use_cuda_graph=False, device=device)
    args.update(kw)
    return HybridEngine(cfg, arena, **args)


def stream_logits(eng, tokens, portions):
    """Feed `tokens` through one stream in the given portion sizes (the rest one by one); logits of every position."""
    s = eng.open_stream()
    out, at = [], 0
    sizes = list(portions)
    while at < len(tokens):
        k = sizes.pop(0) if sizes else 1
        k = min(k, len(tokens) - at)
        out.append(eng.feed([(s, tokens[at:at + k], list(range(k)))]))
        at += k
    eng.close_stream(s)
    return torch.cat(out).double().cpu()


def rel_err(got, ref):
    """Worst position: rms over the vocabulary of the difference (mean removed) over the rms of the reference."""
    d = got.double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    r = ref.double() - ref.double().mean(-1, keepdim=True)
    return (d.pow(2).mean(-1).sqrt() / r.pow(2).mean().sqrt()).max().item()


def tokens_for(config, n, seed=1):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, config["vocab"], (n,), generator=g).tolist()


def oracle_logits(config, wt, tokens):
    return bo.forward(config, wt, tokens)


def write_checkpoint(folder, config, wt):
    (folder / "config.json").write_text(json.dumps(config))
    header, blobs, at = {}, [], 0
    for name, t in wt.items():
        raw = t.to(torch.bfloat16).contiguous().view(torch.int16).numpy().tobytes()
        header[name] = dict(dtype="BF16", shape=list(t.shape), data_offsets=[at, at + len(raw)])
        blobs.append(raw)
        at += len(raw)
    hj = json.dumps(header).encode()
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(hj)))
        f.write(hj)
        for b in blobs:
            f.write(b)
