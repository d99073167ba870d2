"""Small configurations and helpers for the hybrid-decoder tests (random weights, sizes chosen to be awkward)."""
import copy
import json
import struct

import torch

from oracle import hybrid_oracle as ho


def gla_layer(heads=3, dim=10, vdim=24, tau=5.0, rank=5, mlp=None, **kw):
    return dict(type="gla", mixer=dict(heads=heads, dim=dim, vdim=vdim, tau=tau, rank=rank), mlp=mlp, **kw)


def par_layer(heads=4, kv_heads=2, dim=24, vdim=40, rot=8, base=100.0, scale=0.3, left_scale=0.7, right_scale=1.3,
              s_heads=4, s_vdim=12, state=12, groups=2, conv=3, norm_groups=2, mlp=None, **kw):
    return dict(type="parallel",
                mixer=dict(left=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, rot=dict(dims=rot, base=base), scale=scale),
                           right=dict(heads=s_heads, vdim=s_vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups),
                           left_scale=left_scale, right_scale=right_scale),
                mlp=mlp, **kw)


def dense(ff=56, limit=1.25):
    return dict(kind="dense", ff=ff, limit=limit)


def model(layers, vocab=96, width=72, eps=1e-5, embed_scale=3.0):
    return dict(architecture="Povurax", vocab=vocab, width=width, norm=dict(eps=eps), embedding=dict(scale=embed_scale),
                layers=copy.deepcopy(layers))


def shared(layer, j):
    """A layer entry that runs with layer j's tensors (its own cache / state)."""
    out = copy.deepcopy(layer)
    out["weights_of"] = j
    return out


def build_engine(config, wt, dtype, device, **kw):
    from pipelinerl_b200.hybrid import HybridConfig, HybridEngine
    from pipelinerl_b200.model import ParamArena
    cfg = HybridConfig.from_povurax(config)
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
    return ho.forward(config, wt, tokens)


def write_checkpoint(folder, config, wt):
    """config.json (without the test-only `rank` key: the loader reads it off the tensor shape) + model.safetensors."""
    cfg = copy.deepcopy(config)
    for layer in cfg["layers"]:
        layer["mixer"].pop("rank", None)
    (folder / "config.json").write_text(json.dumps(cfg))
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
