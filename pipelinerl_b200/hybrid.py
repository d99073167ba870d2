"""Hybrid decoders on the sampler engine: layers whose mixer is gated linear attention, or softmax attention running
in parallel with a state-space (Mamba-2 form) mixer, each sublayer normalised on its OUTPUT (x += norm(f(x))), with a
clamped gated feed-forward.  The reference serves any architecture its vLLM serves (pipelinerl/launch.py:191-247,
conf/base.yaml:59-73); this module is how such a family runs on `engine.EngineCore`: the core's slots, page pool,
scheduler, sampler and CUDA graph are shared with the Qwen2 engine, and this file adds only the layer program.

`HybridConfig` is a list of layer specs; every size and constant is a field, nothing is fixed to one model.  The
"Povurax" architecture is one parser of that config (`HybridConfig.from_povurax`): another design built from the same
mixers needs a parser, not new kernels.

Numerics: the residual stream, every norm, softmax, router-like gate, decay, step size and recurrent state are fp32.
GEMM operands and the KV cache are bf16, or fp32 when the arena is fp32 (the true-fp32 mode: CUDA-core GEMMs with fp32
accumulation in a fixed order, no TF32).  One code path serves prompt chunks, single decoded tokens and mixtures of
both ("ragged rows"); a token's result depends only on its own sequence.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib
from .cache import PAGE_SIZE
from .engine import EngineCore


@dataclass(frozen=True)
class AttnSpec:
    heads: int
    kv_heads: int
    dim: int            # query / key size per head
    vdim: int           # value size per head
    rot_dims: int       # leading channels of each head that are rotated (interleaved pairs)
    rot_base: float
    scale: float        # score = (q . k) * scale


@dataclass(frozen=True)
class SsdSpec:
    heads: int
    vdim: int
    state: int          # N
    groups: int         # B / C groups
    conv: int           # taps of the causal convolution over x, B, C
    norm_groups: int    # the gated output is RMS-normed in this many equal parts

    @property
    def inner(self) -> int:
        return self.heads * self.vdim

    @property
    def conv_channels(self) -> int:
        return self.inner + 2 * self.groups * self.state

    @property
    def in_rows(self) -> int:   # [z | x | B | C | dt]
        return 2 * self.inner + 2 * self.groups * self.state + self.heads


@dataclass(frozen=True)
class GlaSpec:
    heads: int
    dim: int
    vdim: int
    tau: float          # decay = sigmoid(z)^(1/tau)
    rank: int           # bottleneck of the decay projection


@dataclass(frozen=True)
class MlpSpec:
    ff: int
    limit: float
    beta: float = 1.702  # g * sigmoid(beta * g)


@dataclass(frozen=True)
class LayerSpec:
    kind: str                       # "gla" | "parallel"
    weights_of: int                 # index of the layer whose tensors this layer uses (its own index if it has its own)
    gla: GlaSpec | None = None
    attn: AttnSpec | None = None
    ssd: SsdSpec | None = None
    left_scale: float = 1.0
    right_scale: float = 1.0
    mlp: MlpSpec | None = None


@dataclass(frozen=True)
class HybridConfig:
    vocab_size: int
    width: int
    eps: float
    embed_scale: float
    layers: tuple

    @property
    def head_rows(self) -> int:
        return self.vocab_size

    @property
    def hidden_size(self) -> int:
        return self.width

    # ---- the "Povurax" reading of config.json ---------------------------------------------------------------------
    @staticmethod
    def from_povurax(d: dict, tensor_shapes: dict | None = None) -> "HybridConfig":
        """config.json of a Povurax checkpoint.  The rank of a GLA layer's decay bottleneck is not a config key: it is
        the row count of the layer's `mix.a1` tensor (tensor_shapes), or `mixer.rank` when building without a file."""
        layers = []
        n_layers = len(d["layers"])

        def owner(i: int) -> int:
            """The layer whose tensors layer i runs with: follow `weights_of` to a layer that has its own."""
            seen = set()
            while "weights_of" in d["layers"][i] and int(d["layers"][i]["weights_of"]) != i:
                if i in seen:
                    raise ValueError(f"layer {i}: weights_of runs in a circle")
                seen.add(i)
                i = int(d["layers"][i]["weights_of"])
                if not 0 <= i < n_layers:
                    raise ValueError(f"weights_of names layer {i}, which does not exist")
            return i
        for i, L in enumerate(d["layers"]):
            j = owner(i)
            if L["type"] != d["layers"][j]["type"]:
                raise ValueError(f"layer {i} ({L['type']}) cannot run with the tensors of layer {j} ({d['layers'][j]['type']})")
            m = L["mixer"]
            mlp = None
            if L.get("mlp") is not None:
                if L["mlp"].get("kind", "dense") != "dense":
                    raise ValueError(f"layer {i}: unknown feed-forward kind {L['mlp'].get('kind')!r}")
                mlp = MlpSpec(ff=int(L["mlp"]["ff"]), limit=float(L["mlp"]["limit"]))
            if L["type"] == "gla":
                rank = m.get("rank")
                if rank is None and tensor_shapes is not None:
                    rank = tensor_shapes[f"l{j}.mix.a1"][0]
                if rank is None:
                    raise ValueError(f"layer {i}: the decay rank is neither in the config nor in a tensor shape")
                layers.append(LayerSpec("gla", j, gla=GlaSpec(int(m["heads"]), int(m["dim"]), int(m["vdim"]),
                                                              float(m["tau"]), int(rank)), mlp=mlp))
            elif L["type"] == "parallel":
                a, s = m["left"], m["right"]
                rot = a.get("rot") or {}                       # no rotary block: no dimension is rotated
                attn = AttnSpec(int(a["heads"]), int(a.get("kv_heads", a["heads"])), int(a["dim"]), int(a.get("vdim", a["dim"])),
                                int(rot.get("dims", 0)), float(rot.get("base", 10000.0)), float(a["scale"]))
                ssd = SsdSpec(int(s["heads"]), int(s["vdim"]), int(s["state"]), int(s["groups"]), int(s["conv"]),
                              int(s["norm_groups"]))
                layers.append(LayerSpec("parallel", j, attn=attn, ssd=ssd, left_scale=float(m["left_scale"]),
                                        right_scale=float(m["right_scale"]), mlp=mlp))
            else:
                raise ValueError(f"layer {i}: unknown mixer type {L['type']!r}")
        cfg = HybridConfig(int(d["vocab"]), int(d["width"]), float(d["norm"]["eps"]), float(d["embedding"]["scale"]),
                           tuple(layers))
        cfg.validate()
        return cfg

    def validate(self) -> None:
        for i, L in enumerate(self.layers):
            if L.kind == "parallel":
                a, s = L.attn, L.ssd
                if a.heads % a.kv_heads or a.rot_dims % 2 or a.rot_dims > a.dim:
                    raise ValueError(f"layer {i}: bad attention geometry {a}")
                if s.heads % s.groups or s.inner % s.norm_groups or s.conv < 1 or s.conv > 16:
                    raise ValueError(f"layer {i}: bad state-space geometry {s}")
                if a.dim > 512 or a.vdim > 256 or s.state > 256:
                    raise ValueError(f"layer {i}: head size beyond what the kernels are built for")
            elif L.gla.dim > 256:
                raise ValueError(f"layer {i}: key size beyond what the scan kernel is built for")

    # ---- the parameter arena: fused tensors in kernel order ---------------------------------------------------------
    def _own(self):
        return [(i, L) for i, L in enumerate(self.layers) if L.weights_of == i]

    def fused_shapes(self) -> list[tuple[str, tuple[int, ...]]]:
        W, out = self.width, []
        for i, L in self._own():
            p = f"l{i}."
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                out += [(p + "mix.in", (2 * nq + 2 * nv + g.rank, W)), (p + "mix.a2", (nq, g.rank)),
                        (p + "mix.a2.b", (nq,)), (p + "mix.norm", (g.vdim,)), (p + "mix.o", (W, nv))]
            else:
                a, s = L.attn, L.ssd
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                ng = a.heads * a.vdim
                out += [(p + "mix.in", (nq + nk + nv + ng + s.in_rows, W)), (p + "mix.left.q.norm", (nq,)),
                        (p + "mix.left.k.norm", (nk,)), (p + "mix.left.o", (W, ng)),
                        (p + "mix.right.conv", (s.conv_channels, s.conv)), (p + "mix.right.conv.b", (s.conv_channels,)),
                        (p + "mix.right.dt_bias", (s.heads,)), (p + "mix.right.A_log", (s.heads,)),
                        (p + "mix.right.D", (s.heads,)), (p + "mix.right.norm", (s.inner,)),
                        (p + "mix.right.o", (W, s.inner))]
            out.append((p + "norm1", (W,)))
            if L.mlp is not None:
                out += [(p + "mlp.gate_up", (2 * L.mlp.ff, W)), (p + "mlp.down", (W, L.mlp.ff)), (p + "norm2", (W,))]
        out += [("embed", (self.vocab_size, W)), ("final.norm", (W,)), ("head", (self.vocab_size, W))]
        return out

    def checkpoint_slices(self) -> dict[str, tuple[str, int, int]]:
        """checkpoint tensor name -> (fused tensor, first row, rows)."""
        m: dict[str, tuple[str, int, int]] = {}

        def rows(fused, parts):
            at = 0
            for name, n in parts:
                m[name] = (fused, at, n)
                at += n
        for i, L in self._own():
            p = f"l{i}."
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                rows(p + "mix.in", [(p + "mix.q", nq), (p + "mix.k", nq), (p + "mix.v", nv), (p + "mix.g", nv),
                                    (p + "mix.a1", g.rank)])
                for name, n in (("mix.a2", nq), ("mix.a2.b", nq), ("mix.norm", g.vdim), ("mix.o", self.width)):
                    m[p + name] = (p + name, 0, n)
            else:
                a, s = L.attn, L.ssd
                nq, nk, nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
                rows(p + "mix.in", [(p + "mix.left.q", nq), (p + "mix.left.k", nk), (p + "mix.left.v", nv),
                                    (p + "mix.left.g", a.heads * a.vdim), (p + "mix.right.in", s.in_rows)])
                for name, n in (("mix.left.q.norm", nq), ("mix.left.k.norm", nk), ("mix.left.o", self.width),
                                ("mix.right.conv", s.conv_channels), ("mix.right.conv.b", s.conv_channels),
                                ("mix.right.dt_bias", s.heads), ("mix.right.A_log", s.heads), ("mix.right.D", s.heads),
                                ("mix.right.norm", s.inner), ("mix.right.o", self.width)):
                    m[p + name] = (p + name, 0, n)
            m[p + "norm1"] = (p + "norm1", 0, self.width)
            if L.mlp is not None:
                rows(p + "mlp.gate_up", [(p + "mlp.gate", L.mlp.ff), (p + "mlp.up", L.mlp.ff)])
                m[p + "mlp.down"] = (p + "mlp.down", 0, self.width)
                m[p + "norm2"] = (p + "norm2", 0, self.width)
        m["embed"] = ("embed", 0, self.vocab_size)
        m["final.norm"] = ("final.norm", 0, self.width)
        m["head"] = ("head", 0, self.vocab_size)
        return m

    def init_param(self, name: str, view: torch.Tensor, gen: torch.Generator) -> None:
        """Random initialisation for benches and tests: unit gains, small biases, weights of std 1/sqrt(fan_in)."""
        leaf = name.split(".")[-1]
        if leaf in ("norm", "norm1", "norm2") or name == "final.norm":
            view.fill_(1.0)
        elif leaf == "A_log":
            view.copy_(torch.log(torch.linspace(1.0, 4.0, view.numel())).to(view.dtype))
        elif leaf in ("D",):
            view.fill_(1.0)
        elif leaf in ("b", "dt_bias"):
            view.copy_((torch.randn(view.shape, generator=gen, device=view.device) * 0.1).to(view.dtype))
        else:
            fan_in = view.shape[-1] if view.dim() > 1 else 1
            std = 0.02 if name == "embed" else 1.0 / math.sqrt(fan_in)
            flat = view.view(-1)
            step = 1 << 26
            for s in range(0, flat.numel(), step):
                n = min(step, flat.numel() - s)
                flat[s:s + n] = (torch.randn(n, generator=gen, device=view.device, dtype=torch.float32) * std).to(view.dtype)

    def num_params(self) -> int:
        n = 0
        for _, shape in self.fused_shapes():
            k = 1
            for s in shape:
                k *= s
            n += k
        return n


class _Rows:
    """Activation buffers and ragged-row metadata for up to `n` rows."""

    def __init__(self, eng: "HybridEngine", n: int, pieces: bool = False):
        cfg, d, T = eng.cfg, eng.dev, eng.op_dtype
        W = cfg.width
        wide_p, wide_aux, wide_o, wide_o2, wide_q, wide_f = W, 1, 1, 1, 1, 1
        for L in cfg.layers:
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                wide_p = max(wide_p, 2 * nq + 2 * nv + g.rank)
                wide_aux, wide_o = max(wide_aux, nq), max(wide_o, nv)
            else:
                a, s = L.attn, L.ssd
                nq = a.heads * a.dim
                wide_p = max(wide_p, nq + a.kv_heads * (a.dim + a.vdim) + a.heads * a.vdim + s.in_rows)
                wide_aux, wide_o = max(wide_aux, s.conv_channels), max(wide_o, a.heads * a.vdim)
                wide_o2, wide_q = max(wide_o2, s.inner), max(wide_q, nq)
            if L.mlp is not None:
                wide_p, wide_f = max(wide_p, 2 * L.mlp.ff), max(wide_f, L.mlp.ff)
        f32 = dict(dtype=torch.float32, device=d)
        i32 = dict(dtype=torch.int32, device=d)
        self.n = n
        self.x = torch.zeros(n * W, **f32)                      # the residual stream
        self.xa = torch.zeros(n * W, dtype=T, device=d)         # its copy in the GEMM operand type
        self.P = torch.zeros(n * wide_p, **f32)                 # projection output of the current sublayer
        self.aux = torch.zeros(n * wide_aux, **f32)             # decay logits (GLA) / convolved x, B, C (state-space)
        self.o = torch.zeros(n * wide_o, **f32)                 # raw mixer output (GLA, attention)
        self.o2 = torch.zeros(n * wide_o2, **f32)               # raw state-space output
        self.ob = torch.zeros(n * wide_o if any(eng.tc_attn.values()) else 1, dtype=torch.bfloat16, device=d)  # tcgen05 attention out
        self.ya = torch.zeros(n * wide_o, dtype=T, device=d)    # gated / normed input of the output projection
        self.yb = torch.zeros(n * wide_o2, dtype=T, device=d)
        ny = max(n, 16 * min(n, 128)) * W                       # up to 16 split-K slices of a <= 128-row projection
        self.y0 = torch.zeros(ny, **f32)
        self.y1 = torch.zeros(ny, **f32)
        self.q = torch.zeros(n * wide_q, dtype=T, device=d)
        self.act = torch.zeros(n * wide_f, dtype=T, device=d)
        self.tokens = torch.zeros(n, **i32)
        self.row_pos = torch.zeros(n, **i32)
        self.row_slot = torch.zeros(n, **i32)
        self.row_back = torch.zeros(n, **i32)
        self.seg = torch.zeros(4, n, **i32)                     # seg_start, seg_len, seg_pos0, seg_slot
        self.want = torch.zeros(n, **i32)
        # side-by-side pieces of long segments (prompt portions only): piece tables, a scratch state and a decay
        # table per piece, sized for the largest recurrence of the model
        self.n_sub, self.max_sub = 0, 0
        if pieces:
            lib, st, dc = eng.lib, 1, 1
            for L in cfg.layers:
                for heads, dk, dv in ([(L.gla.heads, L.gla.dim, L.gla.vdim)] if L.kind == "gla" else
                                      [(L.ssd.heads, L.ssd.state, L.ssd.vdim)]):
                    st = max(st, int(lib.prl_lin_scan_state_floats(heads, dk, dv)))
                    dc = max(dc, int(lib.prl_lin_scan_piece_decay_floats(heads, dk)))
            self.max_sub = n // eng.piece_tokens + 8
            self.scratch = torch.zeros(self.max_sub * st, **f32)
            self.cdec = torch.zeros(self.max_sub * dc, **f32)
            self.sub = torch.zeros(2, self.max_sub, **i32)          # sub_start, sub_len
            self.seg_sub = torch.zeros(2, n, **i32)                 # first piece, piece count of every segment


class HybridEngine(EngineCore):
    recurrent = True

    def __init__(self, cfg: HybridConfig, arena, **kw):
        self.f32 = arena.data.dtype == torch.float32
        self.op_dtype = arena.data.dtype
        if self.op_dtype not in (torch.float32, torch.bfloat16):
            raise ValueError("the hybrid engine runs bf16 or fp32 weights")
        self.force_plain_gemm = False      # tests: route every GEMM through the CUDA-core kernel
        self.unfused_glu = False           # tests: gate_up GEMM + activation kernel instead of the GEMM's gated epilogue
        self.force_plain_attn = False      # tests: the any-geometry attention kernel also where the tcgen05 ones fit
        # Long prompt portions run their recurrences as side-by-side pieces (prl_*_scan_split): same values up to fp32
        # rounding, many times the parallelism.  Off in the true-fp32 mode, whose results do not depend on the cut of
        # a prompt bit for bit.  A batch qualifies when its longest segment has split_min_rows rows.
        self.split_scan = not self.f32
        self.split_min_rows = 256
        self.piece_tokens = 64             # tokens per piece (tests lower it); at most prl_lin_scan_piece_tokens()
        self._rows: _Rows | None = None
        super().__init__(cfg, arena, **kw)

    # ---- caches, states, derived parameters ---------------------------------------------------------------------------
    def _alloc_model(self) -> None:
        cfg, d, lib = self.cfg, self.dev, self.lib
        self.k_pool, self.v_pool, self.conv_state, self.ssd_state, self.gla_state, self.rot_freq = {}, {}, {}, {}, {}, {}
        self.tc_attn: dict[int, bool] = {}
        for i, L in enumerate(cfg.layers):               # one cache / state per layer RUN, also where weights are shared
            if L.kind == "gla":
                g = L.gla
                n = int(lib.prl_lin_scan_state_floats(g.heads, g.dim, g.vdim))
                self.gla_state[i] = self.states.add(f"l{i}.gla", (n,))
            else:
                a, s = L.attn, L.ssd
                if a.dim == a.vdim:    # K and V pools adjacent: [2][page][kv head][64][d], the layout of the Qwen2 engine's pool
                    pair = torch.zeros(2, self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                    self.k_pool[i], self.v_pool[i] = pair[0], pair[1]
                else:
                    self.k_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.dim, dtype=self.op_dtype, device=d)
                    self.v_pool[i] = torch.zeros(self.n_pages, a.kv_heads, PAGE_SIZE, a.vdim, dtype=self.op_dtype, device=d)
                # head size 128 in bf16 is what the tcgen05 chunked-prefill kernel and the TMA paged-decode kernel are built
                # for: such a layer runs the SAME attention kernels as the Qwen2 engine (with this layer's own scale)
                self.tc_attn[i] = (not self.f32 and a.dim == 128 and a.vdim == 128
                                   and a.heads // a.kv_heads in (1, 2, 4, 8, 16))
                self.conv_state[i] = self.states.add(f"l{i}.conv", (s.conv_channels, max(s.conv - 1, 1)))
                n = int(lib.prl_lin_scan_state_floats(s.heads, s.state, s.vdim))
                self.ssd_state[i] = self.states.add(f"l{i}.ssd", (n,))
                half = a.rot_dims // 2
                f = [a.rot_base ** (-2.0 * k / a.rot_dims) for k in range(half)] or [0.0]
                self.rot_freq[i] = torch.tensor(f, dtype=torch.float64, device=d)
        # fp32 copies of the small parameter vectors (gains, biases, taps, per-head constants): exact for bf16 weights
        self.vec: dict[str, torch.Tensor] = {}
        for name, shape in cfg.fused_shapes():
            if len(shape) == 1 or name.endswith("mix.right.conv"):
                self.vec[name] = torch.zeros(shape, dtype=torch.float32, device=d)
        self._on_arena_change()
        B = self.B
        self.attn_splits, ws = {}, 0
        for i, on in self.tc_attn.items():
            if on:
                a = cfg.layers[i].attn
                self.attn_splits[i] = int(lib.prl_paged_attn_splits(B, a.kv_heads, self.max_seq_len))
                ws = max(ws, int(lib.prl_paged_attn_workspace_bytes(B, a.heads, self.attn_splits[i])))
        self.attn_ws = torch.zeros(max(ws, 16), dtype=torch.uint8, device=d)
        self._dec = _Rows(self, B)
        i32 = dict(dtype=torch.int32, device=d)
        self._dec.seg[0].copy_(torch.arange(B, **i32))
        self._dec.seg[3].copy_(torch.arange(B, **i32))

    def _on_arena_change(self) -> None:
        for name, t in self.vec.items():
            t.copy_(self.arena.view(name).float())

    def kv_bytes_per_token(self) -> int:
        e = 4 if self.f32 else 2
        return sum(L.attn.kv_heads * (L.attn.dim + L.attn.vdim) * e for L in self.cfg.layers if L.kind == "parallel")

    # ---- GEMM dispatch ------------------------------------------------------------------------------------------------
    def _mm(self, src: torch.Tensor, K: int, w_name: str, N: int, out: torch.Tensor, n: int, split: bool = False) -> int:
        """out[n, N] (fp32) = src[n, K] @ W[N, K]^T.  bf16 with TMA-expressible sizes: the tcgen05 kernels (weight-
        streaming swap-AB for n <= 128 rows, persistent CTA-pair kernel above); otherwise the CUDA-core kernel.
        `split`: the consumer sums split-K slices (prl_postnorm_residual), so a small-N projection of a decode step may
        spread its K range over the SMs; returns the number of slices written ([slices][n][N])."""
        lib, st, wp = self.lib, self._st, self.arena.ptr(w_name)
        if self.f32 or self.force_plain_gemm or K % 8 or K < 64:
            _lib.check(lib.prl_gemm_any(src.data_ptr(), int(self.f32), K, wp, int(self.f32), K, n, N, K,
                                        out.data_ptr(), N, st))
        elif n <= 128:
            k = int(lib.prl_gemm_auto_split_k(n, N, K)) if split else 1
            _lib.check(lib.prl_gemm_bf16_splitk(wp, None, src.data_ptr(), n, N, K, k, out.data_ptr(), st))
            return k
        else:
            _lib.check(lib.prl_gemm_tn(src.data_ptr(), K, wp, K, n, N, K, out.data_ptr(), N, 1, 0, None, None, 0, 1.0, st))
        return 1

    # ---- the layer program over n ragged rows -------------------------------------------------------------------------
    def _layers(self, R: _Rows, n: int, ns: int, max_q: int, row_pos: torch.Tensor, seg_pos0: torch.Tensor,
                trace=None, decode: bool = False) -> None:
        cfg, lib, st, f32 = self.cfg, self.lib, self._st, int(self.f32)
        W, eps, vec = cfg.width, cfg.eps, self.vec
        seg_start, seg_len, seg_slot = R.seg[0].data_ptr(), R.seg[1].data_ptr(), R.seg[3].data_ptr()
        P, x, xa = R.P.data_ptr(), R.x.data_ptr(), R.xa.data_ptr()
        n_sub = 0 if decode else R.n_sub
        if n_sub:
            pieces = (R.seg_sub[0].data_ptr(), R.seg_sub[1].data_ptr(), R.sub[0].data_ptr(), R.sub[1].data_ptr(), n_sub,
                      R.scratch.data_ptr(), R.cdec.data_ptr())
        for i, L in enumerate(cfg.layers):
            w = f"l{L.weights_of}."
            if L.kind == "gla":
                g = L.gla
                nq, nv = g.heads * g.dim, g.heads * g.vdim
                ld = 2 * nq + 2 * nv + g.rank
                self._mm(R.xa, W, w + "mix.in", ld, R.P, n)                       # [q | k | v | g | a1]
                # decay logits z = W_a2 (W_a1 h): the bottleneck stays fp32 (A operand read from P as stored)
                _lib.check(lib.prl_gemm_any(P + 4 * (2 * nq + 2 * nv), 1, ld, self.arena.ptr(w + "mix.a2"), f32, g.rank,
                                            n, nq, g.rank, R.aux.data_ptr(), nq, st))
                _lib.check(lib.prl_gla_decay(R.aux.data_ptr(), nq, vec[w + "mix.a2.b"].data_ptr(), g.tau, n, nq, st))
                if n_sub:
                    _lib.check(lib.prl_gla_scan_split(P, ld, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                                      g.vdim, seg_slot, ns, *pieces, self.gla_state[i].data_ptr(),
                                                      R.o.data_ptr(), nv, st))
                else:
                    _lib.check(lib.prl_gla_scan(P, ld, 0, nq, 2 * nq, g.dim ** -0.5, R.aux.data_ptr(), nq, g.heads, g.dim,
                                                g.vdim, seg_start, seg_len, seg_slot, ns, self.gla_state[i].data_ptr(),
                                                R.o.data_ptr(), nv, st))
                _lib.check(lib.prl_gate_norm(R.o.data_ptr(), 1, nv, P + 4 * (2 * nq + nv), ld, vec[w + "mix.norm"].data_ptr(),
                                             g.vdim, g.vdim, n, nv, 0, 0, 1, eps, R.ya.data_ptr(), f32, st))
                k0 = self._mm(R.ya, nv, w + "mix.o", W, R.y0, n, split=True)
                _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, k0, None, 0, 0.0, 1, vec[w + "norm1"].data_ptr(),
                                                     eps, n, W, x, xa, f32, st))
            else:
                a, s = L.attn, L.ssd
                nq, nk, nvk, ng = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim, a.heads * a.vdim
                left = nq + nk + nvk + ng
                ld = left + s.in_rows
                self._mm(R.xa, W, w + "mix.in", ld, R.P, n)                       # [q | k | v | g || z | x B C | dt]
                # -- left: softmax attention over the paged cache
                _lib.check(lib.prl_qk_norm_rope_cache(P, ld, 0, nq, nq + nk, n, a.heads, a.kv_heads, a.dim, a.vdim,
                                                      a.rot_dims, self.rot_freq[i].data_ptr(),
                                                      vec[w + "mix.left.q.norm"].data_ptr(),
                                                      vec[w + "mix.left.k.norm"].data_ptr(), eps, row_pos.data_ptr(),
                                                      R.row_slot.data_ptr(), self.block_table.data_ptr(), self.max_blocks,
                                                      PAGE_SIZE, R.q.data_ptr(), self.k_pool[i].data_ptr(),
                                                      self.v_pool[i].data_ptr(), f32, st))
                if self.tc_attn[i] and not self.force_plain_attn:
                    kv = self.k_pool[i].data_ptr()       # K pool, V pool right behind it (one "layer" of the Qwen2 pool layout)
                    if decode:
                        _lib.check(lib.prl_paged_attn_decode(R.q.data_ptr(), kv, self.n_pages, 1, 0, self.block_table.data_ptr(),
                                                             self.max_blocks, self.seq_lens.data_ptr(), n, a.heads, a.kv_heads,
                                                             a.dim, PAGE_SIZE, self.attn_splits[i], a.scale, R.ob.data_ptr(),
                                                             self.attn_ws.data_ptr(), self.attn_ws.numel(), st))
                    else:
                        _lib.check(lib.prl_paged_attn_prefill_tc(R.q.data_ptr(), n, kv, self.n_pages, 1, 0,
                                                                 self.block_table.data_ptr(), self.max_blocks, seg_start,
                                                                 seg_len, seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads,
                                                                 a.kv_heads, a.dim, PAGE_SIZE, a.scale, R.ob.data_ptr(), st))
                    o_ptr, o_f32 = R.ob.data_ptr(), 0
                else:
                    _lib.check(lib.prl_attn_any(R.q.data_ptr(), self.k_pool[i].data_ptr(), self.v_pool[i].data_ptr(), f32,
                                                self.block_table.data_ptr(), self.max_blocks, PAGE_SIZE, seg_start, seg_len,
                                                seg_pos0.data_ptr(), seg_slot, ns, max_q, a.heads, a.kv_heads, a.dim, a.vdim,
                                                a.scale, R.o.data_ptr(), st))
                    o_ptr, o_f32 = R.o.data_ptr(), 1
                _lib.check(lib.prl_gate_norm(o_ptr, o_f32, ng, P + 4 * (nq + nk + nvk), ld, None, 1, ng, n, ng, 1, 0, 0,
                                             eps, R.ya.data_ptr(), f32, st))
                k0 = self._mm(R.ya, ng, w + "mix.left.o", W, R.y0, n, split=True)
                # -- right: state-space mixer
                inner, ch = s.inner, s.conv_channels
                conv_w, conv_b = vec[w + "mix.right.conv"].data_ptr(), vec[w + "mix.right.conv.b"].data_ptr()
                _lib.check(lib.prl_conv_silu(P, ld, left + inner, n, ch, s.conv, conv_w, conv_b, R.row_slot.data_ptr(),
                                             R.row_back.data_ptr(), self.conv_state[i].data_ptr(), R.aux.data_ptr(), st))
                _lib.check(lib.prl_conv_state_update(P, ld, left + inner, ch, s.conv, seg_start, seg_len, seg_slot, ns,
                                                     self.conv_state[i].data_ptr(), st))
                ssd_vec = (vec[w + "mix.right.dt_bias"].data_ptr(), vec[w + "mix.right.A_log"].data_ptr(),
                           vec[w + "mix.right.D"].data_ptr())
                if n_sub:
                    _lib.check(lib.prl_ssd_scan_split(P, ld, left + inner + ch, R.aux.data_ptr(), ch, *ssd_vec, s.heads,
                                                      s.groups, s.state, s.vdim, seg_slot, ns, *pieces,
                                                      self.ssd_state[i].data_ptr(), R.o2.data_ptr(), inner, st))
                else:
                    _lib.check(lib.prl_ssd_scan(P, ld, left + inner + ch, R.aux.data_ptr(), ch, *ssd_vec, s.heads, s.groups,
                                                s.state, s.vdim, seg_start, seg_len, seg_slot, ns,
                                                self.ssd_state[i].data_ptr(), R.o2.data_ptr(), inner, st))
                _lib.check(lib.prl_gate_norm(R.o2.data_ptr(), 1, inner, P + 4 * left, ld, vec[w + "mix.right.norm"].data_ptr(),
                                             inner, inner // s.norm_groups, n, inner, 0, 1, 1, eps, R.yb.data_ptr(), f32, st))
                k1 = self._mm(R.yb, inner, w + "mix.right.o", W, R.y1, n, split=True)
                _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, L.left_scale, k0, R.y1.data_ptr(), W, L.right_scale, k1,
                                                     vec[w + "norm1"].data_ptr(), eps, n, W, x, xa, f32, st))
            if L.mlp is not None:
                F = L.mlp.ff
                tc = not (self.f32 or self.force_plain_gemm or W % 8 or W < 64 or self.unfused_glu)
                if tc and n <= 128 and F % 64 == 0:
                    # the clamped gate in the gate_up GEMM's epilogue (the Qwen2 step's SwiGLU-epilogue kernel): no [n, 2F] tile
                    _lib.check(lib.prl_gemm_glu_clamped_decode(self.arena.ptr(w + "mlp.gate_up"), xa, n, F, W, L.mlp.limit,
                                                               L.mlp.beta, R.act.data_ptr(), st))
                elif tc and n > 128 and F % 128 == 0:
                    _lib.check(lib.prl_gemm_glu_clamped_f32(xa, W, self.arena.ptr(w + "mlp.gate_up"), W, n, F, W, L.mlp.limit,
                                                            L.mlp.beta, R.act.data_ptr(), F, st))
                else:
                    self._mm(R.xa, W, w + "mlp.gate_up", 2 * F, R.P, n)
                    _lib.check(lib.prl_glu_clamped(P, 2 * F, n, F, L.mlp.limit, L.mlp.beta, R.act.data_ptr(), f32, st))
                k0 = self._mm(R.act, F, w + "mlp.down", W, R.y0, n, split=True)
                _lib.check(lib.prl_postnorm_residual(R.y0.data_ptr(), W, 1.0, k0, None, 0, 0.0, 1, vec[w + "norm2"].data_ptr(),
                                                     eps, n, W, x, xa, f32, st))
            if trace is not None:
                trace.append(R.x[:n * W].view(n, W).clone())

    # ---- one token for every slot (captured into the engine's CUDA graph) ---------------------------------------------
    def _step_kernels(self) -> None:
        cfg, lib, R, B = self.cfg, self.lib, self._dec, self.B
        self._st = st = _lib.stream_ptr()
        _lib.check(lib.prl_decode_rows(self.active.data_ptr(), B, R.seg[1].data_ptr(), R.row_slot.data_ptr(), st))
        _lib.check(lib.prl_embed_scale(self.tokens.data_ptr(), self.arena.ptr("embed"), int(self.f32), cfg.embed_scale, B,
                                       cfg.width, cfg.vocab_size, R.x.data_ptr(), R.xa.data_ptr(), st))
        self._layers(R, B, B, 1, self.positions, self.positions, decode=True)
        _lib.check(lib.prl_rmsnorm_rows(R.x.data_ptr(), None, self.vec["final.norm"].data_ptr(), cfg.eps, B, cfg.width,
                                        R.xa.data_ptr(), int(self.f32), st))
        self._mm(R.xa, cfg.width, "head", cfg.vocab_size, self.logits, B)

    # ---- a packed batch of prompt portions (prefill chunks, token streams) --------------------------------------------
    def _forward_rows(self, segs, want_rows, trace=None):
        cfg, lib = self.cfg, self.lib
        if self._rows is None:
            self._rows = _Rows(self, max(self.prefill_chunk, 1), pieces=True)
        R = self._rows
        n = sum(k for _, _, k in segs)
        if n > R.n:
            raise ValueError(f"{n} rows exceed the prefill chunk of {R.n}")
        toks, pos, slot, back, meta = [], [], [], [], [[], [], [], []]
        at = 0
        for req, s0, k in segs:
            toks += req.prompt_ids[s0:s0 + k]
            pos += range(s0, s0 + k)
            slot += [req.slot] * k
            back += range(k)
            meta[0].append(at); meta[1].append(k); meta[2].append(s0); meta[3].append(req.slot)
            at += k
        ns = len(segs)
        i32 = torch.int32
        R.n_sub = 0
        if self.split_scan and max(k for _, _, k in segs) >= self.split_min_rows:
            step = min(self.piece_tokens, int(lib.prl_lin_scan_piece_tokens()))
            sub, seg_sub = [[], []], [[], []]
            for start, k in zip(meta[0], meta[1]):
                seg_sub[0].append(len(sub[0]))
                seg_sub[1].append((k + step - 1) // step)
                sub[0] += range(start, start + k, step)
                sub[1] += [min(step, k - c) for c in range(0, k, step)]
            if len(sub[0]) <= R.max_sub:          # else: many short segments beside the long one, walk them token by token
                R.n_sub = len(sub[0])
                R.sub[:, :R.n_sub].copy_(torch.tensor(sub, dtype=i32), non_blocking=True)
                R.seg_sub[:, :ns].copy_(torch.tensor(seg_sub, dtype=i32), non_blocking=True)
        R.tokens[:n].copy_(torch.tensor(toks, dtype=i32), non_blocking=True)
        R.row_pos[:n].copy_(torch.tensor(pos, dtype=i32), non_blocking=True)
        R.row_slot[:n].copy_(torch.tensor(slot, dtype=i32), non_blocking=True)
        R.row_back[:n].copy_(torch.tensor(back, dtype=i32), non_blocking=True)
        R.seg[:, :ns].copy_(torch.tensor(meta, dtype=i32), non_blocking=True)
        self._st = st = _lib.stream_ptr()
        _lib.check(lib.prl_embed_scale(R.tokens.data_ptr(), self.arena.ptr("embed"), int(self.f32), cfg.embed_scale, n,
                                       cfg.width, cfg.vocab_size, R.x.data_ptr(), R.xa.data_ptr(), st))
        self._layers(R, n, ns, max(k for _, _, k in segs), R.row_pos, R.seg[2], trace=trace)
        self.stats["prefill_tokens"] += n
        if not want_rows:
            return None
        nw = len(want_rows)
        R.want[:nw].copy_(torch.tensor(want_rows, dtype=i32), non_blocking=True)
        _lib.check(lib.prl_rmsnorm_rows(R.x.data_ptr(), R.want.data_ptr(), self.vec["final.norm"].data_ptr(), cfg.eps, nw,
                                        cfg.width, R.xa.data_ptr(), int(self.f32), st))
        out = torch.empty(nw, cfg.vocab_size, dtype=torch.float32, device=self.dev)
        self._mm(R.xa, cfg.width, "head", cfg.vocab_size, out, nw)
        return out
