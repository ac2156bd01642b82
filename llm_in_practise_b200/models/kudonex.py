"""Kudonex: a decoder-only language model whose layers pick one of three mixers — an mLSTM matrix memory, a Mamba-2 style
selective state space, or windowed talking-heads attention whose values are its keys — each behind a short causal
convolution, with a mixture-of-experts feed-forward and layer norms before AND after every sublayer.

The stream x (fp32) starts as ``embed[token] * s_e + P[position]``, P the interleaved sin / cos table with frequencies
10000^(-2i / width). LN is a layer norm with a weight and no bias. Layer i (tensors ``l<i>.*``):

    h = LN1(x);  h <- h + conv(h)          a per-channel causal convolution over time (``canon1`` [width, taps]); the last
                                           taps - 1 rows of h are carried per sequence
    x <- x + LN1b(mixer(h))
    x <- x + LN2b(ff(LN2(x)))              only if the layer has a feed-forward

* ``mlstm``: q = W_q h / sqrt(dim), k = W_k h, v = W_v h per head; log gates i = c tanh((W_i h + b_i) / c) and
  f = logsigmoid(c tanh((W_f h + b_f) / c)) with c = ``gate_cap``; a running maximum m' = max(f + m, i) (m = 0 at the start)
  keeps S' = e^(f + m - m') S + e^(i - m') k v^T and n' = e^(f + m - m') n + e^(i - m') k in range; the read-out is
  S'^T q / (max(|n' . q|, e^(-m')) + 1e-6), each head divided by its root mean square, times a weight over all heads, times
  sigmoid(W_g h), then W_o.
* ``mamba2``: W_in h = [z | x | B | C | dt]; x, B, C pass a causal convolution with bias and silu; dt = softplus(dt + bias);
  per head S' = exp(-exp(A_log) dt) S + dt B x^T (B, C shared by the heads of a group), y = S'^T C + D x; y silu(z) is
  RMS-normed in ``norm_groups`` equal parts, times a weight, then W_o.
* ``attention``: grouped query heads over keys that are also the values (no value projection, no rotation); from every
  score a distance penalty r1_h log(1 + r2_h (i - j)) is taken off, the heads' scores are mixed by ``talk`` [H, H] before
  an ordinary softmax over the last ``mask.size`` positions; the heads' outputs are gated by sigmoid(W_g h), then W_o.
* feed-forward: softmax router in fp32; the ``top`` experts with the largest corrected scores (score + ``correction``) among
  the ``groups.keep`` groups of neighbouring experts whose best corrected score is largest; weights are the uncorrected
  scores, not renormalised; SwiGLU experts plus a shared SwiGLU expert for every token.

The output is ``embed @ LN(x)`` (the embedding table without its scale). What is fp32 whatever the model dtype: the stream,
every norm, the position table, scores / mixing / softmax, routers, the recurrent states and everything between the
projections and the scans (convolutions, gates, decays, step sizes, read-out norms).

Keys live in the paged cache (``kv_layout``: key rows only), the convolution tails, matrix memories, running maxima and
state-space states in its per-sequence state rows (``state_layout``). ``inference/ragged.RaggedGenerator`` and
``serve/engine.LLMEngine`` drive ``forward_ragged``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from ..ops import elementwise as ew
from ..ops.gemm import linear_exact
from ..ops.linear_scan import linear_scan, mlstm_gates, scan_readout, short_conv, ssm_gates
from ..ops.moe import gated_moe_ffn, route_grouped
from ..ops.norm import sandwich_norm
from ..ops.paged_attention import rope_paged_store
from ..ops.talking_attention import talking_attention

MIXERS = ("mlstm", "mamba2", "attention")
MLSTM_DEN_EPS = 1e-6              # added to the mLSTM read-out's denominator: fixed by the design
POS_BASE = 10000.0                # base of the position table's frequencies: fixed by the design
GROUP_TOP = 1                     # a group of experts is ranked by its single best corrected score


@dataclass
class KudonexMixer:
    kind: str
    heads: int
    vdim: int
    dim: int = 0                                # mlstm, attention: query / key size per head; mamba2: the state size N
    kv_heads: int = 0                           # attention: key heads; mamba2: groups that share B and C
    gate_cap: float = 0.0                       # mlstm
    conv: int = 1                               # mamba2: taps of the convolution on x | B | C
    norm_groups: int = 1                        # mamba2
    window: int = 0                             # attention
    scale: float = 1.0                          # attention


@dataclass
class KudonexFF:
    experts: int
    top: int
    ff: int
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0


@dataclass
class KudonexLayerSpec:
    type: str
    mixer: KudonexMixer
    mlp: Optional[KudonexFF]


@dataclass
class KudonexConfig:
    vocab_size: int
    hidden_size: int
    layers: List[KudonexLayerSpec]
    norm_eps: float
    embed_scale: float = 1.0
    canon_taps: int = 1
    model_type: str = "kudonex"
    raw: dict = field(default_factory=dict, repr=False)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, d: dict) -> "KudonexConfig":
        layers = []
        for i, L in enumerate(d["layers"]):
            kind, m = L["type"], L["mixer"]
            if kind not in MIXERS:
                raise ValueError(f"Kudonex has no mixer {kind!r}")
            mx = KudonexMixer(kind=kind, heads=int(m["heads"]), vdim=int(m["vdim"]))
            if kind == "mlstm":
                mx.dim, mx.gate_cap, mx.kv_heads = int(m["dim"]), float(m["gate_cap"]), mx.heads
                if not mx.gate_cap > 0:
                    raise ValueError(f"layer {i}: gate_cap must be positive")
            elif kind == "mamba2":
                mx.dim, mx.kv_heads, mx.conv = int(m["state"]), int(m.get("groups", 1)), int(m.get("conv", 1))
                mx.norm_groups = int(m.get("norm_groups", 1))
                if mx.heads % mx.kv_heads or (mx.heads * mx.vdim) % mx.norm_groups or mx.conv < 1:
                    raise ValueError(f"layer {i}: bad mamba2 sizes")
            else:
                mx.dim, mx.kv_heads = int(m["dim"]), int(m.get("kv_heads", m["heads"]))
                mx.window, mx.scale = int((m.get("mask") or {}).get("size", 0)), float(m["scale"])
                if mx.heads % mx.kv_heads or mx.vdim != mx.dim:
                    raise ValueError(f"layer {i}: keys are the values, so vdim must equal dim, and kv_heads must divide heads")
            f = L.get("mlp")
            ff = None
            if f is not None:
                if f.get("kind", "moe") != "moe":
                    raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
                r, g = f["router"], f["router"].get("groups") or {}
                ff = KudonexFF(experts=int(r["experts"]), top=int(r["top"]), ff=int(f["expert"]["ff"]), groups=int(g.get("count", 1)),
                               keep=int(g.get("keep", g.get("count", 1))), shared_ff=int((f.get("shared") or {}).get("ff", 0)))
                if ff.experts % ff.groups or not 1 <= ff.keep <= ff.groups or ff.top > ff.keep * (ff.experts // ff.groups):
                    raise ValueError(f"layer {i}: bad router sizes")
            layers.append(KudonexLayerSpec(kind, mx, ff))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers, norm_eps=float(d["norm"]["eps"]),
                   embed_scale=float((d.get("embedding") or {}).get("scale", 1.0)),
                   canon_taps=int((d.get("canon") or {}).get("taps", 1)), raw=d)


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class KudonexLayer(nn.Module):
    def __init__(self, cfg: KudonexConfig, idx: int, dtype, device):
        super().__init__()
        spec = cfg.layers[idx]
        m, f, W = spec.mixer, spec.mlp, cfg.hidden_size
        self.spec, self.idx = spec, idx
        f32 = lambda *n, v=0.0: nn.Parameter(torch.full(n, v, dtype=torch.float32, device=device))       # noqa: E731
        wt = lambda *n: nn.Parameter(torch.zeros(*n, dtype=dtype, device=device))                        # noqa: E731
        self.norm1, self.norm1b = f32(W, v=1.0), f32(W, v=1.0)
        self.canon = f32(W, cfg.canon_taps)
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        # projections that read the mixer's input are one weight; parts = name -> (first row, end row); rows padded to 8
        if m.kind == "mlstm":
            parts = [("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv), ("i", H), ("f", H)]
            self.i_bias, self.f_bias = f32(H), f32(H)
            self.mix_norm = f32(H * Dv, v=1.0)
        elif m.kind == "mamba2":
            parts = [("in", 2 * H * Dv + 2 * G * D + H)]
            C = H * Dv + 2 * G * D
            self.conv_w, self.conv_b = f32(C, m.conv), f32(C)
            self.dt_bias, self.A_log, self.D_skip = f32(H), f32(H), f32(H)
            self.mix_norm = f32(H * Dv, v=1.0)
        else:
            parts = [("q", H * D), ("k", G * D), ("g", H * D)]
            self.r1, self.r2 = f32(H), f32(H)
            self.talk = nn.Parameter(torch.eye(H, dtype=torch.float32, device=device))
        self.parts = {}
        lo = 0
        for n, r in parts:
            self.parts[n] = (lo, lo + r)
            lo += r
        self.in_proj = wt(_pad8(lo), W)
        self.o_proj = wt(W, H * Dv)
        if f is not None:
            self.norm2, self.norm2b = f32(W, v=1.0), f32(W, v=1.0)
            self.router = f32(f.experts, W)
            self.correction = f32(f.experts)
            self.experts_gate_up = wt(f.experts, 2 * f.ff, W)
            self.experts_down = wt(f.experts, W, f.ff)
            if f.shared_ff:
                self.shared_gate_up = wt(2 * f.shared_ff, W)
                self.shared_down = wt(W, f.shared_ff)

    # ------------------------------------------------------------------ mixers: h [T, W] (model dtype) -> fp32 [T, W]
    def mlstm(self, h, pos, slot, state, runs, n_runs, eps: float):
        m = self.spec.mixer
        H, D, Dv = m.heads, m.dim, m.vdim
        proj = linear_exact(h, self.in_proj, out_dtype=torch.float32)
        sl = lambda n: proj[:, self.parts[n][0]:self.parts[n][1]]             # noqa: E731
        a, b, e = mlstm_gates(sl("i"), sl("f"), self.i_bias, self.f_bias, m.gate_cap, state[2], pos, slot, runs, n_runs)
        # a column of ones rides along with v: the state's last column is the normaliser n, o's last column n . q
        o = linear_scan(sl("q"), sl("k"), sl("v"), state[1], pos, slot, runs, n_runs, H, H, D, Dv + 1, "gated", g=a, beta=b, ones=True)
        z = scan_readout(o, H, Dv, self.mix_norm, H, eps, h.dtype, e=e, den_eps=MLSTM_DEN_EPS, oscale=D ** -0.5, post=sl("g"))
        return linear_exact(z, self.o_proj, out_dtype=torch.float32)

    def mamba2(self, h, pos, slot, state, runs, n_runs, eps: float):
        m = self.spec.mixer
        H, G, N, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        inner, C = H * Dv, H * Dv + 2 * G * N
        proj = linear_exact(h, self.in_proj, out_dtype=torch.float32)
        xbc = short_conv(proj[:, inner:inner + C], self.conv_w, state[2], pos, slot, runs, n_runs, act=True, bias=self.conv_b)
        x, Bm, Cm = xbc[:, :inner], xbc[:, inner:inner + G * N], xbc[:, inner + G * N:]
        a, b = ssm_gates(proj[:, inner + C:inner + C + H], self.dt_bias, self.A_log)
        o = linear_scan(Cm, Bm, x, state[1], pos, slot, runs, n_runs, H, G, N, Dv, "gated", g=a, beta=b)
        z = scan_readout(o, H, Dv, self.mix_norm, m.norm_groups, eps, h.dtype, skip=self.D_skip, x=x, pre=proj[:, :inner])
        return linear_exact(z, self.o_proj, out_dtype=torch.float32)

    def attention(self, h, pos, slot, cache, pieces, zero):
        m = self.spec.mixer
        H, G, D = m.heads, m.kv_heads, m.dim
        qkg = linear_exact(h, self.in_proj)
        rope_paged_store(qkg[:, H * D:], zero, zero, pos, slot, cache.k[self.idx], None, cache.table, 0, G, D, rot_dims=0)
        ctx = talking_attention(qkg, cache.k[self.idx], cache.table, pos, slot, H, G, D, m.scale, m.window, self.r1, self.r2,
                                self.talk, gate=qkg[:, (H + G) * D:(2 * H + G) * D], pieces=pieces)
        return linear_exact(ctx, self.o_proj, out_dtype=torch.float32)

    def feed_forward(self, h: torch.Tensor) -> torch.Tensor:
        """h [T, W] (already normed) -> the sublayer's output in fp32 [T, W]."""
        f = self.spec.mlp
        top_i, top_p, _ = route_grouped(h, self.router, self.correction, f.top, f.groups, f.keep, GROUP_TOP, softmax=True)
        shared = None
        if f.shared_ff:
            shared = linear_exact(ew.act_glu(linear_exact(h, self.shared_gate_up), "silu"), self.shared_down)
        return gated_moe_ffn(h, top_i, top_p, self.experts_gate_up, self.experts_down, _swiglu, shared=shared)


def _swiglu(gate_up: torch.Tensor) -> torch.Tensor:
    return ew.act_glu(gate_up, "silu")


class KudonexForCausalLM(nn.Module):
    """``forward_ragged`` is the serving step; ``forward(input_ids)`` runs whole sequences through the same step."""
    ragged = True                                   # served by inference.ragged.RaggedGenerator

    def __init__(self, cfg: KudonexConfig, dtype=torch.bfloat16, device=None, init_std: float = 0.02):
        super().__init__()
        self.config = cfg
        self.dtype_ = dtype
        W, V = cfg.hidden_size, cfg.vocab_size
        self.embed_tokens = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self.layers = nn.ModuleList([KudonexLayer(cfg, i, dtype, device) for i in range(len(cfg.layers))])
        self.norm = nn.Parameter(torch.ones(W, dtype=torch.float32, device=device))
        self._pos_table = {}

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.device

    def head_weight(self) -> torch.Tensor:
        return self.embed_tokens                    # the output projection is the embedding table

    def kv_layout(self):
        """(key rows, key row size, value row size) per layer: an attention layer caches its key rows and no values (they are
        the keys); the recurrent layers have no pool."""
        return [(s.mixer.kv_heads, s.mixer.dim, 0) if s.mixer.kind == "attention" else (0, 0, 0) for s in self.config.layers]

    def state_layout(self):
        """Per layer, the shapes of the fp32 tensors a sequence carries from token to token: always the last ``taps - 1``
        inputs of the layer's input convolution; then for mlstm the matrix memory with the normaliser as one more column and
        the running maximum per head, for mamba2 the state per head and the last inputs of the x | B | C convolution."""
        W, L = self.config.hidden_size, self.config.canon_taps - 1
        out = []
        for s in self.config.layers:
            m = s.mixer
            shapes = [(L, W)]
            if m.kind == "mlstm":
                shapes += [(m.heads, m.dim, m.vdim + 1), (m.heads,)]
            elif m.kind == "mamba2":
                shapes += [(m.heads, m.dim, m.vdim), (m.conv - 1, m.heads * m.vdim + 2 * m.kv_heads * m.dim)]
            out.append(shapes)
        return out

    def pos_table(self, device, need: int) -> torch.Tensor:
        """The additive position table for at least ``need`` positions. A table that had to grow leaves the old one alive:
        CUDA graphs captured against a smaller cache still read it."""
        tabs = self._pos_table.setdefault(str(device), [])
        if not tabs or tabs[-1].shape[0] < need:
            tabs.append(ew.sinusoid_table(max(need, 1024), self.config.hidden_size, device, POS_BASE))
        return tabs[-1]

    @torch.no_grad()
    def forward_ragged(self, ids: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache, want: Optional[torch.Tensor] = None,
                       max_pos: int = 0, pieces=None, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """One serving step over a flat token list: ``ids`` long [T], ``pos`` / ``slot`` int32 [T] (position in its sequence
        and cache / state row of every token), ``cache`` a ``PagedKVCache`` whose table rows cover those positions and whose
        state rows belong to the same sequences. Returns fp32 logits of the rows ``want`` (long [n]; default all).
        ``pieces`` describes the runs of consecutive tokens (None: every token is a sequence of its own step, a decode
        batch). ``layer_outputs``: a list that receives the residual stream after every layer."""
        cfg = self.config
        dt = self.embed_tokens.dtype
        eps = cfg.norm_eps
        dev = ids.device
        f32 = torch.float32
        layers = self.layers
        table = self.pos_table(dev, max(int(max_pos) + 1, cache.max_len))
        runs, n_runs = (pieces.runs, pieces.n_runs) if pieces is not None else (None, ids.shape[0])
        zero = torch.zeros(1, 1, dtype=f32, device=dev)          # the (unused) rotary tables of a key store without rotation
        x0 = ew.embedding_pos(ids, self.embed_tokens, cfg.embed_scale, pos, table)
        first = layers[0].norm1 if len(layers) else self.norm
        h, x = sandwich_norm(x0, None, None, first, eps, 0.0, f32 if len(layers) else dt, center=True)
        for li, layer in enumerate(layers):
            m = layer.spec.mixer
            state = cache.state[li]
            # the mixer reads h + conv(h); norms feed the convolution in fp32, its output is the projections' operand
            hc = short_conv(h, layer.canon, state[0], pos, slot, runs, n_runs, act=False, residual=True, out_dtype=dt)
            if m.kind == "mlstm":
                y = layer.mlstm(hc, pos, slot, state, runs, n_runs, eps)
            elif m.kind == "mamba2":
                y = layer.mamba2(hc, pos, slot, state, runs, n_runs, eps)
            else:
                y = layer.attention(hc, pos, slot, cache, pieces, zero)
            last = li + 1 == len(layers)
            nxt, nxt_dt = (self.norm, dt) if last else (layers[li + 1].norm1, f32)
            if layer.spec.mlp is None:
                h, x = sandwich_norm(y, layer.norm1b, x, nxt, eps, 0.0, nxt_dt, center=True)
            else:
                h, x = sandwich_norm(y, layer.norm1b, x, layer.norm2, eps, 0.0, dt, center=True)
                h, x = sandwich_norm(layer.feed_forward(h), layer.norm2b, x, nxt, eps, 0.0, nxt_dt, center=True)
            if layer_outputs is not None:
                layer_outputs.append(x)
        if want is not None:
            h = h.index_select(0, want)
        return linear_exact(h.contiguous(), self.embed_tokens, out_dtype=f32)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, labels=None, **_) -> dict:
        """Whole sequences [B, S] through the serving step with a throw-away cache: ``{"logits": [B, S, V]}`` (fp32)."""
        if labels is not None:
            raise NotImplementedError("Kudonex is an inference model here: no loss / backward")
        from ..inference.ragged import RaggedGenerator
        B, S = input_ids.shape
        gen = RaggedGenerator(self, None, max_len=S)
        per = -(-S // 64)
        cache = gen.make_cache(num_blocks=B * per, block_size=64, max_seqs=B, max_len=S)
        for b in range(B):
            gen.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
        logits = gen.step([(b, 0, input_ids[b].tolist(), list(range(S))) for b in range(B)], cache)
        return {"logits": logits.view(B, S, -1)}

    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 256, **kw) -> torch.Tensor:
        from ..inference.ragged import RaggedGenerator
        g = self.__dict__.get("_generator")
        need = input_ids.shape[1] + int(max_new_tokens)
        if g is None or g.max_len < need:
            g = self.__dict__["_generator"] = RaggedGenerator(self, None, max(need, 4096))
        return g.generate(input_ids.to(self.device), max_new_tokens=max_new_tokens, **kw)

    def num_parameters(self, only_trainable: bool = False) -> int:
        return sum(p.numel() for p in self.parameters() if p.requires_grad or not only_trainable)


# ------------------------------------------------------------------------------------------------------------------
# checkpoint: config.json + model.safetensors with the design's own tensor names
# ------------------------------------------------------------------------------------------------------------------
def _tensor_map(model: KudonexForCausalLM):
    """(checkpoint name, the view of a parameter that holds it) per tensor."""
    out = [("embed", model.embed_tokens), ("final.norm", model.norm)]
    for i, layer in enumerate(model.layers):
        p, m, f = f"l{i}.", layer.spec.mixer, layer.spec.mlp
        out += [(p + "norm1", layer.norm1), (p + "norm1b", layer.norm1b), (p + "canon1", layer.canon)]
        for n, (lo, hi) in layer.parts.items():
            out.append((f"{p}mix.{n}", layer.in_proj[lo:hi]))
        out.append((p + "mix.o", layer.o_proj))
        if m.kind == "mlstm":
            out += [(p + "mix.i.b", layer.i_bias), (p + "mix.f.b", layer.f_bias), (p + "mix.norm", layer.mix_norm)]
        elif m.kind == "mamba2":
            out += [(p + "mix.conv", layer.conv_w), (p + "mix.conv.b", layer.conv_b), (p + "mix.dt_bias", layer.dt_bias),
                    (p + "mix.A_log", layer.A_log), (p + "mix.D", layer.D_skip), (p + "mix.norm", layer.mix_norm)]
        else:
            out += [(p + "mix.r1", layer.r1), (p + "mix.r2", layer.r2), (p + "mix.talk", layer.talk)]
        if f is None:
            continue
        out += [(p + "norm2", layer.norm2), (p + "norm2b", layer.norm2b), (p + "mlp.router", layer.router),
                (p + "mlp.correction", layer.correction)]
        for e in range(f.experts):
            q = f"{p}mlp.e{e}."
            out += [(q + "gate", layer.experts_gate_up[e, :f.ff]), (q + "up", layer.experts_gate_up[e, f.ff:]),
                    (q + "down", layer.experts_down[e])]
        if f.shared_ff:
            out += [(p + "mlp.shared.gate", layer.shared_gate_up[:f.shared_ff]), (p + "mlp.shared.up", layer.shared_gate_up[f.shared_ff:]),
                    (p + "mlp.shared.down", layer.shared_down)]
    return out


@torch.no_grad()
def load_kudonex_weights(model: KudonexForCausalLM, path: str) -> None:
    from ..io.safetensors import safe_open
    with safe_open(os.path.join(path, "model.safetensors")) as f:
        names = set(f.keys())
        used = set()
        for name, dst in _tensor_map(model):
            used.add(name)
            dst.copy_(f.get_tensor(name).to(dst.device, dst.dtype).reshape(dst.shape))
        missing = names - used
        if missing:
            raise ValueError(f"checkpoint tensors the model has no place for: {sorted(missing)[:8]}")


def kudonex_from_pretrained(path: str, dtype=torch.bfloat16, device=None) -> KudonexForCausalLM:
    with open(os.path.join(path, "config.json")) as f:
        cfg = KudonexConfig.from_dict(json.load(f))
    model = KudonexForCausalLM(cfg, dtype=dtype, device=device)
    load_kudonex_weights(model, path)
    model.name_or_path = path
    return model.eval()


@torch.no_grad()
def kudonex_state_dict(model: KudonexForCausalLM) -> dict:
    """Tensors under the checkpoint's names (the inverse of ``load_kudonex_weights``)."""
    return {name: t.detach().contiguous() for name, t in _tensor_map(model)}
