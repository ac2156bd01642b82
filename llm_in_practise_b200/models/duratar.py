"""Duratar: a decoder-only language model that mixes windowed differential attention with two recurrent mixers on
hyper-connected residual streams.

The stream enters as ``rms(embed[token]) * g_embed`` copied into S = ``streams`` residual streams x_1 .. x_S (fp32). Every
sublayer q of layer i (1: the mixer, 2: the feed-forward, if the layer has one) reads and writes all of them:

    u = sum_s in_q[s] x_s          y = sublayer(rms(u) * g_q)          x_t <- sum_s mix_q[s, t] x_s + out_q[t] * (ls_q (.) y)

``g`` are one-number norm weights, ``ls`` per-channel layer scales. A config without ``streams`` is the plain pre-norm
residual sum (S = 1, all coefficients 1). The output is ``head(rms(sum_s x_s) * g_final)``. Mixers (``layers[i].type``):

* ``attention``: H heads over G key/value heads, two attention maps per head (own query and key rows of ``dim``, shared
  values of ``vdim``), RMS-normed q / k rows with a weight, rotary on the first ``rot.dims`` dims in the split-half layout
  with wavelength-band frequency rescaling, a sliding window that keeps the first ``mask.keep_first`` tokens, and the
  differential combination o = a_1 - lambda a_2, o <- rms(o) (1 - diff), lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff.
  ``kv_from: j`` makes the layer attend over layer j's cached keys and values with its own queries.
* ``lightning``: q, k, v = silu of their projections; per head S <- decay_h S + k v^T, o = S^T q; the concatenated heads are
  RMS-normed with a weight, gated by sigmoid(W_g h) and projected.
* ``channel_delta``: q, k, v pass a short causal convolution and silu; q, k become unit vectors (q also / sqrt(dim));
  beta = sigmoid(W_b h); per key channel g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias)); per head
  S <- diag(g) S, u = beta (v - S^T k), S <- S + k u^T, o = S^T q; each head is RMS-normed with a weight shared by the
  heads, gated by sigmoid(W_g2 W_g1 h) and projected.

The feed-forward is ``W_down xIELU(W_up h)``. What is fp32 whatever the model dtype: the streams, every norm, rotary tables,
scores and softmax, the recurrent states and everything that enters the recurrences after the projections.

Keys and values live in the paged cache (``kv_layout``: 2 G key rows and G value rows per token; none for layers that
share another layer's), recurrent states and convolution tails in its per-sequence state rows (``state_layout``).
``inference/ragged.RaggedGenerator`` and ``serve/engine.LLMEngine`` drive ``forward_ragged``.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass, field
from typing import List, Optional

import torch
from torch import nn

from ..ops import elementwise as ew
from ..ops.gemm import linear_exact
from ..ops.hyper import gated_group_norm, hc_entry, hc_read, hc_step, xielu
from ..ops.linear_scan import delta_gates, linear_scan, short_conv, silu_rows_
from ..ops.multimap_attention import multimap_attention, qknorm_rope_store

MAPS = 2                          # attention maps per head: fixed by the design
UNIT_EPS = 1e-6                   # inside the root of the delta rule's unit norm: fixed by the design
MIXERS = ("attention", "lightning", "channel_delta")


@dataclass
class DuratarMixer:
    kind: str
    heads: int
    dim: int
    vdim: int
    kv_heads: int = 0                           # attention: key/value heads; channel_delta: q/k heads
    # attention
    diff: float = 0.0
    scale: float = 1.0
    window: int = 0
    keep_first: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    rot_scaling: Optional[dict] = None          # {"factor", "low", "high", "original"} or None
    kv_from: Optional[int] = None
    # lightning
    decay: Optional[List[float]] = None
    # channel_delta
    conv: int = 1


@dataclass
class DuratarLayerSpec:
    type: str
    mixer: DuratarMixer
    ff: int = 0                                 # 0: the layer has no feed-forward


@dataclass
class DuratarConfig:
    vocab_size: int
    hidden_size: int
    layers: List[DuratarLayerSpec]
    norm_eps: float
    streams: int = 1
    hyper: bool = False                         # the config names ``streams``: hyper-connection coefficients are tensors
    model_type: str = "duratar"
    raw: dict = field(default_factory=dict, repr=False)

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def to_dict(self) -> dict:
        return dict(self.raw)

    @classmethod
    def from_dict(cls, d: dict) -> "DuratarConfig":
        layers = []
        for i, L in enumerate(d["layers"]):
            kind, m = L["type"], L["mixer"]
            if kind not in MIXERS:
                raise ValueError(f"Duratar has no mixer {kind!r}")
            mx = DuratarMixer(kind=kind, heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]))
            if kind == "attention":
                rot, mask = m.get("rot") or {}, m.get("mask") or {}
                mx.kv_heads = int(m.get("kv_heads", m["heads"]))
                mx.diff, mx.scale = float(m["diff"]), float(m["scale"])
                mx.window, mx.keep_first = int(mask.get("size", 0)), int(mask.get("keep_first", 0))
                mx.rot_dims, mx.rot_base = int(rot.get("dims", 0)), float(rot.get("base", 10000.0))
                mx.rot_scaling = rot.get("scaling") or None
                kf = m.get("kv_from")
                if kf is not None:
                    kf = int(kf)
                    src = layers[kf].mixer if 0 <= kf < i else None
                    if src is None or src.kind != "attention" or src.kv_from is not None or \
                            (src.kv_heads, src.dim, src.vdim) != (mx.kv_heads, mx.dim, mx.vdim):
                        raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with its own keys of the same shape")
                mx.kv_from = kf
                if mx.heads % mx.kv_heads or mx.rot_dims % 2 or mx.rot_dims > mx.dim:
                    raise ValueError(f"layer {i}: bad attention sizes")
            elif kind == "lightning":
                mx.kv_heads = mx.heads
                mx.decay = [float(x) for x in m["decay"]]
                if len(mx.decay) != mx.heads:
                    raise ValueError(f"layer {i}: one decay per head")
            else:
                mx.kv_heads = int(m.get("kv_heads", m["heads"]))
                mx.conv = int(m.get("conv", 1))
                if mx.heads % mx.kv_heads or mx.conv < 1:
                    raise ValueError(f"layer {i}: bad channel_delta sizes")
            f = L.get("mlp")
            if f is not None and f.get("kind", "dense") != "dense":
                raise ValueError(f"unknown feed-forward kind {f['kind']!r}")
            layers.append(DuratarLayerSpec(kind, mx, int(f["ff"]) if f is not None else 0))
        return cls(vocab_size=int(d["vocab"]), hidden_size=int(d["width"]), layers=layers, norm_eps=float(d["norm"]["eps"]),
                   streams=int(d.get("streams", 1)), hyper="streams" in d, raw=d)


def _band_scaling(s: Optional[dict]) -> Optional[dict]:
    """The design's {factor, low, high, original} in the key names of ``ops.elementwise.rope_inv_freq``'s wavelength-band
    rule."""
    if not s:
        return None
    return {"rope_type": "llama3", "factor": float(s["factor"]), "low_freq_factor": float(s["low"]),
            "high_freq_factor": float(s["high"]), "original_max_position_embeddings": s["original"]}


def _pad8(n: int) -> int:
    return -(-n // 8) * 8


class DuratarLayer(nn.Module):
    def __init__(self, cfg: DuratarConfig, idx: int, dtype, device):
        super().__init__()
        spec = cfg.layers[idx]
        m, W, S = spec.mixer, cfg.hidden_size, cfg.streams
        self.spec, self.idx = spec, idx
        f32 = lambda *n, v=0.0: nn.Parameter(torch.full(n, v, dtype=torch.float32, device=device))       # noqa: E731
        wt = lambda *n: nn.Parameter(torch.zeros(*n, dtype=dtype, device=device))                        # noqa: E731
        subs = (1, 2) if spec.ff else (1,)
        for q in subs:
            setattr(self, f"norm{q}", f32(1, v=1.0))
            setattr(self, f"ls{q}", f32(W, v=1.0))
            setattr(self, f"hc{q}_in", f32(S, v=1.0))
            setattr(self, f"hc{q}_out", f32(S, v=1.0))
            setattr(self, f"hc{q}_mix", nn.Parameter(torch.eye(S, dtype=torch.float32, device=device)))
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        # projections that read the mixer's input are one weight; parts = (name, rows); rows are padded to a multiple of 8
        if m.kind == "attention":
            parts = [("q", H * MAPS * D)] + ([("k", G * MAPS * D), ("v", G * Dv)] if m.kv_from is None else [])
            self.q_norm = f32(D, v=1.0)
            if m.kv_from is None:
                self.k_norm = f32(D, v=1.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                setattr(self, n, f32(D))
        elif m.kind == "lightning":
            parts = [("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv)]
            self.mix_norm = f32(H * Dv, v=1.0)
            self.decay = nn.Parameter(torch.tensor(m.decay, dtype=torch.float32, device=device), requires_grad=False)
        else:
            parts = [("q", G * D), ("k", G * D), ("v", H * Dv), ("b", H)]
            self.conv_w = f32(2 * G * D + H * Dv, m.conv)
            self.A_log = f32(H)
            self.dt_bias = f32(H * D)
            self.mix_norm = f32(Dv, v=1.0)
        self.parts = {}
        lo = 0
        for n, r in parts:
            self.parts[n] = (lo, lo + r)
            lo += r
        self.in_proj = wt(_pad8(lo), W)
        self.o_proj = wt(W, H * Dv)
        if spec.ff:
            self.up_proj = wt(spec.ff, W)
            self.down_proj = wt(W, spec.ff)
            self.act = f32(2)
        self._lambda = None

    def make_low_rank(self, name: str, rank: int, rows: int, dtype, device) -> None:
        """The two factors of a low-rank projection ``<name>2 (<name>1 h)`` (channel_delta's decay and gate paths)."""
        W = self.in_proj.shape[1]
        setattr(self, name + "1", nn.Parameter(torch.zeros(rank, W, dtype=dtype, device=device)))
        setattr(self, name + "2", nn.Parameter(torch.zeros(rows, rank, dtype=dtype, device=device)))

    def diff_lambda(self) -> float:
        """lambda of the differential combination: a function of the weights only, formed once in float64."""
        if self._lambda is None:
            d = lambda a, b: float((a.double() * b.double()).sum())          # noqa: E731
            self._lambda = math.exp(d(self.lq1, self.lk1)) - math.exp(d(self.lq2, self.lk2)) + self.spec.mixer.diff
        return self._lambda

    # ------------------------------------------------------------------ mixers: h [T, W] -> fp32 [T, W]
    def attention(self, h, cos, sin, pos, slot, cache, src: int, eps: float, pieces, max_pos: int = 0):
        m = self.spec.mixer
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        own = m.kv_from is None
        proj = linear_exact(h, self.in_proj, out_dtype=torch.float32)
        q = qknorm_rope_store(proj, self.q_norm, self.k_norm if own else None, cos, sin, pos, slot,
                              cache.k[self.idx] if own else None, cache.v[self.idx] if own else None, cache.table,
                              H, G, MAPS, D, Dv, m.rot_dims, eps, h.dtype)
        ctx = multimap_attention(q, cache.k[src], cache.v[src], cache.table, pos, slot, H, G, MAPS, D, Dv, m.scale, m.window,
                                 m.keep_first, combine=True, lam=self.diff_lambda(), post=1.0 - m.diff, eps=eps, pieces=pieces,
                                 max_pos=max_pos)
        return linear_exact(ctx, self.o_proj, out_dtype=torch.float32)

    def lightning(self, h, pos, slot, cache, runs, n_runs, eps: float):
        m = self.spec.mixer
        H, D, Dv = m.heads, m.dim, m.vdim
        proj = linear_exact(h, self.in_proj, out_dtype=torch.float32)
        sl = lambda n: proj[:, self.parts[n][0]:self.parts[n][1]]             # noqa: E731
        silu_rows_(proj[:, :self.parts["v"][1]])                              # q | k | v are the leading columns
        o = linear_scan(sl("q"), sl("k"), sl("v"), cache.state[self.idx][0], pos, slot, runs, n_runs, H, H, D, Dv, "decay",
                        decay=self.decay)
        z = gated_group_norm(o, sl("g"), self.mix_norm, 1, eps, h.dtype)
        return linear_exact(z, self.o_proj, out_dtype=torch.float32)

    def channel_delta(self, h, pos, slot, cache, runs, n_runs, eps: float):
        m = self.spec.mixer
        H, G, D, Dv = m.heads, m.kv_heads, m.dim, m.vdim
        C = 2 * G * D + H * Dv
        proj = linear_exact(h, self.in_proj, out_dtype=torch.float32)
        a = linear_exact(linear_exact(h, self.a1), self.a2, out_dtype=torch.float32)
        gate = linear_exact(linear_exact(h, self.g1), self.g2, out_dtype=torch.float32)
        state, tail = cache.state[self.idx]
        qkv = short_conv(proj[:, :C], self.conv_w, tail, pos, slot, runs, n_runs, act=True)
        q, k, v = qkv[:, :G * D], qkv[:, G * D:2 * G * D], qkv[:, 2 * G * D:]
        b = proj[:, C:C + H]
        delta_gates(q, k, a, b, self.dt_bias, self.A_log, G, H, D, D ** -0.5, UNIT_EPS)
        o = linear_scan(q, k, v, state, pos, slot, runs, n_runs, H, G, D, Dv, "delta", g=a, beta=b)
        z = gated_group_norm(o, gate, self.mix_norm, H, eps, h.dtype)
        return linear_exact(z, self.o_proj, out_dtype=torch.float32)

    def feed_forward(self, h):
        return linear_exact(xielu(linear_exact(h, self.up_proj), self.act), self.down_proj, out_dtype=torch.float32)


class DuratarForCausalLM(nn.Module):
    """``forward_ragged`` is the serving step; ``forward(input_ids)`` runs whole sequences through the same step."""
    ragged = True                                   # served by inference.ragged.RaggedGenerator

    def __init__(self, cfg: DuratarConfig, dtype=torch.bfloat16, device=None, init_std: float = 0.02, low_ranks=None):
        super().__init__()
        self.config = cfg
        self.dtype_ = dtype
        W, V = cfg.hidden_size, cfg.vocab_size
        self.embed_tokens = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self.embed_norm = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device))
        self.layers = nn.ModuleList([DuratarLayer(cfg, i, dtype, device) for i in range(len(cfg.layers))])
        # ranks of channel_delta's low-rank paths come from the checkpoint's tensor shapes: {layer: (decay rank, gate rank)}
        for i, layer in enumerate(self.layers):
            m = layer.spec.mixer
            if m.kind == "channel_delta":
                ra, rg = (low_ranks or {}).get(i, (max(8, m.dim // 4), max(8, m.dim // 4)))
                layer.make_low_rank("a", ra, m.heads * m.dim, dtype, device)
                layer.make_low_rank("g", rg, m.heads * m.vdim, dtype, device)
        self.norm = nn.Parameter(torch.ones(1, dtype=torch.float32, device=device))
        self.lm_head = nn.Parameter(torch.empty(V, W, dtype=dtype, device=device).normal_(std=init_std))
        self._rope = {}

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.device

    def head_weight(self) -> torch.Tensor:
        return self.lm_head

    def kv_layout(self):
        """(key rows, key row size, value row size, value heads) per layer: an attention layer with keys of its own caches
        one key row per (kv head, map) and one value row per kv head; every other layer has no pool."""
        out = []
        for s in self.config.layers:
            m = s.mixer
            own = m.kind == "attention" and m.kv_from is None
            out.append((m.kv_heads * MAPS, m.dim, m.vdim, m.kv_heads) if own else (0, 0, 0, 0))
        return out

    def state_layout(self):
        """Per layer, the shapes of the fp32 tensors a sequence carries from token to token: the recurrent matrix per head,
        and for channel_delta the last ``conv - 1`` inputs of the short convolutions."""
        out = []
        for s in self.config.layers:
            m = s.mixer
            if m.kind == "lightning":
                out.append([(m.heads, m.dim, m.vdim)])
            elif m.kind == "channel_delta":
                out.append([(m.heads, m.dim, m.vdim), (m.conv - 1, 2 * m.kv_heads * m.dim + m.heads * m.vdim)])
            else:
                out.append([])
        return out

    def rope(self, li: int, device, need: int):
        a = self.config.layers[li].mixer
        key = (a.rot_dims, a.rot_base, json.dumps(a.rot_scaling, sort_keys=True), str(device))
        t = self._rope.get(key)
        if t is None or t[0].shape[0] < need:
            n = max(need, 4096)
            t = self._rope[key] = ew.rope_tables_partial(n, a.rot_dims, a.rot_base, device, _band_scaling(a.rot_scaling))
        return t

    def _read_coeffs(self, li: int):
        """(stream coefficients, norm weight) of what reads the streams after layer li - 1's last sublayer."""
        if li < len(self.layers):
            return self.layers[li].hc1_in, self.layers[li].norm1
        return None, self.norm

    @torch.no_grad()
    def forward_ragged(self, ids: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor, cache, want: Optional[torch.Tensor] = None,
                       max_pos: int = 0, pieces=None, layer_outputs: Optional[list] = None) -> torch.Tensor:
        """One serving step over a flat token list: ``ids`` long [T], ``pos`` / ``slot`` int32 [T] (position in its sequence
        and cache / state row of every token), ``cache`` a ``PagedKVCache`` whose table rows cover those positions and whose
        state rows belong to the same sequences. Returns fp32 logits of the rows ``want`` (long [n]; default all).
        ``pieces`` describes the runs of consecutive tokens (None: every token is a sequence of its own step, a decode
        batch). ``layer_outputs``: a list that receives the sum of the streams after every layer."""
        cfg = self.config
        dt = self.embed_tokens.dtype
        eps, S = cfg.norm_eps, cfg.streams
        dev = ids.device
        need = max(int(max_pos) + 1, cache.max_len)
        runs, n_runs = (pieces.runs, pieces.n_runs) if pieces is not None else (None, ids.shape[0])
        cin, g = self._read_coeffs(0)
        h, X = hc_entry(ew.embedding(ids, self.embed_tokens), self.embed_norm, S, cin, g, eps, dt)
        for li, layer in enumerate(self.layers):
            m = layer.spec.mixer
            if m.kind == "attention":
                if m.rot_dims:
                    cos, sin = self.rope(li, dev, need)
                else:
                    cos = sin = torch.zeros(1, 1, dtype=torch.float32, device=dev)
                y = layer.attention(h, cos, sin, pos, slot, cache, li if m.kv_from is None else m.kv_from, eps, pieces, max_pos)
            elif m.kind == "lightning":
                y = layer.lightning(h, pos, slot, cache, runs, n_runs, eps)
            else:
                y = layer.channel_delta(h, pos, slot, cache, runs, n_runs, eps)
            cin, g = self._read_coeffs(li + 1)
            last = li + 1 == len(self.layers)
            want_sum = layer_outputs is not None
            if layer.spec.ff:
                h, _ = hc_step(y, layer.ls1, X, layer.hc1_mix, layer.hc1_out, layer.hc2_in, layer.norm2, eps, dt)
                y = layer.feed_forward(h)
                h, xs = hc_step(y, layer.ls2, X, layer.hc2_mix, layer.hc2_out, cin, None if last else g, eps, dt, want_sum)
            else:
                h, xs = hc_step(y, layer.ls1, X, layer.hc1_mix, layer.hc1_out, cin, None if last else g, eps, dt, want_sum)
            if want_sum:
                layer_outputs.append(xs)
        if want is not None:
            X = X.index_select(0, want)
        h = hc_read(X.contiguous(), None, self.norm, eps, dt)
        return linear_exact(h, self.lm_head, out_dtype=torch.float32)

    @torch.no_grad()
    def forward(self, input_ids: torch.Tensor, labels=None, **_) -> dict:
        """Whole sequences [B, S] through the serving step with a throw-away cache: ``{"logits": [B, S, V]}`` (fp32)."""
        if labels is not None:
            raise NotImplementedError("Duratar is an inference model here: no loss / backward")
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
def _tensor_map(model: DuratarForCausalLM):
    """(checkpoint name, parameter, slice of its first dim or None, view shape of that slice or None, required) per tensor."""
    cfg = model.config
    out = [("embed", model.embed_tokens, None, None, True), ("embed.norm", model.embed_norm, None, (), True),
           ("final.norm", model.norm, None, (), True), ("head", model.lm_head, None, None, True)]
    for i, layer in enumerate(model.layers):
        p, m = f"l{i}.", layer.spec.mixer
        G, D = m.kv_heads, m.dim
        for q in (1, 2) if layer.spec.ff else (1,):
            out.append((f"{p}norm{q}", getattr(layer, f"norm{q}"), None, (), True))
            out.append((f"{p}ls{q}", getattr(layer, f"ls{q}"), None, None, True))
            if cfg.hyper:
                out += [(f"{p}hc{q}.{n}", getattr(layer, f"hc{q}_{n}"), None, None, True) for n in ("in", "out", "mix")]
        for n, (lo, hi) in layer.parts.items():
            out.append((f"{p}mix.{n}", layer.in_proj, slice(lo, hi), None, True))
        out.append((p + "mix.o", layer.o_proj, None, None, True))
        if m.kind == "attention":
            out.append((p + "mix.q.norm", layer.q_norm, None, None, True))
            if m.kv_from is None:
                out.append((p + "mix.k.norm", layer.k_norm, None, None, True))
            out += [(f"{p}mix.{n}", getattr(layer, n), None, None, True) for n in ("lq1", "lk1", "lq2", "lk2")]
        elif m.kind == "lightning":
            out.append((p + "mix.norm", layer.mix_norm, None, None, True))
        else:
            c = 0
            for n, r in (("q", G * D), ("k", G * D), ("v", m.heads * m.vdim)):
                out.append((f"{p}mix.{n}.conv", layer.conv_w, slice(c, c + r), None, True))
                c += r
            out += [(p + "mix.A_log", layer.A_log, None, None, True), (p + "mix.dt_bias", layer.dt_bias, None, None, True),
                    (p + "mix.norm", layer.mix_norm, None, None, True)]
            out += [(f"{p}mix.{n}", getattr(layer, n), None, None, True) for n in ("a1", "a2", "g1", "g2")]
        if layer.spec.ff:
            out += [(p + "mlp.up", layer.up_proj, None, None, True), (p + "mlp.down", layer.down_proj, None, None, True),
                    (p + "mlp.act", layer.act, None, None, True)]
    return out


@torch.no_grad()
def load_duratar_weights(model: DuratarForCausalLM, path: str) -> None:
    from ..io.safetensors import safe_open
    with safe_open(os.path.join(path, "model.safetensors")) as f:
        names = set(f.keys())
        used = set()
        for name, param, sl, shape, _ in _tensor_map(model):
            used.add(name)
            dst = param if sl is None else param[sl]
            t = f.get_tensor(name).to(param.device, param.dtype)
            dst.copy_(t.reshape(dst.shape))
        missing = names - used
        if missing:
            raise ValueError(f"checkpoint tensors the model has no place for: {sorted(missing)[:8]}")
    for layer in model.layers:
        layer._lambda = None


def _low_ranks(path: str, cfg: DuratarConfig) -> dict:
    from ..io.safetensors import safe_open
    out = {}
    with safe_open(os.path.join(path, "model.safetensors")) as f:
        for i, s in enumerate(cfg.layers):
            if s.mixer.kind == "channel_delta":
                out[i] = (int(f.info(f"l{i}.mix.a1")[1][0]), int(f.info(f"l{i}.mix.g1")[1][0]))
    return out


def duratar_from_pretrained(path: str, dtype=torch.bfloat16, device=None) -> DuratarForCausalLM:
    with open(os.path.join(path, "config.json")) as f:
        cfg = DuratarConfig.from_dict(json.load(f))
    model = DuratarForCausalLM(cfg, dtype=dtype, device=device, low_ranks=_low_ranks(path, cfg))
    load_duratar_weights(model, path)
    model.name_or_path = path
    return model.eval()


@torch.no_grad()
def duratar_state_dict(model: DuratarForCausalLM) -> dict:
    """Tensors under the checkpoint's names (the inverse of ``load_duratar_weights``)."""
    out = {}
    for name, param, sl, shape, _ in _tensor_map(model):
        t = param if sl is None else param[sl]
        out[name] = (t.reshape(shape) if shape is not None else t).detach().contiguous()
    return out
