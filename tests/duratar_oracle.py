"""Slow float64 statement of the Duratar equations, one function per mechanism, token by token where a mechanism has a
state. Shares no code with the package: the tests compare the package's CPU path and CUDA kernels against it.

``cfg`` is the design's config.json as a dict, ``w`` a dict name -> tensor (any float dtype; read as float64).
"""
import math

import torch

F64 = torch.float64


def f64(t):
    return t.detach().to("cpu", F64)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def softplus(z):
    z = torch.as_tensor(z, dtype=F64)
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def silu(z):
    return z * torch.sigmoid(z)


def xielu(z, p, q):
    """p, q: the two raw numbers of the activation."""
    ap, aq = softplus(p), 0.5 + softplus(q)
    neg = aq * (torch.expm1(torch.clamp(z, max=0)) - z) + 0.5 * z
    return torch.where(z > 0, ap * z * z + 0.5 * z, neg)


def rope_freqs(dims, base, scaling):
    """One frequency per rotated pair; ``scaling`` {factor, low, high, original} rescales by wavelength bands."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling:
            fac, lo, hi, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            lam = 2 * math.pi / f
            if lam < orig / hi:
                pass
            elif lam > orig / lo:
                f = f / fac
            else:
                s = (orig / lam - lo) / (hi - lo)
                f = (1 - s) * f / fac + s * f
        out.append(f)
    return out


def rotate_half(x, p, freqs):
    """x [..., D] at position p: dims i and i + n (n = len(freqs)) form pair i; dims >= 2 n pass."""
    n = len(freqs)
    y = x.clone()
    for i, f in enumerate(freqs):
        a = p * f
        u, v = x[..., i], x[..., i + n]
        y[..., i] = u * math.cos(a) - v * math.sin(a)
        y[..., i + n] = v * math.cos(a) + u * math.sin(a)
    return y


def visible(i, j, size, keep):
    return j <= i and (i - j < size or j < keep)


# ----------------------------------------------------------------------------------------------------------------------
# mixers: each takes h [T, W] (one sequence from position 0) and returns (output [T, W], what a later layer may share)
# ----------------------------------------------------------------------------------------------------------------------
def attention_keys(m, w, pre, h, eps):
    """Normed, rotated keys [T, G, 2, D] and values [T, G, Dv] of one attention layer."""
    T = h.shape[0]
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ f64(w[pre + "k"]).T).view(T, G, 2, D)
    v = (h @ f64(w[pre + "v"]).T).view(T, G, Dv)
    k = rms(k, eps) * f64(w[pre + "k.norm"])
    fr = rope_freqs(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    k = torch.stack([rotate_half(k[t], t, fr) for t in range(T)])
    return k, v


def attend(q, k, v, scale, size, keep, lam, diff, eps):
    """q [T, H, 2, D], k [T, G, 2, D], v [T, G, Dv] of one sequence from position 0 -> [T, H, Dv]: two softmax maps per head
    over the visible keys, combined as a_1 - lam a_2, divided by the root mean square over Dv, times (1 - diff)."""
    T, H = q.shape[:2]
    G, Dv = v.shape[1:]
    rep = H // G
    out = torch.zeros(T, H, Dv, dtype=F64)
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep)]
        kk = k[js].repeat_interleave(rep, 1)                       # [n, H, 2, D]
        vv = v[js].repeat_interleave(rep, 1)                       # [n, H, Dv]
        sc = torch.einsum("hmd,nhmd->hmn", q[i], kk) * scale
        a = torch.einsum("hmn,nhe->hme", torch.softmax(sc, -1), vv)
        out[i] = rms(a[:, 0] - lam * a[:, 1], eps) * (1 - diff)
    return out


def diff_lambda(m, w, pre):
    return (math.exp(float((f64(w[pre + "lq1"]) * f64(w[pre + "lk1"])).sum()))
            - math.exp(float((f64(w[pre + "lq2"]) * f64(w[pre + "lk2"])).sum())) + m["diff"])


def attention(m, w, pre, h, eps, shared=None):
    T = h.shape[0]
    H, D = m["heads"], m["dim"]
    q = (h @ f64(w[pre + "q"]).T).view(T, H, 2, D)
    q = rms(q, eps) * f64(w[pre + "q.norm"])
    fr = rope_freqs(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = torch.stack([rotate_half(q[t], t, fr) for t in range(T)])
    k, v = shared if shared is not None else attention_keys(m, w, pre, h, eps)
    size = m["mask"]["size"] if m["mask"].get("size") else 1 << 60
    out = attend(q, k, v, m["scale"], size, m["mask"].get("keep_first", 0), diff_lambda(m, w, pre), m["diff"], eps)
    return out.reshape(T, -1) @ f64(w[pre + "o"]).T, (k, v)


def lightning(m, w, pre, h, eps):
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ f64(w[pre + "q"]).T).view(T, H, D)
    k = silu(h @ f64(w[pre + "k"]).T).view(T, H, D)
    v = silu(h @ f64(w[pre + "v"]).T).view(T, H, Dv)
    S = torch.zeros(H, D, Dv, dtype=F64)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            S[hh] = m["decay"][hh] * S[hh] + torch.outer(k[t, hh], v[t, hh])
            o[t, hh] = S[hh].T @ q[t, hh]
    y = rms(o.reshape(T, H * Dv), eps) * f64(w[pre + "norm"]) * torch.sigmoid(h @ f64(w[pre + "g"]).T)
    return y @ f64(w[pre + "o"]).T, None


def short_conv(x, cw):
    """x [T, C], cw [C, taps] (last column weighs the current token), zeros before the start."""
    T, C = x.shape
    taps = cw.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                y[t] += cw[:, j] * x[s]
    return y


def channel_delta(m, w, pre, h, eps):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ f64(w[pre + "q"]).T, f64(w[pre + "q.conv"]))).view(T, G, D)
    k = silu(short_conv(h @ f64(w[pre + "k"]).T, f64(w[pre + "k.conv"]))).view(T, G, D)
    v = silu(short_conv(h @ f64(w[pre + "v"]).T, f64(w[pre + "v.conv"]))).view(T, H, Dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * D ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ f64(w[pre + "b"]).T)
    a = (h @ f64(w[pre + "a1"]).T) @ f64(w[pre + "a2"]).T + f64(w[pre + "dt_bias"])
    g = torch.exp(-torch.exp(f64(w[pre + "A_log"]))[None, :, None] * softplus(a).view(T, H, D))
    S = torch.zeros(H, D, Dv, dtype=F64)
    o = torch.zeros(T, H, Dv, dtype=F64)
    for t in range(T):
        for hh in range(H):
            kv = hh // (H // G)
            S[hh] = g[t, hh][:, None] * S[hh]
            u = beta[t, hh] * (v[t, hh] - S[hh].T @ k[t, kv])
            S[hh] = S[hh] + torch.outer(k[t, kv], u)
            o[t, hh] = S[hh].T @ q[t, kv]
    gate = torch.sigmoid((h @ f64(w[pre + "g1"]).T) @ f64(w[pre + "g2"]).T).view(T, H, Dv)
    y = rms(o, eps) * f64(w[pre + "norm"]) * gate
    return y.reshape(T, H * Dv) @ f64(w[pre + "o"]).T, None


def feed_forward(f, w, pre, h):
    assert f["kind"] == "dense"
    act = f64(w[pre + "act"])
    return xielu(h @ f64(w[pre + "up"]).T, act[0], act[1]) @ f64(w[pre + "down"]).T


# ----------------------------------------------------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------------------------------------------------
def scalar_norm(x, g, eps):
    return rms(x, eps) * float(g)


def forward(cfg, w, tokens, layer_outputs=None):
    """Logits [T, vocab] (float64) of one sequence; ``layer_outputs`` receives the sum of the streams after every layer."""
    eps = cfg["norm"]["eps"]
    S = int(cfg.get("streams", 1))
    hyper = "streams" in cfg
    x0 = scalar_norm(f64(w["embed"])[torch.as_tensor(tokens)], w["embed.norm"], eps)
    xs = [x0.clone() for _ in range(S)]
    shared = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        subs = [(1, "mixer")] + ([(2, "ff")] if L.get("mlp") is not None else [])
        for qn, kind in subs:
            if hyper:
                cin, cout, cmix = (f64(w[f"{p}hc{qn}.{n}"]) for n in ("in", "out", "mix"))
                u = sum(cin[s] * xs[s] for s in range(S))
            else:
                u = xs[0]
            hn = scalar_norm(u, w[f"{p}norm{qn}"], eps)
            if kind == "ff":
                y = feed_forward(L["mlp"], w, p + "mlp.", hn)
            else:
                m = L["mixer"]
                if L["type"] == "attention":
                    src = shared[m["kv_from"]] if m.get("kv_from") is not None else None
                    y, shared[i] = attention(m, w, p + "mix.", hn, eps, src)
                elif L["type"] == "lightning":
                    y, _ = lightning(m, w, p + "mix.", hn, eps)
                elif L["type"] == "channel_delta":
                    y, _ = channel_delta(m, w, p + "mix.", hn, eps)
                else:
                    raise ValueError(L["type"])
            y = y * f64(w[f"{p}ls{qn}"])
            if hyper:
                xs = [sum(cmix[s, t] * xs[s] for s in range(S)) + cout[t] * y for t in range(S)]
            else:
                xs = [xs[0] + y]
        if layer_outputs is not None:
            layer_outputs.append(sum(xs))
    x = sum(xs)
    return scalar_norm(x, w["final.norm"], eps) @ f64(w["head"]).T


def greedy(cfg, w, prompt, new):
    toks = list(prompt)
    for _ in range(new):
        toks.append(int(forward(cfg, w, toks)[-1].argmax()))
    return toks


# ----------------------------------------------------------------------------------------------------------------------
# small configurations and random weights for the tests
# ----------------------------------------------------------------------------------------------------------------------
def attention_layer(heads, kv_heads, dim, vdim, size, keep, rot_dims, base=10000.0, scaling=None, diff=0.3, scale=None, kv_from=None,
                    ff=0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff, "scale": scale if scale is not None else 0.6,
         "mask": {"size": size, "keep_first": keep}, "rot": {"base": base, "dims": rot_dims}}
    if scaling:
        m["rot"]["scaling"] = scaling
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def lightning_layer(heads, dim, vdim, decay, ff=0):
    return {"type": "lightning", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def delta_layer(heads, kv_heads, dim, vdim, conv, ff=0):
    return {"type": "channel_delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_config(width, vocab, layers, streams=2, eps=1e-5):
    cfg = {"architecture": "Duratar", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def random_weights(cfg, seed=0, ranks=(12, 8), dtype=torch.bfloat16):
    """Weights under the checkpoint's names, rounded to ``dtype`` (the oracle and the package read the same numbers)."""
    g = torch.Generator().manual_seed(seed)
    W, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams", 1)
    w = {}
    rn = lambda *shape, std=1.0, mean=0.0: (torch.randn(tuple(shape), generator=g) * std + mean)      # noqa: E731
    lin = lambda o, i, gain=1.0: rn(o, i, std=gain * i ** -0.5)                                  # noqa: E731
    w["embed"] = rn(V, W)
    w["embed.norm"] = rn(std=0.1, mean=1.2)
    w["final.norm"] = rn(std=0.1, mean=0.9)
    w["head"] = lin(V, W)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for q in (1, 2) if L.get("mlp") else (1,):
            w[f"{p}norm{q}"] = rn(std=0.2, mean=1.0)
            w[f"{p}ls{q}"] = rn(W, std=0.3, mean=0.8)
            if "streams" in cfg:
                w[f"{p}hc{q}.in"] = rn(S, std=0.4, mean=0.7)
                w[f"{p}hc{q}.out"] = rn(S, std=0.4, mean=0.8)
                w[f"{p}hc{q}.mix"] = torch.eye(S) * 0.9 + rn(S, S, std=0.25)
        H, D, Dv = m["heads"], m["dim"], m["vdim"]
        x = p + "mix."
        if L["type"] == "attention":
            G = m["kv_heads"]
            w[x + "q"] = lin(H * 2 * D, W)
            w[x + "q.norm"] = rn(D, std=0.3, mean=1.0)
            if m.get("kv_from") is None:
                w[x + "k"] = lin(G * 2 * D, W)
                w[x + "v"] = lin(G * Dv, W)
                w[x + "k.norm"] = rn(D, std=0.3, mean=1.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                w[x + n] = rn(D, std=0.25)
        elif L["type"] == "lightning":
            for n, r in (("q", H * D), ("k", H * D), ("v", H * Dv), ("g", H * Dv)):
                w[x + n] = lin(r, W, 1.5)
            w[x + "norm"] = rn(H * Dv, std=0.3, mean=1.0)
        else:
            G = m["kv_heads"]
            for n, r in (("q", G * D), ("k", G * D), ("v", H * Dv)):
                w[x + n] = lin(r, W, 1.5)
                w[x + n + ".conv"] = rn(r, m["conv"], std=0.6)
            w[x + "b"] = lin(H, W, 2.0)
            w[x + "A_log"] = rn(H, std=0.7)
            w[x + "dt_bias"] = rn(H * D, std=1.0)
            w[x + "norm"] = rn(Dv, std=0.3, mean=1.0)
            w[x + "a1"], w[x + "a2"] = lin(ranks[0], W), lin(H * D, ranks[0], 2.0)
            w[x + "g1"], w[x + "g2"] = lin(ranks[1], W), lin(H * Dv, ranks[1], 2.0)
        w[x + "o"] = lin(W, H * Dv)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            w[p + "mlp.up"], w[p + "mlp.down"] = lin(F, W), lin(W, F)
            w[p + "mlp.act"] = rn(2, std=0.7)
    return {k: v.to(dtype) for k, v in w.items()}
