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


def attention(m, w, pre, h, eps, shared=None):
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ f64(w[pre + "q"]).T).view(T, H, 2, D)
    q = rms(q, eps) * f64(w[pre + "q.norm"])
    fr = rope_freqs(m["rot"]["dims"], m["rot"]["base"], m["rot"].get("scaling"))
    q = torch.stack([rotate_half(q[t], t, fr) for t in range(T)])
    k, v = shared if shared is not None else attention_keys(m, w, pre, h, eps)
    lam = (math.exp(float((f64(w[pre + "lq1"]) * f64(w[pre + "lk1"])).sum()))
           - math.exp(float((f64(w[pre + "lq2"]) * f64(w[pre + "lk2"])).sum())) + m["diff"])
    size, keep = m["mask"]["size"], m["mask"]["keep_first"]
    out = torch.zeros(T, H, Dv, dtype=F64)
    rep = H // G
    for i in range(T):
        js = [j for j in range(i + 1) if visible(i, j, size, keep)]
        kk = k[js].repeat_interleave(rep, 1)                       # [n, H, 2, D]
        vv = v[js].repeat_interleave(rep, 1)                       # [n, H, Dv]
        sc = torch.einsum("hmd,nhmd->hmn", q[i], kk) * m["scale"]
        a = torch.einsum("hmn,nhe->hme", torch.softmax(sc, -1), vv)
        o = a[:, 0] - lam * a[:, 1]
        out[i] = rms(o, eps) * (1 - m["diff"])
    return out.reshape(T, H * Dv) @ f64(w[pre + "o"]).T, (k, v)


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
