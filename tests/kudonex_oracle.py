"""A plain float64 statement of the Kudonex equations: one function per mechanism, whole sequences, token by token where
there is a state. It shares nothing with the package (no ops, no cache, no batching) and is what the tests compare the
serving step against.

Weights are a dict name -> tensor under the checkpoint's names (``l<i>.mix.q`` ...); ``cfg`` is the parsed config.json.
"""
import math

import torch

F64 = torch.float64
DEN_EPS = 1e-6                       # added to the mLSTM read-out's denominator


def sinusoid(n, width):
    """[n, width]: column 2i = sin(p w_i), column 2i + 1 = cos(p w_i), w_i = 10000^(-2i / width)."""
    out = torch.zeros(n, width, dtype=F64)
    for p in range(n):
        for c in range(width):
            ang = p * 10000.0 ** (-(2 * (c // 2)) / width)
            out[p, c] = math.sin(ang) if c % 2 == 0 else math.cos(ang)
    return out


def embed(tokens, table, scale):
    return table.to(F64)[torch.as_tensor(tokens)] * scale + sinusoid(len(tokens), table.shape[1])


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w.to(F64)


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv(x, w, bias=None):
    """x [n, C], w [C, taps]: y_t = sum_j w[:, j] x_(t - taps + 1 + j), nothing before t = 0."""
    n, C = x.shape
    taps = w.shape[1]
    y = torch.zeros(n, C, dtype=F64)
    for t in range(n):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j].to(F64) * x[s]
        if bias is not None:
            y[t] += bias.to(F64)
    return y


def silu(z):
    return z * torch.sigmoid(z)


def mlstm(h, P, m, eps):
    """h [n, W] -> [n, W]. P: the layer's mixer tensors by short name."""
    H, D, Dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    n = h.shape[0]
    lin = lambda name: h @ P[name].to(F64).t()                                  # noqa: E731
    q = (lin("q") * D ** -0.5).view(n, H, D)
    k = lin("k").view(n, H, D)
    v = lin("v").view(n, H, Dv)
    gi = cap * torch.tanh((lin("i") + P["i.b"].to(F64)) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((lin("f") + P["f.b"].to(F64)) / cap))
    out = torch.zeros(n, H, Dv, dtype=F64)
    for a in range(H):
        S = torch.zeros(D, Dv, dtype=F64)
        nv = torch.zeros(D, dtype=F64)
        mx = 0.0
        for t in range(n):
            new = max(float(gf[t, a]) + mx, float(gi[t, a]))
            keep, put = math.exp(float(gf[t, a]) + mx - new), math.exp(float(gi[t, a]) - new)
            S = keep * S + put * torch.outer(k[t, a], v[t, a])
            nv = keep * nv + put * k[t, a]
            mx = new
            den = max(abs(float(nv @ q[t, a])), math.exp(-mx)) + DEN_EPS
            out[t, a] = (S.t() @ q[t, a]) / den
    y = rms(out, eps).reshape(n, H * Dv) * P["norm"].to(F64) * torch.sigmoid(lin("g"))
    return y @ P["o"].to(F64).t()


def mamba2(h, P, m, eps):
    H, Dv, N, G, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * Dv
    n = h.shape[0]
    u = h @ P["in"].to(F64).t()
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, P["conv"], P["conv.b"]))
    x = xbc[:, :inner].view(n, H, Dv)
    B = xbc[:, inner:inner + G * N].view(n, G, N)
    C = xbc[:, inner + G * N:].view(n, G, N)
    dt = torch.nn.functional.softplus(dt + P["dt_bias"].to(F64), threshold=1e9)
    rate = torch.exp(P["A_log"].to(F64))
    y = torch.zeros(n, H, Dv, dtype=F64)
    for a in range(H):
        g = a // (H // G)
        S = torch.zeros(N, Dv, dtype=F64)
        for t in range(n):
            S = math.exp(-float(rate[a]) * float(dt[t, a])) * S + float(dt[t, a]) * torch.outer(B[t, g], x[t, a])
            y[t, a] = S.t() @ C[t, g] + float(P["D"][a]) * x[t, a]
    y = y.reshape(n, inner) * silu(z)
    y = rms(y.view(n, NG, inner // NG), eps).reshape(n, inner) * P["norm"].to(F64)
    return y @ P["o"].to(F64).t()


def attention(h, P, m):
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    win, scale = int(m["mask"]["size"]), float(m["scale"])
    n = h.shape[0]
    q = (h @ P["q"].to(F64).t()).view(n, H, D)
    k = (h @ P["k"].to(F64).t()).view(n, G, D)
    r1, r2, T = P["r1"].to(F64), P["r2"].to(F64), P["talk"].to(F64)
    ctx = torch.zeros(n, H, D, dtype=F64)
    for i in range(n):
        lo = max(0, i - win + 1)
        raw = torch.zeros(H, i + 1 - lo, dtype=F64)
        dist = torch.arange(i - lo, -1, -1, dtype=F64)                            # i - j for j = lo .. i
        for a in range(H):
            raw[a] = (k[lo:i + 1, a // (H // G)] @ q[i, a]) * scale - r1[a] * torch.log1p(r2[a] * dist)
        p = torch.softmax(T @ raw, -1)
        for a in range(H):
            ctx[i, a] = p[a] @ k[lo:i + 1, a // (H // G)]
    y = ctx.reshape(n, H * D) * torch.sigmoid(h @ P["g"].to(F64).t())
    return y @ P["o"].to(F64).t()


def expert(h, P, pre):
    return (silu(h @ P[pre + "gate"].to(F64).t()) * (h @ P[pre + "up"].to(F64).t())) @ P[pre + "down"].to(F64).t()


def route(h, P, f):
    """Chosen experts and their weights per token: (list of lists, list of lists)."""
    r = f["router"]
    E, top, groups, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = torch.softmax(h @ P["router"].to(F64).t(), -1)
    pick = s + P["correction"].to(F64)
    per = E // groups
    chosen, weights = [], []
    for t in range(h.shape[0]):
        best = sorted(range(groups), key=lambda g: -float(pick[t, g * per:(g + 1) * per].max()))[:keep]
        allowed = [e for e in range(E) if e // per in best]
        ex = sorted(allowed, key=lambda e: -float(pick[t, e]))[:top]
        chosen.append(ex)
        weights.append([float(s[t, e]) for e in ex])
    return chosen, weights


def moe(h, P, f):
    chosen, weights = route(h, P, f)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(chosen[t], weights[t]):
            out[t] += w * expert(h[t:t + 1], P, f"e{e}.")[0]
    return out + expert(h, P, "shared.") if "shared.gate" in P else out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg, weights, tokens):
    """(logits [n, vocab], [residual stream after every layer])."""
    eps = float(cfg["norm"]["eps"])
    x = embed(tokens, weights["embed"], float(cfg["embedding"]["scale"]))
    streams = []
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, weights[p + "norm1"], eps)
        h = h + causal_conv(h, weights[p + "canon1"])
        P = sub(weights, p + "mix.")
        kind = L["type"]
        y = mlstm(h, P, L["mixer"], eps) if kind == "mlstm" else mamba2(h, P, L["mixer"], eps) if kind == "mamba2" \
            else attention(h, P, L["mixer"])
        x = x + layer_norm(y, weights[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            h = layer_norm(x, weights[p + "norm2"], eps)
            x = x + layer_norm(moe(h, sub(weights, p + "mlp."), L["mlp"]), weights[p + "norm2b"], eps)
        streams.append(x.clone())
    return layer_norm(x, weights["final.norm"], eps) @ weights["embed"].to(F64).t(), streams


# ------------------------------------------------------------------------------------------------------------------
# small random models for the tests
# ------------------------------------------------------------------------------------------------------------------
def moe_spec(experts, top, ff, groups=1, keep=1, shared=0):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}},
            "shared": {"ff": shared}}


def mlstm_layer(heads, dim, vdim, cap=15.0, mlp=None):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def mamba2_layer(heads, vdim, state, groups=1, norm_groups=1, conv=4, mlp=None):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups,
                                        "conv": conv}, "mlp": mlp}


def attention_layer(heads, kv_heads, dim, window, scale=None, mlp=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
                                           "scale": dim ** -0.5 if scale is None else scale}, "mlp": mlp}


def make_config(width, vocab, layers, taps=4, embed_scale=3.0, eps=1e-5):
    return {"architecture": "Kudonex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
            "canon": {"taps": taps}, "layers": layers}


def random_weights(cfg, seed=0):
    """bf16 tensors under the checkpoint's names; scales chosen so that every mechanism matters (gates away from saturation,
    distance penalties and head mixing of the order of the scores, corrections that change which experts are chosen)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}
    rnd = lambda *s, std=1.0: torch.randn(*s, generator=g) * std                       # noqa: E731
    lin = lambda o, i, gain=1.0: rnd(o, i, std=gain * i ** -0.5)                        # noqa: E731
    gain = lambda n: 1.0 + rnd(n, std=0.2)                                             # noqa: E731
    out["embed"] = rnd(cfg["vocab"], W, std=0.5)
    out["final.norm"] = gain(W)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b"):
            out[p + n] = gain(W)
        out[p + "canon1"] = rnd(W, cfg["canon"]["taps"], std=0.4)
        H, Dv = m["heads"], m["vdim"]
        if L["type"] == "mlstm":
            D = m["dim"]
            out.update({p + "mix.q": lin(H * D, W, 2.0), p + "mix.k": lin(H * D, W, 2.0), p + "mix.v": lin(H * Dv, W), p + "mix.g": lin(H * Dv, W),
                        p + "mix.i": lin(H, W, 3.0), p + "mix.f": lin(H, W, 3.0), p + "mix.i.b": rnd(H), p + "mix.f.b": rnd(H) + 2.0,
                        p + "mix.norm": gain(H * Dv), p + "mix.o": lin(W, H * Dv)})
        elif L["type"] == "mamba2":
            N, G = m["state"], m["groups"]
            C = H * Dv + 2 * G * N
            out.update({p + "mix.in": lin(2 * H * Dv + 2 * G * N + H, W, 1.5), p + "mix.conv": rnd(C, m["conv"], std=0.5),
                        p + "mix.conv.b": rnd(C, std=0.3), p + "mix.dt_bias": rnd(H) - 1.0, p + "mix.A_log": rnd(H, std=0.5),
                        p + "mix.D": rnd(H), p + "mix.norm": gain(H * Dv), p + "mix.o": lin(W, H * Dv)})
        else:
            D, G = m["dim"], m["kv_heads"]
            out.update({p + "mix.q": lin(H * D, W, 2.0), p + "mix.k": lin(G * D, W, 2.0), p + "mix.g": lin(H * D, W), p + "mix.o": lin(W, H * D),
                        p + "mix.r1": torch.rand(H, generator=g) * 1.5, p + "mix.r2": torch.rand(H, generator=g) * 2.0 + 0.05,
                        p + "mix.talk": torch.eye(H) + rnd(H, H, std=0.3)})
        f = L.get("mlp")
        if f is None:
            continue
        for n in ("norm2", "norm2b"):
            out[p + n] = gain(W)
        E, F, Fs = f["router"]["experts"], f["expert"]["ff"], f["shared"]["ff"]
        # a peaked router: the experts that carry weight win by a margin that 16-bit rounding of h does not close, and
        # the ones decided by a hair carry little; beside a shared expert the routed ones are the smaller part of the sum, so
        # that a choice that falls the other way in 16 bits does not swamp the recurrent states after it
        out[p + "mlp.router"] = lin(E, W, 12.0)
        out[p + "mlp.correction"] = rnd(E, std=0.15) - 0.1
        for e in range(E):
            out.update({f"{p}mlp.e{e}.gate": lin(F, W), f"{p}mlp.e{e}.up": lin(F, W), f"{p}mlp.e{e}.down": lin(W, F, 0.3 if Fs else 1.0)})
        if Fs:
            out.update({p + "mlp.shared.gate": lin(Fs, W), p + "mlp.shared.up": lin(Fs, W), p + "mlp.shared.down": lin(W, Fs)})
    return {k: v.to(torch.bfloat16).contiguous() for k, v in out.items()}


def greedy(cfg, weights, prompt, new):
    toks = list(prompt)
    for _ in range(new):
        toks.append(int(forward(cfg, weights, toks)[0][-1].argmax()))
    return toks
