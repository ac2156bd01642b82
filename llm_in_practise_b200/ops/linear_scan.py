"""Recurrent mixers of the ragged serving step (``csrc/linear_scan.cu``): short causal convolutions with a carried tail and
linear-attention state scans, all in fp32.

A step is a flat token list; token t sits at position ``pos[t]`` of the sequence whose state lives in row ``slot[t]`` of
the per-layer state tensors (``inference.generate.PagedKVCache.state``). The tokens of one sequence are consecutive: a
*run*. ``runs`` int32 [n, 4] = (first row, rows, position of the first row, state row); ``None`` means every token is its
own run (a decode batch, whose pos / slot are read on the device so that the step can be replayed from a CUDA graph). A
run that starts at position 0 starts from a zero state, so state rows are reused without clearing.

    silu_rows_     x <- silu(x) on a column slice of fp32 rows
    short_conv     y[t, c] = act(sum_j w[c, j] x[t - (taps - 1) + j, c]); the tail [rows, taps - 1, C] holds the last inputs
    delta_gates    unit q / k per head, decays exp(-exp(A_log) softplus(a + bias)), beta = sigmoid(b), in place
    linear_scan    mode "decay":  S <- decay_h S + k v^T;                                  o = S^T q
                   mode "delta":  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T;    o = S^T q
                   mode "gated":  S <- a_t S + b_t k v^T (one a, b per token and head);    o = S^T q
    mlstm_gates    capped log gates of an mLSTM and their running maximum -> (a, b, exp(-m)) for the gated scan
    ssm_gates      dt = softplus(x + bias), a = exp(-exp(A_log) dt), b = dt: the step sizes of a selective state space
    scan_readout   normaliser division / skip term / silu gate, RMS norm over column groups, weight, sigmoid gate

The reference has no recurrent mixers; these sit beside the attention ops of the same step (``ops.paged_attention``).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from . import _native as nv

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _run_list(runs, pos, slot):
    if runs is not None:
        return [tuple(r) for r in runs.tolist()]
    return [(t, 1, p, s) for t, (p, s) in enumerate(zip(pos.tolist(), slot.tolist()))]


def short_conv(x: torch.Tensor, w: torch.Tensor, tail: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
               runs: Optional[torch.Tensor], n_runs: int, act: bool = True, bias: Optional[torch.Tensor] = None,
               residual: bool = False, out_dtype: torch.dtype = torch.float32) -> torch.Tensor:
    """``x`` fp32 [T, C] (rows may be strided) -> y [T, C] in ``out_dtype`` (fp32 / bf16); ``w`` fp32 [C, taps] (last column
    weighs the current token), ``bias`` fp32 [C] or None; ``tail`` fp32 [rows, taps - 1, C] is read for the inputs before each
    run and then advanced over the run. ``residual``: y = x + act(conv(x) + bias)."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.empty(T, C, dtype=out_dtype, device=x.device)
    if nv.use_native(x):
        if x.dtype != torch.float32 or x.stride(1) != 1:
            raise ValueError("short_conv: fp32 rows with a contiguous last dim")
        fn = nv.proto("b200_short_conv_ex", [vp, i64, vp, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(x), x.stride(0), nv.ptr(w), nv.ptr(bias), nv.ptr(tail), nv.ptr(pos), nv.ptr(slot), nv.ptr(y), y.stride(0),
                    T, C, taps, int(act), int(residual), nv.dtype_code(out_dtype), nv.stream()), "short_conv")
        fn = nv.proto("b200_short_conv_tail", [vp, i64, vp, vp, vp, vp, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(x), x.stride(0), nv.ptr(tail), nv.ptr(runs), nv.ptr(pos), nv.ptr(slot), n_runs if runs is not None else T,
                    C, taps, nv.stream()), "short_conv_tail")
        nv.count_launch(2)
        return y
    L = taps - 1
    for first, n, p0, s in _run_list(runs, pos, slot):
        old = tail[s] if p0 > 0 else torch.zeros(L, C, dtype=torch.float32, device=x.device)
        ext = torch.cat([old, x[first:first + n].float()], 0)                 # inputs at positions p0 - L .. p0 + n - 1
        acc = torch.zeros(n, C, dtype=torch.float32, device=x.device)
        if bias is not None:
            acc += bias.float()
        for j in range(taps):
            acc += w[:, j].float() * ext[j:j + n]
        acc = F.silu(acc) if act else acc
        y[first:first + n] = ((acc + x[first:first + n].float()) if residual else acc).to(out_dtype)
        if L:
            tail[s] = ext[n:n + L]
    return y


def silu_rows_(x: torch.Tensor) -> torch.Tensor:
    """In place ``silu`` on an fp32 [T, C] view whose rows may be strided (a column slice of a fused projection)."""
    if nv.use_native(x):
        if x.dtype != torch.float32 or x.stride(1) != 1:
            raise ValueError("silu_rows_: fp32 rows with a contiguous last dim")
        fn = nv.proto("b200_silu_rows", [vp, i64, i64, i32, vp])
        nv.check(fn(nv.ptr(x), x.stride(0), x.shape[0], x.shape[1], nv.stream()), "silu_rows")
        nv.count_launch()
        return x
    x.copy_(F.silu(x))
    return x


def delta_gates(q: torch.Tensor, k: torch.Tensor, a: torch.Tensor, b: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor,
                G: int, H: int, D: int, qscale: float, unit_eps: float = 1e-6) -> None:
    """In place on fp32 views with strided rows: q, k [T, G * D] -> x / sqrt(sum(x^2) + unit_eps) per head (q also times
    ``qscale``); a [T, H * D] -> exp(-exp(A_log[h]) * softplus(a + dt_bias)); b [T, H] -> sigmoid(b)."""
    T = q.shape[0]
    if nv.use_native(q):
        fn = nv.proto("b200_delta_gates", [vp, i64, vp, i64, vp, i64, vp, i64, vp, vp, i32, i32, i32, i32, f32, f32, vp])
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(k), k.stride(0), nv.ptr(a), a.stride(0), nv.ptr(b), b.stride(0), nv.ptr(dt_bias),
                    nv.ptr(A_log), T, G, H, D, float(qscale), float(unit_eps), nv.stream()), "delta_gates")
        nv.count_launch()
        return
    for x, sc in ((q, qscale), (k, 1.0)):
        v = x.view(T, G, D)
        x.copy_((v * torch.rsqrt((v * v).sum(-1, keepdim=True) + unit_eps) * sc).view(T, G * D))
    a.copy_(torch.exp(-torch.exp(A_log.float()).view(1, H, 1) * F.softplus(a.view(T, H, D) + dt_bias.float().view(1, H, D))).view(T, H * D))
    b.copy_(torch.sigmoid(b))


def linear_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, state: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                runs: Optional[torch.Tensor], n_runs: int, H: int, G: int, D: int, Dv: int, mode: str,
                decay: Optional[torch.Tensor] = None, g: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None,
                act: bool = False, ones: bool = False) -> torch.Tensor:
    """o fp32 [T, H * Dv]. q, k fp32 [T, G * D] (head h reads head h // (H / G)), v fp32 [T, H * Dv] (rows may be strided);
    ``state`` fp32 [rows, H, D, Dv] is read at the start of each run and written at its end. ``mode`` "decay" takes
    ``decay`` fp32 [H]; "delta" takes ``g`` fp32 [T, H * D] (per key channel) and ``beta`` fp32 [T, H]; "gated" takes
    ``g`` = a and ``beta`` = b, both fp32 [T, H]. ``act``: silu on q, k and v as they are read. ``ones``: every head of v gets
    one more column, all ones — ``Dv`` counts it, v itself has ``Dv - 1`` columns per head — so the state's last column
    accumulates the decayed b k alone and o's last column is its product with q."""
    T = q.shape[0]
    o = torch.empty(T, H * Dv, dtype=torch.float32, device=q.device)
    delta = mode == "delta"
    gated = mode == "gated"
    if mode not in ("decay", "delta", "gated"):
        raise ValueError(f"linear_scan: no mode {mode!r}")
    if nv.use_native(q):
        fn = nv.proto("b200_linear_scan", [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32,
                                           i32, i32, i32, i32, vp])
        per = delta or gated
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(k), k.stride(0), nv.ptr(v), v.stride(0), nv.ptr(g), g.stride(0) if per else 0,
                    nv.ptr(beta), beta.stride(0) if per else 0, nv.ptr(decay), nv.ptr(state), nv.ptr(runs), nv.ptr(pos),
                    nv.ptr(slot), n_runs if runs is not None else T, nv.ptr(o), H, G, D, Dv, 2 if gated else int(delta), int(act),
                    int(ones), nv.stream()), "linear_scan")
        nv.count_launch()
        return o
    rep = H // G
    qf, kf, vf = q.float().view(T, G, D), k.float().view(T, G, D), v.float().reshape(T, H, Dv - int(ones))
    if ones:
        vf = torch.cat([vf, torch.ones(T, H, 1, dtype=torch.float32, device=q.device)], -1)
    if act:
        qf, kf, vf = F.silu(qf), F.silu(kf), F.silu(vf)
    qf, kf = qf.repeat_interleave(rep, 1), kf.repeat_interleave(rep, 1)
    ov = o.view(T, H, Dv)
    for first, n, p0, s in _run_list(runs, pos, slot):
        S = state[s].clone() if p0 > 0 else torch.zeros(H, D, Dv, dtype=torch.float32, device=q.device)
        for t in range(first, first + n):
            if delta:
                S = S * g[t].view(H, D, 1)
                u = beta[t].view(H, 1) * (vf[t] - torch.einsum("hde,hd->he", S, kf[t]))
                S = S + kf[t][:, :, None] * u[:, None, :]
            elif gated:
                S = g[t].float().view(H, 1, 1) * S + kf[t][:, :, None] * (beta[t].float().view(H, 1) * vf[t])[:, None, :]
            else:
                S = decay.float().view(H, 1, 1) * S + kf[t][:, :, None] * vf[t][:, None, :]
            ov[t] = torch.einsum("hde,hd->he", S, qf[t])
        state[s] = S
    return o


def mlstm_gates(gi: torch.Tensor, gf: torch.Tensor, bi: torch.Tensor, bf: torch.Tensor, cap: float, mstate: torch.Tensor,
                pos: torch.Tensor, slot: torch.Tensor, runs: Optional[torch.Tensor], n_runs: int):
    """Gates of an mLSTM for the "gated" scan. ``gi`` / ``gf`` fp32 [T, H] (rows may be strided): the input and forget gates'
    projections; with i = cap tanh((gi + bi) / cap), f = logsigmoid(cap tanh((gf + bf) / cap)) and the running maximum
    m' = max(f + m, i) (``mstate`` fp32 [rows, H]; 0 before position 0) it returns a = exp(f + m - m'), b = exp(i - m') and
    e = exp(-m'), each fp32 [T, H]: the state is carried divided by exp(m)."""
    T, H = gi.shape
    a = torch.empty(T, H, dtype=torch.float32, device=gi.device)
    b, e = torch.empty_like(a), torch.empty_like(a)
    if nv.use_native(gi):
        fn = nv.proto("b200_mlstm_gates", [vp, i64, vp, i64, vp, vp, f32, vp, vp, vp, vp, i32, i32, vp, vp, vp, vp])
        nv.check(fn(nv.ptr(gi), gi.stride(0), nv.ptr(gf), gf.stride(0), nv.ptr(bi), nv.ptr(bf), float(cap), nv.ptr(mstate),
                    nv.ptr(runs), nv.ptr(pos), nv.ptr(slot), n_runs if runs is not None else T, H, nv.ptr(a), nv.ptr(b), nv.ptr(e),
                    nv.stream()), "mlstm_gates")
        nv.count_launch()
        return a, b, e
    iv = cap * torch.tanh((gi.float() + bi.float()) / cap)
    fv = F.logsigmoid(cap * torch.tanh((gf.float() + bf.float()) / cap))
    for first, n, p0, s in _run_list(runs, pos, slot):
        m = mstate[s].clone() if p0 > 0 else torch.zeros(H, dtype=torch.float32, device=gi.device)
        for t in range(first, first + n):
            mn = torch.maximum(fv[t] + m, iv[t])
            a[t], b[t], e[t] = torch.exp(fv[t] + m - mn), torch.exp(iv[t] - mn), torch.exp(-mn)
            m = mn
        mstate[s] = m
    return a, b, e


def ssm_gates(dt: torch.Tensor, dt_bias: torch.Tensor, A_log: torch.Tensor):
    """``dt`` fp32 [T, H] (rows may be strided) -> (a, b) fp32 [T, H]: b = softplus(dt + dt_bias) (no threshold),
    a = exp(-exp(A_log) b)."""
    T, H = dt.shape
    if nv.use_native(dt):
        a = torch.empty(T, H, dtype=torch.float32, device=dt.device)
        b = torch.empty_like(a)
        fn = nv.proto("b200_ssm_gates", [vp, i64, vp, vp, vp, vp, i64, i32, vp])
        nv.check(fn(nv.ptr(dt), dt.stride(0), nv.ptr(dt_bias), nv.ptr(A_log), nv.ptr(a), nv.ptr(b), T, H, nv.stream()), "ssm_gates")
        nv.count_launch()
        return a, b
    z = dt.float() + dt_bias.float()
    b = z.clamp(min=0) + torch.log1p(torch.exp(-z.abs()))
    return torch.exp(-torch.exp(A_log.float()) * b), b


def scan_readout(o: torch.Tensor, H: int, Dv: int, w: torch.Tensor, groups: int, eps: float, out_dtype: torch.dtype,
                 e: Optional[torch.Tensor] = None, den_eps: float = 0.0, oscale: float = 1.0,
                 skip: Optional[torch.Tensor] = None, x: Optional[torch.Tensor] = None, pre: Optional[torch.Tensor] = None,
                 post: Optional[torch.Tensor] = None) -> torch.Tensor:
    """What follows a scan, per token, in one pass: ``o`` fp32 [T, H * ocols] with ocols = Dv, or Dv + 1 when the scan carried
    a column of ones (``e`` fp32 [T, H] given: v = oscale o[h, :Dv] / (max(|oscale o[h, Dv]|, e[h]) + den_eps)); ``skip`` fp32
    [H] with ``x`` fp32 [T, H * Dv]: v += skip[h] x; ``pre``: v *= silu(pre); RMS norm over ``groups`` equal parts of the
    H * Dv columns; times ``w`` (fp32, one per column, or one per column of a group); ``post``: v *= sigmoid(post). pre / post /
    x are fp32 rows that may be strided. Returns [T, H * Dv] in ``out_dtype``."""
    T = o.shape[0]
    N = H * Dv
    ocols = o.shape[1] // H
    w_full = w.numel() == N
    if nv.use_native(o):
        out = torch.empty(T, N, dtype=out_dtype, device=o.device)
        fn = nv.proto("b200_scan_readout", [vp, i32, vp, f32, f32, vp, vp, i64, vp, i64, vp, i64, vp, i32, vp, i64, i32, i32, i32,
                                            f32, i32, vp])
        st = lambda z: z.stride(0) if z is not None else 0                      # noqa: E731
        nv.check(fn(nv.ptr(o), ocols, nv.ptr(e), float(den_eps), float(oscale), nv.ptr(skip), nv.ptr(x), st(x), nv.ptr(pre), st(pre),
                    nv.ptr(post), st(post), nv.ptr(w), int(w_full), nv.ptr(out), T, H, Dv, groups, float(eps),
                    nv.dtype_code(out_dtype), nv.stream()), "scan_readout")
        nv.count_launch()
        return out
    ov = o.float().view(T, H, ocols)
    v = ov[:, :, :Dv] * oscale
    if e is not None:
        v = v / (torch.maximum((ov[:, :, Dv] * oscale).abs(), e.float()) + den_eps)[:, :, None]
    v = v.reshape(T, N)
    if skip is not None:
        v = v + (skip.float().view(1, H, 1) * x.float().reshape(T, H, Dv)).reshape(T, N)
    if pre is not None:
        v = v * F.silu(pre.float())
    v = v.view(T, groups, N // groups)
    v = (v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)).reshape(T, N)
    v = v * (w.float() if w_full else w.float().repeat(groups))
    if post is not None:
        v = v * torch.sigmoid(post.float())
    return v.to(out_dtype)
