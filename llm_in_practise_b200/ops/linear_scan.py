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
               runs: Optional[torch.Tensor], n_runs: int, act: bool = True) -> torch.Tensor:
    """``x`` fp32 [T, C] (rows may be strided) -> y fp32 [T, C]; ``w`` fp32 [C, taps] (last column weighs the current token);
    ``tail`` fp32 [rows, taps - 1, C] is read for the inputs before each run and then advanced over the run."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.empty(T, C, dtype=torch.float32, device=x.device)
    if nv.use_native(x):
        if x.dtype != torch.float32 or x.stride(1) != 1:
            raise ValueError("short_conv: fp32 rows with a contiguous last dim")
        fn = nv.proto("b200_short_conv", [vp, i64, vp, vp, vp, vp, vp, i64, i32, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(x), x.stride(0), nv.ptr(w), nv.ptr(tail), nv.ptr(pos), nv.ptr(slot), nv.ptr(y), y.stride(0), T, C, taps,
                    int(act), nv.stream()), "short_conv")
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
        for j in range(taps):
            acc += w[:, j].float() * ext[j:j + n]
        y[first:first + n] = F.silu(acc) if act else acc
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
                act: bool = False) -> torch.Tensor:
    """o fp32 [T, H * Dv]. q, k fp32 [T, G * D] (head h reads head h // (H / G)), v fp32 [T, H * Dv] (rows may be strided);
    ``state`` fp32 [rows, H, D, Dv] is read at the start of each run and written at its end. ``mode`` "decay" takes
    ``decay`` fp32 [H]; "delta" takes ``g`` fp32 [T, H * D] (per key channel) and ``beta`` fp32 [T, H]. ``act``: silu on q, k
    and v as they are read."""
    T = q.shape[0]
    o = torch.empty(T, H * Dv, dtype=torch.float32, device=q.device)
    delta = mode == "delta"
    if nv.use_native(q):
        fn = nv.proto("b200_linear_scan", [vp, i64, vp, i64, vp, i64, vp, i64, vp, i64, vp, vp, vp, vp, vp, i32, vp, i32, i32, i32,
                                           i32, i32, i32, vp])
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(k), k.stride(0), nv.ptr(v), v.stride(0), nv.ptr(g), g.stride(0) if delta else 0,
                    nv.ptr(beta), beta.stride(0) if delta else 0, nv.ptr(decay), nv.ptr(state), nv.ptr(runs), nv.ptr(pos),
                    nv.ptr(slot), n_runs if runs is not None else T, nv.ptr(o), H, G, D, Dv, int(delta), int(act), nv.stream()),
                 "linear_scan")
        nv.count_launch()
        return o
    rep = H // G
    qf, kf, vf = q.float().view(T, G, D), k.float().view(T, G, D), v.float().view(T, H, Dv)
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
            else:
                S = decay.float().view(H, 1, 1) * S + kf[t][:, :, None] * vf[t][:, None, :]
            ov[t] = torch.einsum("hde,hd->he", S, qf[t])
        state[s] = S
    return o
