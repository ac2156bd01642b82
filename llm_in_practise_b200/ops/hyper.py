"""Hyper-connected residual streams with a one-number RMS norm, the xIELU activation and the gated group norm
(``csrc/hyper_conn.cu``).

A model with S residual streams keeps ``X`` [T, S, W] in fp32. Around a sublayer with output ``y``:

    write   x_t <- sum_s mix[s, t] x_s + out[t] * (ls * y)          all streams at once from the old ones
    read    u = sum_s in[s] x_s;  h = u / sqrt(mean(u^2) + eps) * g    g one number; h in the GEMM dtype

``hc_step`` is the write of one sublayer fused with the read of the next (one pass over X, like ``norm.sandwich_norm`` for
a single stream); ``hc_entry`` makes the streams from embedding rows; with S = 1 and all coefficients 1 the pair is the
plain pre-norm residual sum. The reference's models use single-stream pre-norm blocks
(LLM_Distributed_Trainning/PyTorch/ddp_basics/ddp_gpt_wikitext2.py:120-140); this generalises that block.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _native as nv

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_HC = [vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i32, i32, f32, i32, i32, i32, vp]


def _read(X, cin, g, eps, dtype):
    u = X.sum(1) if cin is None else (X * cin.view(1, -1, 1)).sum(1)
    return (u * torch.rsqrt((u * u).mean(-1, keepdim=True) + eps) * g.float()).to(dtype)


def _call(y, ls, X, mix, out, g_entry, cin, g, h, xsum, eps, mode, e_dtype):
    T, S, W = X.shape
    fn = nv.proto("b200_hc_step", _HC)
    hd = h.dtype if h is not None else torch.float32
    nv.check(fn(nv.ptr(y), nv.ptr(ls), nv.ptr(X), nv.ptr(mix), nv.ptr(out), nv.ptr(g_entry), nv.ptr(cin), nv.ptr(g), nv.ptr(h),
                nv.ptr(xsum), T, S, W, float(eps), mode, nv.dtype_code(hd), nv.dtype_code(e_dtype), nv.stream()), "hc_step")
    nv.count_launch()


def hc_entry(e: torch.Tensor, g_entry: torch.Tensor, streams: int, cin: Optional[torch.Tensor], g: torch.Tensor, eps: float,
             dtype: torch.dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Embedding rows ``e`` [T, W] -> (h, X): X[:, s] = e / rms(e) * g_entry for every stream (fp32), h the first read
    (coefficients ``cin`` fp32 [S] or None for ones, norm weight ``g``, fp32 one-element tensors)."""
    T, W = e.shape
    X = torch.empty(T, streams, W, dtype=torch.float32, device=e.device)
    if nv.use_native(e):
        h = torch.empty(T, W, dtype=dtype, device=e.device)
        _call(e.contiguous(), None, X, None, None, g_entry, cin, g, h, None, eps, 1, e.dtype)
        return h, X
    ef = e.float()
    X[:] = (ef * torch.rsqrt((ef * ef).mean(-1, keepdim=True) + eps) * g_entry.float())[:, None, :]
    return _read(X, cin, g, eps, dtype), X


def hc_step(y: torch.Tensor, ls: Optional[torch.Tensor], X: torch.Tensor, mix: torch.Tensor, out: torch.Tensor,
            cin: Optional[torch.Tensor], g: Optional[torch.Tensor], eps: float, dtype: torch.dtype,
            want_sum: bool = False) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Write the sublayer output ``y`` (fp32 [T, W], scaled by ``ls`` fp32 [W]) into the streams ``X`` in place
    (``mix`` fp32 [S, S] indexed [from, to], ``out`` fp32 [S]) and read for the next sublayer (``cin`` fp32 [S] or None = a
    plain sum, ``g`` one-element norm weight; ``g`` None: no read). Returns (h or None, sum of the streams if ``want_sum``)."""
    T, S, W = X.shape
    if nv.use_native(X):
        h = torch.empty(T, W, dtype=dtype, device=X.device) if g is not None else None
        xs = torch.empty(T, W, dtype=torch.float32, device=X.device) if want_sum else None
        _call(y.contiguous(), ls, X, mix, out, None, cin, g, h, xs, eps, 0, torch.float32)
        return h, xs
    yv = y.float() * (ls.float() if ls is not None else 1.0)
    new = torch.einsum("st,bsw->btw", mix.float(), X) + out.float().view(1, S, 1) * yv[:, None, :]
    X.copy_(new)
    return (_read(X, cin, g, eps, dtype) if g is not None else None), (X.sum(1) if want_sum else None)


def hc_read(X: torch.Tensor, cin: Optional[torch.Tensor], g: torch.Tensor, eps: float, dtype: torch.dtype) -> torch.Tensor:
    """The read alone: h = norm(sum_s cin[s] x_s) (``cin`` None: the plain sum of the streams)."""
    T, S, W = X.shape
    if nv.use_native(X):
        h = torch.empty(T, W, dtype=dtype, device=X.device)
        _call(None, None, X, None, None, None, cin, g, h, None, eps, 2, torch.float32)
        return h
    return _read(X, cin, g, eps, dtype)


def xielu(z: torch.Tensor, pq: torch.Tensor) -> torch.Tensor:
    """xIELU with the raw parameter pair ``pq`` (fp32 [2]): for z > 0 ``softplus(p) z^2 + z / 2``, else
    ``(1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2``. fp32 arithmetic, output in z's dtype."""
    if nv.use_native(z):
        zc = z.contiguous()
        y = torch.empty_like(zc)
        fn = nv.proto("b200_xielu", [vp, vp, i64, vp, i32, vp])
        nv.check(fn(nv.ptr(zc), nv.ptr(y), zc.numel(), nv.ptr(pq), nv.dtype_code(zc.dtype), nv.stream()), "xielu")
        nv.count_launch()
        return y
    zf = z.float()
    ap, aq = F.softplus(pq[0].float()), 0.5 + F.softplus(pq[1].float())
    neg = aq * (torch.expm1(zf.clamp(max=0)) - zf) + 0.5 * zf
    return torch.where(zf > 0, ap * zf * zf + 0.5 * zf, neg).to(z.dtype)


def gated_group_norm(o: torch.Tensor, gate: Optional[torch.Tensor], w: torch.Tensor, groups: int, eps: float,
                     dtype: torch.dtype) -> torch.Tensor:
    """``o`` fp32 [T, groups * GS]: every group of GS columns is divided by its root mean square, multiplied by ``w`` (fp32
    [GS], shared by the groups) and by ``sigmoid(gate)`` (fp32 [T, groups * GS], rows may be strided; None: no gate)."""
    T, N = o.shape
    GS = N // groups
    if nv.use_native(o):
        out = torch.empty(T, N, dtype=dtype, device=o.device)
        fn = nv.proto("b200_gated_group_norm", [vp, vp, i64, vp, vp, i64, i32, i32, f32, i32, vp])
        nv.check(fn(nv.ptr(o), nv.ptr(gate), gate.stride(0) if gate is not None else 0, nv.ptr(w), nv.ptr(out), T, groups, GS,
                    float(eps), nv.dtype_code(dtype), nv.stream()), "gated_group_norm")
        nv.count_launch()
        return out
    x = o.float().view(T, groups, GS)
    x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()
    if gate is not None:
        x = x * torch.sigmoid(gate.float().reshape(T, groups, GS))
    return x.reshape(T, N).to(dtype)
