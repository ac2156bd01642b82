"""Ragged attention over the paged KV cache (``csrc/paged_attn.cu``): the attention of a serving step whose tokens are a
flat list — prompt pieces of some sequences beside single decoded tokens of others — the way vLLM's scheduler batches
the reference's ``vllm serve`` deployments (LLM_on_Kubernetes/Inference_Platfrom/README.md:1504-1509).

Every token carries its cache row (``slot``) and position (``pos``). ``rope_paged_store`` rotates q and k and writes the
new K/V rows into their pages; ``paged_attention`` then lets token t see keys ``0 .. pos[t]`` (or the last ``window`` of
them) of its own row, whatever else is in the batch. Options other designs can use: partial rotation (``rot_dims`` <
head size), interleaved or split pairs, values that are the un-rotated keys (``v_from_k``, for models without a value
projection), per-head attention sinks (a logit that only enters the softmax denominator), a sliding window.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _native as nv

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _rotate(x, cos, sin, rot, interleaved):
    """x [T, heads, D] fp32; cos / sin [T, rot / 2]."""
    c, s = cos[:, None, :], sin[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:rot:2], x[..., 1:rot:2]
        out[..., 0:rot:2] = u * c - v * s
        out[..., 1:rot:2] = v * c + u * s
    else:
        u, v = x[..., :rot // 2], x[..., rot // 2:rot]
        out[..., :rot // 2] = u * c - v * s
        out[..., rot // 2:rot] = v * c + u * s
    return out


def rope_paged_store(qkv: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                     cache_k: torch.Tensor, cache_v: torch.Tensor, table: torch.Tensor, n_heads: int, n_kv_heads: int,
                     head_dim: int, rot_dims: Optional[int] = None, interleaved: bool = False, v_from_k: bool = False) -> torch.Tensor:
    """Rotate the q and k heads of ``qkv`` [T, (H + Hkv (+ Hkv)) * D] in place (first ``rot_dims`` dims of each head, tables
    ``cos`` / ``sin`` [max_pos, rot_dims / 2] fp32 indexed by ``pos`` int32 [T]) and store token t's keys / values at position
    ``pos[t]`` of cache row ``slot[t]`` (int32 [T]; caches [blocks, Hkv, block_size, D], ``table`` int32 [rows, max_blocks]).
    With ``v_from_k`` the values are the keys as projected, before rotation, and ``qkv`` has no v section; ``cache_v`` None:
    the layer keeps no value pool (its key rows are read as values). Returns ``qkv``."""
    T = qkv.shape[0]
    H, G, D = n_heads, n_kv_heads, head_dim
    rot = D if rot_dims is None else rot_dims
    BS = cache_k.shape[2]
    if nv.use_native(qkv):
        if qkv.stride(1) != 1 or cache_k.dtype != qkv.dtype:
            raise ValueError("rope_paged_store: qkv rows must be contiguous and share the cache dtype")
        fn = nv.proto("b200_rope_paged_store", [vp, i64, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(qkv), qkv.stride(0), nv.ptr(cos), nv.ptr(sin), nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1],
                    nv.ptr(cache_k), nv.ptr(cache_v), T, H, G, D, rot, BS, int(interleaved), int(v_from_k), nv.dtype_code(qkv.dtype),
                    nv.stream()), "rope_paged_store")
        nv.count_launch()
        return qkv
    pl, sl = pos.long(), slot.long()
    x = qkv[:, :(H + G) * D].float().view(T, H + G, D)
    r = _rotate(x, cos[pl], sin[pl], rot, interleaved) if rot > 0 else x
    blk = table[sl, pl // BS].long()
    off = pl % BS
    cache_k[blk, :, off] = r[:, H:].to(cache_k.dtype)
    if cache_v is not None:
        cache_v[blk, :, off] = (x[:, H:].to(cache_v.dtype) if v_from_k
                                else qkv[:, (H + G) * D:(H + 2 * G) * D].view(T, G, D).to(cache_v.dtype))
    if rot > 0:
        qkv[:, :(H + G) * D] = r.reshape(T, (H + G) * D).to(qkv.dtype)
    return qkv


_SPLIT_KEYS = int(os.environ.get("B200_PAGED_SPLIT_KEYS", "512"))      # keys per split of a decode-only batch


def paged_attention(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, table: torch.Tensor, pos: torch.Tensor,
                    slot: torch.Tensor, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                    sinks: Optional[torch.Tensor] = None, window: int = 0, max_pos: int = 0, pieces=None) -> torch.Tensor:
    """Context [T, H * D] of token t over keys ``max(0, pos[t] + 1 - window) .. pos[t]`` of cache row ``slot[t]``.
    ``q`` [T, >= H * D] (query heads first; the row may be the whole fused projection). ``sinks`` fp32 [H]: per-head logit
    added to the softmax denominator. ``max_pos``: an upper bound of ``pos`` known on the host (0 = unknown), used to split
    the keys of a small batch over more CTAs. ``pieces``: optional ``Pieces`` describing runs of consecutive tokens of one
    sequence; 16-bit runs then go through the tensor-core kernel."""
    T = q.shape[0]
    H, G, D = n_heads, n_kv_heads, head_dim
    BS = cache_k.shape[2]
    if nv.use_native(q):
        out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
        if pieces is not None and pieces.use_mma(q, D, window, scale) and BS & (BS - 1) == 0:
            fn = nv.proto("b200_paged_attn_mma", [vp, i64, vp, vp, vp, i32, vp, i32, vp, vp, i32, i32, i32, i32, f32, i32, vp])
            nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(cache_k), nv.ptr(cache_v), nv.ptr(pieces.tiles), pieces.n_tiles,
                        nv.ptr(table), table.shape[1], nv.ptr(sinks), nv.ptr(out), H, G, D, BS, scale,
                        nv.dtype_code(q.dtype), nv.stream()), "paged_attn_mma")
            nv.count_launch()
            return out
        nsplit = 1
        if max_pos > 2 * _SPLIT_KEYS and T * G < 296:
            nsplit = min(32, -(-max_pos // _SPLIT_KEYS), max(1, 592 // (T * G)))
        part = torch.empty(T * H * nsplit * (D + 2), dtype=torch.float32, device=q.device) if nsplit > 1 else None
        fn = nv.proto("b200_paged_attn", [vp, i64, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32, i32, i32, vp])
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(cache_k), nv.ptr(cache_v), nv.ptr(pos), nv.ptr(slot), nv.ptr(table),
                    table.shape[1], nv.ptr(sinks), nv.ptr(out), nv.ptr(part), T, H, G, D, BS, scale, int(window), nsplit,
                    nv.dtype_code(q.dtype), nv.stream()), "paged_attn")
        nv.count_launch(2 if nsplit > 1 else 1)
        return out
    # PyTorch path (CPU): one token at a time over its own row
    out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
    rep = H // G
    pl, sl = pos.tolist(), slot.tolist()
    for t in range(T):
        n = pl[t] + 1
        lo = max(0, n - window) if window > 0 else 0
        nb = -(-n // BS)
        blks = table[sl[t], :nb].long()
        k = cache_k[blks].permute(1, 0, 2, 3).reshape(G, nb * BS, D)[:, lo:n].float().repeat_interleave(rep, 0)
        v = cache_v[blks].permute(1, 0, 2, 3).reshape(G, nb * BS, D)[:, lo:n].float().repeat_interleave(rep, 0)
        qt = q[t, :H * D].float().view(H, D)
        sc = torch.einsum("hd,hnd->hn", qt, k) * scale
        if sinks is not None:
            sc = torch.cat([sc, sinks.float().view(H, 1)], 1)
        p = sc.softmax(-1)
        if sinks is not None:
            p = p[:, :-1]
        out[t] = torch.einsum("hn,hnd->hd", p, v).reshape(H * D).to(q.dtype)
    return out
