"""Multi-map attention over the paged KV cache (``csrc/multimap_attn.cu``): every head has M attention maps (own query and
key rows, one set of values), the mask is a sliding window that also keeps the first tokens of the sequence, and two maps
can be combined differentially:

    token at position p sees key j of its own cache row  iff  j <= p and (p - j < window or j < keep_first)
    a_m = softmax_j(scale q_{h,m} . k_{g,m,j}) V_g                     g = h // (H / G)
    o   = a_0 - lambda a_1;   o <- o / sqrt(mean(o^2) + eps) * post     (``combine``; M = 2)

Keys live in ``cache_k`` [blocks, G * M, block, D] (after norm and rotation), values in ``cache_v`` [blocks, G, block, Dv];
Dv need not equal D. A layer may attend over the pools another layer filled (shared K/V). ``qknorm_rope_store`` is the step
in front: per-row RMS norm with a weight, split-half rotary on the first ``rot`` dims, the page writes. Beside
``ops.paged_attention`` (one map, values sized like keys, sinks) and ``ops.latent_attention`` (latent rows), which serve
the same ragged step (the reference reaches it through vLLM, LLM_on_Kubernetes/Inference_Platfrom/README.md:1504-1509).
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _native as nv

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
_MMA_D, _MMA_DV = (32, 48, 64, 96, 128), (32, 64, 96, 128)        # sizes the tensor-core kernel is built for
_SPLIT_KEYS = int(os.environ.get("B200_PAGED_SPLIT_KEYS", "512"))  # keys per range of a small batch with many visible keys


def qknorm_rope_store(proj: torch.Tensor, wq: torch.Tensor, wk: Optional[torch.Tensor], cos: torch.Tensor, sin: torch.Tensor,
                      pos: torch.Tensor, slot: torch.Tensor, cache_k: Optional[torch.Tensor], cache_v: Optional[torch.Tensor],
                      table: torch.Tensor, H: int, G: int, M: int, D: int, Dv: int, rot: int, eps: float,
                      dtype: torch.dtype) -> torch.Tensor:
    """``proj`` fp32 [T, >= (H M + G M) D + G Dv] = q rows | k rows | v rows (the k / v part is absent when ``cache_k`` is
    None: a layer that attends over another layer's pools). Returns q [T, H * M * D] in ``dtype``, normed and rotated; the
    token's keys and values are written at (slot, pos) of the pools."""
    T = proj.shape[0]
    has_kv = cache_k is not None
    q_out = torch.empty(T, H * M * D, dtype=dtype, device=proj.device)
    if nv.use_native(proj):
        if proj.dtype != torch.float32 or proj.stride(1) != 1:
            raise ValueError("qknorm_rope_store: fp32 rows with a contiguous last dim")
        BS = cache_k.shape[2] if has_kv else 1
        fn = nv.proto("b200_qknorm_rope_store", [vp, i64, vp, vp, vp, vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32,
                                                 i32, i32, f32, i32, i32, vp])
        nv.check(fn(nv.ptr(proj), proj.stride(0), nv.ptr(wq), nv.ptr(wk), nv.ptr(cos), nv.ptr(sin), nv.ptr(pos), nv.ptr(slot),
                    nv.ptr(table), table.shape[1], nv.ptr(q_out), nv.ptr(cache_k), nv.ptr(cache_v), T, H, G, M, D, Dv, rot, BS,
                    float(eps), int(has_kv), nv.dtype_code(dtype), nv.stream()), "qknorm_rope_store")
        nv.count_launch()
        return q_out
    pl, sl = pos.long(), slot.long()
    hr = rot // 2
    c, s = (cos[pl][:, None, :], sin[pl][:, None, :]) if rot else (None, None)

    def prep(x, w):
        x = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()
        y = x.clone()
        if rot:
            u, v = x[..., :hr], x[..., hr:rot]
            y[..., :hr] = u * c - v * s
            y[..., hr:rot] = v * c + u * s
        return y

    nq, nk = H * M * D, G * M * D
    q_out.copy_(prep(proj[:, :nq].float().view(T, H * M, D), wq).reshape(T, nq).to(dtype))
    if has_kv:
        BS = cache_k.shape[2]
        blk = table[sl, pl // BS].long()
        off = pl % BS
        cache_k[blk, :, off] = prep(proj[:, nq:nq + nk].float().view(T, G * M, D), wk).to(cache_k.dtype)
        cache_v[blk, :, off] = proj[:, nq + nk:nq + nk + G * Dv].view(T, G, Dv).to(cache_v.dtype)
    return q_out


def multimap_attention(q: torch.Tensor, cache_k: torch.Tensor, cache_v: torch.Tensor, table: torch.Tensor, pos: torch.Tensor,
                       slot: torch.Tensor, H: int, G: int, M: int, D: int, Dv: int, scale: float, window: int = 0,
                       keep_first: int = 0, combine: bool = False, lam: float = 0.0, post: float = 1.0, eps: float = 0.0,
                       pieces=None, max_pos: int = 0) -> torch.Tensor:
    """Context [T, H * Dv] (q's dtype) of ``q`` [T, H * M * D] over the pools; see the module docstring for the mask and the
    combination. ``pieces`` (``inference.ragged.Pieces``): bf16 steps with a run of 8 or more tokens go through the tensor-core
    kernel; everything else (fp32, decode batches, sizes it is not built for) through the per-token kernels. ``max_pos``: an upper
    bound of ``pos`` known on the host (0 = unknown), used to cut the keys of a small batch into ranges."""
    T = q.shape[0]
    BS = cache_k.shape[2]
    out = torch.empty(T, H * Dv, dtype=q.dtype, device=q.device)
    if nv.use_native(q):
        if cache_k.dtype != q.dtype or not q.is_contiguous():
            raise ValueError("multimap_attention: contiguous q in the cache dtype")
        if (pieces is not None and pieces.longest >= 8 and q.dtype == torch.bfloat16 and D in _MMA_D and Dv in _MMA_DV and scale > 0
                and BS & (BS - 1) == 0 and os.environ.get("B200_PAGED_MMA", "1") != "0"):
            fn = nv.proto("b200_multimap_attn_mma", [vp, vp, vp, vp, i32, vp, i32, vp, i32, i32, i32, i32, i32, i32, f32, i32, i32, i32,
                                                     f32, f32, f32, i32, vp])
            nv.check(fn(nv.ptr(q), nv.ptr(cache_k), nv.ptr(cache_v), nv.ptr(pieces.tiles), pieces.n_tiles, nv.ptr(table),
                        table.shape[1], nv.ptr(out), H, G, M, D, Dv, BS, float(scale), int(window), int(keep_first), int(combine),
                        float(lam), float(post), float(eps), nv.dtype_code(q.dtype), nv.stream()), "multimap_attn_mma")
            nv.count_launch()
            return out
        # few tokens with many visible keys (a small decode batch with a wide window or none): cut the keys into ranges
        seen = max_pos + 1 if max_pos > 0 else 0
        if window > 0:
            seen = min(seen, window + max(keep_first, 0))
        nsplit = 1
        if seen > 2 * _SPLIT_KEYS and T * G < 296:
            nsplit = min(32, -(-seen // _SPLIT_KEYS), max(1, 592 // (T * G)))
        part = torch.empty(T * H * M * nsplit * (Dv + 2), dtype=torch.float32, device=q.device) if nsplit * M > 1 else None
        fn = nv.proto("b200_multimap_attn", [vp, vp, vp, vp, vp, vp, i32, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, i32,
                                             i32, i32, f32, f32, f32, i32, vp])
        nv.check(fn(nv.ptr(q), nv.ptr(cache_k), nv.ptr(cache_v), nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1],
                    nv.ptr(out), nv.ptr(part), T, H, G, M, D, Dv, BS, float(scale), int(window), int(keep_first), nsplit, int(combine),
                    float(lam), float(post), float(eps), nv.dtype_code(q.dtype), nv.stream()), "multimap_attn")
        nv.count_launch(2 if nsplit * M > 1 else 1)
        return out
    rep = H // G
    pl, sl = pos.tolist(), slot.tolist()
    qf = q.float().view(T, H, M, D)
    for t in range(T):
        p = pl[t]
        lo = max(0, p + 1 - window) if window > 0 else 0
        idx = list(range(min(max(keep_first, 0), lo))) + list(range(lo, p + 1))
        it = torch.tensor(idx, dtype=torch.long, device=q.device)
        blk = table[sl[t], it // BS].long()
        off = it % BS
        k = cache_k[blk, :, off].float().view(len(idx), G, M, D).repeat_interleave(rep, 1)        # [n, H, M, D]
        v = cache_v[blk, :, off].float().repeat_interleave(rep, 1)                                 # [n, H, Dv]
        sc = torch.einsum("hmd,nhmd->hmn", qf[t], k) * scale
        a = torch.einsum("hmn,nhe->hme", sc.softmax(-1), v)
        o = a[:, 0] - lam * a[:, 1] if M == 2 else a[:, 0]
        if combine:
            o = o * torch.rsqrt((o * o).mean(-1, keepdim=True) + eps) * post
        out[t] = o.reshape(H * Dv).to(q.dtype)
    return out
