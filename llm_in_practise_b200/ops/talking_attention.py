"""Talking-heads attention over the paged key cache (``csrc/talking_attn.cu``, ``csrc/talking_attn_mma.cu``): the attention of
a ragged serving step in which the heads' scores are mixed by a learned [H, H] matrix before the softmax.

For token t at position i = ``pos[t]`` of cache row ``slot[t]`` and the keys j with 0 <= i - j < ``window``:

    raw_g(i, j) = scale * q_g(i) . k_kv(g)(j) - r1[g] * log(1 + r2[g] * (i - j))          a logarithmic distance penalty
    s_h(i, j)   = sum_g talk[h, g] * raw_g(i, j)                                          mixing over ALL heads
    out_h(i)    = sum_j softmax_j(s_h(i, .))[j] * k_kv(h)(j)   (* sigmoid(gate_h(i)))     keys are the values

The layer caches key rows only (``PagedKVCache`` with a value row size of 0; ``ops.paged_attention.rope_paged_store`` with
``cache_v=None`` writes them). Scores, mixing, softmax and accumulators are fp32 whatever the cache dtype. Other designs
can switch the parts off: ``talk`` the identity and ``r1`` zero give plain windowed attention over shared keys / values.

The reference's models use plain causal softmax attention (LLM_Distributed_Trainning/PyTorch/transformer_basics/
miniGPT_with_wikitext2.py:60-88); this sits beside ``ops.paged_attention`` for designs that need the head mixing.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _native as nv

vp, i32, i64, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float
SPLIT_MAX = 8                        # most CTAs that share one decode token's keys


def talking_attention(q: torch.Tensor, cache_k: torch.Tensor, table: torch.Tensor, pos: torch.Tensor, slot: torch.Tensor,
                      n_heads: int, n_kv_heads: int, head_dim: int, scale: float, window: int, r1: torch.Tensor,
                      r2: torch.Tensor, talk: torch.Tensor, gate: Optional[torch.Tensor] = None, pieces=None) -> torch.Tensor:
    """Context [T, H * D] in q's dtype. ``q`` [T, >= H * D] (query heads first; rows may be strided: a slice of a fused
    projection), ``gate`` [T, H * D] or None (same dtype, rows may be strided), ``cache_k`` [blocks, G, block_size, D],
    ``r1`` / ``r2`` fp32 [H], ``talk`` fp32 [H, H] indexed [to, from]. ``window`` 0: every earlier key is visible.
    ``pieces``: optional ``Pieces`` of the step (None: every token stands alone, a decode batch). bf16 runs with at most 16
    heads of a size the tensor-core kernel takes go through it, pieces and single tokens alike; everything else (fp32 runs,
    other sizes) through the per-token kernel."""
    T = q.shape[0]
    H, G, D = n_heads, n_kv_heads, head_dim
    BS = cache_k.shape[2]
    if nv.use_native(q):
        if q.stride(1) != 1 or (gate is not None and gate.stride(1) != 1) or cache_k.dtype != q.dtype:
            raise ValueError("talking_attention: rows must be contiguous and share the cache dtype")
        out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
        if (q.dtype == torch.bfloat16 and D % 16 == 0 and D <= 128 and H <= 16 and nv.has("b200_talking_attn_mma")
                and os.environ.get("B200_TALKING_MMA", "1") != "0"):
            # every 64-row tile of the step becomes up to four CTAs of 16 rows, and without pieces (a decode batch) every
            # token is a tile of one row; sizes the kernel does not take come back as "unsupported" and go to the
            # per-token kernel below
            fn = nv.proto("b200_talking_attn_mma", [vp, i64, vp, i64, vp, vp, i32, vp, vp, vp, i32, vp, vp, vp, vp, i32, i32, i32, i32,
                                                    f32, i32, vp, i32, vp])
            tiles, n = (pieces.tiles, pieces.n_tiles) if pieces is not None else (None, T)
            # a decode batch smaller than the machine: a token's keys are shared out over several CTAs (at least four
            # chunks of 32 keys each) and merged by a second kernel; the count depends on static sizes only, so a captured
            # graph replays it
            nsplit, part = 1, None
            if pieces is None:
                keys = window if window > 0 else table.shape[1] * BS
                nsplit = max(1, min(SPLIT_MAX, nv.sm_count(q.device) // T, (keys // 32 + 1) // 4))
                if nsplit > 1:
                    part = torch.empty(T, nsplit, H, D + 2, dtype=torch.float32, device=q.device)
            rc = fn(nv.ptr(q), q.stride(0), nv.ptr(gate), gate.stride(0) if gate is not None else 0, nv.ptr(cache_k),
                    nv.ptr(tiles), n, nv.ptr(pos), nv.ptr(slot), nv.ptr(table), table.shape[1], nv.ptr(r1), nv.ptr(r2), nv.ptr(talk),
                    nv.ptr(out), H, G, D, BS, float(scale), int(window), nv.ptr(part), nsplit, nv.stream())
            if rc == 0:
                nv.count_launch()
                return out
            if rc != nv.ERR_UNSUPPORTED:
                nv.check(rc, "talking_attn_mma")
        fn = nv.proto("b200_talking_attn", [vp, i64, vp, i64, vp, vp, i32, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32, i32, f32, i32,
                                            i32, vp])
        nv.check(fn(nv.ptr(q), q.stride(0), nv.ptr(gate), gate.stride(0) if gate is not None else 0, nv.ptr(cache_k), nv.ptr(table),
                    table.shape[1], nv.ptr(pos), nv.ptr(slot), nv.ptr(r1), nv.ptr(r2), nv.ptr(talk), nv.ptr(out), T, H, G, D, BS,
                    float(scale), int(window), nv.dtype_code(q.dtype), nv.stream()), "talking_attn")
        nv.count_launch()
        return out
    # PyTorch path (CPU): one token at a time over its own row
    out = torch.empty(T, H * D, dtype=q.dtype, device=q.device)
    rep = H // G
    pl, sl = pos.tolist(), slot.tolist()
    tk = talk.float()
    for t in range(T):
        n = pl[t] + 1
        lo = max(0, n - window) if window > 0 else 0
        nb = -(-n // BS)
        blks = table[sl[t], :nb].long()
        k = cache_k[blks].permute(1, 0, 2, 3).reshape(G, nb * BS, D)[:, lo:n].float().repeat_interleave(rep, 0)     # [H, n, D]
        qt = q[t, :H * D].float().view(H, D)
        dist = torch.arange(n - 1 - lo, -1, -1, dtype=torch.float32, device=q.device)
        raw = torch.einsum("hd,hnd->hn", qt, k) * scale - r1.float()[:, None] * torch.log1p(r2.float()[:, None] * dist[None, :])
        p = (tk @ raw).softmax(-1)
        ctx = torch.einsum("hn,hnd->hd", p, k).reshape(H * D)
        if gate is not None:
            ctx = ctx * torch.sigmoid(gate[t, :H * D].float())
        out[t] = ctx.to(q.dtype)
    return out
