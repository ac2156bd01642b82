"""Kudonex beside Duratar (the framework's closest design: windowed attention over pages beside recurrent scans with short
convolutions, on an fp32 stream) at equal layer sizes, random weights: prefill and decode throughput through each model's own
generator, and the time of each Kudonex kernel next to the Duratar (or, for the norm and the router, Gorozen) kernel that
does the like job, as fractions of the measured roofline (``MEASURED_PEAKS.json``: copy bandwidth and cuBLAS bf16 rate of
this pool's B200). Scans are given against the nominal fp32 FMA rate, as in the Duratar bench.

    python bench.py --workload kudonex [--steps K --warmup W]

Timing: CUDA events on the launching stream, W >= 3 warm-up iterations; the single-kernel rows (both designs) are replayed
from a CUDA graph with an L2 flush (a 256 MB write) between timed iterations; the end-to-end rows run steps whose weights and
caches together exceed L2.
"""
from __future__ import annotations

import json
import time

import torch

from duratar_bench import FP32_TFLOPS, duratar_config
from gorozen_bench import Timer, _peaks
from segorax_bench import GraphTimer

SIZES = {
    # name: (width, attention heads, kv heads, head size, window, scan heads, scan key size, scan value size, state-space groups,
    #        taps, dense-equivalent ff, experts, top, vocab)
    "2k wide, 16 heads": (2048, 16, 4, 128, 1024, 16, 128, 128, 4, 4, 6144, 8, 2, 32768),
    "4k wide, 16 attention heads, 32 scan heads": (4096, 16, 4, 128, 1024, 32, 128, 128, 8, 4, 12288, 8, 2, 32768),
}


def kudonex_config(W, H, G, D, win, SH, SD, SDv, SG, taps, F, E, top, V):
    # the feed-forward multiplies as much per token as a dense one of F: `top` experts of F / 4 and a shared one of F / 2
    mlp = {"kind": "moe", "expert": {"ff": F // 4}, "router": {"experts": E, "top": top, "groups": {"count": 2, "keep": 1}},
           "shared": {"ff": F // 2}}
    att = {"heads": H, "kv_heads": G, "dim": D, "vdim": D, "scale": D ** -0.5, "mask": {"size": win}}
    layers = [{"type": "attention", "mixer": att, "mlp": mlp},
              {"type": "mamba2", "mixer": {"heads": SH, "vdim": SDv, "state": SD, "groups": SG, "norm_groups": SG, "conv": taps}, "mlp": mlp},
              {"type": "attention", "mixer": att, "mlp": mlp},
              {"type": "mlstm", "mixer": {"heads": SH, "dim": SD, "vdim": SDv, "gate_cap": 15.0}, "mlp": mlp}]
    return {"architecture": "Kudonex", "layers": layers, "norm": {"eps": 1e-6}, "embedding": {"scale": W ** 0.5}, "canon": {"taps": taps},
            "vocab": V, "width": W}


def build_models(size, dev):
    from llm_in_practise_b200.models.duratar import DuratarConfig, DuratarForCausalLM
    from llm_in_practise_b200.models.kudonex import KudonexConfig, KudonexForCausalLM
    W, H, G, D, win, SH, SD, SDv, SG, taps, F, E, top, V = SIZES[size]
    torch.manual_seed(0)
    kx = KudonexForCausalLM(KudonexConfig.from_dict(kudonex_config(*SIZES[size])), dtype=torch.bfloat16, device=dev).eval()
    for n, p in kx.named_parameters():
        leaf = n.split(".")[-1]
        if p.dtype == torch.bfloat16 and p.dim() >= 2 and leaf != "embed_tokens":
            p.data.normal_(std=p.shape[-1] ** -0.5)
        elif leaf in ("canon", "conv_w", "router"):
            p.data.normal_(std=0.3)
        elif leaf in ("r1", "r2"):
            p.data.uniform_(0.1, 1.0)
        elif leaf == "talk":
            p.data.add_(torch.randn_like(p) * 0.1)
    du = DuratarForCausalLM(DuratarConfig.from_dict(duratar_config(W, H, G, D // 2, D, win, 4, SH, SD, SDv, SG, taps, F, V)),
                            dtype=torch.bfloat16, device=dev, low_ranks={1: (64, 64)}).eval()
    for n, p in du.named_parameters():
        if p.dtype == torch.bfloat16 and n.split(".")[-1] in ("in_proj", "o_proj", "up_proj", "down_proj", "a1", "a2", "g1", "g2"):
            p.data.normal_(std=p.shape[1] ** -0.5)
        elif n.endswith("conv_w"):
            p.data.normal_(std=0.5)
    return kx, du


@torch.no_grad()
def end_to_end(size, dev, steps, warmup, prompt=2048, batch=32, ctx=1024):
    """tokens/s of (a) one prompt of ``prompt`` tokens, (b) one decode step of ``batch`` sequences at context ``ctx``."""
    from llm_in_practise_b200.inference import RaggedGenerator
    t = Timer(dev, flush=False)
    out = {}
    V = SIZES[size][-1]
    toks = torch.randint(0, V, (prompt,)).tolist()
    for name, model in zip(("kudonex", "duratar"), build_models(size, dev)):
        g = RaggedGenerator(model, None, max(prompt, ctx + 64))
        per = -(-max(prompt, ctx + 64) // 64)
        cache = g.make_cache(batch * per, 64, batch, per * 64)
        for b in range(batch):
            g.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
        ms = t(lambda: g.step([(0, 0, toks, [prompt - 1])], cache), steps, warmup)
        out[f"{name}_prefill_tok_s"] = prompt / ms * 1e3
        out[f"{name}_prefill_ms"] = ms
        last = [1] * batch
        ms = t(lambda: g.decode(last, [ctx] * batch, list(range(batch)), cache), steps * 4, warmup)
        out[f"{name}_decode_tok_s"] = batch / ms * 1e3
        out[f"{name}_decode_ms"] = ms
        out[f"{name}_kv_bytes_per_token"] = g.kv_token_bytes()
        out[f"{name}_state_bytes_per_sequence"] = g.state_bytes()
        del g, cache, model
        torch.cuda.empty_cache()
    return out


@torch.no_grad()
def kernel_rows(size, dev, steps, warmup, root):
    """Single kernels at the layer sizes: (name, Kudonex ms, fraction of roofline, like kernel or None, ms, fraction, bound)."""
    from llm_in_practise_b200.inference.ragged import make_pieces
    from llm_in_practise_b200.ops import elementwise as ew
    from llm_in_practise_b200.ops.hyper import gated_group_norm
    from llm_in_practise_b200.ops.linear_scan import delta_gates, linear_scan, mlstm_gates, scan_readout, short_conv, ssm_gates
    from llm_in_practise_b200.ops.moe import ROUTE_SOFTMAX_SELECTED, route_grouped, route_topk
    from llm_in_practise_b200.ops.multimap_attention import multimap_attention, qknorm_rope_store
    from llm_in_practise_b200.ops.norm import sandwich_norm
    from llm_in_practise_b200.ops.paged_attention import rope_paged_store
    from llm_in_practise_b200.ops.talking_attention import talking_attention
    hbm, tf, which = _peaks(root)
    W, H, G, D, win, SH, SD, SDv, SG, taps, F, E, top, V = SIZES[size]
    t = GraphTimer(dev)
    rows = []
    bf = torch.bfloat16
    T = 4096

    def frac_bw(nbytes, ms):
        return nbytes / (ms * 1e-3) / 1e9 / hbm

    def frac_fl(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / tf

    def frac_fma(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / FP32_TFLOPS

    # --- layer-norm sandwich (fp32 h out, as the input convolution wants it) vs the RMS sandwich of Gorozen (bf16 h out)
    y32, res = torch.randn(T, W, device=dev), torch.randn(T, W, device=dev)
    wn = torch.ones(W, device=dev)
    ms_k = t(lambda: sandwich_norm(y32, wn, res, wn, 1e-6, 0.0, torch.float32, center=True), steps, warmup)
    w2 = torch.zeros(W, dtype=bf, device=dev)
    ms_g = t(lambda: sandwich_norm(y32, w2, res, w2, 1e-6, 1.0, bf), steps, warmup)
    rows.append(("post layer norm + residual + pre layer norm (fp32 out)", ms_k, frac_bw(T * W * 16, ms_k),
                 "Gorozen: post RMS norm + residual + pre RMS norm", ms_g, frac_bw(T * W * 14, ms_g), "HBM"))
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    pieces = make_pieces([(0, T, 0, 0)], dev)
    runs = pieces.runs
    # --- input convolution on the width (residual, bf16 out) vs Duratar's q | k | v convolution
    h32 = torch.randn(T, W, device=dev)
    cw = torch.randn(W, taps, device=dev) * 0.3
    tail = torch.zeros(65, taps - 1, W, device=dev)
    ms_k = t(lambda: short_conv(h32, cw, tail, pos, slot, runs, 1, act=False, residual=True, out_dtype=bf), steps, warmup)
    C = 2 * SG * SD + SH * SDv
    xin = torch.randn(T, C + 8, device=dev)
    cw2 = torch.randn(C, taps, device=dev) * 0.5
    tail2 = torch.zeros(65, taps - 1, C, device=dev)
    ms_d = t(lambda: short_conv(xin[:, :C], cw2, tail2, pos, slot, runs, 1), steps, warmup)
    rows.append((f"input convolution ({taps} taps) + residual + tail, {W} channels, bf16 out", ms_k, frac_bw(T * W * 6, ms_k),
                 f"Duratar: short convolution + silu + tail, {C} channels", ms_d, frac_bw(T * C * 8, ms_d), "HBM"))
    ms_k = t(lambda: short_conv(xin[:, :C], cw2, tail2, pos, slot, runs, 1, act=True, bias=cw2[:, 0].contiguous()), steps, warmup)
    rows.append((f"x | B | C convolution + bias + silu + tail, {C} channels", ms_k, frac_bw(T * C * 8, ms_k),
                 "Duratar: the same kernel without bias", ms_d, frac_bw(T * C * 8, ms_d), "HBM"))
    # --- key page store vs Duratar's q/k norm + rotary + store
    BS = 64
    nb = T // BS
    ck = torch.zeros(nb + 1, G, BS, D, dtype=bf, device=dev)
    table = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).view(1, nb)
    qkg = torch.randn(T, (2 * H + G) * D, device=dev).to(bf)
    zero = torch.zeros(1, 1, device=dev)
    ms_k = t(lambda: rope_paged_store(qkg[:, H * D:], zero, zero, pos, slot, ck, None, table, 0, G, D, rot_dims=0), steps, warmup)
    Dm = D // 2
    dk, dv_ = torch.zeros(nb + 1, G * 2, BS, Dm, dtype=bf, device=dev), torch.zeros(nb + 1, G, BS, D, dtype=bf, device=dev)
    ncol = (H + G) * 2 * Dm + G * D
    proj = torch.randn(T, ncol, device=dev)
    wq = torch.ones(Dm, device=dev)
    cos, sin = ew.rope_tables_partial(T, Dm, 1e6, dev)
    ms_d = t(lambda: qknorm_rope_store(proj, wq, wq, cos, sin, pos, slot, dk, dv_, table, H, G, 2, Dm, D, Dm, 1e-6, bf), steps, warmup)
    rows.append(("key page store (no rotation, no value pool)", ms_k, frac_bw(T * G * D * 4, ms_k),
                 "Duratar: q/k norm + rotary + K/V page store (fp32 in)", ms_d, frac_bw(T * (ncol * 4 + ((H + G) * 2 * Dm + G * D) * 2), ms_d), "HBM"))
    # --- prompt attention over a window: talking heads (all heads in one CTA) vs Duratar's two maps per head
    ck.normal_()
    dk.normal_()
    dv_.normal_()
    r1, r2 = torch.rand(H, device=dev), torch.rand(H, device=dev)
    talk = torch.eye(H, device=dev) + torch.randn(H, H, device=dev) * 0.1
    seen = sum(min(p + 1, win) for p in range(T))
    ms_k = t(lambda: talking_attention(qkg, ck, table, pos, slot, H, G, D, D ** -0.5, win, r1, r2, talk, gate=qkg[:, (H + G) * D:], pieces=pieces),
             steps, warmup)
    qd2 = torch.randn(T, H * 2 * Dm, device=dev).to(bf)
    ms_d = t(lambda: multimap_attention(qd2, dk, dv_, table, pos, slot, H, G, 2, Dm, D, Dm ** -0.5, win, 4, True, 0.4, 0.7, 1e-6, pieces), steps, warmup)
    # the mixing is H fp32 FMAs per score, which the design wants in 32 bits: at these sizes it takes the CUDA cores longer
    # (at their nominal rate) than both products take the tensor cores, so it is the kernel's roofline
    roof_k = max(frac_fl(4 * H * D * seen, ms_k), frac_fma(2 * H * H * seen, ms_k))
    rows.append((f"prompt attention, window {win}, head mixing (mma.sync + fp32 mixing)", ms_k, roof_k,
                 f"Duratar: prompt attention, 2 maps, window {win} + 4 kept (mma.sync)", ms_d, frac_fl(2 * H * 2 * (Dm + D) * (seen + 4 * T), ms_d),
                 "slower of bf16 tensor and fp32 FMA (mixing); Duratar: bf16 tensor"))
    # --- decode attention: 64 sequences at context 4032
    Bq, ctx = 64, 4032
    nbd = Bq * (ctx // BS + 1)
    ckd = torch.randn(nbd + 1, G, BS, D, device=dev).to(bf)
    tabd = torch.arange(1, nbd + 1, dtype=torch.int32, device=dev).view(Bq, -1)
    posd = torch.full((Bq,), ctx, dtype=torch.int32, device=dev)
    slotd = torch.arange(Bq, dtype=torch.int32, device=dev)
    qd = torch.randn(Bq, (2 * H + G) * D, device=dev).to(bf)
    ms_k = t(lambda: talking_attention(qd, ckd, tabd, posd, slotd, H, G, D, D ** -0.5, win, r1, r2, talk, gate=qd[:, (H + G) * D:]), steps, warmup)
    del ckd
    dkd, dvd = torch.randn(nbd + 1, G * 2, BS, Dm, device=dev).to(bf), torch.randn(nbd + 1, G, BS, D, device=dev).to(bf)
    qdd = torch.randn(Bq, H * 2 * Dm, device=dev).to(bf)
    ms_d = t(lambda: multimap_attention(qdd, dkd, dvd, tabd, posd, slotd, H, G, 2, Dm, D, Dm ** -0.5, win, 4, True, 0.4, 0.7, 1e-6), steps, warmup)
    del dkd, dvd
    rows.append((f"decode attention, 64 seqs at 4032, window {win}, head mixing", ms_k, frac_bw(Bq * G * win * D * 2, ms_k),
                 f"Duratar: decode attention, 2 maps, window {win} + 4", ms_d, frac_bw(Bq * G * (win + 4) * (2 * Dm + D) * 2, ms_d), "HBM"))
    # --- gates
    gi = torch.randn(T, 2 * SH, device=dev) * 3
    bi = torch.zeros(SH, device=dev)
    mst = torch.zeros(65, SH, device=dev)
    ms_k = t(lambda: mlstm_gates(gi[:, :SH], gi[:, SH:], bi, bi, 15.0, mst, pos, slot, runs, 1), steps, warmup)
    qs = torch.randn(T, SG * SD, device=dev)
    ks = torch.randn(T, SG * SD, device=dev)
    aa, bb = torch.randn(T, SH * SD, device=dev), torch.randn(T, SH, device=dev)
    dtb, alog = torch.zeros(SH * SD, device=dev), torch.zeros(SH, device=dev)
    ms_d = t(lambda: delta_gates(qs, ks, aa, bb, dtb, alog, SG, SH, SD, 1.0), steps, warmup)
    rows.append((f"mLSTM gates + running maximum, one prompt of {T} tokens (max-plus scans, 256 tokens per round)", ms_k, frac_bw(T * SH * 20, ms_k),
                 "Duratar: unit q / k, decays, beta (no recurrence)", ms_d, frac_bw(T * (2 * SG * SD + SH * SD + SH) * 8, ms_d), "HBM"))
    ms_k = t(lambda: ssm_gates(gi[:, :SH], bi, bi), steps, warmup)
    rows.append(("state-space step sizes and decays", ms_k, frac_bw(T * SH * 12, ms_k), None, 0.0, 0.0, "HBM"))
    # --- scans: one prompt of 4096 tokens, and a decode batch of 64
    q16, k16 = torch.randn(T, SH * SD, device=dev) * SD ** -0.5, torch.randn(T, SH * SD, device=dev) * SD ** -0.5
    vs = torch.randn(T, SH * SDv, device=dev)
    ga, gb = torch.rand(T, SH, device=dev) * 0.1 + 0.9, torch.rand(T, SH, device=dev)
    dec = torch.full((SH,), 0.99, device=dev)
    st0 = torch.zeros(65, SH, SD, SDv, device=dev)
    st1 = torch.zeros(65, SH, SD, SDv + 1, device=dev)
    pd, sd_ = torch.full((Bq,), 77, dtype=torch.int32, device=dev), torch.arange(Bq, dtype=torch.int32, device=dev)
    ms_d = t(lambda: linear_scan(q16, k16, vs, st0, pos, slot, runs, 1, SH, SH, SD, SDv, "decay", decay=dec), steps, warmup)
    ms_db = t(lambda: linear_scan(q16[:Bq], k16[:Bq], vs[:Bq], st0, pd, sd_, None, Bq, SH, SH, SD, SDv, "decay", decay=dec), steps, warmup)
    fl = SH * 2 * 2 * SD * SDv * T
    for name, state, cols, g_, ones in (("mLSTM: gated scan with the normaliser column", st1, SDv + 1, SH, True),
                                        ("state space: gated scan, B / C shared by groups", st0, SDv, SG, False)):
        qq, kk = (q16, k16) if g_ == SH else (qs, ks)
        ms_k = t(lambda: linear_scan(qq, kk, vs, state, pos, slot, runs, 1, SH, g_, SD, cols, "gated", g=ga, beta=gb, ones=ones), steps, warmup)
        rows.append((f"{name}, one prompt of {T} tokens, {SH} heads of {SD} x {SDv}", ms_k, frac_fma(fl, ms_k),
                     "Duratar: state scan (decay per head)", ms_d, frac_fma(fl, ms_d), "nominal fp32 FMA rate"))
        ms_b = t(lambda: linear_scan(qq[:Bq], kk[:Bq], vs[:Bq], state, pd, sd_, None, Bq, SH, g_, SD, cols, "gated", g=ga, beta=gb, ones=ones),
                 steps, warmup)
        rows.append((f"{name}, decode batch of {Bq}", ms_b, frac_bw(Bq * SH * SD * cols * 8, ms_b),
                     "Duratar: state scan (decay), decode batch", ms_db, frac_bw(Bq * SH * SD * SDv * 8, ms_db), "HBM"))
    # --- read-outs vs Duratar's per-head norm + gate
    o1, e1 = torch.randn(T, SH * (SDv + 1), device=dev), torch.rand(T, SH, device=dev)
    gate = torch.randn(T, SH * SDv, device=dev)
    wfull = torch.ones(SH * SDv, device=dev)
    ms_k = t(lambda: scan_readout(o1, SH, SDv, wfull, SH, 1e-6, bf, e=e1, den_eps=1e-6, oscale=SD ** -0.5, post=gate), steps, warmup)
    o32 = torch.randn(T, SH * SDv, device=dev)
    wn1 = torch.ones(SDv, device=dev)
    ms_d = t(lambda: gated_group_norm(o32, gate, wn1, SH, 1e-6, bf), steps, warmup)
    rows.append(("mLSTM read-out: normaliser, per-head norm, weight, sigmoid gate", ms_k, frac_bw(T * SH * SDv * 10, ms_k),
                 "Duratar: per-head norm + sigmoid gate", ms_d, frac_bw(T * SH * SDv * 10, ms_d), "HBM"))
    skip = torch.ones(SH, device=dev)
    ms_k = t(lambda: scan_readout(o32, SH, SDv, wfull, SG, 1e-6, bf, skip=skip, x=vs, pre=gate), steps, warmup)
    rows.append(("state-space read-out: skip, silu gate, grouped norm, weight", ms_k, frac_bw(T * SH * SDv * 14, ms_k),
                 "Duratar: per-head norm + sigmoid gate", ms_d, frac_bw(T * SH * SDv * 10, ms_d), "HBM"))
    # --- router vs Gorozen's
    hb = torch.randn(T, W, device=dev).to(bf)
    wr, corr = torch.randn(E, W, device=dev) * 0.05, torch.zeros(E, device=dev)
    ms_k = t(lambda: route_grouped(hb, wr, corr, top, 2, 1, 1, softmax=True), steps, warmup)
    ms_g = t(lambda: route_topk(hb, wr, corr, top, ROUTE_SOFTMAX_SELECTED), steps, warmup)
    rows.append((f"router: softmax over {E}, correction, best group of 2, top {top}", ms_k, frac_bw(T * W * 2, ms_k),
                 "Gorozen: router with bias, top-k, softmax over the chosen", ms_g, frac_bw(T * W * 2, ms_g), "HBM"))
    return rows, which


def run(args, root):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from llm_in_practise_b200.ops import _native as nv
    nv.lib()
    n0 = nv.launch_count
    t0 = time.time()
    res = {"metric": "Kudonex vs Duratar at equal layer sizes: prefill / decode tok/s", "unit": "tok/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16", "data": "synthetic", "sizes": {}, "kernels": {}}
    first = next(iter(SIZES))
    for size in SIZES:
        res["sizes"][size] = {k: round(v, 2) for k, v in end_to_end(size, dev, args.steps, args.warmup).items()}
        torch.cuda.empty_cache()
    for size in SIZES:
        rows, which = kernel_rows(size, dev, args.steps, args.warmup, root)
        res["kernels"][size] = [{"kudonex": a, "ms": round(b, 4), "of_roofline": round(c, 3), "like": d, "like_ms": round(e, 4),
                                 "like_of_roofline": round(f, 3), "bound": g, "gap_ratio": round(f / c, 2) if c and d else None}
                                for a, b, c, d, e, f, g in rows]
        res["roofline"] = which
        torch.cuda.empty_cache()
    res["gpu_launches"] = nv.launch_count - n0
    res["seconds"] = round(time.time() - t0, 1)
    res["value"] = res["sizes"][first]["kudonex_decode_tok_s"]
    res["config"] = {"model": "kudonex: attention, mamba2, attention, mlstm; one layer each, MoE feed-forwards of a dense layer's active size",
                     "sizes": {k: list(v) for k, v in SIZES.items()},
                     "l2": "single kernels: replayed from a CUDA graph, 256 MB flush between iterations; steps: weights + cache exceed L2"}
    print(json.dumps(res))
    return 0
