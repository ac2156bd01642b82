"""Duratar beside Gorozen (the framework's closest design: an fp32 stream, fused norm steps, paged windowed attention) at
equal layer sizes, random weights: prefill and decode throughput through each model's own generator, and the time of each
Duratar kernel next to the Gorozen kernel that does the like job, as fractions of the measured roofline
(``MEASURED_PEAKS.json``: copy bandwidth and cuBLAS bf16 rate of this pool's B200). The recurrent scans have no like kernel
in Gorozen; they are given against HBM bytes and against the nominal fp32 FMA rate.

    python bench.py --workload duratar [--steps K --warmup W]

Timing: CUDA events on the launching stream, W >= 3 warm-up iterations; the single-kernel rows (both designs) are replayed
from a CUDA graph with an L2 flush (a 256 MB write) between timed iterations; the end-to-end rows run steps whose weights and
caches together exceed L2.
"""
from __future__ import annotations

import json
import time

import torch

from gorozen_bench import Timer, _peaks, gorozen_config
from segorax_bench import GraphTimer

FP32_TFLOPS = 148 * 128 * 2 * 1.965e9 / 1e12          # nominal FMA rate of the CUDA cores at the maximum SM clock

SIZES = {
    # name: (width, heads, kv heads, dim per map, value dim, window, kept, scan heads, scan key dim, scan value dim, delta q/k heads,
    #        conv taps, ff, vocab)
    "2k wide, 16 heads": (2048, 16, 4, 64, 128, 1024, 4, 16, 128, 128, 4, 4, 6144, 32768),
    "4k wide, 32 heads": (4096, 32, 8, 64, 128, 1024, 4, 32, 128, 128, 8, 4, 12288, 32768),
}


def duratar_config(W, H, G, D, Dv, win, keep, SH, SD, SDv, SG, taps, F, V, streams=2):
    rot = {"base": 1e6, "dims": D, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    att = {"heads": H, "kv_heads": G, "dim": D, "vdim": Dv, "diff": 0.3, "scale": D ** -0.5, "mask": {"size": win, "keep_first": keep}, "rot": rot}
    mlp = {"kind": "dense", "ff": F}
    layers = [{"type": "attention", "mixer": att, "mlp": mlp},
              {"type": "channel_delta", "mixer": {"heads": SH, "kv_heads": SG, "dim": SD, "vdim": SDv, "conv": taps}, "mlp": mlp},
              {"type": "attention", "mixer": dict(att, kv_from=0), "mlp": mlp},
              {"type": "lightning", "mixer": {"heads": SH, "dim": SD, "vdim": SDv, "decay": [1.0 - 2.0 ** -(3 + h % 8) for h in range(SH)]}, "mlp": mlp}]
    return {"architecture": "Duratar", "layers": layers, "norm": {"eps": 1e-6}, "streams": streams, "vocab": V, "width": W}


def build_models(size, dev):
    from llm_in_practise_b200.models.duratar import DuratarConfig, DuratarForCausalLM
    from llm_in_practise_b200.models.gorozen import GorozenConfig, GorozenForCausalLM
    W, H, G, D, Dv, win, keep, SH, SD, SDv, SG, taps, F, V = SIZES[size]
    torch.manual_seed(0)
    cfg = DuratarConfig.from_dict(duratar_config(*SIZES[size]))
    du = DuratarForCausalLM(cfg, dtype=torch.bfloat16, device=dev, low_ranks={1: (64, 64)}).eval()
    for n, p in du.named_parameters():
        if p.dtype == torch.bfloat16 and n.split(".")[-1] in ("in_proj", "o_proj", "up_proj", "down_proj", "a1", "a2", "g1", "g2"):
            p.data.normal_(std=p.shape[1] ** -0.5)
        elif n.endswith("conv_w"):
            p.data.normal_(std=0.5)
    gz = GorozenForCausalLM(GorozenConfig.from_dict(gorozen_config(W, H, G, 2 * D, F, 4, V)), dtype=torch.bfloat16, device=dev).eval()
    for p in gz.parameters():
        if p.dim() == 1 and p.dtype == torch.bfloat16:
            p.data.normal_(std=0.1)
    return du, gz


@torch.no_grad()
def end_to_end(size, dev, steps, warmup, prompt=2048, batch=32, ctx=1024):
    """tokens/s of (a) one prompt of ``prompt`` tokens, (b) one decode step of ``batch`` sequences at context ``ctx``."""
    from llm_in_practise_b200.inference import RaggedGenerator
    t = Timer(dev, flush=False)
    out = {}
    V = SIZES[size][-1]
    toks = torch.randint(0, V, (prompt,)).tolist()
    for name, model in zip(("duratar", "gorozen"), build_models(size, dev)):
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
    """Single kernels at the layer sizes: (name, Duratar ms, fraction of roofline, Gorozen like-kernel or None, ms, fraction, bound)."""
    from llm_in_practise_b200.inference.ragged import TILE_Q, Pieces
    from llm_in_practise_b200.ops import elementwise as ew
    from llm_in_practise_b200.ops.hyper import gated_group_norm, hc_step, xielu
    from llm_in_practise_b200.ops.linear_scan import delta_gates, linear_scan, short_conv
    from llm_in_practise_b200.ops.multimap_attention import multimap_attention, qknorm_rope_store
    from llm_in_practise_b200.ops.norm import sandwich_norm
    from llm_in_practise_b200.ops.paged_attention import paged_attention, rope_paged_store
    hbm, tf, which = _peaks(root)
    W, H, G, D, Dv, win, keep, SH, SD, SDv, SG, taps, F, V = SIZES[size]
    gD = 2 * D
    t = GraphTimer(dev)
    rows = []
    bf = torch.bfloat16
    T = 4096

    def frac_bw(nbytes, ms):
        return nbytes / (ms * 1e-3) / 1e9 / hbm

    def frac_fl(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / tf

    # --- stream write + read + norm (2 streams) vs post-norm + residual + pre-norm
    S = 2
    y32, X = torch.randn(T, W, device=dev), torch.randn(T, S, W, device=dev)
    ls, mix, co, ci, gn = torch.ones(W, device=dev), torch.eye(S, device=dev), torch.ones(S, device=dev), torch.ones(S, device=dev), torch.ones(1, device=dev)
    ms_d = t(lambda: hc_step(y32, ls, X, mix, co, ci, gn, 1e-6, bf), steps, warmup)
    res = torch.randn(T, W, device=dev)
    w2 = torch.zeros(W, dtype=bf, device=dev)
    ms_g = t(lambda: sandwich_norm(y32, w2, res, w2, 1e-6, 1.0, bf), steps, warmup)
    rows.append(("stream write + read + one-number norm, 2 streams", ms_d, frac_bw(T * W * (4 + 8 * S + 2), ms_d),
                 "post-norm + residual + pre-norm", ms_g, frac_bw(T * W * 14, ms_g), "HBM"))
    # --- q/k norm + rotary + page store vs rotary + page store
    BS = 64
    nb = T // BS
    ck, cv = torch.zeros(nb + 1, G * 2, BS, D, dtype=bf, device=dev), torch.zeros(nb + 1, G, BS, Dv, dtype=bf, device=dev)
    table = torch.arange(1, nb + 1, dtype=torch.int32, device=dev).view(1, nb)
    pos = torch.arange(T, dtype=torch.int32, device=dev)
    slot = torch.zeros(T, dtype=torch.int32, device=dev)
    ncol = (H + G) * 2 * D + G * Dv
    proj = torch.randn(T, ncol, device=dev)
    wq, wk = torch.ones(D, device=dev), torch.ones(D, device=dev)
    cos, sin = ew.rope_tables_partial(T, D, 1e6, dev)
    ms_d = t(lambda: qknorm_rope_store(proj, wq, wk, cos, sin, pos, slot, ck, cv, table, H, G, 2, D, Dv, D, 1e-6, bf), steps, warmup)
    gk, gv = torch.zeros(nb + 1, G, BS, gD, dtype=bf, device=dev), torch.zeros(nb + 1, G, BS, gD, dtype=bf, device=dev)
    qk = torch.randn(T, (H + G) * gD, device=dev).to(bf)
    cos2, sin2 = ew.rope_tables_partial(T, gD, 1e6, dev)
    ms_g = t(lambda: rope_paged_store(qk, cos2, sin2, pos, slot, gk, gv, table, H, G, gD, gD, True, True), steps, warmup)
    rows.append(("q/k norm + rotary + K/V page store (fp32 in)", ms_d, frac_bw(T * (ncol * 4 + ((H + G) * 2 * D + G * Dv) * 2), ms_d),
                 "rotary + K/V page store", ms_g, frac_bw(T * ((H + G) * gD * 2 * 2 + 2 * G * gD * 2), ms_g), "HBM"))
    # --- prompt attention, 4096 tokens of one sequence
    tiles = torch.tensor([[q0, min(TILE_Q, T - q0), q0, 0] for q0 in range(0, T, TILE_Q)], dtype=torch.int32, device=dev)
    pieces = Pieces(tiles, tiles.shape[0], T, torch.tensor([[0, T, 0, 0]], dtype=torch.int32, device=dev), 1)
    ck.normal_()
    cv.normal_()
    q = torch.randn(T, H * 2 * D, device=dev).to(bf)
    seen = sum(min(p + 1, win) + max(0, min(keep, p + 1 - win)) for p in range(T))
    ms_w = t(lambda: multimap_attention(q, ck, cv, table, pos, slot, H, G, 2, D, Dv, D ** -0.5, win, keep, True, 0.4, 0.7, 1e-6, pieces), steps, warmup)
    ms_d = t(lambda: multimap_attention(q, ck, cv, table, pos, slot, H, G, 2, D, Dv, D ** -0.5, 0, 0, True, 0.4, 0.7, 1e-6, pieces), steps, warmup)
    gk.normal_()
    gv.normal_()
    sinks = torch.zeros(H, device=dev)
    ms_g = t(lambda: paged_attention(qk, gk, gv, table, pos, slot, H, G, gD, gD ** -0.5, sinks=sinks, max_pos=T - 1, pieces=pieces), steps, warmup)
    fl = lambda keys: 2 * H * 2 * (D + Dv) * keys                                                            # noqa: E731
    rows.append(("prompt attention, 2 maps, causal (mma.sync)", ms_d, frac_fl(fl(T * (T + 1) / 2), ms_d),
                 "prompt attention (paged, sinks, mma.sync)", ms_g, frac_fl(4 * H * gD * T * T / 2, ms_g), "bf16 tensor"))
    rows.append((f"prompt attention, 2 maps, window {win} + {keep} kept (mma.sync)", ms_w, frac_fl(fl(seen), ms_w), None, 0.0, 0.0, "bf16 tensor"))
    # --- decode attention: 64 sequences at context 4032, window on both sides
    Bq, ctx = 64, 4032
    nbd = Bq * (ctx // BS + 1)
    ckd, cvd = torch.randn(nbd + 1, G * 2, BS, D, device=dev).to(bf), torch.randn(nbd + 1, G, BS, Dv, device=dev).to(bf)
    tabd = torch.arange(1, nbd + 1, dtype=torch.int32, device=dev).view(Bq, -1)
    posd = torch.full((Bq,), ctx, dtype=torch.int32, device=dev)
    slotd = torch.arange(Bq, dtype=torch.int32, device=dev)
    qd = torch.randn(Bq, H * 2 * D, device=dev).to(bf)
    ms_d = t(lambda: multimap_attention(qd, ckd, cvd, tabd, posd, slotd, H, G, 2, D, Dv, D ** -0.5, win, keep, True, 0.4, 0.7, 1e-6), steps, warmup)
    ms_f = t(lambda: multimap_attention(qd, ckd, cvd, tabd, posd, slotd, H, G, 2, D, Dv, D ** -0.5, 0, 0, True, 0.4, 0.7, 1e-6), steps, warmup)
    del ckd, cvd
    gkd, gvd = torch.randn(nbd + 1, G, BS, gD, device=dev).to(bf), torch.randn(nbd + 1, G, BS, gD, device=dev).to(bf)
    qgd = torch.randn(Bq, (H + G) * gD, device=dev).to(bf)
    ms_g = t(lambda: paged_attention(qgd, gkd, gvd, tabd, posd, slotd, H, G, gD, gD ** -0.5, sinks=sinks, window=win, max_pos=ctx), steps, warmup)
    ms_gf = t(lambda: paged_attention(qgd, gkd, gvd, tabd, posd, slotd, H, G, gD, gD ** -0.5, sinks=sinks, max_pos=ctx), steps, warmup)
    del gkd, gvd
    rows.append((f"decode attention, 64 seqs at 4032, window {win} + {keep}", ms_d, frac_bw(Bq * G * (win + keep) * (2 * D + Dv) * 2, ms_d),
                 f"decode attention (paged, sinks), window {win}", ms_g, frac_bw(Bq * G * win * gD * 2 * 2, ms_g), "HBM"))
    rows.append(("decode attention, 64 seqs at 4032, no window", ms_f, frac_bw(Bq * G * (ctx + 1) * (2 * D + Dv) * 2, ms_f),
                 "decode attention (paged, sinks), no window", ms_gf, frac_bw(Bq * G * (ctx + 1) * gD * 2 * 2, ms_gf), "HBM"))
    # --- activation
    z = torch.randn(T, F, device=dev).to(bf)
    pq = torch.tensor([0.3, -0.5], device=dev)
    gu = torch.randn(T, 2 * F, device=dev).to(bf)
    ms_d = t(lambda: xielu(z, pq), steps, warmup)
    ms_g = t(lambda: ew.clamped_glu(gu, 7.0, 1.702, 1.0), steps, warmup)
    rows.append(("xIELU", ms_d, frac_bw(T * F * 2 * 2, ms_d), "clamped gated unit", ms_g, frac_bw(T * F * 2 * 3, ms_g), "HBM"))
    # --- recurrent mixers: one prompt of 4096 tokens, and a decode batch of 64
    C = 2 * SG * SD + SH * SDv
    runs = torch.tensor([[0, T, 0, 0]], dtype=torch.int32, device=dev)
    xin = torch.randn(T, C + 8, device=dev)
    cw = torch.randn(C, taps, device=dev) * 0.5
    tail = torch.zeros(65, taps - 1, C, device=dev)
    ms_d = t(lambda: short_conv(xin[:, :C], cw, tail, pos, slot, runs, 1), steps, warmup)
    rows.append((f"short convolution ({taps} taps) + silu + tail, {C} channels", ms_d, frac_bw(T * C * 8, ms_d), None, 0.0, 0.0, "HBM"))
    qs = torch.randn(T, SG * SD, device=dev) * SD ** -0.5
    ks = torch.nn.functional.normalize(torch.randn(T, SG, SD, device=dev), dim=-1).view(T, -1)
    vs = torch.randn(T, SH * SDv, device=dev)
    ga, be = torch.rand(T, SH * SD, device=dev) * 0.1 + 0.9, torch.rand(T, SH, device=dev)
    aa, bb = torch.randn(T, SH * SD, device=dev), torch.randn(T, SH, device=dev)
    dtb, alog = torch.zeros(SH * SD, device=dev), torch.zeros(SH, device=dev)
    ms_d = t(lambda: delta_gates(qs, ks, aa, bb, dtb, alog, SG, SH, SD, 1.0), steps, warmup)
    rows.append(("unit q / k, decays, beta (in place)", ms_d, frac_bw(T * (2 * SG * SD + SH * SD + SH) * 8, ms_d), None, 0.0, 0.0, "HBM"))
    state = torch.zeros(65, SH, SD, SDv, device=dev)
    dec = torch.full((SH,), 0.99, device=dev)
    q16, k16 = torch.randn(T, SH * SD, device=dev) * SD ** -0.5, torch.randn(T, SH * SD, device=dev) * SD ** -0.5
    for mode, fl_tok, args in (("decay", 2 * 2 * SD * SDv, dict(decay=dec)), ("delta", 3 * 2 * SD * SDv, dict(g=ga, beta=be))):
        qq, kk, g_ = (q16, k16, SH) if mode == "decay" else (qs, ks, SG)
        ms_d = t(lambda: linear_scan(qq, kk, vs, state, pos, slot, runs, 1, SH, g_, SD, SDv, mode, **args), steps, warmup)
        fr = SH * fl_tok * T / (ms_d * 1e-3) / 1e12 / FP32_TFLOPS
        rows.append((f"state scan ({mode}), one prompt of {T} tokens, {SH} heads of {SD} x {SDv}", ms_d, fr, None, 0.0, 0.0, "nominal fp32 FMA rate"))
        pd, sd_ = torch.full((Bq,), 77, dtype=torch.int32, device=dev), torch.arange(Bq, dtype=torch.int32, device=dev)
        ms_b = t(lambda: linear_scan(qq[:Bq], kk[:Bq], vs[:Bq], state, pd, sd_, None, Bq, SH, g_, SD, SDv, mode, **args), steps, warmup)
        rows.append((f"state scan ({mode}), decode batch of {Bq}", ms_b, frac_bw(Bq * SH * SD * SDv * 8, ms_b), None, 0.0, 0.0, "HBM"))
    o32, gate = torch.randn(T, SH * SDv, device=dev), torch.randn(T, SH * SDv, device=dev)
    wn = torch.ones(SDv, device=dev)
    ms_d = t(lambda: gated_group_norm(o32, gate, wn, SH, 1e-6, bf), steps, warmup)
    rows.append(("per-head norm + sigmoid gate", ms_d, frac_bw(T * SH * SDv * 10, ms_d), None, 0.0, 0.0, "HBM"))
    return rows, which


def run(args, root):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    from llm_in_practise_b200.ops import _native as nv
    nv.lib()
    n0 = nv.launch_count
    t0 = time.time()
    res = {"metric": "Duratar vs Gorozen at equal layer sizes: prefill / decode tok/s", "unit": "tok/s", "n_gpus": 1,
           "steps": args.steps, "warmup": max(3, args.warmup), "dtype": "bf16", "data": "synthetic", "sizes": {}, "kernels": {}}
    first = next(iter(SIZES))
    for size in SIZES:
        res["sizes"][size] = {k: round(v, 2) for k, v in end_to_end(size, dev, args.steps, args.warmup).items()}
        torch.cuda.empty_cache()
    for size in SIZES:
        rows, which = kernel_rows(size, dev, args.steps, args.warmup, root)
        res["kernels"][size] = [{"duratar": a, "ms": round(b, 4), "of_roofline": round(c, 3), "gorozen": d, "gorozen_ms": round(e, 4),
                                 "gorozen_of_roofline": round(f, 3), "bound": g, "gap_ratio": round(f / c, 2) if c and d else None}
                                for a, b, c, d, e, f, g in rows]
        res["roofline"] = which
        torch.cuda.empty_cache()
    res["gpu_launches"] = nv.launch_count - n0
    res["seconds"] = round(time.time() - t0, 1)
    res["value"] = res["sizes"][first]["duratar_decode_tok_s"]
    res["config"] = {"model": "duratar: attention, channel_delta, attention on shared keys, lightning; one layer each",
                     "sizes": {k: list(v) for k, v in SIZES.items()},
                     "l2": "single kernels: replayed from a CUDA graph, 256 MB flush between iterations; steps: weights + cache exceed L2"}
    print(json.dumps(res))
    return 0
