"""Replay recorded traffic through the serving engine and write the logits it produces (no sampling).

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N  < steps.jsonl

Each input line is one engine step, ``{"step": n, "entries": [{"id": .., "tokens": [..], "want": [..]}, ..], "end": [..]}``:
the next tokens of some requests (whole prompts, pieces of prompts and single tokens may share a step) and the indices
among them whose logits are wanted. A step with wanted logits writes ``<out>/<step>.f32`` (little-endian fp32
[wanted, vocab], entry order) and every step answers ``done <step>`` on standard output. Requests listed under ``end``
return their sequence slot and cache blocks to the pools. The model class comes from ``config.json`` through the model
registry, the steps run on ``LLMEngine.replay_step`` — the engine's own slots, block allocator, paged cache and model
step. ``--max-tokens`` sizes the KV block pool (blocks of 64 tokens); four sequences may be live at a time.

The first call in a fresh checkout compiles the kernels the model needs (``_build.ensure_built``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

# kernel sources (csrc/<stem>.cu) behind each served design: what a fresh checkout has to compile before the first step
NATIVE_SOURCES = {
    "Gorozen": ["gemm_tcgen05", "gemv", "gemm_simt", "norm", "elementwise", "paged_attn", "moe"],
    "Segorax": ["gemm_tcgen05", "gemv", "gemm_simt", "norm", "elementwise", "latent_attn", "moe"],
    "Duratar": ["gemm_tcgen05", "gemv", "gemm_simt", "elementwise", "hyper_conn", "multimap_attn", "multimap_attn_mma",
                "linear_scan"],
    "Kudonex": ["gemm_tcgen05", "gemv", "gemm_simt", "norm", "elementwise", "paged_attn", "moe", "linear_scan", "talking_attn",
                "talking_attn_mma"],
}
BLOCK = 64
MAX_LIVE = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", dest="max_tokens", type=int, required=True)
    ap.add_argument("--device", default=None)
    a = ap.parse_args(argv)

    with open(os.path.join(a.model, "config.json")) as f:
        arch = json.load(f).get("architecture")
    import torch
    dev = a.device or ("cuda" if torch.cuda.is_available() else "cpu")
    if dev.startswith("cuda"):
        from .. import _build
        _build.ensure_built(NATIVE_SOURCES.get(arch) or [s.stem for s in _build.CSRC.glob("*.cu")])
    from ..io.hf import from_pretrained
    from ..serve.engine import EngineArgs, LLMEngine

    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    model = from_pretrained(a.model, dtype=getattr(torch, a.dtype), device=torch.device(dev))
    if not getattr(model, "ragged", False):
        print(f"{arch or 'this model'} has no ragged step to replay on", file=sys.stderr)
        return 3
    blocks = -(-a.max_tokens // BLOCK)
    eng = LLMEngine(model, None, EngineArgs(max_num_seqs=MAX_LIVE, max_model_len=blocks * BLOCK, block_size=BLOCK,
                                            num_kv_blocks=blocks, enable_prefix_caching=False, warmup=False))
    os.makedirs(a.out, exist_ok=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        st = json.loads(line)
        entries = [(e["id"], e["tokens"], e.get("want") or []) for e in st.get("entries", [])]
        logits = eng.replay_step(entries, st.get("end") or [])
        if logits is not None:
            tmp = os.path.join(a.out, f".{st['step']}.tmp")
            with open(tmp, "wb") as f:
                f.write(logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4").tobytes())
            os.replace(tmp, os.path.join(a.out, f"{st['step']}.f32"))
        elif dev.startswith("cuda"):
            torch.cuda.synchronize()
        sys.stdout.write(f"done {st['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
