"""Runner for models whose compute path is the ragged serving step (``model.forward_ragged``): one call takes any mix of
prompt pieces and single decoded tokens of different sequences, with all K/V in a paged cache.

``RaggedGenerator`` is what ``Generator`` is for the Qwen family — the object ``serve.engine.LLMEngine`` schedules onto and
``model.generate`` runs — but it has ONE forward entry, ``step``: whole prompts, pieces of prompts, decode batches and
mixtures of them are the same call with different token lists, so a position's logits cannot depend on how its prompt was
cut or on what shared the batch. The cache helpers of ``Generator`` (block rows, host off-load of cached prefixes) are
inherited: they only touch the cache object.

The reference reaches the same behaviour through vLLM's scheduler (chunked prefill mixed into decode batches,
Deployment/Ray/serve_run_examples/deepseek.py:29-34).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import torch

from ..ops.gemm import ensure_graph_workspace
from ..utils.graph_step import no_gc

from .generate import GenerationConfig, Generator, PagedKVCache, sample_next

TILE_Q = 64          # query rows per tile of the tensor-core attention kernel


@dataclass
class Pieces:
    """Runs of consecutive tokens of one sequence inside a step, cut into tiles of at most ``TILE_Q`` query rows:
    ``tiles`` int32 [n_tiles, 4] = (first row in the batch, rows, position of the first row, cache row)."""
    tiles: torch.Tensor
    n_tiles: int
    longest: int                    # tokens of the longest run
    runs: Optional[torch.Tensor] = None     # int32 [n_runs, 4] = (first row, rows, position of the first row, cache row): whole runs,
    n_runs: int = 0                         # walked in order by the recurrent mixers (ops.linear_scan)

    def use_mma(self, q: torch.Tensor, head_dim: int, window: int, scale: float = 1.0) -> bool:
        return (self.longest >= 8 and scale > 0 and q.dtype == torch.bfloat16 and head_dim % 16 == 0 and head_dim <= 128
                and window == 0 and os.environ.get("B200_PAGED_MMA", "1") != "0")


def make_pieces(runs: Sequence[Sequence[int]], device) -> Pieces:
    """``Pieces`` of a step from its runs ``(first row, rows, position of the first row, cache row)``: every run whole (for
    the recurrent mixers) and cut into tiles of at most ``TILE_Q`` rows (for the tensor-core attention kernels)."""
    runs = [[int(v) for v in r] for r in runs if r[1] > 0]
    tiles = [[first + q0, min(TILE_Q, n - q0), p0 + q0, row] for first, n, p0, row in runs for q0 in range(0, n, TILE_Q)]
    tl = torch.tensor(tiles + runs, dtype=torch.int32)
    tl = tl.pin_memory().to(device, non_blocking=True) if torch.device(device).type == "cuda" else tl
    return Pieces(tl[:len(tiles)], len(tiles), max((r[1] for r in runs), default=0), tl[len(tiles):], len(runs))


Entry = Tuple[int, int, Sequence[int], Sequence[int]]       # (cache row, first position, tokens, wanted indices into tokens)


class RaggedGenerator(Generator):
    ragged = True

    def __init__(self, model, tokenizer=None, max_len: int = 4096):
        super().__init__(model, tokenizer, max_len)
        self._graph_decode = os.environ.get("B200_RAGGED_GRAPH", "1") != "0"

    # ------------------------------------------------------------------ cache
    def make_cache(self, num_blocks: int, block_size: int, max_seqs: int, max_len: int) -> PagedKVCache:
        """A paged cache with one pool per layer, each sized from that layer's own (kv heads, head size). Physical block 0
        is left to unset table entries; callers hand out blocks 1 .. num_blocks."""
        m = self.model
        lay = self._kv_layout()
        states = m.state_layout() if hasattr(m, "state_layout") else None
        cache = PagedKVCache(len(lay), num_blocks + 1, [e[0] for e in lay], block_size, [e[1] for e in lay], m.embed_tokens.dtype,
                             m.embed_tokens.device, max_seqs + 1, max_len, Dv=[e[2] for e in lay], Hv=[e[3] for e in lay],
                             state_shapes=states)
        cache.scratch_row = max_seqs             # a row that never gets blocks: padding tokens of a bucketed batch write to block 0
        return cache

    def _kv_layout(self):
        """(key rows per token, key row size, value row size, value heads) per layer; a model's ``kv_layout`` may give pairs
        (values sized like keys), triples (value size 0: the layer keeps no value pool, e.g. a latent cache whose rows serve
        as both) or all four (several key rows per value head; 0 key rows: the layer has no pool of its own)."""
        return [(e[0], e[1], e[2] if len(e) > 2 else e[1], e[3] if len(e) > 3 else e[0]) for e in self.model.kv_layout()]

    def kv_token_bytes(self) -> int:
        es = self.model.embed_tokens.element_size()
        return sum((g * d + gv * dv) * es for g, d, dv, gv in self._kv_layout())

    def state_bytes(self) -> int:
        """Bytes of recurrent state one live sequence holds (fp32), over all layers."""
        m = self.model
        if not hasattr(m, "state_layout"):
            return 0
        n = 0
        for shapes in m.state_layout():
            for shp in shapes:
                k = 4
                for d in shp:
                    k *= d
                n += k
        return n

    # ------------------------------------------------------------------ the step
    @torch.no_grad()
    def step(self, entries: Sequence[Entry], cache: PagedKVCache, layer_outputs: Optional[list] = None) -> Optional[torch.Tensor]:
        """Run the tokens of ``entries`` as one batch; their cache rows must already list blocks for the positions they
        write. Returns the fp32 logits of the wanted tokens in entry order [n_wanted, vocab], or None if nothing is wanted
        (the K/V of the tokens are stored all the same)."""
        dev = self.model.embed_tokens.device
        if (dev.type == "cuda" and layer_outputs is None and self._graph_decode and entries
                and all(len(e[2]) == 1 and list(e[3]) == [0] for e in entries)):
            return self.decode([e[2][0] for e in entries], [e[1] for e in entries], [e[0] for e in entries], cache)
        ids: List[int] = []
        pos: List[int] = []
        slot: List[int] = []
        want: List[int] = []
        runs: List[List[int]] = []
        max_pos = 0
        for row, pos0, toks, wanted in entries:
            n = len(toks)
            if n == 0:
                continue
            if pos0 + n > cache.max_len:
                raise ValueError(f"sequence of {pos0 + n} tokens does not fit the cache rows of {cache.max_len}")
            base = len(ids)
            ids.extend(int(t) for t in toks)
            pos.extend(range(pos0, pos0 + n))
            slot.extend([row] * n)
            want.extend(base + int(w) for w in wanted)
            runs.append([base, n, pos0, row])
            max_pos = max(max_pos, pos0 + n - 1)
        if not ids:
            return None
        meta = torch.tensor(pos + slot, dtype=torch.int32).view(2, -1)
        if dev.type == "cuda":
            meta = meta.pin_memory().to(dev, non_blocking=True)
            ids_t = torch.tensor(ids, dtype=torch.long).pin_memory().to(dev, non_blocking=True)
        else:
            ids_t = torch.tensor(ids, dtype=torch.long)
        pieces = make_pieces(runs, dev)
        want_t = torch.tensor(want, dtype=torch.long, device=dev) if want else torch.zeros(1, dtype=torch.long, device=dev)
        logits = self.model.forward_ragged(ids_t, meta[0], meta[1], cache, want_t, max_pos=max_pos, pieces=pieces,
                                           layer_outputs=layer_outputs)
        return logits if want else None

    @torch.no_grad()
    def decode(self, tokens: Sequence[int], positions: Sequence[int], rows: Sequence[int], cache: PagedKVCache) -> torch.Tensor:
        """One token per sequence (``tokens[i]`` at ``positions[i]`` of cache row ``rows[i]``), replayed from a CUDA graph: a
        decode step is ~10 short launches per layer, so eager execution is bound by the launch rate. One graph per
        (batch bucket, context bucket, cache); token ids, positions and rows are read from device tensors, padding rows of
        the bucket write to the cache's scratch row. Returns fp32 logits [len(tokens), vocab]."""
        dev = self.model.embed_tokens.device
        n = len(tokens)
        nb = 1
        while nb < n:
            nb *= 2
        mp = 64
        while mp < max(positions) + 1:
            mp *= 2
        mp = min(mp, cache.max_len)
        pad = nb - n
        host = torch.tensor([list(tokens) + [0] * pad, list(positions) + [0] * pad, list(rows) + [cache.scratch_row] * pad], dtype=torch.int64)
        # the graphs live on the cache they were captured against (they hold its addresses): they go when it goes, and a new
        # cache that happens to get the old one's id() cannot pick them up
        graphs = cache.__dict__.setdefault("_decode_graphs", {})
        key = (nb, mp)
        g = graphs.get(key)
        if g is None:
            st = {"ids": torch.zeros(nb, dtype=torch.long, device=dev), "pos": torch.zeros(nb, dtype=torch.int32, device=dev),
                  "slot": torch.full((nb,), cache.scratch_row, dtype=torch.int32, device=dev)}
            ensure_graph_workspace(dev)
            self.model.forward_ragged(st["ids"], st["pos"], st["slot"], cache, None, max_pos=mp - 1)       # warm-up: lazily built buffers
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with no_gc(), torch.cuda.graph(graph):
                st["logits"] = self.model.forward_ragged(st["ids"], st["pos"], st["slot"], cache, None, max_pos=mp - 1)
            g = graphs[key] = (graph, st)
        graph, st = g
        hd = host.pin_memory().to(dev, non_blocking=True)
        st["ids"].copy_(hd[0])
        st["pos"].copy_(hd[1])
        st["slot"].copy_(hd[2])
        graph.replay()
        return st["logits"][:n].clone()          # the graph's output buffer is rewritten by the next replay

    # ------------------------------------------------------------------ single-process generation
    def _generate(self, input_ids: torch.Tensor, config: Optional[GenerationConfig], streamer, seed: Optional[int],
                  return_logprobs: bool, **kw):
        """Same interface as ``Generator.generate``: [B, S] prompts -> [B, S + new] ids. The prompts are one ragged step, every
        following step decodes one token per unfinished sequence."""
        cfg = config or GenerationConfig(**{k: v for k, v in kw.items() if k in GenerationConfig.__dataclass_fields__})
        eos = cfg.eos_token_id
        eos = [] if cfg.ignore_eos else ([eos] if isinstance(eos, int) else list(eos or []))
        B, S = input_ids.shape
        dev = input_ids.device
        total = min(self.max_len, S + cfg.max_new_tokens)
        bs = 64
        per = -(-total // bs)
        key = ("gen", B, per)
        cache = self._caches.get(key)
        if cache is None:
            self._caches.clear()
            cache = self._caches[key] = self.make_cache(B * per, bs, B, per * bs)
            for b in range(B):
                self.set_block_row(cache, b, list(range(1 + b * per, 1 + (b + 1) * per)))
        gen = torch.Generator(device=dev).manual_seed(seed) if seed is not None else None
        rows = input_ids.tolist()
        logits = self.step([(b, 0, rows[b], [S - 1]) for b in range(B)], cache)
        out = input_ids
        done = torch.zeros(B, dtype=torch.bool, device=dev)
        logprobs: List[torch.Tensor] = []
        for n in range(S, total):
            nxt = sample_next(logits, cfg, out, gen)
            if return_logprobs:
                logprobs.append(logits.float().log_softmax(-1).gather(1, nxt[:, None]).squeeze(1))
            nxt = torch.where(done, torch.full_like(nxt, cfg.pad_token_id), nxt)
            out = torch.cat([out, nxt[:, None]], 1)
            if streamer is not None:
                streamer.put(nxt)
            for e in eos:
                done |= nxt == e
            if bool(done.all()) or n + 1 >= total:
                break
            last = nxt.tolist()
            logits = self.step([(b, n, [last[b]], [0]) for b in range(B)], cache)
        return (out, torch.stack(logprobs, 1)) if return_logprobs else out
