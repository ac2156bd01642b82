"""Duratar against the plain float64 oracle in ``duratar_oracle.py``: every mechanism alone, then the model through the ragged
step, the serving engine's block / slot / state pools and its scheduler. Small random models of several shapes; the same
tests run on the CPU path and (marked ``gpu``) on the CUDA kernels in fp32 and bf16."""
import json

import pytest
import torch

import duratar_oracle as O

CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]


def tol(dtype):
    return 2e-4 if dtype == torch.float32 else 6e-2


def row_errs(got, want):
    """Per row: RMS difference over RMS of the oracle, means over the last axis removed."""
    got, want = got.double().cpu(), want.double().cpu()
    d = got - want
    d = d - d.mean(-1, keepdim=True)
    w = want - want.mean(-1, keepdim=True)
    return d.pow(2).mean(-1).sqrt() / w.pow(2).mean().sqrt()


def rel_err(got, want):
    return float(row_errs(got.reshape(1, -1), want.reshape(1, -1))[0])


def assert_rows(got, want, dtype, what=""):
    e = row_errs(got, want)
    assert float(e.max()) < tol(dtype), (what, float(e.max()), int(e.argmax()))


def build(tmp_path, cfg, W, device, dtype, name="m"):
    from llm_in_practise_b200.io.hf import from_pretrained
    from llm_in_practise_b200.io.safetensors import save_file
    d = tmp_path / name
    d.mkdir(exist_ok=True)
    (d / "config.json").write_text(json.dumps(cfg))
    save_file(W, str(d / "model.safetensors"))
    return from_pretrained(str(d), dtype=dtype, device=torch.device(device))


def fresh_cache(gen, n_seqs, max_len, block=64, poison=True):
    """A cache whose rows list their blocks in a scrambled physical order and whose state rows hold garbage: a sequence that
    starts at position 0 must not read what an earlier user of its row left."""
    per = -(-max_len // block)
    cache = gen.make_cache(n_seqs * per, block, n_seqs, per * block)
    ids = list(range(1, n_seqs * per + 1))[::-1]
    for s in range(n_seqs):
        gen.set_block_row(cache, s, ids[s::n_seqs][:per])
    if poison:
        for layer in cache.state:
            for t in layer:
                t.fill_(37.0)
    return cache


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


BANDS = {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}       # with base 100 and 16 dims: kept, blended and divided dims

VARIANTS = {
    # all three mixers, shared keys, a layer without a feed-forward; sizes the tensor-core attention kernel takes
    "mixed": lambda: O.make_config(64, 96, [
        O.attention_layer(4, 2, 32, 64, 40, 6, 16, base=100.0, scaling=BANDS, ff=80),
        O.delta_layer(4, 2, 16, 24, 4, ff=72),
        O.attention_layer(4, 2, 32, 64, 24, 3, 16, base=100.0, scaling=BANDS, kv_from=0, ff=0),
        O.lightning_layer(3, 16, 32, [0.7, 0.95, 0.999], ff=64)], streams=2),
    # recurrent layers first, three streams, one kv head for many heads, whole-head rotary, a window larger than any prompt
    "recurrent_first": lambda: O.make_config(48, 80, [
        O.lightning_layer(2, 24, 8, [0.9, 0.5], ff=0),
        O.delta_layer(2, 2, 8, 40, 2, ff=56),
        O.attention_layer(6, 1, 16, 16, 4096, 0, 16, base=50.0, scaling=None, diff=0.1, scale=0.9, ff=40)], streams=3),
    # one stream with coefficients, as many kv heads as heads, no rotary, a window of one token plus kept ones, conv of one tap
    "single_stream": lambda: O.make_config(40, 64, [
        O.attention_layer(2, 2, 16, 32, 1, 5, 0, diff=0.5, scale=1.2, ff=48),
        O.delta_layer(3, 1, 32, 8, 1, ff=0),
        O.attention_layer(2, 2, 16, 32, 7, 0, 8, base=10.0, kv_from=0, ff=32)], streams=1, eps=1e-3),
    # no ``streams`` in the config: the plain residual sum
    "plain_residual": lambda: O.make_config(32, 50, [
        O.delta_layer(2, 1, 16, 16, 3, ff=40),
        O.attention_layer(2, 1, 16, 16, 9, 2, 8, base=1e4, ff=0)], streams=None),
}

# sizes that are not multiples of the kernels' vector widths, ranks of 5 and 3, 4 streams, 5 taps
ODD = {
    "w72": lambda: O.make_config(72, 75, [
        O.attention_layer(6, 3, 20, 12, 33, 4, 10, base=1e4, scaling=BANDS, ff=100),
        O.delta_layer(6, 3, 12, 20, 5, ff=36),
        O.lightning_layer(5, 10, 14, [0.3, 0.6, 0.9, 0.99, 1.0], ff=20)], streams=4),
    "w100": lambda: O.make_config(100, 130, [
        O.lightning_layer(1, 40, 72, [0.97], ff=52),
        O.attention_layer(3, 3, 24, 40, 65, 64, 6, base=1e6, diff=0.05, ff=90),
        O.delta_layer(2, 2, 72, 36, 4, ff=0)], streams=2),
}


# ------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("S,W", [(1, 40), (2, 72), (3, 64), (4, 100), (8, 24), (13, 16)])
def test_hyper_connection_steps(device, dtype, S, W):
    from llm_in_practise_b200.ops.hyper import hc_entry, hc_read, hc_step
    g = torch.Generator().manual_seed(S)
    n, eps = 5, 1e-5
    e = torch.randn(n, W, generator=g).to(dtype)
    ge, g1, g2 = (torch.randn(1, generator=g) * 0.2 + 1 for _ in range(3))
    cin1, cin2, cout = (torch.randn(S, generator=g) for _ in range(3))
    mix = torch.randn(S, S, generator=g)
    ls = torch.randn(W, generator=g)
    y = torch.randn(n, W, generator=g) * 3
    dv = lambda t: t.to(device)                                     # noqa: E731
    h, X = hc_entry(dv(e), dv(ge), S, dv(cin1), dv(g1), eps, dtype)
    x0 = O.scalar_norm(e.double(), ge, eps)
    assert X.dtype == torch.float32 and X.shape == (n, S, W) and h.dtype == dtype
    for s in range(S):
        torch.testing.assert_close(X[:, s].cpu().double(), x0, rtol=1e-5, atol=1e-5)
    t = tol(dtype) / 4
    torch.testing.assert_close(h.cpu().double(), O.scalar_norm(sum(cin1[s].double() * x0 for s in range(S)), g1, eps), rtol=t, atol=t)
    # streams that differ, then one write + read
    X0 = torch.randn(n, S, W, generator=g)
    Xd = dv(X0.clone())
    h2, xs = hc_step(dv(y), dv(ls), Xd, dv(mix), dv(cout), dv(cin2), dv(g2), eps, dtype, want_sum=True)
    new = [sum(mix[s, to].double() * X0[:, s].double() for s in range(S)) + cout[to].double() * (y.double() * ls.double()) for to in range(S)]
    for s in range(S):
        torch.testing.assert_close(Xd[:, s].cpu().double(), new[s], rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(xs.cpu().double(), sum(new), rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(h2.cpu().double(), O.scalar_norm(sum(cin2[s].double() * new[s] for s in range(S)), g2, eps), rtol=t, atol=t)
    h3 = hc_read(Xd, None, dv(g1), eps, dtype)
    torch.testing.assert_close(h3.cpu().double(), O.scalar_norm(sum(new), g1, eps), rtol=t, atol=t)
    # no read: the last sublayer only writes
    assert hc_step(dv(y), None, Xd, dv(mix), dv(cout), None, None, eps, dtype)[0] is None


@pytest.mark.parametrize("device,dtype", CASES)
def test_xielu_and_gated_group_norm(device, dtype):
    from llm_in_practise_b200.ops.hyper import gated_group_norm, xielu
    g = torch.Generator().manual_seed(2)
    t = tol(dtype) / 4
    for pq in ([0.3, -0.8], [-2.0, 1.5], [0.0, 0.0]):
        z = (torch.randn(9, 52, generator=g) * 3).to(dtype)
        pqt = torch.tensor(pq)
        got = xielu(z.to(device), pqt.to(device))
        assert got.dtype == dtype
        torch.testing.assert_close(got.cpu().double(), O.xielu(z.double(), pq[0], pq[1]), rtol=t, atol=2 * t)
    # both branches meet at 0 with slope 1/2 and differ in curvature
    a = O.xielu(torch.tensor([-1e-4, 1e-4], dtype=torch.float64), 0.3, -0.8)
    assert abs(float(a[1] + a[0])) < 1e-7 and abs(float(a[1]) - 5e-5) < 1e-7
    for groups, GS in ((1, 56), (4, 24), (3, 40)):
        n = 6
        o = torch.randn(n, groups * GS, generator=g) * 2
        wide = torch.randn(n, groups * GS + 16, generator=g)           # the gate is a column slice of a wider projection
        gate = wide[:, 8:8 + groups * GS]
        w = torch.randn(GS, generator=g)
        got = gated_group_norm(o.to(device), wide.to(device)[:, 8:8 + groups * GS], w.to(device), groups, 1e-5, dtype)
        ref = (O.rms(o.double().view(n, groups, GS), 1e-5) * w.double()).view(n, -1) * torch.sigmoid(gate.double())
        torch.testing.assert_close(got.cpu().double(), ref, rtol=t, atol=t)


def test_band_scaled_frequencies():
    from llm_in_practise_b200.models.duratar import _band_scaling
    from llm_in_practise_b200.ops.elementwise import rope_inv_freq
    f0 = O.rope_freqs(16, 100.0, None)
    f = O.rope_freqs(16, 100.0, BANDS)
    ratio = [a / b for a, b in zip(f, f0)]
    assert any(abs(r - 1.0) < 1e-12 for r in ratio) and any(abs(r - 1 / 4) < 1e-12 for r in ratio)
    assert any(1 / 4 + 1e-6 < r < 1 - 1e-6 for r in ratio)
    for dims, base, sc in ((16, 100.0, BANDS), (8, 1e4, {"factor": 8.0, "low": 2.0, "high": 16.0, "original": 256}), (6, 7.0, None),
                           (32, 5e5, {"factor": 2.0, "low": 0.5, "high": 3.0, "original": 1000})):
        inv, att = rope_inv_freq(dims, base, _band_scaling(sc), dtype=torch.float64)
        torch.testing.assert_close(inv, torch.tensor(O.rope_freqs(dims, base, sc), dtype=torch.float64), rtol=1e-9, atol=0)
        assert att == 1.0


def _table(n_rows, per, device):
    """Block table rows with scrambled physical blocks (block 0 unused)."""
    ids = list(range(1, n_rows * per + 1))[::-1]
    return torch.tensor([ids[s::n_rows][:per] for s in range(n_rows)], dtype=torch.int32, device=device)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,G,D,Dv,rot,own", [(4, 2, 32, 64, 16, True), (3, 1, 20, 12, 20, True), (2, 2, 16, 8, 0, True), (4, 4, 24, 40, 6, False)])
def test_qknorm_rope_store(device, dtype, H, G, D, Dv, rot, own):
    from llm_in_practise_b200.ops.elementwise import rope_tables_partial
    from llm_in_practise_b200.ops.multimap_attention import qknorm_rope_store
    g = torch.Generator().manual_seed(3)
    BS, eps = 64, 1e-5
    pos = [0, 1, 63, 64, 65, 127, 128, 1023, 700]
    n = len(pos)
    nq, nk = H * 2 * D, G * 2 * D
    cols = -(-(nq + (nk + G * Dv if own else 0)) // 8) * 8
    proj = torch.randn(n, cols, generator=g) * 2
    wq, wk = torch.randn(D, generator=g), torch.randn(D, generator=g)
    cos, sin = rope_tables_partial(1024, rot, 300.0, device) if rot else (torch.zeros(1, 1, device=device),) * 2
    table = _table(1, 16, device)
    ck = torch.zeros(17, G * 2, BS, D, dtype=dtype, device=device) if own else None
    cv = torch.zeros(17, G, BS, Dv, dtype=dtype, device=device) if own else None
    pt = torch.tensor(pos, dtype=torch.int32, device=device)
    q = qknorm_rope_store(proj.to(device), wq.to(device), wk.to(device) if own else None, cos, sin, pt, torch.zeros_like(pt), ck, cv,
                          table, H, G, 2, D, Dv, rot, eps, dtype)
    fr = O.rope_freqs(rot, 300.0, None) if rot else []
    t = tol(dtype) / 4
    for i, p in enumerate(pos):
        qr = O.rotate_half(O.rms(proj[i, :nq].double().view(H * 2, D), eps) * wq.double(), p, fr)
        torch.testing.assert_close(q[i].cpu().double().view(H * 2, D), qr, rtol=t, atol=t)
        if own:
            kr = O.rotate_half(O.rms(proj[i, nq:nq + nk].double().view(G * 2, D), eps) * wk.double(), p, fr)
            blk = int(table[0, p // BS])
            torch.testing.assert_close(ck[blk, :, p % BS].cpu().double(), kr, rtol=t, atol=t)
            torch.testing.assert_close(cv[blk, :, p % BS].cpu().double(), proj[i, nq + nk:nq + nk + G * Dv].double().view(G, Dv), rtol=t, atol=t)


def _attention_case(device, dtype, H, G, D, Dv, size, keep, n, seed, targets, as_piece, max_pos=0):
    """Random q / k / v of one sequence with, for each (query position, key position) in ``targets``, the key scaled so that
    its score dominates if it is seen; the values of target keys are large, so a wrong mask moves the output by its size."""
    from llm_in_practise_b200.inference.ragged import Pieces
    from llm_in_practise_b200.ops.multimap_attention import multimap_attention
    g = torch.Generator().manual_seed(seed)
    BS = 64
    q = torch.randn(n, H, 2, D, generator=g).to(dtype)
    k = (torch.randn(n, G, 2, D, generator=g) * 0.3).to(dtype)
    v = torch.randn(n, G, Dv, generator=g).to(dtype)
    for qi, kj in targets:
        if 0 <= kj < n:
            k[kj] = (q[qi].float().view(G, H // G, 2, D)[:, 0] * 1.5).to(dtype)
            v[kj] = v[kj] * 8
    per = -(-n // BS)
    table = _table(2, per, device)
    ck = torch.zeros(2 * per + 1, G * 2, BS, D, dtype=dtype, device=device)
    cv = torch.zeros(2 * per + 1, G, BS, Dv, dtype=dtype, device=device)
    pl = torch.arange(n)
    blk = table[1, pl // BS].long().cpu()
    ck[blk, :, pl % BS] = k.view(n, G * 2, D).to(device)
    cv[blk, :, pl % BS] = v.to(device)
    lam, diff, eps, scale = 0.45, 0.3, 1e-5, 0.5
    ref = O.attend(q.double(), k.double(), v.double(), scale, size if size > 0 else 1 << 60, keep, lam, diff, eps)
    rows = sorted({qi for qi, _ in targets})
    if as_piece:                                          # the last rows as one prompt piece that starts in the middle of a page
        first = max(0, min(rows) - 3)
        sel = list(range(first, n))
        tiles = [[i, min(64, len(sel) - i), first + i, 1] for i in range(0, len(sel), 64)]
        pieces = Pieces(torch.tensor(tiles, dtype=torch.int32, device=device), len(tiles), len(sel),
                        torch.tensor([[0, len(sel), first, 1]], dtype=torch.int32, device=device), 1)
    else:
        sel, pieces = rows, None
    pos = torch.tensor(sel, dtype=torch.int32, device=device)
    out = multimap_attention(q[sel].reshape(len(sel), -1).to(device), ck, cv, table, pos, torch.ones_like(pos), H, G, 2, D, Dv, scale,
                             size, keep, combine=True, lam=lam, post=1 - diff, eps=eps, pieces=pieces, max_pos=max_pos)
    got = out.view(len(sel), H, Dv)
    for i, p in enumerate(sel):
        assert rel_err(got[i], ref[p]) < tol(dtype), (p, as_piece)
    return ref, rows


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("as_piece", [False, True])
@pytest.mark.parametrize("H,G,D,Dv", [(4, 2, 32, 64), (2, 1, 48, 96), (6, 3, 24, 40), (2, 2, 128, 128)])
def test_attention_window_edges_and_far_keys(device, dtype, as_piece, H, G, D, Dv):
    size, keep, n = 70, 5, 330
    # (query, key): just inside and just outside the window, the last kept token and the first one not kept, keys hundreds
    # back that are kept, page borders, the query's own key
    targets = [(329, 329 - 69), (328, 328 - 70), (327, 4), (326, 5), (325, 0), (324, 324), (323, 256), (322, 255), (321, 192)]
    ref, rows = _attention_case(device, dtype, H, G, D, Dv, size, keep, n, 5, targets, as_piece)
    # the construction works: a seen target dominates its row, an unseen one leaves it small
    big = ref[[329, 327, 325, 324]].abs().amax((-1, -2))
    assert float(big.min()) > 0
    # no window, nothing kept: a key 300 back is seen
    _attention_case(device, dtype, H, G, D, Dv, 0, 0, n, 6, [(329, 20), (328, 0), (300, 299)], as_piece)
    # the window covers less than the kept tokens near the start of a sequence
    _attention_case(device, dtype, H, G, D, Dv, 3, 10, 40, 7, [(12, 9), (12, 10), (12, 8), (2, 0), (11, 2), (39, 9), (39, 36), (38, 35)], as_piece)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,G,D,Dv,size,keep", [(4, 2, 32, 64, 0, 0), (2, 1, 24, 40, 0, 0), (4, 1, 64, 128, 1200, 30)])
def test_attention_long_context_decode_in_key_ranges(device, dtype, H, G, D, Dv, size, keep):
    """Few single tokens far into a sequence: their visible keys are cut into ranges that are merged afterwards; dominant
    keys sit in the first, a middle and the last range, at range borders and (with a window) on both sides of its edge."""
    n = 1400
    targets = [(1399, 0), (1398, 511), (1397, 512), (1396, 1396), (1395, 700), (1394, 1394 - 1199), (1393, 1393 - 1200), (1392, 29), (1391, 30)]
    _attention_case(device, dtype, H, G, D, Dv, size, keep, n, 9, targets, False, max_pos=n - 1)


@pytest.mark.parametrize("device,dtype", [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)])
@pytest.mark.parametrize("C,taps", [(24, 4), (7, 2), (40, 1), (16, 7)])
def test_short_conv_across_cuts(device, dtype, C, taps):
    from llm_in_practise_b200.ops.linear_scan import short_conv
    g = torch.Generator().manual_seed(C)
    n = 50
    xs = [torch.randn(L, C + 8, generator=g) for L in (n, 9, 1)]
    w = torch.randn(C, taps, generator=g)
    refs = [torch.nn.functional.silu(O.short_conv(x[:, 4:4 + C].double(), w.double())) for x in xs]
    tail = torch.full((4, taps - 1, C), 9.0, device=device)           # garbage: position 0 must not read it
    plans = [[20, 1, 2, 0, 1, 5, 21], [0, 9, 0, 0, 0, 0, 0], [0, 0, 0, 1, 0, 0, 0]]
    rows = [2, 0, 3]
    done = [0, 0, 0]
    outs = [[], [], []]
    for step in range(7):
        parts, runs, pos, slot = [], [], [], []
        for s in range(3):
            c = plans[s][step]
            if c:
                runs.append([len(pos), c, done[s], rows[s]])
                parts.append((s, c))
                pos += list(range(done[s], done[s] + c))
                slot += [rows[s]] * c
        x = torch.cat([xs[s][done[s]:done[s] + c] for s, c in parts], 0).to(device)
        single = all(c == 1 for _, c in parts)                        # a decode batch passes no runs
        rt = None if single else torch.tensor(runs, dtype=torch.int32, device=device)
        y = short_conv(x[:, 4:4 + C], w.to(device), tail, torch.tensor(pos, dtype=torch.int32, device=device),
                       torch.tensor(slot, dtype=torch.int32, device=device), rt, len(runs))
        o = 0
        for s, c in parts:
            outs[s].append(y[o:o + c])
            o += c
            done[s] += c
    for s in range(3):
        torch.testing.assert_close(torch.cat(outs[s], 0).cpu().double(), refs[s], rtol=1e-5, atol=1e-5)


def _scan_oracle(mode, q, k, v, H, G, decay=None, gk=None, beta=None):
    n, D, Dv = q.shape[0], q.shape[2], v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=torch.float64)
    o = torch.zeros(n, H, Dv, dtype=torch.float64)
    for t in range(n):
        for h in range(H):
            kv = h // (H // G)
            if mode == "decay":
                S[h] = decay[h] * S[h] + torch.outer(k[t, kv], v[t, h])
            else:
                S[h] = gk[t, h][:, None] * S[h]
                u = beta[t, h] * (v[t, h] - S[h].T @ k[t, kv])
                S[h] = S[h] + torch.outer(k[t, kv], u)
            o[t, h] = S[h].T @ q[t, kv]
    return o, S


@pytest.mark.parametrize("device,dtype", [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)])
@pytest.mark.parametrize("mode,H,G,D,Dv", [("decay", 3, 3, 16, 32), ("decay", 2, 2, 40, 12), ("decay", 1, 1, 128, 128), ("delta", 4, 2, 16, 24),
                                           ("delta", 2, 2, 72, 36), ("delta", 6, 1, 8, 8), ("delta", 2, 1, 128, 64)])
def test_linear_scan_across_cuts(device, dtype, mode, H, G, D, Dv):
    """The state carried in a reused row equals the sequential recurrence, however the sequence is cut; a second sequence in
    the same steps has its own state."""
    from llm_in_practise_b200.ops.linear_scan import linear_scan
    g = torch.Generator().manual_seed(D + Dv)
    lens = [90, 17]
    data, refs = [], []
    decay = torch.rand(H, generator=g) * 0.5 + 0.5
    for L in lens:
        q, k = torch.randn(L, G, D, generator=g) * D ** -0.5, torch.nn.functional.normalize(torch.randn(L, G, D, generator=g), dim=-1)
        v = torch.randn(L, H, Dv, generator=g)
        gk, beta = torch.rand(L, H, D, generator=g) * 0.3 + 0.7, torch.rand(L, H, generator=g)
        data.append((q, k, v, decay, gk, beta))
        refs.append(_scan_oracle(mode, q.double(), k.double(), v.double(), H, G, decay.double(), gk.double(), beta.double()))
    state = torch.full((3, H, D, Dv), 5.0, device=device)
    plans = [[33, 1, 1, 2, 16, 37], [0, 0, 1, 16, 0, 0]]
    rows = [2, 0]
    done = [0, 0]
    outs = [[], []]
    for step in range(6):
        parts, runs, pos, slot = [], [], [], []
        for s in range(2):
            c = plans[s][step]
            if c:
                runs.append([len(pos), c, done[s], rows[s]])
                parts.append((s, c))
                pos += list(range(done[s], done[s] + c))
                slot += [rows[s]] * c
        cat = lambda i: torch.cat([data[s][i][done[s]:done[s] + c].reshape(c, -1) for s, c in parts], 0).to(device)      # noqa: E731
        single = all(c == 1 for _, c in parts)
        rt = None if single else torch.tensor(runs, dtype=torch.int32, device=device)
        o = linear_scan(cat(0), cat(1), cat(2), state, torch.tensor(pos, dtype=torch.int32, device=device),
                        torch.tensor(slot, dtype=torch.int32, device=device), rt, len(runs), H, G, D, Dv, mode, decay=decay.to(device),
                        g=cat(4) if mode == "delta" else None, beta=cat(5) if mode == "delta" else None)
        i = 0
        for s, c in parts:
            outs[s].append(o[i:i + c])
            i += c
            done[s] += c
    for s in range(2):
        got = torch.cat(outs[s], 0).cpu().double().view(lens[s], H, Dv)
        assert rel_err(got, refs[s][0]) < 1e-4, (mode, s)
        assert rel_err(state[rows[s]].cpu(), refs[s][1]) < 1e-4


@pytest.mark.parametrize("device,dtype", [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)])
def test_delta_gates(device, dtype):
    from llm_in_practise_b200.ops.linear_scan import delta_gates
    g = torch.Generator().manual_seed(4)
    n, G, H, D = 7, 2, 4, 24
    buf = torch.randn(n, 2 * G * D + 5, generator=g) * 3
    a, b = torch.randn(n, H * D, generator=g) * 3, torch.randn(n, H + 3, generator=g) * 2
    bias, A = torch.randn(H * D, generator=g), torch.randn(H, generator=g)
    bd, ad, bb = buf.clone().to(device), a.clone().to(device), b.clone().to(device)
    delta_gates(bd[:, :G * D], bd[:, G * D:2 * G * D], ad, bb[:, 1:1 + H], bias.to(device), A.to(device), G, H, D, D ** -0.5)
    x = buf.double()
    unit = lambda t: t / torch.sqrt((t * t).sum(-1, keepdim=True) + 1e-6)                                   # noqa: E731
    torch.testing.assert_close(bd[:, :G * D].cpu().double(), (unit(x[:, :G * D].view(n, G, D)) * D ** -0.5).view(n, -1), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(bd[:, G * D:2 * G * D].cpu().double(), unit(x[:, G * D:2 * G * D].view(n, G, D)).view(n, -1), rtol=1e-5, atol=1e-6)
    ref = torch.exp(-torch.exp(A.double())[None, :, None] * O.softplus(a.double() + bias.double()).view(n, H, D)).view(n, -1)
    torch.testing.assert_close(ad.cpu().double(), ref, rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(bb[:, 1:1 + H].cpu().double(), torch.sigmoid(b[:, 1:1 + H].double()), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(bb[:, 0].cpu(), b[:, 0])                # neighbours of the strided views are untouched


# ------------------------------------------------------------------------------------------------------------------
# the model through the ragged step
# ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("variant", list(VARIANTS))
def test_whole_prompt_and_residuals(tmp_path, device, dtype, variant):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS[variant]()
    W = O.random_weights(cfg, seed=11)
    model = build(tmp_path, cfg, W, device, dtype)
    toks = _tokens(90, cfg["vocab"], 1)
    res_ref = []
    ref = O.forward(cfg, W, toks, res_ref)
    gen = RaggedGenerator(model, None, 128)
    cache = fresh_cache(gen, 1, 128)
    res = []
    got = gen.step([(0, 0, toks, list(range(len(toks))))], cache, layer_outputs=res)
    assert got.dtype == torch.float32
    for i, L in enumerate(cfg["layers"]):                        # layers that share keys or carry a state hold no pool of their own
        own = L["type"] == "attention" and "kv_from" not in L["mixer"]
        assert (cache.k[i].numel() > 0) == own and (len(cache.state[i]) > 0) == (L["type"] != "attention")
    for a, b in zip(res, res_ref):
        assert_rows(a, b, dtype, variant)
    assert_rows(got, ref, dtype, variant)
    # the first tokens of a sequence: a one-token request and the start of a longer one agree with the oracle row by row
    one = gen.step([(0, 0, toks[:1], [0])], fresh_cache(gen, 1, 64))
    assert rel_err(one, ref[:1]) < 2 * tol(dtype)
    assert rel_err(got[:3], ref[:3]) < 2 * tol(dtype)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("name", list(ODD))
def test_odd_sizes(tmp_path, device, dtype, name):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = ODD[name]()
    W = O.random_weights(cfg, seed=3, ranks=(5, 3))
    model = build(tmp_path, cfg, W, device, dtype)
    n = 140
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    gen = RaggedGenerator(model, None, 192)
    cache = fresh_cache(gen, 2, 192)
    p, outs = 0, []
    for c in [30, 34, 2, 3, 61, 1, 1, 1, 7]:
        outs.append(gen.step([(1, p, toks[p:p + c], list(range(c)))], cache))
        p += c
    assert_rows(torch.cat(outs, 0), ref, dtype, name)


@pytest.mark.parametrize("device,dtype", CASES)
def test_portions_decode_and_long_decode(tmp_path, device, dtype):
    """Whatever way a sequence is cut into steps — whole, portions down to two tokens that straddle page borders and window
    edges, one token at a time for 150 tokens (the window and the kept tokens pass over decoded positions) — every
    position's logits equal the oracle's for the whole sequence."""
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=12)
    model = build(tmp_path, cfg, W, device, dtype)
    n = 230
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)
    gen = RaggedGenerator(model, None, 256)
    for cuts in ([60, 2, 2, 3, 61, 1, 2, 64, 35], [63, 2, 64, 101], [80] + [1] * 150, [1, 1, 2, 36, 2, 188]):
        assert sum(cuts) == n
        cache = fresh_cache(gen, 1, 256)
        p, outs = 0, []
        for c in cuts:
            outs.append(gen.step([(0, p, toks[p:p + c], list(range(c)))], cache))
            p += c
        assert_rows(torch.cat(outs, 0), ref, dtype, cuts[:4])


@pytest.mark.parametrize("device,dtype", CASES)
def test_mixed_batch_equals_each_alone(tmp_path, device, dtype):
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS["recurrent_first"]()
    W = O.random_weights(cfg, seed=13)
    model = build(tmp_path, cfg, W, device, dtype)
    lens = [150, 9, 70, 1]
    seqs = [_tokens(L, cfg["vocab"], 20 + i) for i, L in enumerate(lens)]
    refs = [O.forward(cfg, W, s) for s in seqs]
    gen = RaggedGenerator(model, None, 192)
    cache = fresh_cache(gen, 4, 192)
    plans = [[64, 2, 0, 50, 1, 1, 32], [0, 9, 0, 0, 0, 0, 0], [3, 1, 60, 1, 1, 2, 2], [0, 0, 1, 0, 0, 0, 0]]
    done = [0] * 4
    outs = [[] for _ in seqs]
    for step in range(7):
        entries, who = [], []
        for s, plan in enumerate(plans):
            c = plan[step]
            if c:
                entries.append((s, done[s], seqs[s][done[s]:done[s] + c], list(range(c))))
                who.append((s, c))
                done[s] += c
        got = gen.step(entries, cache)
        o = 0
        for s, c in who:
            outs[s].append(got[o:o + c])
            o += c
    assert done == lens
    for s in range(4):
        assert_rows(torch.cat(outs[s], 0), refs[s], dtype, s)


@pytest.mark.parametrize("device,dtype", CASES)
def test_engine_replay_reuses_pages_slots_and_state(tmp_path, device, dtype):
    """The engine's own slot pool (4 rows, each with its recurrent state) and block pool (sized for the live requests only):
    six requests come and go, so rows, their state and pages are handed out again while neighbours still use theirs."""
    from llm_in_practise_b200.serve.engine import EngineArgs, LLMEngine
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=14)
    model = build(tmp_path, cfg, W, device, dtype)
    lens = {"a": 130, "b": 64, "c": 65, "d": 20, "e": 128, "f": 70}
    seqs = {k: _tokens(L, cfg["vocab"], 30 + i) for i, (k, L) in enumerate(lens.items())}
    refs = {k: O.forward(cfg, W, s) for k, s in seqs.items()}
    eng = LLMEngine(model, None, EngineArgs(max_num_seqs=4, max_model_len=192, block_size=64, num_kv_blocks=7,
                                            enable_prefix_caching=False, warmup=False))
    done = {k: 0 for k in lens}
    outs = {k: [] for k in lens}

    def run(parts, end=()):
        entries = []
        for k, c in parts:
            entries.append((k, seqs[k][done[k]:done[k] + c], list(range(c))))
            done[k] += c
        got = eng.replay_step(entries, end)
        o = 0
        for k, c in parts:
            outs[k].append(got[o:o + c])
            o += c

    run([("a", 100), ("b", 30)])
    run([("a", 30), ("b", 34), ("c", 65)], end=["b"])
    run([("d", 20), ("c", 0), ("e", 60)], end=["a"])
    run([("e", 68), ("d", 0)], end=["d", "c"])
    run([("f", 2)])
    run([("f", 62), ("e", 0)])
    run([("f", 6)], end=["e", "f"])
    assert done == lens
    for k in lens:
        assert_rows(torch.cat([o for o in outs[k] if o.shape[0]], 0), refs[k], dtype, k)
    assert len(eng.free) == 4 and len(eng._free_blocks) == 7


@pytest.mark.parametrize("device,dtype", [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)])
def test_greedy_generation_through_engine_and_generate(tmp_path, device, dtype):
    from llm_in_practise_b200.inference import GenerationConfig
    from llm_in_practise_b200.serve.engine import EngineArgs, LLMEngine
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=15)
    model = build(tmp_path, cfg, W, device, dtype)
    prompts = [_tokens(L, cfg["vocab"], 40 + i) for i, L in enumerate([5, 70, 17, 33, 2, 64])]
    new = 12
    refs = [O.greedy(cfg, W, p, new) for p in prompts]
    # scheduler: 4 rows for 6 requests, 24 prompt tokens per iteration, so prompts are cut and mixed with decode tokens; the
    # engine is asked for prefix caching and must switch it off by itself (a recurrent state cannot restart mid-sequence)
    eng = LLMEngine(model, None, EngineArgs(max_num_seqs=4, max_model_len=128, max_prefill_tokens=24, block_size=64,
                                            enable_prefix_caching=True, warmup=False))
    assert not eng.args.enable_prefix_caching
    reqs = eng.generate(prompts, GenerationConfig(max_new_tokens=new, ignore_eos=True))
    for r, p, ref in zip(reqs, prompts, refs):
        assert r.finish_reason == "length"
        assert p + r.output_ids == ref
    again = eng.generate([prompts[1], prompts[5]], GenerationConfig(max_new_tokens=new, ignore_eos=True))
    assert prompts[1] + again[0].output_ids == refs[1] and prompts[5] + again[1].output_ids == refs[5]
    out = model.generate(torch.tensor([prompts[2], prompts[2][::-1]], device=device), max_new_tokens=new)
    assert out[0].tolist() == refs[2]
    assert out[1].tolist() == O.greedy(cfg, W, prompts[2][::-1], new)
    lg = model(torch.tensor([prompts[3]], device=device))["logits"][0]
    assert rel_err(lg, O.forward(cfg, W, prompts[3])) < tol(dtype)


def test_checkpoint_names_round_trip(tmp_path):
    from llm_in_practise_b200.models.duratar import DuratarConfig, duratar_state_dict
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=16)
    model = build(tmp_path, cfg, W, "cpu", torch.bfloat16)
    sd = duratar_state_dict(model)
    assert set(sd) == set(W)
    for k in W:
        assert sd[k].shape == W[k].shape, k
        assert torch.equal(sd[k].to(torch.bfloat16).cpu(), W[k]), k
    c = DuratarConfig.from_dict(cfg)
    assert [l.ff for l in c.layers] == [80, 72, 0, 64] and c.layers[2].mixer.kv_from == 0 and c.streams == 2 and c.hyper
    assert model.kv_layout() == [(4, 32, 64, 2), (0, 0, 0, 0), (0, 0, 0, 0), (0, 0, 0, 0)]
    assert not DuratarConfig.from_dict(VARIANTS["plain_residual"]()).hyper
    for breakage in (lambda b: b["layers"][0].__setitem__("type", "recurrent"), lambda b: b["layers"][2]["mixer"].__setitem__("kv_from", 1),
                     lambda b: b["layers"][2]["mixer"].__setitem__("kv_from", 2)):
        bad = json.loads(json.dumps(cfg))
        breakage(bad)
        with pytest.raises(ValueError):
            DuratarConfig.from_dict(bad)
