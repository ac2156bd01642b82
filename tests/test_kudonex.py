"""Kudonex against the plain float64 oracle in ``kudonex_oracle.py``: every mechanism alone, then the model through the ragged
step, the serving engine's block / slot / state pools and its scheduler. Small random models of several shapes; the same
tests run on the CPU path and (marked ``gpu``) on the CUDA kernels in fp32 and bf16."""
import json
import math

import pytest
import torch

import kudonex_oracle as O

CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu),
         pytest.param("cuda", torch.bfloat16, marks=pytest.mark.gpu)]
F32_CASES = [("cpu", torch.float32), pytest.param("cuda", torch.float32, marks=pytest.mark.gpu)]


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
    """Every position against the oracle. In fp32 each row must agree. In 16 bits a router score that the oracle decides by a
    hair can fall the other way and move that token's row (and, through the recurrent states, later ones a little) by more
    than rounding, so there nine rows in ten are held to the tolerance and the median to half of it."""
    e = row_errs(got, want)
    if dtype == torch.float32:
        assert float(e.max()) < tol(dtype), (what, float(e.max()), int(e.argmax()))
    else:
        assert float(e.quantile(0.9)) < tol(dtype) and float(e.median()) < tol(dtype) / 2, (what, float(e.quantile(0.9)), float(e.median()))


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
        for k in cache.k:
            k.fill_(9.0)
    return cache


def _tokens(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _i32(x, device):
    return torch.tensor(x, dtype=torch.int32, device=device)


VARIANTS = {
    # all three mixers; expert groups with some dropped; kv heads shared by two heads; sizes the tensor-core kernel takes
    "mixed": lambda: O.make_config(64, 96, [
        O.mlstm_layer(2, 16, 24, cap=8.0, mlp=O.moe_spec(6, 2, 32, groups=3, keep=2, shared=40)),
        O.mamba2_layer(4, 8, 16, groups=2, norm_groups=2, conv=3, mlp=O.moe_spec(4, 1, 24, groups=1, keep=1, shared=16)),
        O.attention_layer(4, 2, 16, 40, mlp=O.moe_spec(8, 3, 16, groups=4, keep=2, shared=24)),
        O.mlstm_layer(4, 8, 8, cap=15.0, mlp=None)], taps=3),
    # attention first, one kv head for all heads, a window larger than any prompt, every expert chosen, no convolution taps
    # beyond the token itself, one norm group, one state-space group
    "attention_first": lambda: O.make_config(48, 80, [
        O.attention_layer(6, 1, 16, 4096, scale=0.2, mlp=O.moe_spec(3, 3, 20, groups=1, keep=1, shared=8)),
        O.mamba2_layer(2, 24, 8, groups=1, norm_groups=1, conv=1, mlp=None),
        O.mlstm_layer(1, 32, 48, cap=4.0, mlp=O.moe_spec(4, 2, 12, groups=2, keep=2, shared=0))], taps=1, embed_scale=1.0, eps=1e-3),
    # as many kv heads as heads, a window of one token, state-space groups = heads, norm groups = heads, two taps
    "narrow_window": lambda: O.make_config(40, 64, [
        O.mamba2_layer(3, 16, 12, groups=3, norm_groups=3, conv=2, mlp=O.moe_spec(6, 1, 16, groups=2, keep=1, shared=16)),
        O.attention_layer(2, 2, 32, 1, mlp=None),
        O.attention_layer(4, 4, 16, 7, scale=0.4, mlp=O.moe_spec(2, 1, 24, groups=2, keep=1, shared=8))], taps=2, embed_scale=7.5),
}

# sizes that are not multiples of the kernels' vector widths
ODD = {
    "w72": lambda: O.make_config(72, 75, [
        O.attention_layer(6, 3, 20, 33, mlp=O.moe_spec(5, 2, 36, groups=5, keep=3, shared=20)),
        O.mlstm_layer(3, 12, 20, cap=11.0, mlp=O.moe_spec(9, 4, 12, groups=3, keep=2, shared=28)),
        O.mamba2_layer(5, 10, 14, groups=5, norm_groups=2, conv=5, mlp=None)], taps=5),
    "w100": lambda: O.make_config(100, 130, [
        O.mamba2_layer(2, 36, 72, groups=1, norm_groups=4, conv=4, mlp=O.moe_spec(4, 2, 52, groups=2, keep=1, shared=12)),
        O.attention_layer(3, 3, 24, 65, mlp=None),
        O.mlstm_layer(2, 40, 72, cap=15.0, mlp=None)], taps=4),
}


# ------------------------------------------------------------------------------------------------------------------
# mechanisms alone
# ------------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("W", [40, 72, 100, 256])
def test_layer_norm_sandwich(device, dtype, W):
    from llm_in_practise_b200.ops.norm import sandwich_norm
    g = torch.Generator().manual_seed(W)
    n, eps = 5, 1e-3
    y = torch.randn(n, W, generator=g) * 3 + 1.5                 # a mean far from zero: an RMS norm would give something else
    x = torch.randn(n, W, generator=g) * 2
    w1, w2 = torch.randn(W, generator=g), torch.randn(W, generator=g)
    h, xn = sandwich_norm(y.to(device), w1.to(device), x.to(device), w2.to(device), eps, 0.0, dtype, center=True)
    want_x = x.double() + O.layer_norm(y.double(), w1, eps)
    torch.testing.assert_close(xn.cpu().double(), want_x, rtol=1e-5, atol=1e-5)
    assert h.dtype == dtype and xn.dtype == torch.float32
    t = tol(dtype) / 4
    torch.testing.assert_close(h.cpu().double(), O.layer_norm(want_x, w2, eps), rtol=t, atol=t)
    # the stream's entry: nothing normed on the way in, the first pre-norm on the way out
    h0, x0 = sandwich_norm(y.to(device), None, None, w2.to(device), eps, 0.0, torch.float32, center=True)
    torch.testing.assert_close(x0.cpu(), y)
    torch.testing.assert_close(h0.cpu().double(), O.layer_norm(y.double(), w2, eps), rtol=1e-5, atol=1e-5)
    # without `center` the same call is the RMS form
    hr, _ = sandwich_norm(y.to(device), None, None, w2.to(device), eps, 0.0, torch.float32)
    torch.testing.assert_close(hr.cpu().double(), O.rms(y.double(), eps) * w2.double(), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("W", [16, 50, 33])
def test_embedding_with_position_table(device, dtype, W):
    from llm_in_practise_b200.ops import elementwise as ew
    g = torch.Generator().manual_seed(W)
    table = torch.randn(20, W, generator=g).to(dtype)
    ids = [3, 19, 0, 3, 7]
    pos = [0, 1, 700, 64, 2047]
    tab = ew.sinusoid_table(2048, W, device)
    got = ew.embedding_pos(torch.tensor(ids, device=device), table.to(device), 2.5, _i32(pos, device), tab)
    assert got.dtype == torch.float32
    ref = O.sinusoid(2048, W)
    want = table.double()[ids] * 2.5 + ref[pos]
    torch.testing.assert_close(got.cpu().double(), want, rtol=1e-6, atol=2e-6)
    assert abs(float(ref[700, 0]) - math.sin(700.0)) < 1e-12 and abs(float(ref[5, 1]) - math.cos(5.0)) < 1e-12


def _cut_runs(lens, plans, rows):
    """Yield per step (parts, runs, pos, slot) for sequences cut by `plans` (one list of counts per sequence)."""
    done = [0] * len(lens)
    for step in range(len(plans[0])):
        parts, runs, pos, slot = [], [], [], []
        for s in range(len(lens)):
            c = plans[s][step]
            if c:
                runs.append([len(pos), c, done[s], rows[s]])
                parts.append((s, done[s], c))
                pos += list(range(done[s], done[s] + c))
                slot += [rows[s]] * c
                done[s] += c
        yield parts, runs, pos, slot


PLANS = [[33, 1, 1, 2, 16, 37], [0, 0, 1, 16, 0, 0]]


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("C,taps,residual,bias,act", [(24, 4, True, False, False), (10, 1, True, False, False), (36, 3, False, True, True),
                                                      (7, 5, False, True, True), (16, 2, True, True, False)])
def test_short_conv_with_residual_bias_and_tail(device, dtype, C, taps, residual, bias, act):
    from llm_in_practise_b200.ops.linear_scan import short_conv
    g = torch.Generator().manual_seed(C + taps)
    lens = [90, 17]
    xs = [torch.randn(L, C, generator=g) for L in lens]
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    refs = []
    for x in xs:
        y = O.causal_conv(x.double(), w, b if bias else None)
        y = O.silu(y) if act else y
        refs.append(y + x.double() if residual else y)
    tail = torch.full((3, taps - 1, C), 5.0, device=device)
    rows = [2, 0]
    outs = [[], []]
    for parts, runs, pos, slot in _cut_runs(lens, PLANS, rows):
        x = torch.cat([xs[s][p:p + c] for s, p, c in parts], 0).to(device)
        single = all(c == 1 for _, _, c in parts)
        y = short_conv(x, w.to(device), tail, _i32(pos, device), _i32(slot, device), None if single else _i32(runs, device), len(runs),
                       act=act, bias=b.to(device) if bias else None, residual=residual, out_dtype=dtype)
        assert y.dtype == dtype
        i = 0
        for s, _, c in parts:
            outs[s].append(y[i:i + c])
            i += c
    for s in range(2):
        t = 1e-5 if dtype == torch.float32 else 3e-2
        torch.testing.assert_close(torch.cat(outs[s], 0).cpu().double(), refs[s], rtol=t, atol=t)


@pytest.mark.parametrize("device,dtype", F32_CASES)
@pytest.mark.parametrize("H,cap", [(3, 15.0), (1, 2.0), (5, 40.0)])
def test_mlstm_gates_across_cuts(device, dtype, H, cap):
    """The running maximum is carried per sequence and head in a reused row; a, b and exp(-m) equal the sequential
    recurrence however the sequence is cut. Gate inputs reach far past the cap on both sides."""
    from llm_in_practise_b200.ops.linear_scan import mlstm_gates
    g = torch.Generator().manual_seed(H)
    lens = [90, 17]
    gi = [torch.randn(L, H + 2, generator=g) * 12 for L in lens]
    gf = [torch.randn(L, H, generator=g) * 12 + 3 for L in lens]
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g)
    refs = []
    for s, L in enumerate(lens):
        iv = cap * torch.tanh((gi[s][:, 1:1 + H].double() + bi.double()) / cap)
        fv = torch.nn.functional.logsigmoid(cap * torch.tanh((gf[s].double() + bf.double()) / cap))
        m = torch.zeros(H, dtype=torch.float64)
        rows = []
        for t in range(L):
            mn = torch.maximum(fv[t] + m, iv[t])
            rows.append(torch.stack([torch.exp(fv[t] + m - mn), torch.exp(iv[t] - mn), torch.exp(-mn)]))
            m = mn
        refs.append(torch.stack(rows))                                   # [L, 3, H]
    mstate = torch.full((3, H), -50.0, device=device)
    outs = [[], []]
    for parts, runs, pos, slot in _cut_runs(lens, PLANS, [2, 0]):
        ci = torch.cat([gi[s][p:p + c] for s, p, c in parts], 0).to(device)
        cf = torch.cat([gf[s][p:p + c] for s, p, c in parts], 0).to(device)
        single = all(c == 1 for _, _, c in parts)
        a, b, e = mlstm_gates(ci[:, 1:1 + H], cf, bi.to(device), bf.to(device), cap, mstate, _i32(pos, device), _i32(slot, device),
                              None if single else _i32(runs, device), len(runs))
        i = 0
        for s, _, c in parts:
            outs[s].append(torch.stack([a[i:i + c], b[i:i + c], e[i:i + c]], 1))
            i += c
    for s in range(2):
        torch.testing.assert_close(torch.cat(outs[s], 0).cpu().double(), refs[s], rtol=2e-4, atol=1e-7)


@pytest.mark.parametrize("device,dtype", F32_CASES)
def test_ssm_gates(device, dtype):
    from llm_in_practise_b200.ops.linear_scan import ssm_gates
    g = torch.Generator().manual_seed(2)
    n, H = 9, 5
    buf = torch.randn(n, H + 3, generator=g) * 8                          # softplus far on both sides, and no threshold above
    buf[0, 1] = 30.0
    bias, A = torch.randn(H, generator=g), torch.randn(H, generator=g)
    a, b = ssm_gates(buf.to(device)[:, 1:1 + H], bias.to(device), A.to(device))
    dt = torch.nn.functional.softplus(buf[:, 1:1 + H].double() + bias.double(), threshold=1e9)
    torch.testing.assert_close(b.cpu().double(), dt, rtol=1e-5, atol=1e-9)
    torch.testing.assert_close(a.cpu().double(), torch.exp(-torch.exp(A.double()) * dt), rtol=1e-5, atol=1e-9)


def _gated_oracle(q, k, v, a, b, H, G, ones):
    n, D = q.shape[0], q.shape[2]
    if ones:
        v = torch.cat([v, torch.ones(n, H, 1, dtype=torch.float64)], -1)
    Dv = v.shape[2]
    S = torch.zeros(H, D, Dv, dtype=torch.float64)
    o = torch.zeros(n, H, Dv, dtype=torch.float64)
    for t in range(n):
        for h in range(H):
            kv = h // (H // G)
            S[h] = a[t, h] * S[h] + b[t, h] * torch.outer(k[t, kv], v[t, h])
            o[t, h] = S[h].T @ q[t, kv]
    return o, S


@pytest.mark.parametrize("device,dtype", F32_CASES)
@pytest.mark.parametrize("H,G,D,Dv,ones", [(3, 3, 16, 32, True), (2, 2, 40, 12, True), (1, 1, 128, 127, True), (4, 2, 16, 24, False),
                                           (6, 1, 8, 8, False), (5, 5, 14, 10, False), (2, 2, 72, 36, True)])
def test_gated_scan_across_cuts(device, dtype, H, G, D, Dv, ones):
    """S <- a S + b k v^T with one a, b per token and head, with and without the column of ones, in reused rows that hold
    garbage, however the sequences are cut; a second sequence in the same steps has its own state."""
    from llm_in_practise_b200.ops.linear_scan import linear_scan
    g = torch.Generator().manual_seed(D + Dv)
    lens = [90, 17]
    data, refs = [], []
    cols = Dv + int(ones)
    for L in lens:
        q, k = torch.randn(L, G, D, generator=g) * D ** -0.5, torch.randn(L, G, D, generator=g)
        v = torch.randn(L, H, Dv, generator=g)
        a, b = torch.rand(L, H, generator=g) * 0.6 + 0.4, torch.rand(L, H, generator=g) * 2
        data.append((q, k, v, a, b))
        refs.append(_gated_oracle(q.double(), k.double(), v.double(), a.double(), b.double(), H, G, ones))
    state = torch.full((3, H, D, cols), 5.0, device=device)
    rows = [2, 0]
    outs = [[], []]
    for parts, runs, pos, slot in _cut_runs(lens, PLANS, rows):
        cat = lambda i: torch.cat([data[s][i][p:p + c].reshape(c, -1) for s, p, c in parts], 0).to(device)      # noqa: E731
        single = all(c == 1 for _, _, c in parts)
        o = linear_scan(cat(0), cat(1), cat(2), state, _i32(pos, device), _i32(slot, device), None if single else _i32(runs, device),
                        len(runs), H, G, D, cols, "gated", g=cat(3), beta=cat(4), ones=ones)
        i = 0
        for s, _, c in parts:
            outs[s].append(o[i:i + c])
            i += c
    for s in range(2):
        got = torch.cat(outs[s], 0).cpu().double().view(lens[s], H, cols)
        assert rel_err(got, refs[s][0]) < 1e-4, s
        assert rel_err(state[rows[s]].cpu(), refs[s][1]) < 1e-4


@pytest.mark.parametrize("device,dtype", CASES)
def test_scan_readout_forms(device, dtype):
    from llm_in_practise_b200.ops.linear_scan import scan_readout
    g = torch.Generator().manual_seed(8)
    n, H, Dv, eps = 6, 3, 20, 1e-4
    t = 1e-5 if dtype == torch.float32 else 2e-2
    # matrix-memory form: normaliser column, floor exp(-m), per-head norm, a weight over all heads, sigmoid gate after the norm
    o = torch.randn(n, H, Dv + 1, generator=g)
    o[0, :, Dv] = 1e-3                                                    # |n . q| below the floor: the floor divides
    e = torch.rand(n, H, generator=g) + 0.05
    w, gate = torch.randn(H * Dv, generator=g), torch.randn(n, H * Dv + 4, generator=g)
    got = scan_readout(o.reshape(n, -1).to(device), H, Dv, w.to(device), H, eps, dtype, e=e.to(device), den_eps=1e-6, oscale=0.25,
                       post=gate.to(device)[:, 4:])
    od = o.double() * 0.25
    v = od[:, :, :Dv] / (torch.maximum(od[:, :, Dv].abs(), e.double()) + 1e-6)[:, :, None]
    want = O.rms(v, eps).reshape(n, -1) * w.double() * torch.sigmoid(gate[:, 4:].double())
    torch.testing.assert_close(got.cpu().double(), want, rtol=t, atol=t)
    # state-space form: skip term, silu gate before the norm, norm over 2 groups that are not the heads, a weight per column
    o2 = torch.randn(n, H * Dv, generator=g)
    x, z, skip = torch.randn(n, H * Dv, generator=g), torch.randn(n, H * Dv + 8, generator=g), torch.randn(H, generator=g)
    got2 = scan_readout(o2.to(device), H, Dv, w.to(device), 2, eps, dtype, skip=skip.to(device), x=x.to(device), pre=z.to(device)[:, :H * Dv])
    y = (o2.double().view(n, H, Dv) + skip.double()[None, :, None] * x.double().view(n, H, Dv)).reshape(n, -1) * O.silu(z[:, :H * Dv].double())
    want2 = O.rms(y.view(n, 2, -1), eps).reshape(n, -1) * w.double()
    torch.testing.assert_close(got2.cpu().double(), want2, rtol=t, atol=t)
    # a weight shared by the groups
    got3 = scan_readout(o2.to(device), H, Dv, w[:Dv].to(device), H, eps, torch.float32)
    torch.testing.assert_close(got3.cpu().double(), (O.rms(o2.double().view(n, H, Dv), eps) * w[:Dv].double()).reshape(n, -1), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("device,dtype", F32_CASES)
@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (4, 4, 1, 1), (12, 1, 4, 4), (9, 3, 3, 1), (5, 2, 5, 3)])
def test_softmax_router_with_groups(device, dtype, E, top, groups, keep):
    """Corrections below zero make every choice score of some tokens negative: dropped groups must count as minus infinity,
    and the weights are the scores without the correction, not renormalised."""
    from llm_in_practise_b200.ops.moe import route_grouped
    g = torch.Generator().manual_seed(E * 7 + top)
    n, W = 40, 24
    h = torch.randn(n, W, generator=g)
    wr = torch.randn(E, W, generator=g) * 0.5
    corr = torch.randn(E, generator=g) * 0.4 - 1.2
    f = O.moe_spec(E, top, 8, groups, keep)
    want_i, want_p = O.route(h.double(), {"router": wr, "correction": corr}, f)
    ti, tp, _ = route_grouped(h.to(device), wr.to(device), corr.to(device), top, groups, keep, 1, softmax=True)
    assert ti.tolist() == want_i
    torch.testing.assert_close(tp.cpu().double(), torch.tensor(want_p, dtype=torch.float64), rtol=1e-4, atol=1e-7)
    assert float((h @ wr.t()).softmax(-1).add(corr).max(-1).values.min()) < 0          # some tokens choose among negative scores only


def _attn_setup(device, dtype, H, G, D, n_pos, window, hot=None, seed=0, identity=False):
    """Keys of positions 0 .. n_pos - 1 of one sequence written into scrambled pages through the store op; returns what the
    attention call needs and the float64 tensors of the oracle. `hot` = (query position, key position): that query and key
    are scaled so that, if the key is visible, its score dwarfs all others."""
    from llm_in_practise_b200.inference.generate import PagedKVCache
    from llm_in_practise_b200.ops.paged_attention import rope_paged_store
    g = torch.Generator().manual_seed(seed)
    BS = 64
    nb = -(-n_pos // BS)
    q = torch.randn(n_pos, H * D, generator=g)
    k = torch.randn(n_pos, G * D, generator=g)
    if hot is not None:
        qi, kj = hot
        unit = torch.nn.functional.normalize(torch.randn(D, generator=g), dim=0)
        k[kj] = (unit * 4).repeat(G)
        q[qi] = (unit * 40).repeat(H)
    gate = torch.randn(n_pos, H * D, generator=g)
    q, k, gate = q.to(dtype), k.to(dtype), gate.to(dtype)
    r1, r2 = torch.rand(H, generator=g), torch.rand(H, generator=g) + 0.1
    talk = torch.eye(H) if identity else torch.eye(H) + torch.randn(H, H, generator=g) * 0.2
    cache = PagedKVCache(1, nb + 1, [G], BS, [D], dtype, torch.device(device), 3, nb * BS, Dv=[0])
    cache.k[0].fill_(50.0)
    cache.set_row(1, list(range(nb, 0, -1)))
    pos, slot = _i32(list(range(n_pos)), device), _i32([1] * n_pos, device)
    zero = torch.zeros(1, 1, device=device)
    rope_paged_store(k.to(device), zero, zero, pos, slot, cache.k[0], None, cache.table, 0, G, D, rot_dims=0)
    return cache, q, k, gate, r1, r2, talk


def _attn_oracle(q, k, gate, r1, r2, talk, H, G, D, scale, window, rows):
    P = {"q": torch.eye(H * D), "k": torch.eye(G * D), "g": torch.eye(H * D), "o": torch.eye(H * D), "r1": r1, "r2": r2, "talk": talk}
    # the oracle's attention projects h itself, so give it identity projections of three different inputs, one at a time
    n = q.shape[0]
    qd, kd = q.double().view(n, H, D), k.double().view(n, G, D)
    out = torch.zeros(len(rows), H * D, dtype=torch.float64)
    for x, i in enumerate(rows):
        lo = max(0, i - window + 1) if window > 0 else 0
        dist = torch.arange(i - lo, -1, -1, dtype=torch.float64)
        raw = torch.stack([(kd[lo:i + 1, a // (H // G)] @ qd[i, a]) * scale - r1[a].double() * torch.log1p(r2[a].double() * dist) for a in range(H)])
        p = torch.softmax(talk.double() @ raw, -1)
        ctx = torch.stack([p[a] @ kd[lo:i + 1, a // (H // G)] for a in range(H)]).reshape(-1)
        out[x] = ctx * torch.sigmoid(gate[i].double())
    assert P["talk"] is talk
    return out


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,G,D,window", [(4, 2, 16, 40), (6, 1, 20, 33), (2, 2, 32, 1), (8, 4, 64, 72), (3, 3, 24, 0), (16, 2, 128, 100),
                                           (16, 16, 96, 150)])          # the last: kv rows so wide that fewer keys are staged at a time
def test_talking_attention_tokens_and_pieces(device, dtype, H, G, D, window):
    """Single tokens (decode) and prompt pieces that start in the middle of a page, against the oracle: distance penalty,
    head mixing, window, keys as values, output gate."""
    from llm_in_practise_b200.inference.ragged import Pieces, make_pieces
    from llm_in_practise_b200.ops.talking_attention import talking_attention
    n_pos = 200
    scale = D ** -0.5
    cache, q, k, gate, r1, r2, talk = _attn_setup(device, dtype, H, G, D, n_pos, window, seed=H + D)
    dv = lambda t: t.to(device)                                     # noqa: E731
    rows = [0, 1, 2, 63, 64, 65, 127, 128, 199]
    got = talking_attention(dv(q)[rows], cache.k[0], cache.table, _i32(rows, device), _i32([1] * len(rows), device), H, G, D, scale,
                            window, dv(r1), dv(r2), dv(talk), gate=dv(gate)[rows])
    want = _attn_oracle(q, k, gate, r1, r2, talk, H, G, D, scale, window, rows)
    assert_rows(got, want, dtype, "tokens")
    for first, cnt in ((0, 200), (37, 100), (60, 9), (126, 2)):
        rows = list(range(first, first + cnt))
        pieces = make_pieces([(0, cnt, first, 1)], device)
        got = talking_attention(dv(q)[rows], cache.k[0], cache.table, _i32(rows, device), _i32([1] * cnt, device), H, G, D, scale, window,
                                dv(r1), dv(r2), dv(talk), gate=dv(gate)[rows], pieces=pieces)
        want = _attn_oracle(q, k, gate, r1, r2, talk, H, G, D, scale, window, rows)
        e = row_errs(got, want)
        assert float(e.max()) < tol(dtype), (first, cnt, float(e.max()), int(e.argmax()))
    assert isinstance(pieces, Pieces)


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("H,G,D,window", [(4, 2, 32, 0), (16, 4, 64, 300), (6, 3, 48, 1000), (5, 1, 16, 0)])
def test_talking_attention_few_tokens_over_long_contexts(device, dtype, H, G, D, window):
    """A handful of decode tokens over a long cache row: the 16-bit kernel shares a token's keys out over several CTAs and
    merges their partial softmaxes. Tokens near the start (most CTAs get no key at all), at chunk and page borders and at
    the end of the row, alone and as a batch, agree with the oracle and with each other."""
    from llm_in_practise_b200.ops.talking_attention import talking_attention
    n_pos = 1100
    scale = D ** -0.5
    cache, q, k, gate, r1, r2, talk = _attn_setup(device, dtype, H, G, D, n_pos, window, seed=3 * H + D)
    dv = lambda t: t.to(device)                                     # noqa: E731
    rows = [0, 1, 31, 32, 33, 127, 128, 129, 255, 256, 700, 1023, 1024, 1099]
    want = _attn_oracle(q, k, gate, r1, r2, talk, H, G, D, scale, window, rows)
    got = talking_attention(dv(q)[rows], cache.k[0], cache.table, _i32(rows, device), _i32([1] * len(rows), device), H, G, D, scale,
                            window, dv(r1), dv(r2), dv(talk), gate=dv(gate)[rows])
    e = row_errs(got, want)
    assert float(e.max()) < tol(dtype), (float(e.max()), rows[int(e.argmax())])
    for x in (0, 4, 9, 13):                                         # one token alone: the most CTAs per token
        one = talking_attention(dv(q)[rows[x]:rows[x] + 1], cache.k[0], cache.table, _i32(rows[x:x + 1], device), _i32([1], device),
                                H, G, D, scale, window, dv(r1), dv(r2), dv(talk), gate=dv(gate)[rows[x]:rows[x] + 1])
        assert float(row_errs(one, want[x:x + 1]).max()) < tol(dtype), rows[x]
        assert float((one.float() - got[x:x + 1].float()).abs().max()) < (1e-5 if dtype == torch.float32 else 0.04), rows[x]


@pytest.mark.parametrize("device,dtype", CASES)
@pytest.mark.parametrize("as_piece", [False, True])
def test_one_dominant_key_at_the_window_edges(device, dtype, as_piece):
    """One key is made to dominate a query's scores. Inside the window (its far edge, a page border, the query's own
    position, the first token) the head outputs are that key; one step outside the window it must leave no trace."""
    from llm_in_practise_b200.inference.ragged import make_pieces
    from llm_in_practise_b200.ops.talking_attention import talking_attention
    H, G, D, window, n_pos = 4, 2, 32, 70, 330
    scale = D ** -0.5
    dv = lambda t: t.to(device)                                     # noqa: E731
    for qi, kj, seen in ((300, 231, True), (300, 230, False), (320, 256, True), (320, 255, True), (320, 250, False), (69, 0, True),
                         (70, 0, False), (70, 1, True), (191, 191, True), (192, 128, True), (5, 0, True), (329, 260, True), (329, 259, False)):
        cache, q, k, gate, r1, r2, talk = _attn_setup(device, dtype, H, G, D, n_pos, window, hot=(qi, kj), seed=qi, identity=True)
        if as_piece:
            first = max(0, qi - 20)
            rows = list(range(first, qi + 1))
            pieces = make_pieces([(0, len(rows), first, 1)], device)
        else:
            rows, pieces = [qi], None
        got = talking_attention(dv(q)[rows], cache.k[0], cache.table, _i32(rows, device), _i32([1] * len(rows), device), H, G, D, scale,
                                window, dv(r1), dv(r2), dv(talk), gate=None, pieces=pieces)[-1].float().cpu().view(H, D)
        want = _attn_oracle(q, k, torch.full_like(gate, 50.0), r1, r2, talk, H, G, D, scale, window, [qi])[0].view(H, D)
        key = k[kj].float().view(G, D).repeat_interleave(H // G, 0)
        close = float((got - key).abs().max()) < 0.1
        assert close == seen, (qi, kj, seen)
        assert float((got.double() - want).abs().max()) < (1e-3 if dtype == torch.float32 else 0.1), (qi, kj)


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
    ref, res_ref = O.forward(cfg, W, toks)
    gen = RaggedGenerator(model, None, 128)
    cache = fresh_cache(gen, 1, 128)
    res = []
    got = gen.step([(0, 0, toks, list(range(len(toks))))], cache, layer_outputs=res)
    assert got.dtype == torch.float32
    for i, L in enumerate(cfg["layers"]):                        # only attention layers hold pages, and no value pool
        assert (cache.k[i].numel() > 0) == (L["type"] == "attention") and cache.v[i].numel() == 0
        assert len(cache.state[i]) == (1 if L["type"] == "attention" else 3)
    for li, (a, b) in enumerate(zip(res, res_ref)):
        assert_rows(a, b, dtype, (variant, li))
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
    W = O.random_weights(cfg, seed=3)
    model = build(tmp_path, cfg, W, device, dtype)
    n = 140
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)[0]
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
    edges, one token at a time for 150 tokens (the window passes over decoded positions) — every position's logits equal
    the oracle's for the whole sequence."""
    from llm_in_practise_b200.inference.ragged import RaggedGenerator
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=12)
    model = build(tmp_path, cfg, W, device, dtype)
    n = 230
    toks = _tokens(n, cfg["vocab"], 2)
    ref = O.forward(cfg, W, toks)[0]
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
    cfg = VARIANTS["attention_first"]()
    W = O.random_weights(cfg, seed=13)
    model = build(tmp_path, cfg, W, device, dtype)
    lens = [150, 9, 70, 1]
    seqs = [_tokens(L, cfg["vocab"], 20 + i) for i, L in enumerate(lens)]
    refs = [O.forward(cfg, W, s)[0] for s in seqs]
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
    refs = {k: O.forward(cfg, W, s)[0] for k, s in seqs.items()}
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


@pytest.mark.parametrize("device,dtype", F32_CASES)
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
    assert rel_err(lg, O.forward(cfg, W, prompts[3])[0]) < tol(dtype)


def test_checkpoint_names_round_trip(tmp_path):
    from llm_in_practise_b200.models.kudonex import KudonexConfig, kudonex_state_dict
    cfg = VARIANTS["mixed"]()
    W = O.random_weights(cfg, seed=16)
    model = build(tmp_path, cfg, W, "cpu", torch.bfloat16)
    sd = kudonex_state_dict(model)
    assert set(sd) == set(W)
    for k in W:
        assert sd[k].shape == W[k].shape, k
        assert torch.equal(sd[k].to(torch.bfloat16).cpu(), W[k]), k
    c = KudonexConfig.from_dict(cfg)
    assert [l.mlp.experts if l.mlp else 0 for l in c.layers] == [6, 4, 8, 0] and c.canon_taps == 3 and c.embed_scale == 3.0
    assert model.kv_layout() == [(0, 0, 0), (0, 0, 0), (2, 16, 0), (0, 0, 0)]
    assert model.state_layout()[0] == [(2, 64), (2, 16, 25), (2,)] and model.state_layout()[1] == [(2, 64), (4, 16, 8), (2, 96)]
    for breakage in (lambda b: b["layers"][0].__setitem__("type", "recurrent"), lambda b: b["layers"][2]["mixer"].__setitem__("vdim", 8),
                     lambda b: b["layers"][2]["mlp"]["router"].__setitem__("top", 5), lambda b: b["layers"][2]["mixer"].__setitem__("kv_heads", 3)):
        bad = json.loads(json.dumps(cfg))
        breakage(bad)
        with pytest.raises(ValueError):
            KudonexConfig.from_dict(bad)
