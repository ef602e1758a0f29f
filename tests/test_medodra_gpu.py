"""The Medodra architecture on the GPU against the plain implementation (``plain_medodra``): each mechanism's kernel
alone, then whole models of five small configurations through the engine's step function, its cache and state and its
generation loop, in true 32-bit and in bfloat16.

The models carry a planted key (``tiny_medodra.make_model``): a probe token's attention output is one needle token's
value, so a dropped key, a distance that lands in the wrong row of the bias table, a page of another sequence or a
slot's old content changes a probe's logits by many times the tolerance; decays and update gates are slow, so a lost
state shows for hundreds of tokens. The 32-bit runs are the sharp ones for everything else.
"""
import json
import math
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_medodra as PM
import tiny
import tiny_medodra as TM

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64


@pytest.fixture(scope="module")
def K():
    from kindi_b200.kernels import lib
    lib.load()
    return lib


def _status():
    return torch.zeros(1, dtype=torch.int32, device="cuda")


def _rel(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / (b.abs().max() + 1e-30))


def _i32(x):
    return torch.tensor(list(x), dtype=torch.int32, device="cuda")


def _packed(lens, first):
    """pos, seq, q_start of a packed step: sequence b brings lens[b] rows from position first[b] on"""
    pos = [p for b, n in enumerate(lens) for p in range(first[b], first[b] + n)]
    seq = [b for b, n in enumerate(lens) for _ in range(n)]
    return _i32(pos), _i32(seq), _i32([0] + list(np.cumsum(lens)))


def _slots(B, extra=3, seed=3):
    s = list(range(B + extra))
    random.Random(seed).shuffle(s)
    return s[:B], B + extra


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("T,E", [(1, 64), (7, 72), (40, 200)])
def test_sinusoidal_positions(K, T, E):
    freq = torch.tensor([10000.0 ** (-2.0 * i / E) for i in range((E + 1) // 2)], dtype=torch.float64)
    x = torch.randn(T, E)
    pos = torch.tensor([0, 1, 5, 63, 64, 1000, 40000][:T] + list(range(7, T)), dtype=torch.int64)[:T]
    got = x.clone().cuda()
    K.sinusoid_add(got, pos.to(torch.int32).cuda(), freq.cuda())
    want = x.double() + PM.sinusoid(pos, E)
    assert _rel(got, want) < 2e-6


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("C,taps,lens,act,planes", [(5, 3, [7, 1, 2], True, 1), (130, 4, [1, 1, 1], False, 2),
                                                    (64, 2, [3, 40], True, 1), (24, 5, [2, 3, 9, 70], False, 3),
                                                    (33, 1, [4, 2], True, 1), (200, 8, [5, 6], False, 1)])
def test_short_convolution_and_its_tails(K, dtype, C, taps, lens, act, planes):
    """three steps over several sequences in shuffled slots: the first rows of a sequence see zeros, later steps the
    tails the earlier ones left, also when a step brings fewer rows than there are taps"""
    g = torch.Generator().manual_seed(C * taps)
    tdt = DT[dtype]
    B = len(lens)
    takes = [lens, [1] * B, [2 if b % 2 else taps + 1 for b in range(B)]]
    total = [sum(t[b] for t in takes) for b in range(B)]
    col0 = 3
    seqs = [torch.randn(total[b], col0 + C + 2, generator=g) for b in range(B)]
    if planes == 1:
        seqs = [s.to(tdt).float() for s in seqs]
    w = torch.randn(C, taps, generator=g)
    bias = torch.randn(C, generator=g)
    slots, n_slots = _slots(B)
    tails = torch.randn(n_slots, max(1, (taps - 1) * C) + 5, generator=g)
    tails[slots] = 0.0
    tails = tails.cuda()
    want = []
    for b in range(B):
        y = PM.short_conv(seqs[b][:, col0:col0 + C].double() + bias.double(), w.double())
        want.append(PM.silu(y) if act else y)
    got = [[] for _ in range(B)]
    at = [0] * B
    for take in takes:
        rows = torch.cat([seqs[b][at[b]:at[b] + take[b]] for b in range(B)])
        if planes > 1:
            parts = torch.randn(planes, *rows.shape, generator=g)
            parts[0] = rows - parts[1:].sum(0)
            src = parts.cuda()
        else:
            src = rows.to(tdt).cuda()
        pos, seq, q_start = _packed(take, at)
        out = torch.full((rows.shape[0], C), float("nan"), dtype=torch.float32, device="cuda")
        K.short_conv(src, col0, C, bias.cuda(), w.cuda(), act, tails, pos, seq, _i32(slots), q_start, out)
        o = 0
        for b in range(B):
            got[b].append(out[o:o + take[b]].cpu())
            o += take[b]
            at[b] += take[b]
    for b in range(B):
        assert _rel(torch.cat(got[b]), want[b]) < 1e-5, b


def _unit(x, eps):
    return x / torch.sqrt((x * x).sum(-1, keepdim=True) + eps)


@pytest.mark.parametrize("pdtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,d,dv,lens", [(2, 1, 16, 24, [5, 1, 40]), (4, 4, 32, 64, [70, 3]), (3, 1, 40, 9, [1, 1, 1, 1]),
                                           (2, 2, 128, 16, [19, 130]), (1, 1, 256, 8, [17]),
                                           (4, 2, 128, 128, [300, 64, 65]), (6, 2, 64, 128, [257]),
                                           (2, 1, 36, 20, [150, 20, 129])])
def test_gated_delta_rule_and_its_state(K, pdtype, H, G, d, dv, lens):
    """S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q over several sequences in one packed step, then a
    second step that goes on from the stored state (one token for some, several for others), in slots out of order
    among slots with stale content; the per-head norm with a gate"""
    g = torch.Generator().manual_seed(H * d + dv)
    tdt = DT[pdtype]
    B = len(lens)
    # (the second step: one token, a few, and - from a state that is not zero - enough for the form for long prompts)
    more = [1 if b % 2 == 0 else 200 if lens[0] == 150 else 7 for b in range(B)]
    C = 2 * G * d + H * dv
    qkv = [torch.randn(lens[b] + more[b], C, generator=g) for b in range(B)]
    proj = [(torch.randn(lens[b] + more[b], 2 + 2 * H + H * dv, generator=g) * 2).to(tdt).float() for b in range(B)]
    a_log = -4.0 + 4.0 * torch.rand(H, generator=g)
    dt_bias = torch.randn(H, generator=g)
    wn = torch.rand(dv, generator=g) + 0.5
    slots, n_slots = _slots(B)
    state = torch.randn(n_slots, H * dv * d + 3, generator=g)
    state[slots] = 0.0
    state = state.cuda()
    ob, oa, og = 2, 2 + H, 2 + 2 * H
    want_o, want_y = [], []
    for b in range(B):
        x, pj = qkv[b].double(), proj[b].double()
        q = _unit(x[:, :G * d].view(-1, G, d), 1e-6) * d ** -0.5
        k = _unit(x[:, G * d:2 * G * d].view(-1, G, d), 1e-6)
        v = x[:, 2 * G * d:].view(-1, H, dv)
        beta = PM.sigmoid(pj[:, ob:ob + H])
        decay = torch.exp(-torch.exp(a_log.double()) * PM.softplus(pj[:, oa:oa + H] + dt_bias.double()))
        o = PM.delta_recurrence(q, k, v, beta, decay)
        want_o.append(o.reshape(-1, H * dv))
        want_y.append((PM.rms(o, 1e-5) * wn.double()).reshape(-1, H * dv) * PM.silu(pj[:, og:]))
    got_o = [[] for _ in range(B)]
    got_y = [[] for _ in range(B)]
    at = [0] * B
    for take in (lens, more):
        rows = torch.cat([qkv[b][at[b]:at[b] + take[b]] for b in range(B)]).cuda()
        pr = torch.cat([proj[b][at[b]:at[b] + take[b]] for b in range(B)]).to(tdt).cuda()
        T = rows.shape[0]
        _, _, q_start = _packed(take, at)
        o = torch.full((T, H * dv), float("nan"), dtype=torch.float32, device="cuda")
        K.delta_rule(rows, pr, ob, oa, a_log.cuda(), dt_bias.cuda(), B, H, G, d, dv, 1e-6, q_start, _i32(slots), state, o,
                     max_rows=max(take))
        y = torch.empty((T, H * dv), dtype=tdt, device="cuda")
        K.head_norm_gate(o, H, dv, wn.cuda(), 1e-5, pr, og, "silu", y)
        n = 0
        for b in range(B):
            got_o[b].append(o[n:n + take[b]].cpu())
            got_y[b].append(y[n:n + take[b]].cpu())
            n += take[b]
            at[b] += take[b]
    for b in range(B):
        assert _rel(torch.cat(got_o[b]), want_o[b]) < 3e-5, b
        assert _rel(torch.cat(got_y[b]), want_y[b]) < (3e-5 if pdtype == "float32" else 1.2e-2), b


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,lens,planes", [(5, [7, 1, 2], 1), (130, [1, 1, 1], 2), (384, [64, 65, 63], 1),
                                           (72, [300, 2], 3), (1024, [700], 1)])
def test_min_gru_and_its_state(K, dtype, W, lens, planes):
    """S <- (1 - z) S + z c over packed sequences of unequal lengths, then two more steps from the stored state"""
    g = torch.Generator().manual_seed(W)
    tdt = DT[dtype]
    B = len(lens)
    takes = [lens, [1] * B, [130 if b == 0 else 3 for b in range(B)]]
    total = [sum(t[b] for t in takes) for b in range(B)]
    seqs = [torch.randn(total[b], 3 * W + 8, generator=g) * 2 for b in range(B)]
    if planes == 1:
        seqs = [s.to(tdt).float() for s in seqs]
    bz, bx = torch.randn(W, generator=g) - 2.0, torch.randn(W, generator=g)
    slots, n_slots = _slots(B)
    state = torch.randn(n_slots, W + 2, generator=g)
    state[slots] = 0.0
    state = state.cuda()
    oz, ox, og = 8, 8 + W, 8 + 2 * W
    want = []
    for b in range(B):
        x = seqs[b].double()
        S = PM.min_gru_scan(PM.sigmoid(x[:, oz:oz + W] + bz.double()), x[:, ox:ox + W] + bx.double())
        want.append(S * PM.silu(x[:, og:og + W]))
    got = [[] for _ in range(B)]
    at = [0] * B
    for take in takes:
        rows = torch.cat([seqs[b][at[b]:at[b] + take[b]] for b in range(B)])
        if planes > 1:
            parts = torch.randn(planes, *rows.shape, generator=g)
            parts[0] = rows - parts[1:].sum(0)
            src = parts.cuda()
        else:
            src = rows.to(tdt).cuda()
        _, _, q_start = _packed(take, at)
        out = torch.full((rows.shape[0], W), float("nan"), dtype=tdt, device="cuda")
        K.min_gru(src, oz, ox, og, W, bz.cuda(), bx.cuda(), B, q_start, _i32(slots), state, out, max_rows=max(take))
        n = 0
        for b in range(B):
            got[b].append(out[n:n + take[b]].cpu())
            n += take[b]
            at[b] += take[b]
    for b in range(B):
        assert _rel(torch.cat(got[b]), want[b]) < (2e-5 if dtype == "float32" else 1e-2), b


@pytest.mark.parametrize("T,E,n", [(1, 64, 2), (9, 200, 1), (70, 72, 3)])
def test_mean_of_normed_branches(K, T, E, n):
    g = torch.Generator().manual_seed(T + E)
    branches, want = [], torch.zeros(T, E, dtype=F64)
    for i in range(n):
        planes = torch.randn(1 + i, T, E, generator=g) * (3.0 ** i)
        bias = torch.randn(E, generator=g) if i % 2 == 0 else None
        gain = torch.rand(E, generator=g) + 0.5
        v = planes.double().sum(0) + (bias.double() if bias is not None else 0.0)
        want += PM.rms(v, 1e-5) * gain.double() / n
        branches.append((planes.cuda(), None if bias is None else bias.cuda(), gain.cuda()))
    out = torch.empty(T, E, dtype=torch.float32, device="cuda")
    K.branch_norm_mean(branches, 1e-5, out)
    assert _rel(out, want) < 1e-5


def _cache(lengths, nkv, hd, dtype, seed, extra=3):
    """pool [pages, 2, nkv, 64, hd] with every sequence's pages scattered, and the page table"""
    rng = random.Random(seed)
    n_blocks = [-(-n // 64) for n in lengths]
    n_pages = sum(n_blocks) + extra
    order = list(range(n_pages))
    rng.shuffle(order)
    table = torch.full((len(lengths), max(n_blocks) + 1), -1, dtype=torch.int32)
    at = 0
    for s, nb in enumerate(n_blocks):
        for b in range(nb):
            table[s, b] = order[at]
            at += 1
    # (what a page holds past its sequence's end is some other sequence's old content: finite, and large here)
    pool = (torch.randn((n_pages, 2, nkv, 64, hd), generator=torch.Generator().manual_seed(seed)) * 50).to(dtype)
    return pool, table, n_pages


def _sigmoid_attention_case(K, kind, dtype, nh, nkv, hd, q_lens, kv_lens, rows, far, seed, boost):
    """rows q_lens[b] at the end of sequences of kv_lens[b] positions; a distance table of `rows` rows folded with the
    heads' constants into one table over the distance, as the part does; `boost` = (sequence, key position): that
    key and every query are scaled so that its score stands far out of the others, which weigh about 0.01"""
    from kindi_b200.parts.sigmoid_attention import distance_bucket
    g = torch.Generator().manual_seed(seed)
    tdt = DT[dtype]
    B = len(q_lens)
    pool, table, n_pages = _cache(kv_lens, nkv, hd, tdt, seed)
    ks = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    qs = [torch.randn(n, nh, hd, generator=g) for n in q_lens]
    rel = torch.randn(rows, nh, generator=g)
    pb = -4.5 + 0.5 * torch.randn(nh, generator=g)
    if boost is not None:
        b, p = boost
        ks[b][p, :, 0] = 30.0
        for q in qs:
            q[:, :, 0] = 2.0
    scale = 0.17
    want = []
    for b in range(B):
        k, v, q = ks[b].to(tdt).double(), vs[b].to(tdt).double(), qs[b].to(tdt).double()
        want.append(PM.sigmoid_attention(q, k, v, scale, rel.double(), far, pb.double(), kv_lens[b] - q_lens[b]))
        for p in range(kv_lens[b]):
            page = int(table[b, p // 64])
            pool[page, 0, :, p % 64] = ks[b][p].to(tdt)
            pool[page, 1, :, p % 64] = vs[b][p].to(tdt)
    n = int(math.ceil(far)) + 1
    idx = torch.tensor([distance_bucket(i, rows, far) if i < far else rows - 1 for i in range(n)])
    bias = (rel[idx].t() + pb.view(nh, 1)).contiguous().cuda()
    q = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).to(tdt).cuda()
    out = torch.full_like(q, float("nan"))
    first = [kv_lens[b] - q_lens[b] for b in range(B)]
    pos, seq, q_start = _packed(q_lens, first)
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    kvl = _i32(kv_lens)
    st = _status()
    pool, table = pool.cuda(), table.cuda()
    if kind == "generic":
        K.sigmoid_attn(q, out, pos, seq, slot, nh, nkv, hd, scale, bias, pool, table, n_pages, st)
    elif kind == "tc":
        K.sigattn_tc(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, bias, pool, table, n_pages,
                     grid_x=-(-max(q_lens) // (128 // (nh // nkv))), status=st)
    else:
        K.sigattn_decode(q, out, slot, kvl, B, nh, nkv, hd, scale, bias, pool, table, n_pages, splits=int(kind[3:]),
                         status=st)
    assert int(st.item()) == 0
    return _rel(out.view(-1, nh, hd), torch.cat(want))


@pytest.mark.parametrize("kind,dtype,hd", [("generic", "float32", 24), ("generic", "bfloat16", 64),
                                           ("generic", "float32", 128), ("tc", "bfloat16", 64),
                                           ("tc", "bfloat16", 128)])
@pytest.mark.parametrize("rows,far", [(6, 7.5), (16, 64), (12, 200)])
def test_attention_without_a_softmax(K, kind, dtype, hd, rows, far):
    """prompt-sized steps: whole prompts and portions at the end of longer sequences, one to several query heads per
    key/value head; the key that stands out sits at the first position, at page borders, at the distances where the
    table's rows change and where its last row begins, and far back"""
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    fl = int(math.floor(far))
    for nh, nkv in ((4, 4), (6, 2), (8, 1)):
        L = 300
        for p in (0, 63, 64, L - 1 - rows // 2, L - rows // 2, L - fl, L - 1 - fl, L - 2 - fl, 5):
            if 0 <= p < L:
                err = _sigmoid_attention_case(K, kind, dtype, nh, nkv, hd, [L], [L], rows, far, p, (0, p))
                assert err < tol, (nh, nkv, p, err)
        err = _sigmoid_attention_case(K, kind, dtype, nh, nkv, hd, [2, 70, 1, 33], [66, 200, 129, 33], rows, far, 1, (1, 3))
        assert err < tol, (nh, nkv, err)
        err = _sigmoid_attention_case(K, kind, dtype, nh, nkv, hd, [130, 5], [130, 700], rows, far, 2, None)
        assert err < tol, (nh, nkv, err)


@pytest.mark.parametrize("kind", ["generic", "dec1", "dec2", "dec7"])
@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("rows,far", [(6, 7.5), (16, 64), (12, 200)])
def test_attention_without_a_softmax_single_tokens(K, kind, hd, rows, far):
    """decode steps in bfloat16: one row per sequence, contexts from one position to many pages, the key that stands
    out at a split's edge, at the table's edges and far back"""
    fl = int(math.floor(far))
    for nh, nkv in ((4, 4), (6, 2), (8, 1), (16, 1)):
        lens = [1, 64, 65, 700, 130, 2]
        for b, p in ((3, 0), (3, 699 - fl), (3, 698 - fl), (3, 700 - fl), (3, 447), (3, 448), (4, 129), (1, 63), (0, 0)):
            if p < 0:
                continue
            err = _sigmoid_attention_case(K, kind, "bfloat16", nh, nkv, hd, [1] * 6, lens, rows, far, p + b, (b, p))
            assert err < 1.5e-2, (nh, nkv, b, p, err)


@pytest.mark.parametrize("T,E,top", [(1, 4, 1), (9, 12, 3), (70, 8, 8), (33, 130, 2)])
def test_router_with_sigmoid_scores(K, T, E, top):
    """the `top` largest logits of a row; each one's weight is its own logistic function, not normalised"""
    g = torch.Generator().manual_seed(T * E)
    z = torch.randn(T, E, generator=g) * 2
    idx, wts = K.moe_topk(z.cuda(), None, top, "sigmoid")
    idx, wts = idx.cpu(), wts.cpu()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(z[t, e]), e))[:top]
        assert sorted(int(i) for i in idx[t]) == sorted(order), t
        for j in range(top):
            assert abs(float(wts[t, j]) - float(PM.sigmoid(z[t, int(idx[t, j])].double()))) < 1e-6


# ------------------------------------------------------------------------------------------- whole models
def _plain(folder, reqs):
    cfg, w = PM.load_model(folder)
    return {rid: PM.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def _compare(got, reqs, want, tol, what):
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        err = tiny.rel_err(mine, want[rid])
        row = int(np.argmax(np.max(np.abs(mine - want[rid]), axis=1)))
        assert err <= tol, "%s %s: %.3g at position %d of %d" % (what, rid, err, row, len(toks))


def _table_edges(raw):
    """the distances at which a distance table changes rows for good: where its logarithmic half begins and where its
    last row begins, over the layers"""
    out = set()
    for l in raw["layers"]:
        if l["type"] == "parallel":
            out |= {l["_rows"] // 2, int(math.floor(l["mixer"]["left"]["bias_max"]))}
    return sorted(out)


def _edge_requests(raw, seed, longest=420):
    """requests whose needle stands at the places that matter - the first position, a page's last and first position,
    just before, at and just behind each edge of the distance tables as seen from the probes at the end, far back -
    with probes over the last positions; and the shortest sequences there are"""
    rng = random.Random(seed)
    vocab = raw["vocab"]
    edges = [e for e in _table_edges(raw) if e < longest - 60]
    L = min(longest, max(edges, default=70) + 150)        # (a model of delta layers alone has no table)
    places = {0, 1, 63, 64, 127, 128}
    for e in edges:
        places |= {L - 3 - e, L - 2 - e, L - 1 - e, L - e}
    reqs = {}
    for p in sorted(x for x in places if 0 <= x < L - 8):
        reqs["n%d" % p] = TM.needle_request(vocab, L, p, list(range(L - 6, L)), rng)
    reqs["one"] = [rng.randrange(5, vocab)]
    reqs["two"] = [rng.randrange(5, vocab), TM.PROBE]
    reqs["three"] = [TM.NEEDLE, rng.randrange(5, vocab), TM.PROBE]
    return reqs


def _engine(folder, steps, dtype, **kw):
    from kindi_b200.engine.engine import Engine
    return Engine(folder, ctx=tiny.max_live_tokens(steps) + 64, dtype=dtype,
                  max_batch=max(len(s["entries"]) for s in steps), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TM.TINY))
def test_whole_prompts_and_token_by_token(tmp_path, name, dtype):
    """every request whole in one step, then again with its last 40 tokens one by one (the table's edges pass over
    decoded tokens; the recurrent states and the convolutions' tails go on from the prompt's), in the same engine,
    slots and pages"""
    raw = TM.TINY[name][0]
    folder = TM.make_model(tmp_path, name, dtype)
    reqs = _edge_requests(raw, seed=3)
    want = _plain(folder, reqs)
    steps = tiny.trace_whole(reqs)
    later = tiny.trace_last_n(reqs, 40)
    for s in later:
        s["step"] += len(steps)
    eng = _engine(folder, steps + later, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s whole" % (name, dtype))
    tiny.run_replay(eng, later, out)
    _compare(tiny.collect(out, later, raw["vocab"]), reqs, want, TOL[dtype], "%s %s decoded" % (name, dtype))
    eng.check_status()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_prompts_in_portions(tmp_path, name, dtype):
    """a prompt cut into portions of 2, 3, 31, 64 and 65 tokens, and a step limit that cuts it inside the engine: the
    logits are those of the whole prompt"""
    from kindi_b200.engine.engine import Engine
    raw = TM.TINY[name][0]
    folder = TM.make_model(tmp_path, name, dtype)
    reqs = {k: v for k, v in _edge_requests(raw, seed=4, longest=200).items() if k in ("n0", "n64", "three")}
    want = _plain(folder, reqs)
    for portion in (2, 3, 31, 64, 65):
        steps = []
        for rid, toks in reqs.items():
            for a in range(0, len(toks), portion):
                part = toks[a:a + portion]
                steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": part,
                                                               "want": list(range(len(part)))}],
                              "end": [rid] if a + portion >= len(toks) else []})
        eng = _engine(folder, steps, dtype)
        out = str(tmp_path / ("out%d" % portion))
        tiny.run_replay(eng, steps, out)
        eng.check_status()
        _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s by %d" % (name, dtype, portion))
    steps = tiny.trace_whole(reqs)
    eng = Engine(folder, ctx=tiny.max_live_tokens(steps) + 64, dtype=dtype, max_batch=2, max_step_tokens=64)
    out = str(tmp_path / "outcut")
    tiny.run_replay(eng, steps, out)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s cut inside" % (name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TM.TINY))
def test_unequal_batches_and_reused_slots(tmp_path, name, dtype):
    """batches of unequal requests that start together and are decoded together, shorter ones ending earlier, a
    second batch in the slots, pages and state the first gave back: every row as if its request ran alone"""
    raw = TM.TINY[name][0]
    folder = TM.make_model(tmp_path, name, dtype)
    reqs = _edge_requests(raw, seed=5, longest=300)
    ids = list(reqs)
    rng = random.Random(9)
    decode = {r: min(len(reqs[r]) - 1, rng.choice([0, 3, 9, 30])) for r in ids}
    half = len(ids) // 2
    steps = tiny.trace_group({r: reqs[r] for r in ids[:half]}, decode)
    steps += tiny.trace_group({r: reqs[r] for r in ids[half:]}, decode, first_step=len(steps))
    want = _plain(folder, reqs)
    eng = _engine(folder, steps, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    eng.cache.check()
    assert eng.cache.slots.n_held == 0 and all(g.pages.pool.n_held == 0 for g in eng.cache.groups)
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "%s %s batches" % (name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_in_a_batch(tmp_path, dtype):
    """three requests decoded together for 330 steps (recorded decode steps; states, tails and pages carried all the
    way), probes throughout, a needle near the start, at a page's first position and late"""
    raw = TM.TINY["B"][0]
    folder = TM.make_model(tmp_path, "B", dtype)
    rng = random.Random(2)
    reqs = {"a": TM.needle_request(raw["vocab"], 400, 2, list(range(60, 400, 3)), rng),
            "b": TM.needle_request(raw["vocab"], 350, 64, list(range(200, 350, 2)), rng),
            "c": TM.needle_request(raw["vocab"], 340, 300, list(range(100, 340, 5)), rng)}
    steps = tiny.trace_group(reqs, {"a": 330, "b": 330, "c": 330})
    want = _plain(folder, reqs)
    eng = _engine(folder, steps, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    assert eng.graph_replays > 300
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "long %s" % dtype)


@pytest.mark.parametrize("dtype,tie", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype, tie):
    from kindi_b200 import Engine
    raw = TM.TINY[name][0]
    folder = TM.make_model(tmp_path, name, dtype)
    cfg, w = PM.load_model(folder)
    eng = Engine(folder, ctx=2048, dtype=dtype, max_batch=3)
    prompts = list(tiny.random_requests(raw["vocab"], [5, 9, 1, 80, 13], seed=3).values())
    res = eng.generate_batch(prompts, temperature=0.0, max_tokens=10, stop_token_ids=())
    assert res.stats.batches == 2 and eng.cache.slots.n_held == 0
    for p, got in zip(prompts, res.tokens):
        assert len(got) == 10
        seq = list(p)
        for t in got:
            z = PM.forward(cfg, w, seq)[-1].numpy()
            best = int(np.argmax(z))
            assert t == best or z[best] - z[t] <= tie * np.abs(z).max(), (len(seq), t, best)
            seq.append(t)
    eng.cache.check()


def test_trace_run_and_command_line_as_programs(tmp_path):
    folder = TM.make_model(tmp_path, "A", "bfloat16")
    vocab = TM.MD_A["vocab"]
    reqs = tiny.random_requests(vocab, [5, 40], seed=2)
    steps = tiny.trace_batched(reqs, batch=2, decode=4)
    out = str(tmp_path / "out")
    env = dict(os.environ, PYTHONDONTWRITEBYTECODE="1")
    r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", "bfloat16", "--out", out,
                        "--max-tokens", str(tiny.max_live_tokens(steps))],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, env=env,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    got = tiny.collect(out, steps, vocab)
    _compare(got, reqs, _plain(folder, reqs), TOL["bfloat16"], "trace_run")
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", folder, "--ctx", "512", "generate",
                        "--prompt-ids", "1,2,3", "--prompt-ids", "9 8", "--temperature", "0", "--max-tokens", "5"],
                       capture_output=True, text=True, cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.strip().split("\n")]
    assert len(lines) == 2 and all(len(l["tokens"]) == 5 for l in lines)
    r = subprocess.run([sys.executable, "-m", "kindi_b200", "--model", folder, "info"], capture_output=True, text=True,
                       cwd=ROOT, env=env, timeout=600)
    assert r.returncode == 0 and "Medodra" in r.stdout + r.stderr, r.stderr[-2000:]
