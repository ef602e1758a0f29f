"""The Nilatar architecture on the GPU against the plain implementation (``plain_nilatar``): each mechanism's kernel
alone, then whole models of five small configurations through the engine's step function, its cache and state and
its generation loop, in true 32-bit and in bfloat16.

The models carry a planted key (``tiny_nilatar.make_model``): a probe token's attention rests on one needle token, so
a dropped key, a window that is one position off, a page of another sequence or a slot's old content changes a
probe's logits by many times the tolerance; the sinks carry a good part of a softmax's mass. The 32-bit runs are the
sharp ones for everything else (rotation, decay, state, scales).
"""
import json
import os
import random
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_nilatar as PN
import tiny
import tiny_nilatar as TN

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# (bfloat16: with activations stored in 16 bits the typical row of these models lies 0.3 % of the largest logit away
# from the 64-bit result and single rows up to 4 %, with the general kernels as with the tensor-core ones; what the
# planted key changes is 17 % to 110 %. The 32-bit runs are the sharp ones.)
TOL = {"float32": 3e-5, "bfloat16": 6e-2}
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


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


def _ctx(T, tdt, fast, **kw):
    from kindi_b200.parts.base import StepContext
    base = dict(T=T, B=1, tok=None, pos=None, seq=None, slot=None, q_start=None, kv_len=None, h_slot=None,
                h_q_start=None, h_kv_len=None, decode=False, max_q=T, max_kv=T, dtype=tdt, device=torch.device("cuda"),
                status=_status(), fast=fast)
    base.update(kw)
    return StepContext(**base)


# ------------------------------------------------------------------------------------------- kernels alone
@pytest.mark.parametrize("T,E,planes,ydtype", [(1, 64, 1, "float32"), (5, 200, 3, "float32"), (33, 72, 1, "bfloat16"),
                                               (3, 4100, 2, "float32"), (200, 256, 9, "bfloat16"),
                                               (600, 384, 2, "bfloat16"), (2100, 1024, 1, "bfloat16"),
                                               (520, 3200, 1, "bfloat16")])
def test_scaled_branch_add_and_rms_norm(K, T, E, planes, ydtype):
    """x += ls * (sum of the planes), then the RMS norm: every form of the norm kernel (a block a row, four warps a
    row, a warp a row in registers and in passes)"""
    g = torch.Generator().manual_seed(T * 1000 + E)
    tdt = DT[ydtype]
    x = torch.randn(T, E, generator=g) * 2
    d = torch.randn(planes, T, E, generator=g)
    w = (torch.randn(E, generator=g) * 0.3 + 1).to(tdt)
    ls = (torch.randn(E, generator=g) * 0.5 + 1).to(tdt)
    v = x.double() + d.double().sum(0) * ls.double()
    want = PN.rms_norm(v, w.double(), 1e-5)
    xd, out = x.cuda(), torch.empty(T, E, dtype=tdt, device="cuda")
    st = _status()
    K.add_rmsnorm(xd, d.cuda(), w.cuda(), 1e-5, out, None, True, st, branch_scale=ls.cuda())
    assert _rel(out, want) < (1e-5 if ydtype == "float32" else 8e-3) and int(st.item()) == 0
    assert _rel(xd, v) < 1e-6                                 # the scaled sum was written back
    # chosen rows, nothing written back
    rows = torch.tensor([T - 1, 0], dtype=torch.int32, device="cuda")
    x2, out2 = x.cuda(), torch.empty(2, E, dtype=tdt, device="cuda")
    K.add_rmsnorm(x2, d.cuda(), w.cuda(), 1e-5, out2, rows, False, st, branch_scale=ls.cuda())
    assert _rel(out2, want[[T - 1, 0]]) < (1e-5 if ydtype == "float32" else 8e-3) and torch.equal(x2.cpu(), x)


@pytest.mark.parametrize("dtype,fast", [("float32", False), ("bfloat16", False), ("bfloat16", True)])
@pytest.mark.parametrize("M,width,F", [(1, 64, 48), (8, 256, 512), (20, 128, 96), (70, 72, 20), (300, 256, 640),
                                       (1500, 512, 1024)])
def test_gated_feed_forward_with_gelu(K, dtype, fast, M, width, F):
    """act(W_gate y) * (W_up y) with the tanh form of GELU: the stand-alone kernel and the products that finish it in
    their epilogues (decode form, prompt form, pairs of SMs); silu stays what it was"""
    from kindi_b200.kernels import linear as L
    g = torch.Generator().manual_seed(M + F)
    tdt = DT[dtype]
    y = (torch.randn(M, width, generator=g)).to(tdt)
    wg, wu = ((torch.randn(F, width, generator=g) * 0.15).to(tdt) for _ in range(2))
    wgu, group = L.join_gate_up(wg.cuda(), wu.cuda())
    for act, fn in (("gelu_tanh", PN.gelu_tanh), ("silu", PN.silu)):
        want = fn(y.double() @ wg.double().T) * (y.double() @ wu.double().T)
        ctx = _ctx(M, tdt, fast)
        got = L.gate_up_swiglu(ctx, y.cuda(), wgu, group, F, tdt, act)
        assert int(ctx.status.item()) == 0
        assert _rel(got, want) < (2e-5 if dtype == "float32" else 1.5e-2), (act, dtype, fast)


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


def _attention_case(K, kind, dtype, nh, nkv, hd, q_lens, kv_lens, window, seed, boost, sink_mean, gated):
    """rows q_lens[b] at the end of sequences of kv_lens[b] positions, a sink per head, optionally an output gate;
    `boost` = (sequence, key position): that key and every query are scaled so that its score stands out"""
    g = torch.Generator().manual_seed(seed)
    tdt = DT[dtype]
    B = len(q_lens)
    pool, table, n_pages = _cache(kv_lens, nkv, hd, tdt, seed)
    ks = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    vs = [torch.randn(n, nkv, hd, generator=g) for n in kv_lens]
    qs = [torch.randn(n, nh, hd, generator=g) for n in q_lens]
    gs = [torch.randn(n, nh, hd, generator=g) * 2 for n in q_lens]
    sink = torch.randn(nh, generator=g) + sink_mean
    if boost is not None:
        b, p = boost
        ks[b][p, :, 0] = 30.0
        for q in qs:
            q[:, :, 0] = 2.0
    scale = 0.17
    want = []
    rep = nh // nkv
    for b in range(B):
        k, v, q = ks[b].to(tdt).double(), vs[b].to(tdt).double(), qs[b].to(tdt).double()
        full = torch.zeros(kv_lens[b], nh, hd, dtype=torch.float64)
        full[kv_lens[b] - q_lens[b]:] = q
        o = PN.softmax_attention(full.transpose(0, 1), k.transpose(0, 1).repeat_interleave(rep, dim=0),
                                 v.transpose(0, 1).repeat_interleave(rep, dim=0), scale, window, sink.double())
        o = o.transpose(0, 1)[kv_lens[b] - q_lens[b]:]
        if gated:
            o = o * torch.sigmoid(gs[b].to(tdt).double())
        want.append(o)
        for p in range(kv_lens[b]):
            page = int(table[b, p // 64])
            pool[page, 0, :, p % 64] = ks[b][p].to(tdt)
            pool[page, 1, :, p % 64] = vs[b][p].to(tdt)
    q = torch.cat([x.reshape(x.shape[0], -1) for x in qs]).to(tdt).cuda()
    gate = torch.cat([x.reshape(x.shape[0], -1) for x in gs]).to(tdt).cuda() if gated else None
    out = torch.full_like(q, float("nan"))
    pos = torch.cat([torch.arange(kv_lens[b] - q_lens[b], kv_lens[b]) for b in range(B)]).to(torch.int32).cuda()
    seq = torch.cat([torch.full((q_lens[b],), b) for b in range(B)]).to(torch.int32).cuda()
    slot = torch.arange(B, dtype=torch.int32, device="cuda")
    q_start = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32, device="cuda")
    kvl = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    st = _status()
    pool, table, sk = pool.cuda(), table.cuda(), sink.cuda()
    if kind == "generic":
        K.attn_generic(q, out, pos, seq, slot, nh, nkv, hd, scale, window or 0, pool, table, n_pages, st, 0, sk, gate)
    elif kind == "tc":
        K.attn_tc(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages,
                  grid_x=-(-max(q_lens) // (128 // (nh // nkv))), status=st, sink=sk, gate=gate)
    elif kind == "mma":
        K.attn_mma(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages, decode=False,
                   grid_x=-(-max(q_lens) * (nh // nkv) // 64), status=st, sink=sk)
    else:
        K.attn_mma(q, out, slot, q_start, kvl, B, nh, nkv, hd, scale, window or 0, pool, table, n_pages, decode=True,
                   grid_x=int(kind[3:]), status=st, sink=sk)
    if gated and kind not in ("generic", "tc"):
        K.gate_mul(out, gate, out)
    assert int(st.item()) == 0
    return _rel(out.view(-1, nh, hd), torch.cat(want))


@pytest.mark.parametrize("kind,dtype,hd", [("generic", "float32", 24), ("generic", "bfloat16", 64),
                                           ("generic", "float32", 320), ("tc", "bfloat16", 64), ("tc", "bfloat16", 128),
                                           ("mma", "bfloat16", 64), ("dec1", "bfloat16", 128), ("dec3", "bfloat16", 64),
                                           ("dec7", "bfloat16", 64)])
@pytest.mark.parametrize("window", [1, 37, 64, 130, None])
def test_attention_with_a_sink_and_a_gate(K, kind, dtype, hd, window):
    """a sink that weighs like many keys (and one that weighs nothing beside a key that stands out), with the key
    placed just inside and just outside the window, at page borders and far back: prompt rows and single decoded rows,
    with and without the output gate"""
    tol = 2e-5 if dtype == "float32" else 1.5e-2
    dec = kind.startswith("dec")
    L = 321
    w = window or L
    places = {0, L - w - 1, L - w, L - w + 1, 63, 64, L - 1}
    for n, p in enumerate(sorted(x for x in places if 0 <= x < L)):
        q_lens = [1, 1] if dec else [L - 200, 37]
        err = _attention_case(K, kind, dtype, 6, 2, hd, q_lens, [L, 150], window, seed=L + p, boost=(0, p),
                              sink_mean=3.0, gated=n % 2 == 0)
        assert err < tol, (kind, L, p, err)
    # no key stands out: the sink is a large share of every row's denominator
    err = _attention_case(K, kind, dtype, 6, 2, hd, [1, 1] if dec else [90, 37], [L, 150], window, seed=5, boost=None,
                          sink_mean=2.0, gated=True)
    assert err < tol, (kind, "sink", err)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("T,q_rank,kv_rank,rot,D,planes,scaling", [
    (7, 24, 20, 8, 64, 1, None), (40, 64, 48, 16, 64, 3, (8.0, 64, 4.0, 1.0)), (3, 72, 96, 32, 128, 2, (4.0, 32, 8.0, 0.5)),
    (65, 20, 18, 6, 24, 1, (2.0, 16, 2.0, 1.0)), (9, 40, 100, 64, 168, 4, (16.0, 128, 32.0, 1.0))])
def test_latent_norms_rotation_and_store(K, dtype, T, q_rank, kv_rank, rot, D, planes, scaling):
    """the query latent normalised; the key/value latent normalised and stored as the cached head's keys and values;
    the shared key part rotated by interleaved pairs with stretched frequencies; from rows and from 32-bit planes"""
    from kindi_b200.parts.rope import yarn_frequencies
    g = torch.Generator().manual_seed(T + q_rank)
    tdt = DT[dtype]
    extra = 11
    row = torch.randn(T, q_rank + kv_rank + rot + extra, generator=g) * 2
    wq, wkv = ((torch.rand(n, generator=g) + 0.5).to(tdt) for n in (q_rank, kv_rank))
    if planes == 1:
        row = row.to(tdt).float()
    pos = torch.tensor([3 * t + 60 for t in range(T)], dtype=torch.int32)      # positions that cross a page
    pos[0] = 0
    rspec = {"base": 10000.0, "dims": rot}
    if scaling:
        rspec["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    freq, mult = PN.rotation_table(rspec)
    r64 = row.double()
    want_cq = PN.rms_norm(r64[:, :q_rank], wq.double(), 1e-5)
    want_c = PN.rms_norm(r64[:, q_rank:q_rank + kv_rank], wkv.double(), 1e-5)
    want_kr = PN.rotate_pairs(r64[:, q_rank + kv_rank:q_rank + kv_rank + rot], pos, freq, mult)
    if planes > 1:
        parts = torch.randn(planes, *row.shape, generator=g)
        parts[0] = row - parts[1:].sum(0)
        src = parts.cuda()
    else:
        src = row.to(tdt).cuda()
    pool, table, n_pages = _cache([int(pos.max()) + 1], 1, D, tdt, seed=T)
    pool, table = pool.cuda(), table.cuda()
    f, m = yarn_frequencies(10000.0, rot, rspec.get("scaling"))
    assert abs(m - mult) < 1e-12 and float((f - freq).abs().max()) < 1e-12
    cq = torch.empty(T, q_rank, dtype=tdt, device="cuda")
    zeros = torch.zeros(T, dtype=torch.int32, device="cuda")
    st = _status()
    K.latent_prep(src, q_rank, kv_rank, rot, wq.cuda(), wkv.cuda(), 1e-5, f.float().cuda(), m, pos.cuda(), zeros,
                  zeros[:1], cq, D, pool, table, n_pages, st)
    assert int(st.item()) == 0
    tol = 2e-5 if dtype == "float32" else 1.2e-2
    assert _rel(cq, want_cq) < tol
    for t in range(T):
        p = int(pos[t])
        page = int(table[0, p // 64])
        kd, vd = pool[page, 0, 0, p % 64], pool[page, 1, 0, p % 64]
        assert _rel(kd[:kv_rank], want_c[t]) < tol and _rel(vd[:kv_rank], want_c[t]) < tol
        assert _rel(kd[kv_rank:kv_rank + rot], want_kr[t]) < tol
        assert float(kd[kv_rank + rot:].float().abs().max() if D > kv_rank + rot else 0) == 0
        assert float(vd[kv_rank:].float().abs().max()) == 0
    # the queries' rotated parts
    H, dim = 3, 10
    q = (torch.randn(T, H * (dim + rot), generator=g)).to(tdt)
    out = torch.full((T, H * D), float("nan"), dtype=tdt, device="cuda")
    K.latent_qrope(q.cuda(), dim, rot, f.float().cuda(), m, pos.cuda(), out, kv_rank, D, H)
    want_q = PN.rotate_pairs(q.double().view(T, H, dim + rot)[..., dim:].transpose(0, 1), pos, freq,
                             mult).transpose(0, 1)                                             # [T, H, rot]
    got = out.view(T, H, D)
    assert _rel(got[..., kv_rank:kv_rank + rot], want_q) < tol
    assert float(got[..., kv_rank + rot:].float().abs().max() if D > kv_rank + rot else 0) == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("M,H,N,Kd,planes", [(1, 2, 5, 7, 1), (70, 4, 20, 16, 2), (130, 8, 48, 32, 0), (9, 3, 100, 130, 1),
                                             (300, 8, 96, 128, 0), (65, 5, 41, 72, 2), (8, 16, 128, 96, 1)])
def test_products_per_head(K, dtype, M, H, N, Kd, planes):
    """out[t][h] = W[h] a[t][h] over strided heads, with and without the gate in the epilogue; bf16 operands with
    aligned rows on the tensor cores, everything else by 32-bit multiply-adds"""
    g = torch.Generator().manual_seed(M + N)
    tdt = DT[dtype]
    sa, so = Kd + (8 if Kd % 8 == 0 else 3), N + 5       # head strides wider than the heads
    a = torch.randn(M, H * sa, generator=g).to(tdt)
    w = (torch.randn(H, N, Kd, generator=g) * 0.3).to(tdt)
    want = torch.einsum("thk,hnk->thn", a.double().view(M, H, sa)[..., :Kd], w.double())
    gate = None
    if planes:
        gate = torch.randn(planes, M, H * N, generator=g) if planes > 1 else torch.randn(M, H * N, generator=g).to(tdt)
        want = want * torch.sigmoid((gate.double().sum(0) if planes > 1 else gate.double()).view(M, H, N))
    out = torch.zeros(M, H * so, dtype=tdt, device="cuda")
    K.head_gemm(a.cuda(), sa, w.cuda(), out, so, gate=gate.cuda() if gate is not None else None)
    got = out.view(M, H, so)
    assert _rel(got[..., :N], want) < (2e-5 if dtype == "float32" else 1e-2)
    assert float(got[..., N:].float().abs().max()) == 0    # nothing written between the heads
    out2 = torch.zeros(M, H * so, dtype=tdt, device="cuda")
    K.head_gemm(a.cuda(), sa, w.cuda(), out2, so, gate=gate.cuda() if gate is not None else None, tensor_cores=False)
    assert _rel(out2.view(M, H, so)[..., :N], want) < (2e-5 if dtype == "float32" else 1e-2)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("chunk", [0, 16, 64])
@pytest.mark.parametrize("H,d,dv,lens,planes", [(2, 16, 24, [5, 1, 40], 1), (4, 32, 64, [70, 3], 3), (1, 64, 32, [33], 1),
                                                (3, 40, 9, [1, 1, 1, 1], 2), (2, 128, 16, [19, 130], 1),
                                                (1, 256, 8, [17], 1), (2, 128, 128, [300, 64, 65], 1)])
def test_decayed_recurrence_and_its_state(K, dtype, H, d, dv, lens, planes, chunk):
    """S <- decay S + k v^T, o = S^T q over several sequences in one packed step, then a second step that goes on from
    the stored state (one token for some sequences, several for others), in slots that are not in order; token by
    token (chunk 0) and with a sequence's runs of `chunk` tokens side by side; the gated norm over the heads"""
    g = torch.Generator().manual_seed(H * d + dv)
    tdt = DT[dtype]
    B = len(lens)
    more = [1 if b % 2 == 0 else 7 for b in range(B)]
    decay = torch.tensor([0.5, 0.9, 0.99, 1.0][:H], dtype=torch.float32)
    ncol = 2 * H * d + 2 * H * dv
    seqs = [torch.randn(lens[b] + more[b], ncol, generator=g) for b in range(B)]
    if planes == 1:
        seqs = [s.to(tdt).float() for s in seqs]
    n_slots = B + 3
    slots = list(range(n_slots))
    random.Random(3).shuffle(slots)
    slots = slots[:B]
    state = torch.randn(n_slots, H, dv, d, generator=g)              # stale content everywhere ...
    for s in slots:
        state[s] = 0.0                                                 # ... but a taken slot starts at zero
    state = state.cuda()
    wn = (torch.rand(H * dv, generator=g) + 0.5).to(tdt)
    want = []
    for b in range(B):
        x = seqs[b].double()
        q = PN.silu(x[:, :H * d]).view(-1, H, d)
        k = PN.silu(x[:, H * d:2 * H * d]).view(-1, H, d)
        v = PN.silu(x[:, 2 * H * d:2 * H * d + H * dv]).view(-1, H, dv)
        S = torch.zeros(H, d, dv, dtype=torch.float64)
        o = torch.empty(x.shape[0], H, dv, dtype=torch.float64)
        for t in range(x.shape[0]):
            S = decay.double()[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
            o[t] = torch.einsum("hde,hd->he", S, q[t])
        o = o.view(-1, H * dv)
        want.append((o, PN.rms_norm(o, wn.double(), 1e-5) * torch.sigmoid(x[:, 2 * H * d + H * dv:])))
    got_o = [[] for _ in range(B)]
    got_y = [[] for _ in range(B)]
    for step, take in enumerate([lens, more]):
        rows = torch.cat([seqs[b][(0 if step == 0 else lens[b]):(lens[b] if step == 0 else lens[b] + more[b])]
                          for b in range(B)])
        T = rows.shape[0]
        if planes > 1:
            parts = torch.randn(planes, *rows.shape, generator=g)
            parts[0] = rows - parts[1:].sum(0)
            src = parts.cuda()
        else:
            src = rows.to(tdt).cuda()
        q_start = torch.tensor([0] + list(np.cumsum(take)), dtype=torch.int32, device="cuda")
        o = torch.full((T, H * dv), float("nan"), dtype=torch.float32, device="cuda")
        K.decay_scan(src, B, H, d, dv, decay.cuda(), q_start, torch.tensor(slots, dtype=torch.int32, device="cuda"),
                     state, o, chunk=chunk, max_rows=max(take) + (5 if chunk else 0))
        y = torch.empty(T, H * dv, dtype=tdt, device="cuda")
        K.gated_rmsnorm(o, wn.cuda(), 1e-5, src[..., 2 * H * d + H * dv:], y)
        at = 0
        for b in range(B):
            got_o[b].append(o[at:at + take[b]].cpu())
            got_y[b].append(y[at:at + take[b]].cpu())
            at += take[b]
    tol = 3e-5 if dtype == "float32" else 1.2e-2
    for b in range(B):
        assert _rel(torch.cat(got_o[b]), want[b][0]) < tol, b
        assert _rel(torch.cat(got_y[b]), want[b][1]) < tol, b


# ------------------------------------------------------------------------------------------- whole models
def _plain(folder, reqs):
    cfg, w = PN.load_model(folder)
    return {rid: PN.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def _compare(got, reqs, want, tol, what):
    for rid, toks in reqs.items():
        mine = np.stack([got[(rid, i)] for i in range(len(toks))])
        err = tiny.rel_err(mine, want[rid])
        row = int(np.argmax(np.max(np.abs(mine - want[rid]), axis=1)))
        assert err <= tol, "%s %s: %.3g at position %d of %d" % (what, rid, err, row, len(toks))


def _windows(raw):
    return sorted({l["mixer"]["mask"]["size"] for l in raw["layers"] if l["type"] == "attention" and "mask" in l["mixer"]})


def _edge_requests(raw, seed):
    """requests whose needle stands at the places that matter - the first position, just inside and just outside each
    window as seen from the probes at the end, at a page border, far back - with probes over the last positions; and
    the shortest sequences there are"""
    rng = random.Random(seed)
    vocab = raw["vocab"]
    windows = _windows(raw) or [50]
    reqs = {}
    L = max(windows) + 150
    places = {0, 1, 63, 64}
    for w in windows:
        places |= {L - 4 - w, L - 3 - w, L - 2 - w, L - 1 - w}
    for p in sorted(x for x in places if 0 <= x < L - 8):
        reqs["n%d" % p] = TN.needle_request(vocab, L, p, list(range(L - 6, L)), rng)
    reqs["one"] = [rng.randrange(5, vocab)]
    reqs["two"] = [rng.randrange(5, vocab), TN.PROBE]
    return reqs


def _engine(folder, steps, dtype, **kw):
    from kindi_b200.engine.engine import Engine
    return Engine(folder, ctx=tiny.max_live_tokens(steps) + 64, dtype=dtype,
                  max_batch=max(len(s["entries"]) for s in steps), **kw)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TN.TINY))
def test_whole_prompts_and_token_by_token(tmp_path, name, dtype):
    """every request whole in one step, then again with its last 40 tokens one by one (the windows pass over decoded
    tokens and the needle leaves them; the recurrent state goes on from the prompt's), in the same engine, slots and
    pages"""
    raw = TN.TINY[name][0]
    folder = TN.make_model(tmp_path, name, dtype)
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
    raw = TN.TINY[name][0]
    folder = TN.make_model(tmp_path, name, dtype)
    reqs = {k: v for k, v in _edge_requests(raw, seed=4).items() if k in ("n0", "n64", "two")}
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
@pytest.mark.parametrize("name", sorted(TN.TINY))
def test_unequal_batches_and_reused_slots(tmp_path, name, dtype):
    """batches of unequal requests that start together and are decoded together, shorter ones ending earlier, a
    second batch in the slots, pages and state the first gave back: every row as if its request ran alone"""
    raw = TN.TINY[name][0]
    folder = TN.make_model(tmp_path, name, dtype)
    # (seed 5 draws a request of which one row is ill-conditioned in bfloat16 for configuration B: 0.07 of the largest
    # logit also when the request runs alone, twice what any other row shows; the test is about batches, not that row)
    reqs = _edge_requests(raw, seed=6)
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
    """three requests decoded together for 330 steps (recorded decode steps; the windows' pages are given back, the
    state is carried), probes all the way, a needle far back for the layers that see everything"""
    raw = TN.TINY["B"][0]
    folder = TN.make_model(tmp_path, "B", dtype)
    rng = random.Random(2)
    reqs = {"a": TN.needle_request(raw["vocab"], 400, 2, list(range(60, 400, 3)), rng),
            "b": TN.needle_request(raw["vocab"], 350, 69, list(range(200, 350, 2)), rng),
            "c": TN.needle_request(raw["vocab"], 340, 300, list(range(100, 340, 5)), rng)}
    steps = tiny.trace_group(reqs, {"a": 330, "b": 330, "c": 330})
    want = _plain(folder, reqs)
    eng = _engine(folder, steps, dtype)
    out = str(tmp_path / "out")
    tiny.run_replay(eng, steps, out)
    eng.check_status()
    assert eng.graph_replays > 300
    # a window group holds what the widest window that reads it touches, not the sequences
    for g in eng.cache.groups:
        if g.need.window is not None:
            assert g.need.window == 70 and g.n_pool_pages <= 3 * (-(-g.need.window // 64) + 4) + 128
    _compare(tiny.collect(out, steps, raw["vocab"]), reqs, want, TOL[dtype], "long %s" % dtype)


@pytest.mark.parametrize("dtype,tie", [("float32", 1e-5), ("bfloat16", 2e-2)])
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_entry_point(tmp_path, name, dtype, tie):
    from kindi_b200 import Engine
    raw = TN.TINY[name][0]
    folder = TN.make_model(tmp_path, name, dtype)
    cfg, w = PN.load_model(folder)
    eng = Engine(folder, ctx=2048, dtype=dtype, max_batch=3)
    prompts = list(tiny.random_requests(raw["vocab"], [5, 9, 1, 80, 13], seed=3).values())
    res = eng.generate_batch(prompts, temperature=0.0, max_tokens=10, stop_token_ids=())
    assert res.stats.batches == 2 and eng.cache.slots.n_held == 0
    for p, got in zip(prompts, res.tokens):
        assert len(got) == 10
        seq = list(p)
        for t in got:
            z = PN.forward(cfg, w, seq)[-1].numpy()
            best = int(np.argmax(z))
            assert t == best or z[best] - z[t] <= tie * np.abs(z).max(), (len(seq), t, best)
            seq.append(t)
    eng.cache.check()


def test_trace_run_and_command_line_as_programs(tmp_path):
    folder = TN.make_model(tmp_path, "A", "bfloat16")
    vocab = TN.NL_A["vocab"]
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
    assert r.returncode == 0 and "Nilatar" in r.stdout + r.stderr, r.stderr[-2000:]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["B", "C"])
def test_recorded_prompt_steps_and_their_padding_rows(tmp_path, name, dtype):
    """short prompt steps are padded to a multiple of 64 rows and replayed from a recording once their shape has come
    twice: the padding rows go through the norms and products like any row, store nothing, touch no state and change
    no other row; in 32-bit a recorded step gives the bits of an engine that records nothing"""
    from kindi_b200.engine.batch import StepEntry
    from kindi_b200.engine.engine import Engine
    raw = TN.TINY[name][0]
    folder = TN.make_model(tmp_path, name, dtype)
    cfg, w = PN.load_model(folder)
    rng = random.Random(9)
    eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4)
    plain_eng = Engine(folder, ctx=4096, dtype=dtype, max_batch=4, cuda_graphs=False)

    def run(e, groups, follow=3):
        out = []
        for group in groups:
            slots = [e.alloc() for _ in group]
            k = [len(t) - follow for t in group]
            logits = e.step([StepEntry(s, tuple(t[:n]), (n - 1,)) for s, t, n in zip(slots, group, k)])
            rows = [[logits[i].cpu().numpy()] for i in range(len(group))]
            for j in range(follow):
                lg = e.step([StepEntry(s, (t[n + j],), (0,)) for s, t, n in zip(slots, group, k)])
                for i in range(len(group)):
                    rows[i].append(lg[i].cpu().numpy())
            e.check_status()
            for s in slots:
                e.free(s)
            out.append([np.stack(r) for r in rows])
        return out

    lengths = [[103], [93], [131], [68], [73], [40, 71], [64, 9], [8, 100], [200], [260], [300]]
    groups = [[TN.needle_request(raw["vocab"], n, 1, list(range(n - 5, n)), rng) for n in g] for g in lengths]
    got = run(eng, groups)
    assert sum(1 for k in eng._graphs if k[0] == "prompt") >= 2 and eng.graph_replays >= 6
    same = run(plain_eng, groups)
    for g, mine, other in zip(groups, got, same):
        for toks, a, b in zip(g, mine, other):
            want = PN.forward(cfg, w, toks).numpy()[len(toks) - 4:]
            assert tiny.rel_err(a, want) <= TOL[dtype], (len(toks), tiny.rel_err(a, want))
            if dtype == "float32":
                assert np.array_equal(a, b), len(toks)
    eng.cache.check()
    assert eng.cache.slots.n_held == 0
