"""The Luzerax architecture without a GPU: its configuration reader, names and shapes, cache needs, the plain
implementation's own sanity (the planted key decides a probe's logits; the router's groups and correction), and the
layouts the mixer part gives its weights (an interleaved rotation as a row permutation, differential attention as
grouped-query attention over twice the heads) checked against the plain mixers in 64-bit."""
import copy
import math
import random

import numpy as np
import pytest
import torch

import plain_luzerax as PL
import tiny
import tiny_luzerax as TL
from kindi_b200.config import ConfigError
from kindi_b200.config.registry import model_from_config, part_class
from kindi_b200.parts.base import KVNeed, WeightView
from kindi_b200.parts.model import cache_needs, expected_tensors, tensor_inits


def test_config_reads_every_size_from_the_nested_keys():
    cfg, spec = model_from_config(TL.LZ_A)
    assert (cfg.vocab, cfg.width, cfg.eps) == (211, 64, 1e-5)
    assert [l.kind for l in cfg.layers] == ["attention", "attention", "attention_2"]
    m = cfg.layers[0].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.diff, m.temp_coef, m.temp_every) == \
        (4, 2, 16, 24, 0.5, 0.55, 0.5, 16)
    m = cfg.layers[2].mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.rot_base, m.rot_dims) == (4, 2, 16, 24, 10000.0, 8)
    f = cfg.layers[0].ff
    assert (f.experts, f.identity, f.top, f.groups, f.keep, f.ff, f.limit, f.shared_ff) == (4, 0, 2, 1, 1, 24, 0.7, None)
    assert cfg.layers[1].ff is None and cfg.layers[2].ff == 40
    for name in TL.TINY:
        assert model_from_config(TL.TINY[name][0])[0].to_dict() == TL.TINY[name][0]
    names = expected_tensors(spec)
    assert names["embed"] == (211, 64) and names["head"] == (211, 64) and names["final.norm"] == (64,)
    assert names["l0.mix.q"] == (128, 64) and names["l0.mix.k"] == (64, 64) and names["l0.mix.v"] == (48, 64)
    assert names["l0.mix.o"] == (64, 96) and names["l0.mix.q.norm"] == (16,) and names["l0.mix.lk2"] == (16,)
    assert names["l0.mlp.router"] == (4, 64) and names["l0.mlp.correction"] == (4,)
    assert names["l0.mlp.e3.gate"] == (24, 64) and names["l0.mlp.e3.down"] == (64, 24)
    assert not any(n.startswith(("l1.mlp", "l1.norm2", "l1.ls2", "l0.mlp.shared", "l0.mix.g")) for n in names)
    assert names["l2.mix.q"] == (64, 64) and names["l2.mix.k"] == (32, 64) and names["l2.mix.g"] == (4, 64)
    assert names["l2.mlp.gate"] == (40, 64) and names["l2.ls2"] == (64,) and names["l1.ls1"] == (64,)
    names = expected_tensors(model_from_config(TL.LZ_B)[1])
    assert names["l0.mlp.router"] == (16, 128) and names["l0.mlp.correction"] == (16,)
    assert "l0.mlp.e13.up" in names and "l0.mlp.e14.up" not in names and names["l0.mlp.shared.down"] == (128, 48)
    inits = tensor_inits(spec)
    assert inits["l0.ls1"] == "gain" and inits["l0.mix.q.norm"] == "gain" and inits["l2.norm2"] == "gain"


@pytest.mark.parametrize("change,word", [
    (lambda c: c.update(bogus=1), "bogus"),
    (lambda c: c["layers"][0]["mixer"].update(softcap=3.0), "softcap"),
    (lambda c: c["layers"][0].update(type="recurrent"), "recurrent"),
    (lambda c: c["layers"][2]["mlp"].update(kind="glu"), "glu"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv_heads"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=7), "dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=18), "dims"),
    (lambda c: c["layers"][2]["mixer"].update(diff=0.5), "diff"),
    (lambda c: c["layers"][0]["mixer"].update(rot={"base": 10.0, "dims": 4}), "rot"),
    (lambda c: c["layers"][0]["mixer"].pop("diff"), "diff"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=2, keep=3), "groups"),
    (lambda c: c["layers"][0]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(noise=0.1), "noise"),
    (lambda c: c["norm"].pop("eps"), "eps"),
])
def test_config_errors_name_the_key(change, word):
    c = copy.deepcopy(TL.LZ_A)
    change(c)
    with pytest.raises(ConfigError) as e:
        model_from_config(c)
    assert word in str(e.value)


@pytest.mark.parametrize("name", sorted(TL.TINY))
def test_cache_needs_follow_the_mixers(name):
    raw = TL.TINY[name][0]
    cfg, spec = model_from_config(raw)
    needs = cache_needs(spec)
    assert [e.layer for e in spec.schedule] == list(range(len(raw["layers"])))
    for layer, need in zip(raw["layers"], needs):
        m = layer["mixer"]
        maps = 2 if layer["type"] == "attention" else 1
        assert isinstance(need, KVNeed) and need.window is None
        assert need.n_kv_heads == maps * m["kv_heads"] and need.head_dim >= max(m["dim"], m["vdim"])


def test_the_plain_router():
    z = torch.tensor([2.0, 1.0, 0.5, 0.0, 1.9, -1.0], dtype=torch.float64)
    none = torch.zeros(6, dtype=torch.float64)
    assert PL.route(z, none, 2, 1, 1)[0] == [0, 4]
    assert PL.route(z, none, 2, 3, 1)[0] == [0, 1]                       # the best group alone: experts 0 and 1
    assert PL.route(z, none, 2, 2, 1)[0] == [0, 1]                       # groups of three
    corr = torch.tensor([-1.0, 0.0, 0.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    chosen, w = PL.route(z, corr, 2, 1, 1)
    s = torch.softmax(z, 0)
    assert chosen == [4, 1] and abs(sum(w) - 1.0) < 1e-12 and abs(w[0] - float(s[4] / (s[4] + s[1]))) < 1e-12
    # a group whose members' choice scores are all negative still beats no group: it is kept, not treated as zero
    corr = torch.full((6,), -2.0, dtype=torch.float64)
    assert PL.route(z, corr, 1, 3, 1)[0] == [0]


def test_the_planted_key_matters(tmp_path):
    """on the plain model: without the needle a probe's logits move by far more than any tolerance of the GPU tests"""
    for name in sorted(TL.TINY):
        raw = TL.TINY[name][0]
        folder = TL.make_model(tmp_path, name, "float32")
        cfg, w = PL.load_model(folder)
        rng = random.Random(1)
        toks = TL.needle_request(raw["vocab"], 90, 5, [88, 89], rng)
        other = list(toks)
        other[5] = 7
        a, b = PL.forward(cfg, w, toks).numpy(), PL.forward(cfg, w, other).numpy()
        assert tiny.rel_err(a[88:], b[88:]) > 0.3, name


def _kernel_view_of_the_mixer(part, h):
    """what the kernels compute from the part's re-laid weights, written with tensor operations in 64-bit: heads by the
    plain grouped-query rule, rotate-half on the first ``rot`` elements, the norm per head over the true size"""
    T = h.shape[0]
    hd, nhq, nkvq = part.hd, part.nhq, part.nkvq
    rows = h @ part.wqkv.double().T
    q = rows[:, :nhq * hd].view(T, nhq, hd)
    k = rows[:, nhq * hd:(nhq + nkvq) * hd].view(T, nkvq, hd)
    v = rows[:, (nhq + nkvq) * hd:part.n_main].view(T, nkvq, hd)
    pos = torch.arange(T, dtype=torch.float64)

    def norm(x, gain):
        x = x / torch.sqrt((x * x).sum(-1, keepdim=True) / part.qk_dim + part.norm_eps)
        return x if gain is None else x * gain.double()

    def rotate(x):
        half = part.rot // 2
        if not half:
            return x
        ang = pos[:, None] * part.inv_freq64[None, :half]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
        a, b = x[..., :half], x[..., half:part.rot]
        return torch.cat([a * c - b * s, b * c + a * s, x[..., part.rot:]], dim=-1)

    if part.norm_when == "before":
        q, k = rotate(norm(q, part.gq)), rotate(norm(k, part.gk))
    else:
        q, k = norm(rotate(q), part.gq), norm(rotate(k), part.gk)
    if part.t_coef:
        q = q * PL.query_temperature(T, part.t_coef, part.t_every).view(T, 1, 1)
    r = nhq // nkvq
    att = torch.stack([PL.causal_softmax_attention(q[:, j], k[:, j // r], v[:, j // r], part.scale)
                       for j in range(nhq)], dim=1)                         # [T, nhq, hd]
    if part.diff is not None:
        lam, eps, mult = part.diff
        a = att.view(T, part.nkv, 2, part.group, hd)
        o = (a[:, :, 0] - lam * a[:, :, 1]).reshape(T, part.nh, hd)
        out = torch.zeros_like(o)
        out[..., :part.v_dim] = PL.rms(o[..., :part.v_dim], eps) * mult
        att = out
    elif part.has_gate:
        att = att * PL.sigmoid(rows[:, part.n_main:part.n_main + part.nh])[:, :, None]
    return att.reshape(T, -1) @ part.wo.double().T


@pytest.mark.parametrize("name", sorted(TL.TINY))
def test_the_mixers_weight_layouts_compute_the_plain_mixers(tmp_path, name):
    raw = TL.TINY[name][0]
    folder = TL.make_model(tmp_path, name, "float32")
    cfg, w = PL.load_model(folder)
    _, spec = model_from_config(cfg)
    g = torch.Generator().manual_seed(5)
    h = torch.randn(21, raw["width"], generator=g, dtype=torch.float64)
    for i, layer in enumerate(raw["layers"]):
        ms = spec.layers[i].block["mixer"]
        part = part_class("mixer", ms.kind)(ms, raw["width"], WeightView(w, "l%d.mix." % i), dtype=torch.float32,
                                            device=torch.device("cpu"))
        plain = PL.differential_attention if layer["type"] == "attention" else PL.gated_rotary_attention
        want = plain(w, "l%d.mix." % i, cfg["layers"][i]["mixer"], h, raw["norm"]["eps"])
        got = _kernel_view_of_the_mixer(part, h)
        assert float((got - want).abs().max()) < 1e-9 * max(1.0, float(want.abs().max())), (name, i)
