"""Small Medodra configurations with seeded random weights for the tests, with one key that stands out.

The configurations differ in every size and option: the order of the two kinds of layer, a repeated stretch over the
middle, over everything, over one layer, and none; head counts and groups (one key/value head, one per query head),
values wider and narrower than keys, head sizes the tensor-core kernels take and sizes no vector load takes, short
convolutions of one tap (a factor per channel) to five and none at all, distance tables of 6 to 32 rows whose last row begins below, at and above a
cache page and at a distance that is no integer, temperatures that switch on at every position, late and never, one
to all experts per token, layers with and without a shared expert or a feed-forward at all, residual multipliers
and embedding scales above and below one.
"""
from __future__ import annotations

import json
import math
import os
import random
from typing import List

NEEDLE, PROBE = 3, 4            # token ids: the needle's key stands out for every probe's query
CODE = 6.0                      # the size of the planted embedding features, far above the random ones


def _moe(experts, top, ff, shared=None):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
            "shared": None if shared is None else {"ff": shared}}


def _par(heads, kv, dim, vdim, conv, scale, far, coef, every, right, mlp=None, rows=16):
    left = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv, "scale": scale, "bias_max": far,
            "q_temp": {"coef": coef, "every": every}}
    if conv is None:
        del left["conv"]
    return {"type": "parallel", "mixer": {"left": left, "right": {"width": right}}, "mlp": mlp, "_rows": rows}


def _delta(heads, kv, dim, vdim, conv, mlp=None):
    mixer = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "conv": conv}
    if conv is None:
        del mixer["conv"]
    return {"type": "delta", "mixer": mixer, "mlp": mlp}


def _config(vocab, width, eps, emb_scale, mult, layers, loop=None):
    cfg = {"architecture": "Medodra", "vocab": vocab, "width": width, "norm": {"eps": eps},
           "embedding": {"scale": emb_scale}, "residual_mult": mult, "layers": layers}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# A: small everything, no repeated stretch; values wider than keys; a table of 8 rows whose last row begins well
#    below a page; a layer without feed-forward, one without a shared expert; a delta layer with two taps
MD_A = _config(211, 64, 1e-5, 1.7, 1.0, [
    _par(4, 2, 16, 24, 3, 0.3, 40, 0.5, 16, 48, _moe(4, 2, 24, 16), rows=8),
    _delta(4, 2, 16, 8, 2),
    _par(2, 1, 16, 24, 2, 0.25, 33, 0.2, 7, 32, _moe(3, 1, 40), rows=10)])
# B: head size 64 (the tensor-core attention kernel runs in bfloat16), three query heads per key/value head, the
#    middle two layers three times, four taps, a delta layer with a key head per value head, three experts of eight
MD_B = _config(300, 128, 1e-6, 0.6, 0.5, [
    _delta(4, 4, 32, 64, 4, _moe(8, 3, 32, 48)),
    _par(6, 2, 64, 64, 4, 0.125, 100, 0.3, 64, 128, _moe(8, 3, 32, 48), rows=16),
    _delta(2, 1, 64, 32, 3, _moe(2, 1, 64)),
    _par(2, 2, 64, 64, 3, 0.11, 64, 0.4, 100, 96, None, rows=12)], loop=(1, 3, 3))
# C: head size 128 with values of 64 (widened in the cache), one key/value head, convolutions of one tap and none, everything
#    twice, a table of 32 rows that reaches far beyond a page, a temperature that grows from the first position on,
#    all experts chosen, a width that is no power of two
MD_C = _config(257, 200, 2e-6, 14.142, 0.7, [
    _par(4, 1, 128, 64, 1, 0.09, 300, 0.1, 1, 200, _moe(2, 2, 136, 72), rows=32),
    _delta(3, 3, 24, 40, None, _moe(2, 2, 136, 72)),
    _delta(2, 1, 128, 16, 1, None),
    _par(4, 1, 128, 64, None, 0.08, 129, 0.15, 2, 104, _moe(6, 4, 16, 8), rows=20)], loop=(0, 4, 2))
# D: sizes that no vector load or tensor-core tile takes: width 72, heads of 24 with values of 10, a key/value head per
#    query head, five taps, a table of 6 rows whose last row begins at a distance that is no integer, no temperature,
#    one layer four times, a delta head of 40 with values of 9
MD_D = _config(131, 72, 1e-5, 1.0, 0.25, [
    _par(5, 5, 24, 10, 5, 0.2, 7.5, 0.0, 3, 20, _moe(5, 2, 20, 12), rows=6),
    _delta(3, 1, 40, 9, 5, _moe(5, 2, 20)),
    _par(3, 1, 10, 24, 3, 0.3, 17, 0.9, 5, 72, None, rows=7)], loop=(1, 2, 4))
# E: a head size of 96 (keys 48, values 96), a table whose last row begins far away, one pass "repeated" once, a
#    delta layer first and last
MD_E = _config(401, 160, 1e-5, 2.5, 1.5, [
    _delta(2, 1, 64, 32, 3, _moe(4, 1, 64, 32)),
    _par(4, 2, 48, 96, 3, 0.14, 1000, 0.5, 128, 160, _moe(4, 1, 64, 32), rows=12),
    _delta(4, 2, 32, 48, 4, _moe(3, 2, 24, 40))], loop=(0, 2, 1))
TINY = {"A": (MD_A, 31), "B": (MD_B, 32), "C": (MD_C, 33), "D": (MD_D, 34), "E": (MD_E, 35)}


def config(name: str) -> dict:
    """the config.json object of a configuration (the row counts of the distance tables are the tensors' own)"""
    cfg = json.loads(json.dumps(TINY[name][0]))
    for l in cfg["layers"]:
        l.pop("_rows", None)
    return cfg


def planted_columns(width: int):
    """(needle's column, probe's column): even columns near the end, where the position vector's sine is almost zero
    over any length these tests use"""
    return width - 2, width - 4


def make_model(tmp_path, name: str, dtype: str = "bfloat16", strength: float = 12.0) -> str:
    """a model folder with seeded random weights in which every mechanism moves the logits by far more than rounding:

    * attention without a softmax: a PROBE token's query against a NEEDLE token's key scores about ``strength`` in
      the query heads of the first key/value head, wherever the two stand, while the per-head constants sit near -5,
      so that an ordinary key weighs about 0.01 and the needle about 1: a probe row's output is the needle's value
      even among hundreds of keys. The distance table is drawn from N(0, 1): a key in a wrong row of it changes its
      weight by a factor of e.
    * short convolutions: taps drawn from N(0, 0.5) (the planted channels read the current token only), biases from
      N(0, 0.1).
    * recurrences that remember: the delta rule's decays lie between exp(-0.0017) and exp(-0.25) per token, the
      minGRU's update gates around sigmoid(-2.5), so a state that is lost or taken from another sequence shows for
      hundreds of tokens.
    * the product that begins a pass keeps most of the stream and mixes the embedding output in.

    How the needle is planted: its embedding row has one large feature (an even column near the end, where the
    position vector is almost zero), a probe's another; the key projection of the first key/value head reads the
    first into its last dimension, the query projections of that group's heads read the second into the same
    dimension; no branch writes into the two columns."""
    import torch
    from kindi_b200.config.registry import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    from kindi_b200.weights.safetensors_io import write_file
    raw, seed = TINY[name]
    cfg = config(name)
    d = os.path.join(str(tmp_path), "md_%s_%s" % (name, dtype))
    if os.path.isfile(os.path.join(d, "model.safetensors")):
        return d
    os.makedirs(d, exist_ok=True)
    _, spec = model_from_config(cfg)
    shapes = dict(expected_tensors(spec))
    for i, l in enumerate(raw["layers"]):
        if l["type"] == "parallel":
            shapes["l%d.mix.left.rel" % i] = (l["_rows"], l["mixer"]["left"]["heads"])
    t = random_tensors(shapes, seed, dtype=torch.float32, inits=tensor_inits(spec))
    g = torch.Generator().manual_seed(seed + 1)
    width, s = cfg["width"], cfg["embedding"]["scale"]
    cn, cp = planted_columns(width)
    emb = t["embed"]
    emb[:, cn] = 0.0
    emb[:, cp] = 0.0
    emb[NEEDLE, cn] = CODE / s
    emb[PROBE, cp] = CODE / s
    # what the first norm makes of a planted feature: CODE over the root mean square of a row that holds it, the
    # position vector (mean square one half) and small random features
    feature = CODE / math.sqrt((CODE * CODE + width * (0.5 + (0.02 * s) ** 2)) / width)
    for n in list(t):
        if n.endswith(".conv"):
            t[n] = 0.5 * torch.randn(t[n].shape, generator=g)
        elif n.endswith(".b") and t[n].dim() == 1:
            t[n] = 0.1 * torch.randn(t[n].shape, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        m, p = layer["mixer"], "l%d.mix." % i
        if layer["type"] == "parallel":
            a = m["left"]
            H, G, dim = a["heads"], a["kv_heads"], a["dim"]
            at = dim - 1
            q, k, v = t[p + "left.q"], t[p + "left.k"], t[p + "left.v"]
            k[at, :] = 0.0
            k[at, cn] = 1.0
            t[p + "left.k.b"][at] = 0.0
            v[:, cn] = 0.25 * torch.sign(v[:, 0])
            for h in range(H // G):
                q[h * dim + at, :] = 0.0
                q[h * dim + at, cp] = strength / (a["scale"] * feature * feature)
                t[p + "left.q.b"][h * dim + at] = 0.0
                if a.get("conv"):
                    t[p + "left.q.conv"][h * dim + at] = 0.0
                    t[p + "left.q.conv"][h * dim + at, -1] = 1.0
            if a.get("conv"):
                t[p + "left.k.conv"][at] = 0.0
                t[p + "left.k.conv"][at, -1] = 1.0
            t[p + "left.rel"] = torch.randn(t[p + "left.rel"].shape, generator=g)
            t[p + "left.pb"] = -5.0 + 0.5 * torch.randn(H, generator=g)
            t[p + "right.z.b"] = -2.5 + torch.randn(m["right"]["width"], generator=g)
        else:
            H = m["heads"]
            t[p + "A_log"] = -6.0 + 5.0 * torch.rand(H, generator=g)
            t[p + "dt_bias"] = 0.5 * torch.randn(H, generator=g)
    if "loop.in" in t:
        w = 0.02 * torch.randn(width, 2 * width, generator=g)
        w[:, :width] += 0.7 * torch.eye(width)
        w[:, width:] += 0.5 * torch.eye(width)
        for c in (cn, cp):
            w[c, :] = 0.0
            w[:, c] = 0.0
            w[:, width + c] = 0.0
            w[c, c] = 0.7
            w[c, width + c] = 0.5
        t["loop.in"] = w
    # no branch writes into the planted columns: what the planted keys and queries read stays the tokens' own
    for n in list(t):
        if n.endswith(".o") or n.endswith(".down"):
            t[n][cn, :] = 0.0
            t[n][cp, :] = 0.0
        if n.endswith(".o.b"):
            t[n][cn] = 0.0
            t[n][cp] = 0.0
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    t = {n: v.to(tdt).contiguous() for n, v in t.items()}
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_file(os.path.join(d, "model.safetensors"), t, metadata={"format": "pt"})
    return d


def needle_request(vocab: int, length: int, needle_at: int, probes: List[int], rng: random.Random) -> List[int]:
    """random tokens (neither needle nor probe) with the needle at `needle_at` and probes at the listed places"""
    toks = []
    for i in range(length):
        t = rng.randrange(vocab)
        while t in (NEEDLE, PROBE):
            t = rng.randrange(vocab)
        toks.append(NEEDLE if i == needle_at else PROBE if i in probes else t)
    return toks
