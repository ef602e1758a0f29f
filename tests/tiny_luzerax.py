"""Small Luzerax configurations with seeded random weights for the tests, with one key that stands out.

The configurations differ in every size and option: the order of the two mixers, head counts and groups (one
key/value head, one per query head), values wider and narrower than keys, head sizes the tensor-core kernels take and
sizes no vector load takes, rotations of the whole head and of a part, temperatures that switch on at the first
position, late and never, dense feed-forwards, none at all, and experts with one group and several, with and without
identity experts, a correction and a shared expert, one pick a row and several.
"""
from __future__ import annotations

import json
import os
import random
from typing import List

NEEDLE, PROBE = 3, 4            # token ids: the needle's key stands out for every probe's query
CODE = 3.0                      # the size of the planted embedding features, far above the random ones
KEPT = 10                       # the stream's first columns keep the token's own features through all layers


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, groups, keep, ff, limit, shared=None):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit},
            "router": {"experts": experts, "identity": identity, "top": top, "groups": {"count": groups, "keep": keep}},
            "shared": None if shared is None else {"ff": shared[0], "limit": shared[1]}}


def _diff(heads, kv, dim, vdim, scale, diff, coef, every, mlp=None):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff,
                      "q_temp": {"coef": coef, "every": every}}}


def _rot(heads, kv, dim, vdim, scale, base, dims, mlp=None):
    return {"type": "attention_2", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
                      "rot": {"base": base, "dims": dims}}}


def _config(vocab, width, eps, layers):
    return {"architecture": "Luzerax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A: small everything; two differential layers in a row; values wider than keys; half of a head rotated; experts in
#    one group without identity experts or a shared expert; a layer without a feed-forward
LZ_A = _config(211, 64, 1e-5, [
    _diff(4, 2, 16, 24, 0.5, 0.55, 0.5, 16, _moe(4, 0, 2, 1, 1, 24, 0.7)),
    _diff(2, 1, 16, 8, 0.45, 0.3, 0.25, 7),
    _rot(4, 2, 16, 24, 0.6, 10000.0, 8, _dense(40))])
# B: head size 64 (the tensor-core attention kernels run in bfloat16), three query heads per key/value head, whole
#    heads rotated, a temperature from the first position on, 14 experts and two identity experts in four groups of
#    which two are kept, four picks a row, a shared expert with a limit of its own
LZ_B = _config(300, 128, 1e-6, [
    _rot(6, 2, 64, 64, 0.16, 500000.0, 64, _moe(14, 2, 4, 4, 2, 32, 1.2, (48, 2.0))),
    _diff(4, 2, 64, 64, 0.15, 0.5, 0.4, 1, _dense(96)),
    _rot(2, 2, 64, 64, 0.14, 500000.0, 64),
    _diff(6, 2, 64, 64, 0.17, 0.2, 0.1, 50, _moe(14, 2, 4, 4, 2, 32, 1.2, (48, 2.0)))])
# C: head size 128 with values of 64 (widened in the cache), one key/value head, a differential layer with a key/value
#    head per query head, a temperature that never switches on, a width that is no power of two, six experts and two
#    identity experts in four groups of two with three kept, a quarter of the head rotated
LZ_C = _config(257, 200, 2e-6, [
    _diff(2, 2, 128, 64, 0.09, 0.6, 0.3, 100000, _moe(6, 2, 2, 4, 3, 40, 3.0, (24, 0.5))),
    _rot(4, 1, 128, 64, 0.1, 10000.0, 32, _dense(136)),
    _diff(4, 1, 128, 64, 0.08, 0.45, 1.5, 33, _moe(6, 2, 2, 4, 3, 40, 3.0, (24, 0.5)))])
# D: sizes that no vector load or tensor-core tile takes: width 72, heads of 24 with values of 10, a key/value head per
#    query head, six of 24 elements rotated, five experts of 20 and one identity expert in three groups of two with one
#    kept (a row picks the whole group), ONE layer kind only at the start
LZ_D = _config(131, 72, 1e-5, [
    _rot(5, 5, 24, 10, 0.25, 30000.0, 6, _moe(5, 1, 2, 3, 1, 20, 1.0)),
    _rot(3, 1, 24, 10, 0.2, 100.0, 24, _dense(20)),
    _diff(3, 3, 10, 24, 0.9, 0.4, 0.3, 5, _moe(5, 1, 2, 3, 1, 20, 1.0, (12, 1.5)))])
# E: values far wider than keys, one pick a row, more identity experts than the kept groups hold experts, every group
#    kept, no rotation at all in a rotated layer's configuration (dims 0)
LZ_E = _config(401, 160, 1e-5, [
    _diff(8, 4, 32, 80, 0.3, 0.35, 0.6, 64, _moe(5, 3, 1, 2, 2, 64, 0.9, (32, 0.9))),
    _rot(8, 2, 32, 16, 0.2, 1000000.0, 0, _moe(9, 3, 3, 3, 2, 16, 1.1))])
TINY = {"A": (LZ_A, 31), "B": (LZ_B, 32), "C": (LZ_C, 33), "D": (LZ_D, 34), "E": (LZ_E, 35)}


def make_model(tmp_path, name: str, dtype: str = "bfloat16", strength: float = 12.0) -> str:
    """a model folder with random weights N(0, 0.02) (gains and layer scales around one) in which the score of a PROBE
    token's query against a NEEDLE token's key stands out in every attention layer, wherever the two stand.

    How: the needle's embedding row has one large feature (column 0), a probe's another (column 1), and no branch
    writes into those columns with a changed sign. The key projection of the first key/value head (its first map, in a
    differential layer) reads column 0 into its last dimension with a weight far above the random ones, and the query
    projections of that group's heads read column 1 into the same dimension: after the heads' norms both are about
    sqrt(dim) in that dimension, and the layer's scale is set so that the score is ``strength``. The value projection
    reads column 0 with a large weight. The routers read nothing but eight further kept columns, which hold features of
    the token's own of size one: a row's picks then follow from its token with logits of ordinary size, the correction
    changes them, and the 16-bit rounding of activations cannot (the products of stored numbers are exact in both
    implementations). Lambda stays within a tenth of ``diff``, and ``diff`` well below one: where both maps see the same few keys (a sequence's first positions) the head is ``(1 - lambda)`` times a value, and 16-bit rounding of the maps' outputs is amplified by ``1 / (1 - lambda)``. With plain random weights attention is nearly
    uniform, and a key that is dropped moves the logits by less than the rounding error of bfloat16."""
    import torch
    from kindi_b200.config.registry import model_from_config
    from kindi_b200.parts.model import expected_tensors, tensor_inits
    from kindi_b200.weights.random_init import random_tensors
    from kindi_b200.weights.safetensors_io import write_file
    cfg, seed = TINY[name]
    cfg = json.loads(json.dumps(cfg))
    d = os.path.join(str(tmp_path), "lz_%s_%s" % (name, dtype))
    if os.path.isfile(os.path.join(d, "model.safetensors")):
        return d
    os.makedirs(d, exist_ok=True)
    for layer in cfg["layers"]:
        layer["mixer"]["scale"] = strength / layer["mixer"]["dim"]
    _, spec = model_from_config(cfg)
    t = random_tensors(expected_tensors(spec), seed, dtype=torch.float32, inits=tensor_inits(spec))
    emb = t["embed"]
    g = torch.Generator().manual_seed(seed + 1)
    emb[:, 0:2] = 0.0
    emb[NEEDLE, 0] = CODE
    emb[PROBE, 1] = CODE
    emb[:, 2:KEPT] = torch.randn(emb.shape[0], KEPT - 2, generator=g)
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        p = "l%d.mix." % i
        H, G, dim = m["heads"], m["kv_heads"], m["dim"]
        maps = 2 if layer["type"] == "attention" else 1
        at = dim - 1
        t[p + "k"][at, :] = 0.0
        t[p + "k"][at, 0] = 1.0
        t[p + "v"][:, 0] = 0.25 * torch.sign(t[p + "v"][:, 1])
        for h in range(H // G):
            t[p + "q"][h * maps * dim + at, :] = 0.0
            t[p + "q"][h * maps * dim + at, 1] = 1.0
        if layer["type"] == "attention":
            for n in ("q.norm", "k.norm"):
                t[p + n][at] = 1.0
            for n in ("lq1", "lk1", "lq2", "lk2"):
                t[p + n] = 0.3 * torch.randn(dim, generator=g) / dim ** 0.5
        f = layer["mlp"]
        if f is not None and f["kind"] == "moe":
            q = "l%d.mlp." % i
            t[q + "router"][:] = 0.0
            t[q + "router"][:, 2:KEPT] = 0.6 * torch.randn(t[q + "router"].shape[0], KEPT - 2, generator=g)
            t[q + "correction"] = 0.1 * torch.randn(t[q + "correction"].shape, generator=g)
    # the needle's and the probes' own picks are no close calls (they stand in every request): their kept features are
    # drawn again until every routed layer picks with a clear gap, also when an identity expert has stretched them
    from plain_luzerax import route_margin
    routed = [(t["l%d.mlp.router" % i].double(), t["l%d.mlp.correction" % i].double(), l["mlp"]["router"])
              for i, l in enumerate(cfg["layers"]) if l["mlp"] is not None and l["mlp"]["kind"] == "moe"]
    for tok in (NEEDLE, PROBE):
        for _ in range(500):
            feat = emb[tok].double()
            if all(route_margin(wr @ feat * sc, corr, r["top"], r["groups"]["count"], r["groups"]["keep"], 0.0) >= 0.05
                   for wr, corr, r in routed for sc in (0.7, 1.0, 1.4)):
                break
            emb[tok, 2:KEPT] = torch.randn(KEPT - 2, generator=g)
        else:
            raise RuntimeError("no features with clear picks found for token %d" % tok)
    # no branch writes into the kept columns: what the planted keys and queries and the routers read stays the tokens'
    # own (an identity expert hands them through: that changes their size, not their direction)
    for n in list(t):
        if n.endswith(".mix.o") or n.endswith(".down"):
            t[n][0:KEPT, :] = 0.0
    tdt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    t = {n: v.to(tdt) for n, v in t.items()}
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
