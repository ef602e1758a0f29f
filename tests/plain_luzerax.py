"""A plain, slow implementation of the Luzerax decoder: one function per mechanism, 64-bit, whole sequences, no cache.

It shares no code with the library: tensors come as a ``{name: tensor}`` mapping, sizes and constants from the nested
configuration (a dict shaped like config.json). Every function works on ONE sequence given from its first token on;
attention is an explicit loop over the queries, each reduced over its visible keys.

Notation: ``h`` is a mixer's or feed-forward's input ``[T, width]``; linear weights are ``[out, in]``.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Mapping

import torch

F64 = torch.float64


def load_model(model_dir: str):
    """(the JSON object of config.json, {name: tensor}) of a model folder"""
    from safetensors.torch import load_file
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(model_dir, "model.safetensors"))


def _w(t: Mapping[str, torch.Tensor], name: str) -> torch.Tensor:
    return t[name].to(F64)


def sigmoid(x):
    return 1.0 / (1.0 + torch.exp(-x))


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis"""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def causal_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float) -> torch.Tensor:
    """q [T, d], k [T, d], v [T, dv] of one head: row i is softmax_j<=i(scale q_i . k_j) v"""
    T = q.shape[0]
    out = torch.zeros((T, v.shape[1]), dtype=F64)
    for i in range(T):
        s = (k[: i + 1] @ q[i]) * scale
        p = torch.exp(s - s.max())
        out[i] = (p / p.sum()) @ v[: i + 1]
    return out


def query_temperature(T: int, coef: float, every: int) -> torch.Tensor:
    """[T]: 1 + coef ln(floor((p + 1) / every) + 1)"""
    return torch.tensor([1.0 + coef * math.log((p + 1) // every + 1) for p in range(T)], dtype=F64)


def differential_lambda(t, p: str, diff: float) -> float:
    a = math.exp(float((_w(t, p + "lq1") * _w(t, p + "lk1")).sum()))
    b = math.exp(float((_w(t, p + "lq2") * _w(t, p + "lk2")).sum()))
    return a - b + diff


def differential_attention(t, p: str, m: Mapping, h: torch.Tensor, eps: float) -> torch.Tensor:
    """two softmax maps per head over the same values, the second subtracted lambda times; no rotation"""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    diff = float(m["diff"])
    q = (h @ _w(t, p + "q").T).view(T, H, 2, d)
    k = (h @ _w(t, p + "k").T).view(T, G, 2, d)
    v = (h @ _w(t, p + "v").T).view(T, G, dv)
    q = rms(q, eps) * _w(t, p + "q.norm")
    k = rms(k, eps) * _w(t, p + "k.norm")
    temp = query_temperature(T, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))
    q = q * temp.view(T, 1, 1, 1)
    lam = differential_lambda(t, p, diff)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        a1 = causal_softmax_attention(q[:, hh, 0], k[:, g, 0], v[:, g], float(m["scale"]))
        a2 = causal_softmax_attention(q[:, hh, 1], k[:, g, 1], v[:, g], float(m["scale"]))
        heads.append(rms(a1 - lam * a2, eps) * (1.0 - diff))
    return torch.cat(heads, dim=1) @ _w(t, p + "o").T


def rotate_interleaved(x: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, n, d]: on the first ``dims`` elements of every head the pair (2i, 2i + 1) at position p turns by
    p base^(-2i / dims); the rest passes"""
    T = x.shape[0]
    out = x.clone()
    pos = torch.arange(T, dtype=F64)
    for i in range(dims // 2):
        a = pos * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a).view(T, 1), torch.sin(a).view(T, 1)
        u, w = x[:, :, 2 * i], x[:, :, 2 * i + 1]
        out[:, :, 2 * i] = u * c - w * s
        out[:, :, 2 * i + 1] = w * c + u * s
    return out


def gated_rotary_attention(t, p: str, m: Mapping, h: torch.Tensor, eps: float) -> torch.Tensor:
    """rotation of adjacent pairs, then a unit RMS per head on q and k, softmax attention, a sigmoid gate per head"""
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = (h @ _w(t, p + "q").T).view(T, H, d)
    k = (h @ _w(t, p + "k").T).view(T, G, d)
    v = (h @ _w(t, p + "v").T).view(T, G, dv)
    base, dims = float(m["rot"]["base"]), int(m["rot"]["dims"])
    q = rms(rotate_interleaved(q, base, dims), eps)
    k = rms(rotate_interleaved(k, base, dims), eps)
    gate = sigmoid(h @ _w(t, p + "g").T)                                   # [T, H]
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        heads.append(causal_softmax_attention(q[:, hh], k[:, g], v[:, g], float(m["scale"])) * gate[:, hh:hh + 1])
    return torch.cat(heads, dim=1) @ _w(t, p + "o").T


def dense_feed_forward(t, p: str, h: torch.Tensor) -> torch.Tensor:
    g = h @ _w(t, p + "gate").T
    return (g * sigmoid(g) * (h @ _w(t, p + "up").T)) @ _w(t, p + "down").T


def clamped_expert(t, p: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ _w(t, p + "gate").T, max=limit)
    u = torch.clamp(h @ _w(t, p + "up").T, min=-limit, max=limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ _w(t, p + "down").T


def route(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int):
    """z [n] router logits of one row -> (chosen indices, weights): softmax over all, choice by score + correction
    inside the ``keep`` best of ``groups`` groups of neighbours, weights the chosen scores over their sum"""
    n = z.numel()
    s = torch.exp(z - z.max())
    s = s / s.sum()
    c = s + correction
    size = n // groups
    best = sorted(range(groups), key=lambda g: (-float(c[g * size:(g + 1) * size].max()), g))[:keep]
    allowed = [e for e in range(n) if e // size in best]
    chosen = sorted(allowed, key=lambda e: (-float(c[e]), e))[:top]
    total = sum(float(s[e]) for e in chosen) + 1e-20
    return chosen, [float(s[e]) / total for e in chosen]


def route_margin(z: torch.Tensor, correction: torch.Tensor, top: int, groups: int, keep: int,
                 weight: float = 0.02) -> float:
    """how far the row is from another pick that would matter: the gap between the last choice score that was taken
    and the best that was not (experts inside the kept groups, and the groups' own scores), counted only where the
    experts that would change places hold more than ``weight`` of the chosen ones' scores"""
    n = z.numel()
    s = torch.exp(z - z.max())
    s = s / s.sum()
    c = s + correction
    size = n // groups
    chosen, _ = route(z, correction, top, groups, keep)
    total = sum(float(s[e]) for e in chosen) + 1e-20
    order = sorted(range(groups), key=lambda g: (-float(c[g * size:(g + 1) * size].max()), g))
    margin = float("inf")
    if keep < groups:
        last, nxt = order[keep - 1], order[keep]
        moved = max(float(s[e]) for g in (last, nxt) for e in range(g * size, (g + 1) * size))
        if moved > weight * total:
            margin = float(c[last * size:(last + 1) * size].max() - c[nxt * size:(nxt + 1) * size].max())
    rest = [e for e in range(n) if e // size in order[:keep] and e not in chosen]
    if rest:
        k = min(chosen, key=lambda e: float(c[e]))
        u = max(rest, key=lambda e: float(c[e]))
        if max(float(s[k]), float(s[u])) > weight * total:
            margin = min(margin, float(c[k] - c[u]))
    return margin


def expert_feed_forward(t, p: str, f: Mapping, h: torch.Tensor, margins: list = None) -> torch.Tensor:
    """``margins`` (a list) receives a tensor [T]: every row's ``route_margin``"""
    r = f["router"]
    E, n_id, top = int(r["experts"]), int(r["identity"]), int(r["top"])
    limit = float(f["expert"]["limit"])
    z = h @ _w(t, p + "router").T
    corr = _w(t, p + "correction")
    out = torch.zeros_like(h)
    for i in range(h.shape[0]):
        chosen, wts = route(z[i], corr, top, int(r["groups"]["count"]), int(r["groups"]["keep"]))
        for e, w in zip(chosen, wts):
            if e >= E:
                out[i] += w * h[i]                       # an identity expert
            else:
                out[i] += w * clamped_expert(t, p + "e%d." % e, h[i:i + 1], limit)[0]
    if margins is not None:
        margins.append(torch.tensor([route_margin(z[i], corr, top, int(r["groups"]["count"]), int(r["groups"]["keep"]))
                                     for i in range(h.shape[0])], dtype=F64))
    if f.get("shared"):
        out = out + clamped_expert(t, p + "shared.", h, float(f["shared"]["limit"]))
    return out


def forward(cfg: Mapping, t: Mapping[str, torch.Tensor], tokens: List[int], residuals: list = None,
            margins: list = None) -> torch.Tensor:
    """logits [T, vocab] of one sequence; ``residuals`` (a list) receives the stream after every layer, ``margins`` (a
    list) every routed layer's ``route_margin`` per row"""
    eps = float(cfg["norm"]["eps"])
    x = _w(t, "embed")[torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        p = "l%d." % i
        mix = differential_attention if layer["type"] == "attention" else gated_rotary_attention
        x = x + rms(mix(t, p + "mix.", layer["mixer"], x, eps), eps) * _w(t, p + "norm1") * _w(t, p + "ls1")
        f = layer.get("mlp")
        if f is not None:
            y = dense_feed_forward(t, p + "mlp.", x) if f["kind"] == "dense" else \
                expert_feed_forward(t, p + "mlp.", f, x, margins)
            x = x + rms(y, eps) * _w(t, p + "norm2") * _w(t, p + "ls2")
        if residuals is not None:
            residuals.append(x.clone())
    return (rms(x, eps) * _w(t, "final.norm")) @ _w(t, "head").T
